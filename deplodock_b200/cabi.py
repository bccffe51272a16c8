"""ctypes binding of ``libemk.so`` — the only route from Python to the kernels.

There is no fallback: if the library is missing or a call fails, an exception is raised. The status-to-exception
mapping mirrors what the reference raises from its CUDA runtime layer (``emmy/compiler/backend/cuda/program.py``:
``ValueError`` for shape/capacity problems ``:379-384``, ``HungKernelError(RuntimeError)`` for a launch that does not
finish ``:525``, ``RuntimeError`` for everything else ``:1027-1031``).
"""

from __future__ import annotations

import ctypes
import threading
from ctypes import c_char_p, c_float, c_int, c_int64, c_void_p
from pathlib import Path

import os

#: ``EMK_BOUNDS_CHECK=1`` selects the bounds-check build of the library (``python -m deplodock_b200.build
#: --bounds-check``): out-of-range token ids, rotary positions and cu_seqlens entries are then reported by
#: ``device_status`` as ``IndexError`` (status ``EMK_ERR_BOUNDS``) instead of being clamped silently
BOUNDS_CHECK = os.environ.get("EMK_BOUNDS_CHECK", "0") not in ("", "0")
LIB_PATH = Path(__file__).resolve().parent / ("libemk_check.so" if BOUNDS_CHECK else "libemk.so")

EMK_OK = 0
EMK_ERR_SHAPE = 1
EMK_ERR_DTYPE = 2
EMK_ERR_ALIGN = 3
EMK_ERR_WORKSPACE = 4
EMK_ERR_CUDA = 5
EMK_ERR_TIMEOUT = 6
EMK_ERR_ARG = 7
EMK_ERR_LIMIT = 8
EMK_ERR_BOUNDS = 9

EMK_F32, EMK_BF16, EMK_F16 = 0, 1, 2
EMK_EW_ADD, EMK_EW_MUL, EMK_EW_SILU, EMK_EW_SILU_MUL = 0, 1, 2, 3
EMK_W_NK, EMK_W_KN = 0, 1
EMK_EPI_NONE, EMK_EPI_RESIDUAL, EMK_EPI_SWIGLU, EMK_EPI_BIAS, EMK_EPI_QKNORM_ROPE = 0, 1, 2, 3, 4


class GemmDesc(ctypes.Structure):
    """``emk_gemm_desc_t`` of ``include/emk.h``."""

    _fields_ = [
        ("x", c_void_p), ("w", c_void_p), ("residual", c_void_p), ("y", c_void_p),
        ("M", c_int64), ("N", c_int64), ("K", c_int64),
        ("wlayout", c_int), ("epilogue", c_int),
        ("row_sumsq_in", c_void_p), ("norm_dim", c_int64), ("norm_eps", c_float),
        ("row_sumsq_out", c_void_p),
        ("q_norm_weight", c_void_p), ("k_norm_weight", c_void_p), ("rope_chunk_major", c_void_p),
        ("seq_len", c_int64), ("num_q_heads", c_int64), ("num_kv_heads", c_int64), ("qk_eps", c_float),
        ("positions", c_void_p),
    ]


class HungKernelError(RuntimeError):
    """A device-side bounded wait expired (reference: ``HungKernelError``, ``backend/cuda/program.py:525``)."""


class EmkLibraryMissing(RuntimeError):
    """``libemk.so`` has not been built; run ``python -m deplodock_b200.build``."""


# name -> (argtypes); every function returns int unless listed in _RESTYPES
_SIGNATURES: dict[str, list] = {
    "emk_version": [],
    "emk_bounds_check_enabled": [],
    "emk_status_string": [c_int],
    "emk_create": [c_int, ctypes.POINTER(c_void_p)],
    "emk_destroy": [c_void_p],
    "emk_last_error": [c_void_p],
    "emk_device_status": [c_void_p, c_void_p],
    "emk_set_wait_limit_ms": [c_void_p, c_int],
    "emk_set_launch_overlap": [c_void_p, c_int],
    "emk_rmsnorm": [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_float, c_int, c_void_p],
    "emk_softmax_lastdim": [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_void_p],
    "emk_linear_bf16": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_int,
                        c_void_p],
    "emk_linear_bf16_simt": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int,
                             c_int, c_void_p],
    "emk_linear_f32_simt": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int,
                            c_void_p],
    "emk_linear_f32_tc_workspace_bytes": [c_int64, c_int64, c_int64],
    "emk_linear_f32_tc": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p,
                          c_int64, c_void_p],
    "emk_linear_bf16_qknorm_rope": [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p,
                                    c_void_p, c_void_p, c_int64, c_int64, c_int64, c_float, c_void_p],
    "emk_gemm_bf16_fused": [c_void_p, c_void_p, c_void_p],
    "emk_gemm_bf16_chain_workspace_bytes": [c_int64],
    "emk_gemm_bf16_chain": [c_void_p, c_void_p, c_int, c_void_p, c_int64, c_void_p],
    "emk_linear_residual_rmsnorm_bf16_noalloc": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                 c_int64, c_int64, c_int64, c_float, c_void_p],
    "emk_linear_bf16_w8": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int64,
                           c_void_p],
    "emk_linear_bf16_w8_workspace_bytes": [c_int64, c_int64],
    "emk_elementwise": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p],
    "emk_loop_rope_scores_f32": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                 c_int64, c_float, c_float, c_float, c_void_p],
    "emk_loop_softmax_pv_f32": [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_void_p],
    "emk_loop_linear_f32": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                            c_int64, c_int64, c_int64, c_void_p],
    "emk_sdpa_causal_gqa_bf16": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                 c_int64, c_int64, c_float, c_void_p],
    "emk_sdpa_causal_gqa_bf16_tok": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                     c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_float, c_void_p],
    "emk_sdpa_varlen_workspace_bytes": [c_int64, c_int64],
    "emk_sdpa_causal_gqa_bf16_varlen": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                                        c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_float,
                                        c_void_p, c_int64, c_void_p],
    "emk_pool_norm_l2_varlen": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_float, c_void_p],
    "emk_sdpa_simt": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64,
                      c_int64, c_float, c_int, c_int, c_void_p],
    "emk_embed_gather": [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p],
    "emk_embed_gather_sumsq": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p],
    "emk_qknorm_rope": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                        c_int64, c_float, c_void_p],
    "emk_pool_norm_l2": [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_float, c_void_p],
    "emk_selftest_wait_expiry": [c_void_p, c_int, c_void_p],
}
_RESTYPES = {"emk_status_string": c_char_p, "emk_last_error": c_char_p,
             "emk_linear_bf16_w8_workspace_bytes": c_int64, "emk_sdpa_varlen_workspace_bytes": c_int64,
             "emk_linear_f32_tc_workspace_bytes": c_int64, "emk_gemm_bf16_chain_workspace_bytes": c_int64}

#: every symbol ``include/emk.h`` declares; ``tests/test_cabi_symbols.py`` checks the header against this list
EXPORTED_SYMBOLS = tuple(_SIGNATURES)

_lib = None
_lib_lock = threading.Lock()


def load_library() -> ctypes.CDLL:
    """Load ``libemk.so`` (once). Raises :class:`EmkLibraryMissing` when it has not been built."""
    global _lib
    with _lib_lock:
        if _lib is not None:
            return _lib
        if not LIB_PATH.exists():
            raise EmkLibraryMissing(
                f"{LIB_PATH} not found: build it with `python -m deplodock_b200.build"
                f"{' --bounds-check' if BOUNDS_CHECK else ''}` (needs nvcc). "
                "There is no CPU or PyTorch fallback for the kernels."
            )
        lib = ctypes.CDLL(str(LIB_PATH))
        for name, argtypes in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = _RESTYPES.get(name, c_int)
        _lib = lib
        return lib


class Handle:
    """Per-device library handle (``emk_create``/``emk_destroy``)."""

    def __init__(self, device: int = 0) -> None:
        self.lib = load_library()
        self.device = device
        ptr = c_void_p()
        rc = self.lib.emk_create(int(device), ctypes.byref(ptr))
        if rc != EMK_OK:
            raise RuntimeError(f"emk_create(device={device}) failed: {self.status_string(rc)}")
        self.ptr = ptr

    def status_string(self, rc: int) -> str:
        return self.lib.emk_status_string(int(rc)).decode()

    def last_error(self) -> str:
        return self.lib.emk_last_error(self.ptr).decode()

    def check(self, rc: int, what: str) -> None:
        """Turn a non-zero status into the exception type the reference would raise."""
        if rc == EMK_OK:
            return
        detail = self.last_error()
        msg = f"{what}: {self.status_string(rc)}" + (f" — {detail}" if detail else "")
        if rc in (EMK_ERR_SHAPE, EMK_ERR_ALIGN, EMK_ERR_WORKSPACE, EMK_ERR_LIMIT, EMK_ERR_ARG):
            raise ValueError(msg)
        if rc == EMK_ERR_DTYPE:
            raise TypeError(msg)
        if rc == EMK_ERR_TIMEOUT:
            raise HungKernelError(msg)
        if rc == EMK_ERR_BOUNDS:
            raise IndexError(msg)
        raise RuntimeError(msg)

    def device_status(self, stream: int = 0) -> None:
        """Synchronise ``stream`` and raise if a device-side wait expired or a launch failed."""
        self.check(self.lib.emk_device_status(self.ptr, c_void_p(stream)), "emk_device_status")

    def set_wait_limit_ms(self, ms: int) -> None:
        self.check(self.lib.emk_set_wait_limit_ms(self.ptr, int(ms)), "emk_set_wait_limit_ms")

    def set_launch_overlap(self, on: bool) -> bool:
        """Programmatic dependent launch for the kernels launched from now on; returns the previous setting."""
        prev = int(self.lib.emk_set_launch_overlap(self.ptr, 1 if on else 0))
        if prev < 0:
            self.check(-prev, "emk_set_launch_overlap")
        return bool(prev)

    def close(self) -> None:
        if getattr(self, "ptr", None) is not None and self.ptr.value:
            self.lib.emk_destroy(self.ptr)
            self.ptr = c_void_p()

    def __del__(self) -> None:  # best effort
        try:
            self.close()
        except Exception:
            pass
