"""Launcher for ``oracle/_ref/``: the reference compiler's own emitted kernels (built by ``build_ref_kernels.py``).

TEST AND REFERENCE-TIMING INFRASTRUCTURE, not product code: the product never imports this. It exists so that the parity tests
can compare the hand-written kernels with what the reference itself emits for the same four configurations, and so
that ``bench.py --impl reference`` can report the reference's kernels timed on the same GPU.

The reference launches its cubins through cupy (``emmy/compiler/backend/cuda/program.py:394-424``): positional device
pointers in ``arg_order``, scalar constants as one-element device buffers (``program.py:257-264``), TMA descriptors
encoded with ``cuTensorMapEncodeTiled`` over the C-order shape reversed (innermost first), byte strides of a contiguous
array, interleave / L2 promotion / OOB fill all NONE, placed in device memory and passed by pointer
(``emmy/compiler/backend/cuda/_tma.py:91-170``, ``program.py:470-510``). cupy is not installed here, so the same calls
are made through the driver API with ctypes; tensors are torch tensors.
"""

from __future__ import annotations

import ctypes
import json
from pathlib import Path

import torch

REF_DIR = Path(__file__).resolve().parent / "_ref"

_TORCH_DTYPES = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}
_SWIZZLE = {"NONE": 0, "32B": 1, "64B": 2, "128B": 3}
_TMAP_DTYPE_BY_ITEMSIZE = {1: 0, 2: 6, 4: 7, 8: 8}   # UINT8, FLOAT16, FLOAT32, FLOAT64 (the reference's table)


def available() -> bool:
    return (REF_DIR / "manifest.json").exists()


def _cuda():
    lib = ctypes.CDLL("libcuda.so.1")
    return lib


def _check(res: int, what: str) -> None:
    if res != 0:
        raise RuntimeError(f"{what} failed: CUresult={res}")


def encode_tiled(lib, global_address: int, src_shape, box_extents, elem_size: int, swizzle: str) -> bytes:
    """128-byte tensor map with the reference's conventions (see the module docstring)."""
    rank = len(src_shape)
    rev_shape = [int(d) for d in reversed(src_shape)]
    rev_box = [int(b) for b in reversed(box_extents)]
    global_dim = (ctypes.c_uint64 * rank)(*rev_shape)
    box_dim = (ctypes.c_uint32 * rank)(*rev_box)
    elem_strides = (ctypes.c_uint32 * rank)(*([1] * rank))
    strides = []
    running = rev_shape[0] * elem_size
    for d in rev_shape[1:]:
        strides.append(running)
        running *= d
    global_strides = (ctypes.c_uint64 * max(rank - 1, 1))(*strides) if strides else None
    buf = (ctypes.c_uint8 * 128)()
    fn = lib.cuTensorMapEncodeTiled
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_uint32, ctypes.c_void_p, ctypes.POINTER(ctypes.c_uint64),
                   ctypes.POINTER(ctypes.c_uint64), ctypes.POINTER(ctypes.c_uint32), ctypes.POINTER(ctypes.c_uint32),
                   ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int]
    _check(fn(ctypes.cast(buf, ctypes.c_void_p), _TMAP_DTYPE_BY_ITEMSIZE[elem_size], rank,
              ctypes.c_void_p(int(global_address)), global_dim, global_strides, box_dim, elem_strides, 0,
              _SWIZZLE[swizzle], 0, 0), "cuTensorMapEncodeTiled")
    return bytes(buf)


class RefKernel:
    """One emitted kernel of the reference, bound to freshly allocated device buffers."""

    def __init__(self, name: str, device="cuda") -> None:
        manifest = json.loads((REF_DIR / "manifest.json").read_text())
        if name not in manifest:
            raise KeyError(name)
        self.name, self.meta = name, manifest[name]
        self.lib = _cuda()
        torch.zeros(1, device=device)   # make sure the primary context exists and is current
        image = (REF_DIR / f"{name}.cubin").read_bytes()
        self._image = ctypes.create_string_buffer(image, len(image))
        self.module = ctypes.c_void_p()
        _check(self.lib.cuModuleLoadData(ctypes.byref(self.module), self._image), "cuModuleLoadData")
        self.func = ctypes.c_void_p()
        _check(self.lib.cuModuleGetFunction(ctypes.byref(self.func), self.module, self.meta["kernel_name"].encode()),
               "cuModuleGetFunction")
        if self.meta["smem_bytes"] > 48 * 1024:
            # CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES = 8
            _check(self.lib.cuFuncSetAttribute(self.func, 8, int(self.meta["smem_bytes"])), "cuFuncSetAttribute")
        self.buffers: dict[str, torch.Tensor] = {}
        for bid, info in self.meta["buffers"].items():
            dt = _TORCH_DTYPES[info["dtype"]]
            if info["op"] == "ConstantOp" and info.get("value") is not None:
                self.buffers[bid] = torch.full(info["shape"], float(info["value"]), dtype=dt, device=device)
            else:
                self.buffers[bid] = torch.zeros(info["shape"], dtype=dt, device=device)
        self.descs: dict[str, torch.Tensor] = {}

    def bind(self, **tensors: torch.Tensor) -> None:
        """Copy host or device tensors into the kernel's buffers (by the reference's buffer names)."""
        for bid, t in tensors.items():
            dst = self.buffers[bid]
            if tuple(t.shape) != tuple(dst.shape):
                raise ValueError(f"{bid}: expected shape {tuple(dst.shape)}, got {tuple(t.shape)}")
            dst.copy_(t.to(dst.dtype))
        self.descs = {}
        for d in self.meta["tma_descriptors"]:
            src = self.buffers[d["src_buf"]]
            raw = encode_tiled(self.lib, src.data_ptr(), tuple(src.shape), d["box_extents"], src.element_size(),
                               d["swizzle"])
            self.descs[d["name"]] = torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(src.device)
        torch.cuda.synchronize()

    @property
    def output(self) -> torch.Tensor:
        return self.buffers[self.meta["output"]]

    def launch(self) -> None:
        """One launch on torch's current stream."""
        for z in self.meta["zero_outputs"]:
            self.buffers[z].zero_()
        ptrs = []
        for a in self.meta["arg_order"]:
            t = self.descs[a] if a in self.descs else self.buffers[a]
            ptrs.append(ctypes.c_void_p(t.data_ptr()))
        params = (ctypes.c_void_p * len(ptrs))(*[ctypes.cast(ctypes.pointer(p), ctypes.c_void_p) for p in ptrs])
        g, b = self.meta["grid"], self.meta["block"]
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        # shared memory is declared statically by the emitted kernels up to 48 KB; only larger footprints use a dynamic
        # pool (program.py:419-424)
        dyn = int(self.meta["smem_bytes"]) if self.meta["smem_bytes"] > 48 * 1024 else 0
        _check(self.lib.cuLaunchKernel(self.func, g[0], g[1], g[2], b[0], b[1], b[2], dyn, stream, params, None),
               f"cuLaunchKernel({self.meta['kernel_name']})")
        self._keepalive = ptrs

    def time_us(self, reps: int = 10, iters: int = 5) -> float:
        """Median microseconds per launch, measured as a CUDA graph of ``reps`` back-to-back launches (the protocol
        ``bench.py`` uses for the hand-written kernels)."""
        self.launch()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(reps):
                self.launch()
        graph.replay()
        torch.cuda.synchronize()
        times = []
        for _ in range(iters):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            graph.replay()
            e.record()
            torch.cuda.synchronize()
            times.append(s.elapsed_time(e) * 1e3 / reps)
        times.sort()
        return times[len(times) // 2]
