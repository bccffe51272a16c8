"""Torch-tensor front end of the C-ABI kernels: validates tensors, passes raw device pointers and the current CUDA
stream to ``libemk.so``. PyTorch is used only for device memory and streams; every computation below is one call into
the library (no eager fallback).

Each function names the reference Torch-IR op it stands for (``emmy/compiler/ir/frontend/ir.py``).
"""

from __future__ import annotations

import math
from ctypes import c_void_p

import torch

from deplodock_b200 import cabi

_handles: dict[int, cabi.Handle] = {}


def handle(device: int | None = None) -> cabi.Handle:
    """The library handle of ``device`` (default: torch's current CUDA device), created on first use."""
    if not torch.cuda.is_available():
        raise RuntimeError("deplodock_b200 kernels need a CUDA device (sm_100a); there is no CPU fallback")
    if device is None:
        device = torch.cuda.current_device()
    h = _handles.get(device)
    if h is None:
        with torch.cuda.device(device):
            h = cabi.Handle(device)
        _handles[device] = h
    return h


def _stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: torch.Tensor | None) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def _check_cuda_contig(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            if not torch.cuda.is_available():
                raise RuntimeError("deplodock_b200 kernels need a CUDA device (sm_100a); there is no CPU fallback")
            raise ValueError("expected CUDA tensors")
        if not t.is_contiguous():
            raise ValueError("expected contiguous tensors")


def _check_buffer(name: str, t: torch.Tensor | None, numel: int, dtype: torch.dtype) -> None:
    """A caller-provided buffer the library reads or writes through a raw pointer: its size and dtype are checked here,
    because the kernels cannot (a short buffer would be an out-of-bounds device access, not a Python error)."""
    if t is None:
        return
    if t.dtype != dtype:
        raise TypeError(f"{name} must be {dtype}, got {t.dtype}")
    if t.numel() < numel:
        raise ValueError(f"{name} holds {t.numel()} elements, the call needs {numel}")


_DTYPES = {torch.float32: cabi.EMK_F32, torch.bfloat16: cabi.EMK_BF16}


def _dtype_token(t: torch.Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {t.dtype}; the kernels take float32 and bfloat16") from None


def device_status() -> None:
    """Synchronise the current stream and raise if a kernel recorded an expired wait or a launch error."""
    handle().device_status(torch.cuda.current_stream().cuda_stream)


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6, out: torch.Tensor | None = None) -> torch.Tensor:
    """RmsNormOp (``ir/frontend/ir.py:296-312``) over the last axis."""
    _check_cuda_contig(x, weight, out)
    if weight.dtype != x.dtype or weight.numel() != x.shape[-1]:
        raise ValueError("weight must be a vector of the row length with the dtype of x")
    y = torch.empty_like(x) if out is None else out
    cols = x.shape[-1]
    rows = x.numel() // cols
    h = handle()
    h.check(h.lib.emk_rmsnorm(h.ptr, _ptr(x), _ptr(weight), _ptr(y), rows, cols, float(eps), _dtype_token(x),
                              _stream()), "emk_rmsnorm")
    return y


def softmax_lastdim(x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """SoftmaxOp(axis=-1) (``ir/frontend/ir.py:343-358``)."""
    _check_cuda_contig(x, out)
    y = torch.empty_like(x) if out is None else out
    cols = x.shape[-1]
    rows = x.numel() // cols
    h = handle()
    h.check(h.lib.emk_softmax_lastdim(h.ptr, _ptr(x), _ptr(y), rows, cols, _dtype_token(x), _stream()),
            "emk_softmax_lastdim")
    return y


def _linear_common(fn_name: str, x, w, *, residual, bias, swiglu, w_is_kn, out):
    _check_cuda_contig(x, w, residual, bias, out)
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise TypeError("linear expects bfloat16 operands")
    K = x.shape[-1]
    M = x.numel() // K
    if w_is_kn:
        if w.shape[0] != K:
            raise ValueError("weight [K,N] does not match x")
        N = w.shape[1]
    else:
        if w.shape[1] != K:
            raise ValueError("weight [N,K] does not match x")
        N = w.shape[0]
    if sum(v is not None and v is not False for v in (residual, bias, swiglu or None)) > 1:
        raise ValueError("choose at most one of residual / bias / swiglu")
    epi, extra = cabi.EMK_EPI_NONE, None
    n_out = N
    if residual is not None:
        epi, extra = cabi.EMK_EPI_RESIDUAL, residual
    elif bias is not None:
        epi, extra = cabi.EMK_EPI_BIAS, bias
    elif swiglu:
        epi, n_out = cabi.EMK_EPI_SWIGLU, N // 2
    _check_buffer("out", out, M * n_out, torch.bfloat16)
    _check_buffer("residual", residual, M * N, torch.bfloat16)
    _check_buffer("bias", bias, N, torch.bfloat16)
    y = torch.empty(*x.shape[:-1], n_out, dtype=torch.bfloat16, device=x.device) if out is None else out
    h = handle()
    fn = getattr(h.lib, fn_name)
    h.check(fn(h.ptr, _ptr(x), _ptr(w), _ptr(extra), _ptr(y), M, N, K,
               cabi.EMK_W_KN if w_is_kn else cabi.EMK_W_NK, epi, _stream()), fn_name)
    return y


def linear(x, w, *, residual=None, bias=None, swiglu=False, w_is_kn=False, out=None) -> torch.Tensor:
    """LinearOp ``x @ w.T`` (``ir/frontend/ir.py:202-217``) or, with ``w_is_kn``, MatmulOp ``x @ w`` (``:221-237``), on
    the tcgen05 tensor cores, with an optional fused epilogue."""
    return _linear_common("emk_linear_bf16", x, w, residual=residual, bias=bias, swiglu=swiglu, w_is_kn=w_is_kn,
                          out=out)


def linear_simt(x, w, *, residual=None, bias=None, swiglu=False, w_is_kn=False, out=None) -> torch.Tensor:
    """Same contract on CUDA cores: for K or N not a multiple of 8, and as a cross-check in the tests."""
    return _linear_common("emk_linear_bf16_simt", x, w, residual=residual, bias=bias, swiglu=swiglu, w_is_kn=w_is_kn,
                          out=out)


def rope_chunk_major(cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Re-lay bf16 cos/sin tables ``[S,128]`` as the chunk-major table ``[8,S,16]`` the fused QKV epilogue reads:
    entry ``[q,s]`` = cos(s, 8q..8q+7) then sin(s, 8q..8q+7) of the first 64 elements (element i+64 shares the angle)."""
    S = cos.shape[0]
    c = cos[:, :64].reshape(S, 8, 8)
    s_ = sin[:, :64].reshape(S, 8, 8)
    return torch.cat([c, s_], dim=-1).permute(1, 0, 2).contiguous()


def linear_qknorm_rope(x, w_qkv, q_weight, k_weight, rope_cm, S: int, Hq: int, Hkv: int, eps: float = 1e-6,
                       out=None) -> torch.Tensor:
    """Fused QKV projection ``x @ w_qkv.T`` with per-head q/k RMSNorm and RoPE in the GEMM epilogue; the result is the
    token-major ``[T, (Hq+2*Hkv)*128]`` buffer the attention kernel reads. ``rope_cm`` comes from
    :func:`rope_chunk_major`."""
    _check_cuda_contig(x, w_qkv, q_weight, k_weight, rope_cm, out)
    if not (x.dtype == w_qkv.dtype == rope_cm.dtype == torch.bfloat16):
        raise TypeError("linear_qknorm_rope expects bfloat16 operands and table")
    K = x.shape[-1]
    M = x.numel() // K
    N = w_qkv.shape[0]
    if w_qkv.shape[1] != K or tuple(rope_cm.shape) != (8, S, 16):
        raise ValueError("weight/table shapes do not match")
    y = torch.empty(M, N, dtype=torch.bfloat16, device=x.device) if out is None else out
    h = handle()
    h.check(h.lib.emk_linear_bf16_qknorm_rope(h.ptr, _ptr(x), _ptr(w_qkv), _ptr(y), M, N, K, _ptr(q_weight),
                                              _ptr(k_weight), _ptr(rope_cm), S, Hq, Hkv, float(eps), _stream()),
            "emk_linear_bf16_qknorm_rope")
    return y


def _gemm_desc(x, w, out, *, epilogue: str = "none", residual=None, w_is_kn: bool = False, row_sumsq_in=None,
               norm_dim: int = 0, norm_eps: float = 1e-6, row_sumsq_out=None, q_weight=None,
               k_weight=None, rope_cm=None, S: int = 0, Hq: int = 0, Hkv: int = 0, qk_eps: float = 1e-6,
               positions=None) -> "cabi.GemmDesc":
    """Checks the tensors of one fused GEMM and fills its ``emk_gemm_desc_t``."""
    _check_cuda_contig(x, w, out, residual, row_sumsq_in, row_sumsq_out, q_weight, k_weight, rope_cm)
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise TypeError("gemm_fused expects bfloat16 operands")
    epi = {"none": cabi.EMK_EPI_NONE, "residual": cabi.EMK_EPI_RESIDUAL, "swiglu": cabi.EMK_EPI_SWIGLU,
           "bias": cabi.EMK_EPI_BIAS, "qknorm_rope": cabi.EMK_EPI_QKNORM_ROPE}[epilogue]
    K = x.shape[-1]
    M = x.numel() // K
    N = w.shape[1] if w_is_kn else w.shape[0]
    if (w.shape[0] if w_is_kn else w.shape[1]) != K:
        raise ValueError("weight does not match x")
    _check_buffer("out", out, M * (N // 2 if epilogue == "swiglu" else N), torch.bfloat16)
    _check_buffer("residual", residual, M * N, torch.bfloat16)
    _check_buffer("row_sumsq_out", row_sumsq_out, M * ((N + 127) // 128), torch.float32)
    if row_sumsq_in is not None:
        if norm_dim <= 0 or norm_dim % 128 != 0:
            raise ValueError("row_sumsq_in needs norm_dim > 0 and a multiple of 128")
        _check_buffer("row_sumsq_in", row_sumsq_in, M * (norm_dim // 128), torch.float32)
    d = cabi.GemmDesc()
    d.x, d.w, d.y = x.data_ptr(), w.data_ptr(), out.data_ptr()
    d.residual = residual.data_ptr() if residual is not None else None
    d.M, d.K = x.numel() // K, K
    d.N = w.shape[1] if w_is_kn else w.shape[0]
    d.wlayout = cabi.EMK_W_KN if w_is_kn else cabi.EMK_W_NK
    d.epilogue = epi
    d.row_sumsq_in = row_sumsq_in.data_ptr() if row_sumsq_in is not None else None
    d.norm_dim, d.norm_eps = int(norm_dim), float(norm_eps)
    d.row_sumsq_out = row_sumsq_out.data_ptr() if row_sumsq_out is not None else None
    d.q_norm_weight = q_weight.data_ptr() if q_weight is not None else None
    d.k_norm_weight = k_weight.data_ptr() if k_weight is not None else None
    d.rope_chunk_major = rope_cm.data_ptr() if rope_cm is not None else None
    d.seq_len, d.num_q_heads, d.num_kv_heads, d.qk_eps = int(S), int(Hq), int(Hkv), float(qk_eps)
    if positions is not None:   # rotary position per row (packed sequences); S is then the table length
        _check_cuda_contig(positions)
        _check_buffer("positions", positions, M, torch.int32)
        d.positions = positions.data_ptr()
    return d


def gemm_fused(x, w, out, **kw):
    """``emk_gemm_bf16_fused``: the tcgen05 GEMM with an epilogue (``none | residual | bias | swiglu | qknorm_rope``)
    and an RMSNorm folded around it through per-row partial sum-of-squares buffers ``[M, dim/128]`` fp32 (see
    ``emk_gemm_desc_t``). Keywords: ``epilogue, residual, w_is_kn, row_sumsq_in, norm_dim, norm_eps, row_sumsq_out,
    q_weight, k_weight, rope_cm, S, Hq, Hkv, qk_eps, positions``."""
    import ctypes as _ct

    d = _gemm_desc(x, w, out, **kw)
    h = handle()
    h.check(h.lib.emk_gemm_bf16_fused(h.ptr, _ct.byref(d), _stream()), "emk_gemm_bf16_fused")
    return out


def gemm_chain_workspace(M: int, device) -> torch.Tensor:
    """Zeroed counter workspace for :func:`gemm_chain` over ``M`` rows. One workspace serves any number of chain
    launches that follow each other on a stream (every completed launch leaves it zero)."""
    h = handle()
    n = int(h.lib.emk_gemm_bf16_chain_workspace_bytes(int(M)))
    return torch.zeros((n + 3) // 4, dtype=torch.int32, device=device)


def gemm_chain(phases: list[dict], workspace: torch.Tensor):
    """``emk_gemm_bf16_chain``: 1 to 4 fused GEMMs, each reading the output of the one before it, as one persistent
    launch. ``phases`` are keyword dicts of :func:`gemm_fused` with ``x``, ``w`` and ``out`` entries. Returns the last
    phase's output."""
    import ctypes as _ct

    if not phases:
        raise ValueError("gemm_chain needs at least one phase")
    descs = (cabi.GemmDesc * len(phases))()
    for i, ph in enumerate(phases):
        kw = dict(ph)
        descs[i] = _gemm_desc(kw.pop("x"), kw.pop("w"), kw.pop("out"), **kw)
    _check_cuda_contig(workspace)
    if workspace.dtype != torch.int32:
        raise TypeError("gemm_chain workspace must be int32")
    h = handle()
    h.check(h.lib.emk_gemm_bf16_chain(h.ptr, descs, len(phases), workspace.data_ptr(),
                                      workspace.numel() * 4, _stream()), "emk_gemm_bf16_chain")
    return phases[-1]["out"]


def linear_residual_rmsnorm_noalloc(x, w, residual, norm_weight, eps: float = 1e-6, out_hidden=None, out_norm=None):
    """``emk_linear_residual_rmsnorm_bf16_noalloc``: ``h = bf16(bf16(x @ w.T) + residual)`` and ``RMSNorm(h)`` with the
    scratch between the two kernels held in a fixed array inside the library (no device allocation by the call; the
    output tensors are the caller's). Returns ``(h, norm)``. Size limit ``M * ceil(N/128) <= 2**20``."""
    _check_cuda_contig(x, w, residual, norm_weight, out_hidden, out_norm)
    if not (x.dtype == w.dtype == residual.dtype == norm_weight.dtype == torch.bfloat16):
        raise TypeError("linear_residual_rmsnorm_noalloc expects bfloat16 tensors")
    K = x.shape[-1]
    M = x.numel() // K
    N = w.shape[0]
    if w.shape[1] != K or residual.numel() != M * N or norm_weight.numel() != N:
        raise ValueError("shapes do not match")
    hid = torch.empty(M, N, dtype=torch.bfloat16, device=x.device) if out_hidden is None else out_hidden
    nrm = torch.empty(M, N, dtype=torch.bfloat16, device=x.device) if out_norm is None else out_norm
    h = handle()
    h.check(h.lib.emk_linear_residual_rmsnorm_bf16_noalloc(h.ptr, _ptr(x), _ptr(w), _ptr(residual), _ptr(norm_weight),
                                                           _ptr(hid), _ptr(nrm), M, N, K, float(eps), _stream()),
            "emk_linear_residual_rmsnorm_bf16_noalloc")
    return hid, nrm


#: fp32 problems with at least this many rows go to the tensor cores (split operands); below it the split of the
#: weight costs more than the CUDA-core kernel's whole product
F32_TC_MIN_ROWS = 256
_F32_SCRATCH: dict[int, torch.Tensor] = {}


def _f32_scratch(device: torch.device, nbytes: int) -> torch.Tensor:
    """One grow-only scratch buffer per device for the split operands of :func:`linear_f32`; it holds nothing between
    calls (calls on different streams must not overlap)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    buf = _F32_SCRATCH.get(idx)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(nbytes, dtype=torch.uint8, device=device)
        _F32_SCRATCH[idx] = buf
    return buf


def linear_f32(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None, w_is_kn: bool = False,
               route: str = "auto", out: torch.Tensor | None = None) -> torch.Tensor:
    """fp32 LinearOp / MatmulOp. ``route``: ``"tc"`` — tensor cores on exactly split bf16 operands
    (``emk_linear_f32_tc``; K and N multiples of 8), ``"simt"`` — the register-tiled CUDA-core kernel, ``"auto"`` —
    tensor cores from ``F32_TC_MIN_ROWS`` rows on when the shape allows."""
    _check_cuda_contig(x, w, bias, out)
    if x.dtype != torch.float32 or w.dtype != torch.float32 or (bias is not None and bias.dtype != torch.float32):
        raise TypeError("linear_f32 expects float32 operands")
    K = x.shape[-1]
    M = x.numel() // K
    N = w.shape[1] if w_is_kn else w.shape[0]
    if (w.shape[0] if w_is_kn else w.shape[1]) != K:
        raise ValueError("weight does not match x")
    if route not in ("auto", "tc", "simt"):
        raise ValueError("route must be 'auto', 'tc' or 'simt'")
    _check_buffer("out", out, M * N, torch.float32)
    _check_buffer("bias", bias, N, torch.float32)
    y = torch.empty(*x.shape[:-1], N, dtype=torch.float32, device=x.device) if out is None else out
    h = handle()
    wl = cabi.EMK_W_KN if w_is_kn else cabi.EMK_W_NK
    tc_ok = K % 8 == 0 and N % 8 == 0
    if route == "tc" and not tc_ok:
        raise ValueError("the tensor-core route needs K and N to be multiples of 8")
    if route == "tc" or (route == "auto" and tc_ok and M >= F32_TC_MIN_ROWS):
        ws = _f32_scratch(x.device, int(h.lib.emk_linear_f32_tc_workspace_bytes(M, N, K)))
        h.check(h.lib.emk_linear_f32_tc(h.ptr, _ptr(x), _ptr(w), _ptr(bias), _ptr(y), M, N, K, wl, _ptr(ws),
                                        ws.numel(), _stream()), "emk_linear_f32_tc")
        return y
    h.check(h.lib.emk_linear_f32_simt(h.ptr, _ptr(x), _ptr(w), _ptr(bias), _ptr(y), M, N, K, wl, _stream()),
            "emk_linear_f32_simt")
    return y


_EW_OPS = {"add": cabi.EMK_EW_ADD, "multiply": cabi.EMK_EW_MUL, "silu": cabi.EMK_EW_SILU, "silu_multiply": cabi.EMK_EW_SILU_MUL}


def elementwise(op: str, a: torch.Tensor, b: torch.Tensor | None = None, out=None) -> torch.Tensor:
    """Same-shape ``add`` / ``multiply`` / ``silu`` / ``silu_multiply`` (= ``silu(a) * b``) in fp32 or bf16."""
    _check_cuda_contig(a, b, out)
    if op not in _EW_OPS:
        raise ValueError(f"unknown elementwise op {op!r}")
    if a.dtype not in (torch.float32, torch.bfloat16) or (b is not None and b.dtype != a.dtype):
        raise TypeError("elementwise expects float32 or bfloat16 operands of one dtype")
    if op != "silu" and (b is None or tuple(b.shape) != tuple(a.shape)):
        raise ValueError("elementwise operands must have the same shape (no broadcasting)")
    y = torch.empty_like(a) if out is None else out
    h = handle()
    h.check(h.lib.emk_elementwise(h.ptr, _EW_OPS[op], _ptr(a), _ptr(b), _ptr(y), a.numel(),
                                  cabi.EMK_F32 if a.dtype == torch.float32 else cabi.EMK_BF16, _stream()),
            "emk_elementwise")
    return y


def loop_linear_f32(x: torch.Tensor, w: torch.Tensor, M: int, N: int, K: int, *, x_inner: int | None = None,
                    x_stride_outer: int = 0, x_stride_m: int | None = None, residual=None, gate=None,
                    out=None) -> torch.Tensor:
    """The fp32 contraction of the Loop-IR kernel records: ``y[m,n] = e(sum_k x[m,k] * w[n,k])`` with the blocked
    activation addressing ``(k // x_inner) * x_stride_outer + m * x_stride_m + k % x_inner`` and the epilogue
    ``+ residual`` or ``* silu(gate)`` (see ``emk_loop_linear_f32``). ``x`` is taken as a flat buffer."""
    _check_cuda_contig(x, w, residual, gate, out)
    for t in (x, w, residual, gate):
        if t is not None and t.dtype != torch.float32:
            raise TypeError("loop_linear_f32 expects float32 tensors")
    x_inner = K if x_inner is None else int(x_inner)
    x_stride_m = K if x_stride_m is None else int(x_stride_m)
    need = (K // x_inner - 1) * x_stride_outer + (M - 1) * x_stride_m + x_inner
    if x.numel() < need or tuple(w.shape) != (N, K):
        raise ValueError("operand sizes do not match the addressing")
    for t in (residual, gate):
        if t is not None and t.numel() != M * N:
            raise ValueError("epilogue operand must hold M * N elements")
    y = torch.empty(M, N, dtype=torch.float32, device=x.device) if out is None else out
    h = handle()
    h.check(h.lib.emk_loop_linear_f32(h.ptr, _ptr(x), _ptr(w), _ptr(residual), _ptr(gate), _ptr(y), M, N, K, x_inner,
                                      int(x_stride_outer), x_stride_m, _stream()), "emk_loop_linear_f32")
    return y


def loop_rope_scores_f32(q, k, cos, sin, S: int, H: int, Hkv: int, D: int, scale: float, mask_zero: float,
                         mask_fill: float) -> torch.Tensor:
    """First half of the reference's unfused attention record: RoPE on q and k, scaled dot products, causal fill;
    ``[H, S, S]`` fp32 (see ``emk_loop_rope_scores_f32``)."""
    _check_cuda_contig(q, k, cos, sin)
    if any(t.dtype != torch.float32 for t in (q, k, cos, sin)):
        raise TypeError("loop_rope_scores_f32 expects float32 tensors")
    if q.numel() != S * H * D or k.numel() != S * Hkv * D or cos.numel() != S * D or sin.numel() != S * D:
        raise ValueError("operand sizes do not match S, H, Hkv, D")
    y = torch.empty(H, S, S, dtype=torch.float32, device=q.device)
    h = handle()
    h.check(h.lib.emk_loop_rope_scores_f32(h.ptr, _ptr(q), _ptr(k), _ptr(cos), _ptr(sin), _ptr(y), S, H, Hkv, D,
                                           float(scale), float(mask_zero), float(mask_fill), _stream()),
            "emk_loop_rope_scores_f32")
    return y


def loop_softmax_pv_f32(scores, v, S: int, H: int, Hkv: int, D: int) -> torch.Tensor:
    """Second half: row softmax of ``[H, S, S]`` scores times ``v [S, Hkv*D]`` -> ``[H, S, D]`` fp32."""
    _check_cuda_contig(scores, v)
    if scores.dtype != torch.float32 or v.dtype != torch.float32:
        raise TypeError("loop_softmax_pv_f32 expects float32 tensors")
    if scores.numel() != H * S * S or v.numel() != S * Hkv * D:
        raise ValueError("operand sizes do not match S, H, Hkv, D")
    o = torch.empty(H, S, D, dtype=torch.float32, device=scores.device)
    h = handle()
    h.check(h.lib.emk_loop_softmax_pv_f32(h.ptr, _ptr(scores), _ptr(v), _ptr(o), S, H, Hkv, D, _stream()),
            "emk_loop_softmax_pv_f32")
    return o


_W8_SCRATCH: dict[int, torch.Tensor] = {}


def w8_scratch(device: torch.device, nbytes: int) -> torch.Tensor:
    """One grow-only scratch buffer per device for the expanded weight of :func:`linear_w8`; it holds nothing between
    calls, so every e4m3 layer of a model shares it (calls on different streams must not overlap)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    buf = _W8_SCRATCH.get(idx)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(nbytes, dtype=torch.uint8, device=device)
        _W8_SCRATCH[idx] = buf
    return buf


def linear_w8(x: torch.Tensor, w_e4m3: torch.Tensor, scale: torch.Tensor, out=None, workspace="auto") -> torch.Tensor:
    """bf16 activations times e4m3 weights ``[N,K]`` with one fp32 scale per output channel. ``workspace``: "auto"
    (shared scratch when the row count makes expanding the weight once the faster route), ``None`` (always convert
    inside the main loop, no scratch) or a uint8 CUDA tensor of ``N * K * 2`` bytes."""
    _check_cuda_contig(x, w_e4m3, scale, out)
    if x.dtype != torch.bfloat16 or w_e4m3.dtype != torch.float8_e4m3fn or scale.dtype != torch.float32:
        raise TypeError("linear_w8 expects bfloat16 x, float8_e4m3fn weights and float32 scales")
    K = x.shape[-1]
    M = x.numel() // K
    N = w_e4m3.shape[0]
    if w_e4m3.shape[1] != K or scale.numel() != N:
        raise ValueError("weight/scale shapes do not match x")
    y = torch.empty(*x.shape[:-1], N, dtype=torch.bfloat16, device=x.device) if out is None else out
    h = handle()
    ws = None
    if isinstance(workspace, str):
        if workspace != "auto":
            raise ValueError("workspace must be 'auto', None or a uint8 CUDA tensor")
        if M > 256:
            ws = w8_scratch(x.device, int(h.lib.emk_linear_bf16_w8_workspace_bytes(N, K)))
    elif workspace is not None:
        _check_cuda_contig(workspace)
        ws = workspace
    h.check(h.lib.emk_linear_bf16_w8(h.ptr, _ptr(x), _ptr(w_e4m3), _ptr(scale), _ptr(y), M, N, K, _ptr(ws),
                                     0 if ws is None else ws.numel() * ws.element_size(), _stream()),
            "emk_linear_bf16_w8")
    return y


def sdpa_causal_gqa(q, k, v, scale: float | None = None, out=None) -> torch.Tensor:
    """SdpaOp(is_causal=True) with grouped KV heads (``ir/frontend/ir.py:241-275``); q ``[B,Hq,S,128]``, k/v
    ``[B,Hkv,S,128]`` bf16, on the tcgen05 flash kernel."""
    _check_cuda_contig(q, k, v, out)
    if not (q.dtype == k.dtype == v.dtype == torch.bfloat16):
        raise TypeError("sdpa_causal_gqa expects bfloat16 operands")
    B, Hq, S, D = q.shape
    Hkv = k.shape[1]
    if k.shape != (B, Hkv, S, D) or v.shape != (B, Hkv, S, D):
        raise ValueError("k/v shapes do not match q")
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    o = torch.empty_like(q) if out is None else out
    h = handle()
    h.check(h.lib.emk_sdpa_causal_gqa_bf16(h.ptr, _ptr(q), _ptr(k), _ptr(v), _ptr(o), B, Hq, Hkv, S, D, float(scale),
                                           _stream()), "emk_sdpa_causal_gqa_bf16")
    return o


def sdpa_causal_gqa_tok(qkv: torch.Tensor, B: int, S: int, Hq: int, Hkv: int, out: torch.Tensor,
                        scale: float | None = None) -> torch.Tensor:
    """Same attention reading the fused token-major projection ``qkv [B*S, (Hq+2*Hkv)*128]`` in place and writing
    ``out [B*S, Hq*128]`` — the layout of the traced layer before its transposes."""
    _check_cuda_contig(qkv, out)
    D = 128
    ld = qkv.shape[-1]
    if ld != (Hq + 2 * Hkv) * D or qkv.numel() != B * S * ld or out.numel() != B * S * Hq * D:
        raise ValueError("qkv/out shapes do not match B, S, Hq, Hkv")
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    esz = qkv.element_size()
    h = handle()
    qp = qkv.data_ptr()
    h.check(h.lib.emk_sdpa_causal_gqa_bf16_tok(
        h.ptr, c_void_p(qp), c_void_p(qp + Hq * D * esz), c_void_p(qp + (Hq + Hkv) * D * esz), _ptr(out), B, Hq, Hkv,
        S, D, ld, ld, ld, Hq * D, float(scale), _stream()), "emk_sdpa_causal_gqa_bf16_tok")
    return out


def sdpa_varlen_workspace(B: int, total_tokens: int, device) -> torch.Tensor:
    """Scratch for :func:`sdpa_causal_gqa_varlen` (the table of query blocks built from ``cu_seqlens``)."""
    n = int(handle().lib.emk_sdpa_varlen_workspace_bytes(int(B), int(total_tokens)))
    return torch.empty(max(n, 16), dtype=torch.uint8, device=device)


def sdpa_causal_gqa_varlen(qkv: torch.Tensor, cu_seqlens: torch.Tensor, max_seqlen: int, Hq: int, Hkv: int,
                           out: torch.Tensor, workspace: torch.Tensor | None = None,
                           scale: float | None = None) -> torch.Tensor:
    """Causal GQA attention over packed sequences: ``qkv [T, (Hq+2*Hkv)*128]`` token-major, sequence ``b`` in rows
    ``cu_seqlens[b]:cu_seqlens[b+1]`` (int32 CUDA tensor ``[B+1]``), none longer than ``max_seqlen``; writes
    ``out [T, Hq*128]``. One launch whatever the mix of lengths, no padding between sequences."""
    _check_cuda_contig(qkv, cu_seqlens, out, workspace)
    D = 128
    ld = qkv.shape[-1]
    T = qkv.numel() // ld
    B = cu_seqlens.numel() - 1
    if cu_seqlens.dtype != torch.int32 or B <= 0:
        raise TypeError("cu_seqlens must be an int32 tensor of B + 1 entries")
    if qkv.dtype != torch.bfloat16 or ld != (Hq + 2 * Hkv) * D:
        raise ValueError("qkv must be bfloat16 [T, (Hq + 2*Hkv) * 128]")
    _check_buffer("out", out, T * Hq * D, torch.bfloat16)
    if workspace is None:
        workspace = sdpa_varlen_workspace(B, T, qkv.device)
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    esz = qkv.element_size()
    h = handle()
    qp = qkv.data_ptr()
    h.check(h.lib.emk_sdpa_causal_gqa_bf16_varlen(
        h.ptr, c_void_p(qp), c_void_p(qp + Hq * D * esz), c_void_p(qp + (Hq + Hkv) * D * esz), _ptr(out),
        _ptr(cu_seqlens), B, T, int(max_seqlen), Hq, Hkv, D, ld, ld, ld, Hq * D, float(scale), _ptr(workspace),
        workspace.numel() * workspace.element_size(), _stream()), "emk_sdpa_causal_gqa_bf16_varlen")
    return out


def pool_norm_l2_varlen(hidden_states, weight, cu_seqlens: torch.Tensor, eps: float = 1e-6, out=None) -> torch.Tensor:
    """Last-token pooling of packed sequences + final RMSNorm + L2 normalisation: ``[B, hidden]`` fp32."""
    _check_cuda_contig(hidden_states, weight, cu_seqlens, out)
    if cu_seqlens.dtype != torch.int32:
        raise TypeError("cu_seqlens must be int32")
    B = cu_seqlens.numel() - 1
    hidden = hidden_states.shape[-1]
    y = torch.empty(B, hidden, dtype=torch.float32, device=hidden_states.device) if out is None else out
    _check_buffer("out", y, B * hidden, torch.float32)
    h = handle()
    h.check(h.lib.emk_pool_norm_l2_varlen(h.ptr, _ptr(hidden_states), _ptr(weight), _ptr(y), _ptr(cu_seqlens), B,
                                          hidden, float(eps), _stream()), "emk_pool_norm_l2_varlen")
    return y


def sdpa_simt(q, k, v, causal: bool, scale: float | None = None) -> torch.Tensor:
    """SdpaOp on CUDA cores: fp32 or bf16, head_dim <= 256, causal or full."""
    _check_cuda_contig(q, k, v)
    B, Hq, Sq, D = q.shape
    Hkv, Skv = k.shape[1], k.shape[2]
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    o = torch.empty_like(q)
    h = handle()
    h.check(h.lib.emk_sdpa_simt(h.ptr, _ptr(q), _ptr(k), _ptr(v), _ptr(o), B, Hq, Hkv, Sq, Skv, D, float(scale),
                                int(bool(causal)), _dtype_token(q), _stream()), "emk_sdpa_simt")
    return o


def embed_gather(table: torch.Tensor, ids: torch.Tensor, out=None, row_sumsq=None) -> torch.Tensor:
    """GatherOp of the embedding table (bf16 rows) by int64 token ids; ``row_sumsq`` (fp32 ``[tokens, hidden/128]``)
    optionally receives the sum of squares of every gathered row (slot 0; the other slots are zeroed)."""
    _check_cuda_contig(table, ids, out, row_sumsq)
    if table.dtype != torch.bfloat16 or ids.dtype != torch.int64:
        raise TypeError("embed_gather expects a bfloat16 table and int64 ids")
    vocab, hidden = table.shape
    tokens = ids.numel()
    y = torch.empty(tokens, hidden, dtype=table.dtype, device=table.device) if out is None else out
    h = handle()
    h.check(h.lib.emk_embed_gather_sumsq(h.ptr, _ptr(table), _ptr(ids), _ptr(y), _ptr(row_sumsq), tokens, hidden,
                                         vocab, _stream()), "emk_embed_gather_sumsq")
    return y


def qknorm_rope_(qkv, q_weight, k_weight, cos, sin, S: int, Hq: int, Hkv: int, eps: float = 1e-6) -> torch.Tensor:
    """In place on the fused projection ``[T,(Hq+2Hkv)*128]``: per-head RMSNorm of q and k, then rotate-half RoPE."""
    _check_cuda_contig(qkv, q_weight, k_weight, cos, sin)
    if qkv.dtype != torch.bfloat16 or cos.dtype != torch.bfloat16 or sin.dtype != torch.bfloat16:
        raise TypeError("qknorm_rope_ expects bfloat16 qkv and bfloat16 cos/sin tables")
    tokens = qkv.numel() // qkv.shape[-1]
    if qkv.shape[-1] != (Hq + 2 * Hkv) * 128 or cos.shape[-2:] != (S, 128) or tokens % S != 0:
        raise ValueError("qkv/cos shapes do not match S, Hq, Hkv")
    h = handle()
    h.check(h.lib.emk_qknorm_rope(h.ptr, _ptr(qkv), _ptr(q_weight), _ptr(k_weight), _ptr(cos), _ptr(sin), tokens, S,
                                  Hq, Hkv, float(eps), _stream()), "emk_qknorm_rope")
    return qkv


def pool_norm_l2(hidden_states, weight, B: int, S: int, eps: float = 1e-6, out=None) -> torch.Tensor:
    """Last-token pooling, final RMSNorm and L2 normalisation: ``[B*S, hidden]`` bf16 -> ``[B, hidden]`` fp32."""
    _check_cuda_contig(hidden_states, weight, out)
    hidden = hidden_states.shape[-1]
    y = torch.empty(B, hidden, dtype=torch.float32, device=hidden_states.device) if out is None else out
    h = handle()
    h.check(h.lib.emk_pool_norm_l2(h.ptr, _ptr(hidden_states), _ptr(weight), _ptr(y), B, S, hidden, float(eps),
                                   _stream()), "emk_pool_norm_l2")
    return y


def selftest_wait_expiry(limit_ms: int = 20) -> None:
    """Launch the bounded-wait self test; the following :func:`device_status` raises ``HungKernelError``."""
    h = handle()
    h.check(h.lib.emk_selftest_wait_expiry(h.ptr, int(limit_ms), _stream()), "emk_selftest_wait_expiry")
