"""Parity of the CUDA kernels (called through the C ABI) with the CPU oracle on the same seeded inputs.

Tolerances: fp32 reductions <= 1e-5 relative (absolute floor 1e-6 for outputs near zero); bf16 tensor-core paths
<= 2e-2 absolute (scaled with the output magnitude above 4) and row cosine >= 0.999."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import load_golden
from oracle import cpu_ref, inputs, metrics

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops(libemk):
    from deplodock_b200 import ops as _ops

    assert torch.cuda.is_available()
    return _ops


def _dev(t):
    return t.cuda()


# ------------------------------------------------------------------------------------------------------------
# RMSNorm
# ------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("rows_shape,cols", [((1, 32), 2048), ((3, 5), 100), ((1,), 7), ((2048,), 1024),
                                             ((4, 7), 4096), ((2,), 8200)])
def test_rmsnorm_fp32(ops, rows_shape, cols):
    x, w = inputs.rmsnorm_inputs(rows_shape, cols)
    got = ops.rmsnorm(_dev(x), _dev(w), 1e-6).cpu()
    ops.device_status()
    metrics.assert_fp32_reduction(got, cpu_ref.rmsnorm(x, w, 1e-6), what=f"rmsnorm {rows_shape}x{cols}")


@pytest.mark.parametrize("rows,cols", [(4096, 1024), (33, 4104), (100, 128), (5, 36)])
def test_rmsnorm_bf16_matches_hf_module(ops, rows, cols):
    x, w = inputs.rmsnorm_inputs((rows,), cols, dtype=torch.bfloat16)
    got = ops.rmsnorm(_dev(x), _dev(w), 1e-6).cpu()
    ref = cpu_ref.rmsnorm_hf(x, w, 1e-6)
    metrics.assert_bf16_tensor_path(got, ref, what="rmsnorm bf16")
    # same rounding sequence as the module: at most one bf16 ulp apart, and almost everywhere identical
    assert (got != ref).float().mean().item() < 0.02


def test_rmsnorm_golden(ops):
    ins, outs = load_golden("rmsnorm_readme_shape")
    got = ops.rmsnorm(torch.from_numpy(ins["x"]).cuda(), torch.from_numpy(ins["p_weight"]).cuda(), 1e-6).cpu()
    metrics.assert_fp32_reduction(got, outs["rms_norm"], what="rmsnorm golden")


# ------------------------------------------------------------------------------------------------------------
# Softmax
# ------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("shape", [(1, 2, 64, 2048), (7, 13, 100), (3, 4096), (2, 5000), (1, 1), (5, 33), (4, 1000)])
def test_softmax_fp32(ops, shape):
    x = inputs.softmax_inputs(shape, mask_frac=0.01 if shape[-1] > 1 else 0.0)
    got = ops.softmax_lastdim(_dev(x)).cpu()
    ops.device_status()
    ref = cpu_ref.softmax(x)
    metrics.assert_fp32_reduction(got, ref, abs_floor=1e-30, what=f"softmax {shape}")
    assert torch.equal(got == 0, ref == 0)  # -inf entries give exactly 0
    np.testing.assert_allclose(got.double().sum(-1).numpy(), 1.0, rtol=0, atol=1e-5)


def test_softmax_heavy_mask_and_full_mask_row(ops):
    x = inputs.softmax_inputs((64, 2048), mask_frac=0.9, seed=3)
    x[5] = float("-inf")  # torch returns NaN for a fully masked row; so must the kernel
    got = ops.softmax_lastdim(_dev(x)).cpu()
    ref = cpu_ref.softmax(x)
    assert torch.isnan(got[5]).all() and torch.isnan(ref[5]).all()
    keep = torch.ones(64, dtype=torch.bool)
    keep[5] = False
    metrics.assert_fp32_reduction(got[keep], ref[keep], abs_floor=1e-30, what="softmax heavy mask")


def test_softmax_golden(ops):
    ins, outs = load_golden("softmax_f32")
    got = ops.softmax_lastdim(torch.from_numpy(ins["input"]).cuda()).cpu()
    metrics.assert_fp32_reduction(got, outs["softmax"], abs_floor=1e-30, what="softmax golden")


def test_softmax_full_config_properties(ops):
    """Full benchmark size [1,28,2048,2048]: rows sum to 1, masked entries are 0, argmax preserved, and a slice is
    compared with the oracle."""
    g = torch.Generator(device="cuda").manual_seed(0)
    x = 3.0 * torch.randn(28 * 2048, 2048, device="cuda", generator=g)
    mask = torch.rand(x.shape, device="cuda", generator=g) < 0.01
    mask[:, 0] = False
    x[mask] = float("-inf")
    y = ops.softmax_lastdim(x)
    ops.device_status()
    assert torch.all(y[mask] == 0)
    assert (y.sum(-1) - 1).abs().max().item() < 1e-5
    assert torch.equal(y.argmax(-1), x.argmax(-1))
    sl = slice(12345, 12345 + 64)
    metrics.assert_fp32_reduction(y[sl].cpu(), cpu_ref.softmax(x[sl].cpu()), abs_floor=1e-30, what="softmax slice")


# ------------------------------------------------------------------------------------------------------------
# Linear (bf16 tcgen05), epilogues, layouts
# ------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("M,K,N", [(128, 64, 256), (128, 64, 128), (1, 64, 8), (200, 136, 264), (256, 512, 512),
                                   (1000, 2048, 1024), (130, 72, 520), (4096, 2048, 6144)])
def test_linear_bf16(ops, M, K, N):
    x, w = inputs.linear_inputs(M, K, N)
    got = ops.linear(_dev(x), _dev(w)).cpu()
    ops.device_status()
    metrics.assert_bf16_tensor_path(got, cpu_ref.linear(x, w), what=f"linear {M}x{K}x{N}")


@pytest.mark.parametrize("M,K,N", [(128, 64, 256), (200, 136, 264), (384, 1024, 2048)])
def test_matmul_kn_layout(ops, M, K, N):
    x, w = inputs.linear_inputs(M, K, N)
    wt = w.t().contiguous()  # [K,N] row-major: MatmulOp layout
    got = ops.linear(_dev(x), _dev(wt), w_is_kn=True).cpu()
    ops.device_status()
    metrics.assert_bf16_tensor_path(got, torch.matmul(x, wt), what=f"matmul {M}x{K}x{N}")


def test_linear_tensor_core_equals_cuda_core_path(ops):
    """The tcgen05 kernel against the independent CUDA-core kernel on the device (same inputs, same epilogue)."""
    x, w = inputs.linear_inputs(300, 256, 520, seed=4)
    xd, wd = _dev(x), _dev(w)
    a = ops.linear(xd, wd).float()
    b = ops.linear_simt(xd, wd).float()
    assert (a - b).abs().max().item() <= 2 ** -7 * max(1.0, b.abs().max().item())  # one bf16 ulp of the largest value


def test_linear_residual_bias_swiglu_epilogues(ops):
    M, K, N = 520, 256, 1024
    x, w = inputs.linear_inputs(M, K, N, seed=2)
    g = torch.Generator().manual_seed(9)
    res = torch.randn(M, N, generator=g).bfloat16()
    bias = torch.randn(N, generator=g).bfloat16()
    xd, wd = _dev(x), _dev(w)
    got = ops.linear(xd, wd, residual=_dev(res)).cpu()
    metrics.assert_bf16_tensor_path(got, cpu_ref.linear(x, w) + res, what="linear+residual")
    got = ops.linear(xd, wd, bias=_dev(bias)).cpu()
    metrics.assert_bf16_tensor_path(got, cpu_ref.linear(x, w, bias), what="linear+bias")
    # SwiGLU: interleave gate/up rows the way the model plan does
    wg, wu = w[: N // 2], w[N // 2:]
    wgu = torch.stack([wg, wu], dim=1).reshape(N, K).contiguous()
    got = ops.linear(xd, _dev(wgu), swiglu=True).cpu()
    ops.device_status()
    metrics.assert_bf16_tensor_path(got, cpu_ref.swiglu(x, wg, wu), what="linear+swiglu")


def test_linear_residual_in_place(ops):
    x, w = inputs.linear_inputs(256, 128, 256, seed=3)
    h = torch.randn(256, 256, generator=torch.Generator().manual_seed(1)).bfloat16()
    hd = _dev(h)
    ops.linear(_dev(x), _dev(w), residual=hd, out=hd)
    metrics.assert_bf16_tensor_path(hd.cpu(), cpu_ref.linear(x, w) + h, what="in-place residual")


def test_linear_rejects_unaligned_and_simt_takes_it(ops):
    x, w = inputs.linear_inputs(16, 20, 12)  # K and N not multiples of 8
    with pytest.raises(ValueError):
        ops.linear(_dev(x), _dev(w))
    got = ops.linear_simt(_dev(x), _dev(w)).cpu()
    metrics.assert_bf16_tensor_path(got, cpu_ref.linear(x, w), what="simt linear odd shape")


def test_linear_golden_values_in_bf16(ops):
    ins, outs = load_golden("linear_f32")
    x = torch.from_numpy(ins["input"]).bfloat16()
    w = torch.from_numpy(ins["p_weight"]).bfloat16()
    got = ops.linear(_dev(x), _dev(w)).cpu()
    # inputs rounded to bf16: compare with the fixture at bf16 input precision
    metrics.assert_bf16_tensor_path(got, outs["linear"], abs_tol=6e-2, what="linear golden")
    metrics.assert_bf16_tensor_path(got, cpu_ref.linear(x, w), what="linear golden vs eager bf16")


def test_linear_linearity_at_full_size(ops):
    """Size-independent property at the benchmark size: W(x1 + x2) = W x1 + W x2 up to bf16 rounding."""
    x, w = inputs.linear_inputs(4096, 2048, 6144, seed=5)
    x2 = torch.randn(4096, 2048, generator=torch.Generator().manual_seed(6)).bfloat16()
    wd = _dev(w)
    a = ops.linear(_dev(x), wd).float()
    b = ops.linear(_dev(x2), wd).float()
    c = ops.linear(_dev(x) + _dev(x2), wd).float()
    ops.device_status()
    err = (c - (a + b)).abs().max().item()
    assert err < 0.15, err  # outputs ~N(0, 0.9*sqrt(2)); three bf16 roundings + the rounded sum of inputs


# ------------------------------------------------------------------------------------------------------------
# Linear with e4m3 weights
# ------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("M,K,N", [(128, 64, 256), (200, 144, 264), (512, 1024, 1024), (4096, 2048, 6144)])
def test_linear_w8(ops, M, K, N):
    x, wq, s = inputs.linear_w8_inputs(M, K, N)
    got = ops.linear_w8(_dev(x), _dev(wq), _dev(s)).cpu()
    ops.device_status()
    metrics.assert_bf16_tensor_path(got, cpu_ref.linear_w8(x, wq, s), what=f"linear_w8 {M}x{K}x{N}")


def test_linear_w8_exact_dequant_incl_subnormals(ops):
    """Every e4m3 code (zero, subnormals, max) must dequantise exactly: x = identity picks single weights."""
    K = N = 256
    codes = torch.arange(256, dtype=torch.uint8)
    codes = codes[(codes & 0x7F) != 0x7F]  # drop the two NaN codes
    wq_bits = codes.repeat((N * K + len(codes) - 1) // len(codes))[: N * K].reshape(N, K)
    wq = wq_bits.view(torch.float8_e4m3fn)
    s = torch.ones(N)
    x = torch.eye(K).bfloat16()
    got = ops.linear_w8(_dev(x), _dev(wq), _dev(s)).cpu().float()
    assert torch.equal(got, wq.float().t().contiguous())


def test_linear_w8_nan_codes_stay_nan(ops):
    """The two e4m3 NaN codes take the converter's slow path: a channel that holds one is NaN, the others are exact."""
    K = N = 256
    codes = torch.arange(256, dtype=torch.uint8)
    codes = codes[(codes & 0x7F) != 0x7F]
    bits = codes.repeat((N * K + len(codes) - 1) // len(codes))[: N * K].reshape(N, K).clone()
    bits[5, 7] = 0x7F
    bits[130, 200] = 0xFF
    wq = bits.view(torch.float8_e4m3fn)
    x = torch.eye(K).bfloat16()
    got = ops.linear_w8(_dev(x), _dev(wq), _dev(torch.ones(N)), workspace=None).cpu().float()
    ops.device_status()
    assert torch.isnan(got[:, 5]).all() and torch.isnan(got[:, 130]).all()
    keep = torch.ones(N, dtype=torch.bool)
    keep[[5, 130]] = False
    assert torch.equal(got[:, keep], wq.float().t().contiguous()[:, keep])


@pytest.mark.parametrize("M,K,N", [(512, 1024, 1024), (1000, 144, 264)])
def test_linear_w8_routes_agree(ops, M, K, N):
    """In-loop conversion and expand-once-then-multiply do the same arithmetic (exact e4m3 -> bf16, fp32
    accumulation over k in 16-wide steps, scale on the accumulator)."""
    x, wq, s = inputs.linear_w8_inputs(M, K, N)
    fused = ops.linear_w8(_dev(x), _dev(wq), _dev(s), workspace=None).cpu()
    ws = torch.empty(N * K * 2, dtype=torch.uint8, device="cuda")
    expanded = ops.linear_w8(_dev(x), _dev(wq), _dev(s), workspace=ws).cpu()
    ops.device_status()
    ref = cpu_ref.linear_w8(x, wq, s)
    metrics.assert_bf16_tensor_path(fused, ref, what="linear_w8 in-loop")
    metrics.assert_bf16_tensor_path(expanded, ref, what="linear_w8 expanded")
    # accumulation order over k differs between the two tensor-core kernels only in how K is chunked: allow one ulp
    assert (fused.float() - expanded.float()).abs().max().item() <= 2.0 ** -7 * ref.float().abs().max().item()


def test_linear_w8_expanded_exact_dequant(ops):
    K = N = 256
    codes = torch.arange(256, dtype=torch.uint8)
    codes = codes[(codes & 0x7F) != 0x7F]
    wq = codes.repeat((N * K + len(codes) - 1) // len(codes))[: N * K].reshape(N, K).view(torch.float8_e4m3fn)
    x = torch.zeros(512, K)
    x[:K] = torch.eye(K)
    ws = torch.empty(N * K * 2, dtype=torch.uint8, device="cuda")
    got = ops.linear_w8(_dev(x.bfloat16()), _dev(wq), _dev(torch.ones(N)), workspace=ws).cpu().float()
    assert torch.equal(got[:K], wq.float().t().contiguous())
    assert torch.count_nonzero(got[K:]) == 0


def test_linear_w8_workspace_too_small(ops):
    x, wq, s = inputs.linear_w8_inputs(512, 64, 64)
    with pytest.raises(ValueError, match="workspace"):
        ops.linear_w8(_dev(x), _dev(wq), _dev(s), workspace=torch.empty(64, dtype=torch.uint8, device="cuda"))


# ------------------------------------------------------------------------------------------------------------
# Attention
# ------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("B,Hq,Hkv,S", [(1, 2, 1, 128), (1, 2, 1, 256), (1, 1, 1, 256), (2, 6, 2, 384), (1, 4, 2, 200),
                                        (1, 3, 1, 130), (2, 16, 8, 512), (1, 2, 2, 1)])
def test_sdpa_causal_gqa_bf16(ops, B, Hq, Hkv, S):
    q, k, v = inputs.sdpa_inputs(B, Hq, Hkv, S)
    got = ops.sdpa_causal_gqa(_dev(q), _dev(k), _dev(v)).cpu()
    ops.device_status()
    metrics.assert_bf16_tensor_path(got, cpu_ref.sdpa_causal_gqa(q, k, v), what=f"sdpa {B},{Hq},{Hkv},{S}")
    metrics.assert_bf16_tensor_path(got, cpu_ref.sdpa_causal_gqa_fp32(q, k, v), abs_tol=1.2e-2, what="sdpa vs fp32")


def test_sdpa_full_config(ops):
    q, k, v = inputs.sdpa_inputs(4, 16, 8, 2048)
    got = ops.sdpa_causal_gqa(_dev(q), _dev(k), _dev(v))
    ops.device_status()
    # oracle on a bounded sample: batch 1, one KV group (heads 6,7 share KV head 3)
    ref = cpu_ref.sdpa_causal_gqa(q[1:2, 6:8], k[1:2, 3:4], v[1:2, 3:4])
    metrics.assert_bf16_tensor_path(got[1:2, 6:8].cpu(), ref, what="sdpa full config slice")
    # property: row 0 of every head attends only to key 0 -> output equals v[:, h//2, 0]
    first = got[:, :, 0].cpu().float()
    want = v[:, :, 0].float().repeat_interleave(2, dim=1)
    assert (first - want).abs().max().item() < 1e-2
    # device-side cross-check against the CUDA-core kernel
    alt = ops.sdpa_simt(_dev(q[:1]), _dev(k[:1]), _dev(v[:1]), True)
    metrics.assert_bf16_tensor_path(got[:1].cpu(), alt.cpu(), what="tcgen05 vs simt")


def test_sdpa_token_major_equals_head_major(ops):
    B, S, Hq, Hkv = 2, 300, 4, 2
    g = torch.Generator().manual_seed(7)
    qkv = torch.randn(B * S, (Hq + 2 * Hkv) * 128, generator=g).bfloat16()
    out = torch.empty(B * S, Hq * 128, dtype=torch.bfloat16, device="cuda")
    ops.sdpa_causal_gqa_tok(_dev(qkv), B, S, Hq, Hkv, out)
    ops.device_status()
    q = qkv[:, : Hq * 128].view(B, S, Hq, 128).transpose(1, 2)
    k = qkv[:, Hq * 128: (Hq + Hkv) * 128].view(B, S, Hkv, 128).transpose(1, 2)
    v = qkv[:, (Hq + Hkv) * 128:].view(B, S, Hkv, 128).transpose(1, 2)
    ref = cpu_ref.sdpa_causal_gqa(q, k, v)
    metrics.assert_bf16_tensor_path(out.cpu().view(B, S, Hq, 128).transpose(1, 2), ref, what="token-major sdpa")


def test_sdpa_golden_d128(ops):
    ins, outs = load_golden("sdpa_causal_gqa_d128_f32")
    q, k, v = (torch.from_numpy(ins[n]).bfloat16() for n in "qkv")
    got = ops.sdpa_causal_gqa(_dev(q), _dev(k), _dev(v)).cpu()
    metrics.assert_bf16_tensor_path(got, outs["scaled_dot_product_attention"], abs_tol=4e-2, what="sdpa golden (bf16 in)")
    metrics.assert_bf16_tensor_path(got, cpu_ref.sdpa_causal_gqa(q, k, v), what="sdpa golden vs eager bf16")


@pytest.mark.parametrize("case,causal", [("sdpa_causal_gqa_f32", True), ("sdpa_full_f32", False)])
def test_sdpa_simt_fp32_golden(ops, case, causal):
    ins, outs = load_golden(case)
    q, k, v = (torch.from_numpy(ins[n]).cuda() for n in "qkv")
    got = ops.sdpa_simt(q, k, v, causal).cpu()
    np.testing.assert_allclose(got.numpy(), outs["scaled_dot_product_attention"], rtol=5e-5, atol=2e-6)


def test_sdpa_rejects_head_dim(ops):
    q, k, v = inputs.sdpa_inputs(1, 2, 1, 64, D=64)
    with pytest.raises(ValueError):
        ops.sdpa_causal_gqa(_dev(q), _dev(k), _dev(v))


# ------------------------------------------------------------------------------------------------------------
# Pointwise kernels of the embedding forward
# ------------------------------------------------------------------------------------------------------------
def test_embed_gather_and_clamp(ops):
    table = torch.randn(50, 1024, generator=torch.Generator().manual_seed(0)).bfloat16()
    ids = inputs.token_ids(3, 17, 50)
    got = ops.embed_gather(_dev(table), _dev(ids)).cpu()
    assert torch.equal(got, table[ids.flatten()])


def test_qknorm_rope_bit_exact_vs_eager_module(ops):
    B, S, Hq, Hkv, D = 2, 40, 16, 8, 128
    g = torch.Generator().manual_seed(11)
    qkv = torch.randn(B * S, (Hq + 2 * Hkv) * D, generator=g).bfloat16()
    qw = (1 + 0.1 * torch.randn(D, generator=g)).bfloat16()
    kw = (1 + 0.1 * torch.randn(D, generator=g)).bfloat16()
    cos, sin = inputs.rope_tables(S, D, 1e6)
    cb, sb = cos.bfloat16(), sin.bfloat16()

    def rot(x):
        return torch.cat([-x[..., D // 2:], x[..., : D // 2]], dim=-1)

    ref = qkv.clone()
    q = cpu_ref.rmsnorm_hf(qkv[:, : Hq * D].view(B, S, Hq, D), qw)
    k = cpu_ref.rmsnorm_hf(qkv[:, Hq * D: (Hq + Hkv) * D].view(B, S, Hkv, D), kw)
    c4, s4 = cb[None, :, None, :], sb[None, :, None, :]
    ref[:, : Hq * D] = ((q * c4) + (rot(q) * s4)).reshape(B * S, -1)
    ref[:, Hq * D: (Hq + Hkv) * D] = ((k * c4) + (rot(k) * s4)).reshape(B * S, -1)
    got = ops.qknorm_rope_(_dev(qkv), _dev(qw), _dev(kw), _dev(cb), _dev(sb), S, Hq, Hkv, 1e-6).cpu()
    ops.device_status()
    assert torch.equal(got[:, (Hq + Hkv) * D:], qkv[:, (Hq + Hkv) * D:])  # V untouched
    mism = (got != ref).float().mean().item()
    assert mism < 0.01, mism  # identical rounding sequence; only the fp32 sum order differs
    metrics.assert_bf16_tensor_path(got, ref, what="qknorm_rope")


def test_pool_norm_l2(ops):
    B, S, H = 5, 9, 1024
    g = torch.Generator().manual_seed(2)
    hs = torch.randn(B * S, H, generator=g).bfloat16()
    w = (1 + 0.1 * torch.randn(H, generator=g)).bfloat16()
    got = ops.pool_norm_l2(_dev(hs), _dev(w), B, S).cpu()
    last = hs.view(B, S, H)[:, -1]
    ref = torch.nn.functional.normalize(cpu_ref.rmsnorm_hf(last, w).float(), dim=-1)
    assert (got - ref).abs().max().item() < 2e-4
    np.testing.assert_allclose(got.double().norm(dim=-1).numpy(), 1.0, atol=1e-5)


# ------------------------------------------------------------------------------------------------------------
# Error path: a bounded device-side wait that expires is reported, and the context stays usable
# ------------------------------------------------------------------------------------------------------------
def test_expired_device_wait_is_reported_and_context_survives(ops):
    from deplodock_b200.cabi import HungKernelError

    ops.selftest_wait_expiry(20)
    with pytest.raises(HungKernelError):
        ops.device_status()
    ops.device_status()  # cleared
    x, w = inputs.rmsnorm_inputs((4,), 256)
    got = ops.rmsnorm(_dev(x), _dev(w)).cpu()
    metrics.assert_fp32_reduction(got, cpu_ref.rmsnorm(x, w), what="after expiry")


@pytest.mark.parametrize("B,S", [(2, 40), (3, 130), (1, 512)])
def test_linear_qknorm_rope_fused_equals_two_step(ops, B, S):
    """The fused epilogue against projection + stand-alone q/k-norm+RoPE kernel, and against
    the eager module's rounding sequence."""
    Hq, Hkv, D, K = 16, 8, 128, 256
    T = B * S
    g = torch.Generator().manual_seed(21)
    x = torch.randn(T, K, generator=g).bfloat16()
    w = (0.06 * torch.randn((Hq + 2 * Hkv) * D, K, generator=g)).bfloat16()
    qw = (1 + 0.1 * torch.randn(D, generator=g)).bfloat16()
    kw = (1 + 0.1 * torch.randn(D, generator=g)).bfloat16()
    cos, sin = inputs.rope_tables(S, D, 1e6)
    cb, sb = cos.bfloat16(), sin.bfloat16()
    cm = ops.rope_chunk_major(_dev(cb), _dev(sb))
    fused = ops.linear_qknorm_rope(_dev(x), _dev(w), _dev(qw), _dev(kw), cm, S, Hq, Hkv, 1e-6).cpu()
    two = ops.qknorm_rope_(ops.linear(_dev(x), _dev(w)), _dev(qw), _dev(kw), _dev(cb), _dev(sb), S, Hq, Hkv, 1e-6).cpu()
    ops.device_status()
    assert (fused != two).float().mean().item() < 0.005  # same arithmetic; only the order of the fp32 row sum differs
    metrics.assert_bf16_tensor_path(fused, two, what="fused vs two-step")

    def rot(t):
        return torch.cat([-t[..., D // 2:], t[..., : D // 2]], dim=-1)

    proj = cpu_ref.linear(x, w)
    q = cpu_ref.rmsnorm_hf(proj[:, : Hq * D].view(B, S, Hq, D), qw)
    k = cpu_ref.rmsnorm_hf(proj[:, Hq * D: (Hq + Hkv) * D].view(B, S, Hkv, D), kw)
    c4, s4 = cb[None, :, None, :], sb[None, :, None, :]
    ref = proj.clone()
    ref[:, : Hq * D] = ((q * c4) + (rot(q) * s4)).reshape(T, -1)
    ref[:, Hq * D: (Hq + Hkv) * D] = ((k * c4) + (rot(k) * s4)).reshape(T, -1)
    metrics.assert_bf16_tensor_path(fused, ref, abs_tol=6e-2, what="fused qkv vs eager")


def test_gemm_fused_row_sumsq_protocol(ops):
    """Producer GEMM writes the partial row sums of squares of what it stores; the consumer GEMM scales its rows by
    rsqrt(mean + eps) with the norm weight folded into W: together they equal linear -> rmsnorm -> linear with
    stand-alone kernels. The partial buffer is overwritten, not accumulated, and the result is bitwise repeatable."""
    M, K, H, N2 = 300, 256, 512, 768
    g = torch.Generator().manual_seed(31)
    x = torch.randn(M, K, generator=g).bfloat16()
    w1 = (0.06 * torch.randn(H, K, generator=g)).bfloat16()
    res = torch.randn(M, H, generator=g).bfloat16()
    wn = (1 + 0.1 * torch.randn(H, generator=g)).bfloat16()
    w2 = (0.05 * torch.randn(N2, H, generator=g)).bfloat16()
    xd, w1d, w2d, wnd = _dev(x), _dev(w1), _dev(w2), _dev(wn)
    ss = torch.full((M, H // 128), 123.0, dtype=torch.float32, device="cuda")  # stale contents must not matter
    h = torch.empty(M, H, dtype=torch.bfloat16, device="cuda")
    ops.gemm_fused(xd, w1d, h, epilogue="residual", residual=_dev(res), row_sumsq_out=ss)
    ops.device_status()
    want_ss = h.float().pow(2).sum(-1)
    assert torch.allclose(ss.sum(1), want_ss, rtol=1e-4, atol=1e-3)
    metrics.assert_bf16_tensor_path(h.cpu(), cpu_ref.linear(x, w1) + res, what="producer output")
    w2_folded = (w2d.float() * wnd.float()[None, :]).bfloat16().contiguous()
    y = torch.empty(M, N2, dtype=torch.bfloat16, device="cuda")
    ops.gemm_fused(h, w2_folded, y, epilogue="none", row_sumsq_in=ss, norm_dim=H, norm_eps=1e-6)
    two_step = ops.linear(ops.rmsnorm(h, wnd, 1e-6), w2d)
    ops.device_status()
    metrics.assert_bf16_tensor_path(y.cpu(), two_step.cpu(), what="folded rmsnorm vs stand-alone")
    ref = cpu_ref.linear(cpu_ref.rmsnorm_hf(h.cpu(), wn, 1e-6), w2)
    metrics.assert_bf16_tensor_path(y.cpu(), ref, what="folded rmsnorm vs eager")
    y2 = torch.empty_like(y)
    ss2 = torch.zeros_like(ss)
    h2 = torch.empty_like(h)
    ops.gemm_fused(xd, w1d, h2, epilogue="residual", residual=_dev(res), row_sumsq_out=ss2)
    ops.gemm_fused(h2, w2_folded, y2, epilogue="none", row_sumsq_in=ss2, norm_dim=H, norm_eps=1e-6)
    assert torch.equal(ss, ss2) and torch.equal(y, y2)
    # the gather writes the same layout
    table = torch.randn(64, H, generator=g).bfloat16()
    ids = inputs.token_ids(2, 9, 64)
    ssg = torch.full((18, H // 128), -1.0, dtype=torch.float32, device="cuda")
    rows = ops.embed_gather(_dev(table), _dev(ids), row_sumsq=ssg)
    assert torch.allclose(ssg.sum(1), rows.float().pow(2).sum(-1), rtol=1e-5) and float(ssg[:, 1:].abs().max()) == 0.0


# ------------------------------------------------------------------------------------------------------------
# Whole-tensor comparisons at the benchmark sizes, bf16 softmax, row sums of squares from the single-CTA GEMM
# ------------------------------------------------------------------------------------------------------------
def _fp32_rel_err(got: torch.Tensor, ref: torch.Tensor, abs_floor: float) -> float:
    """max |got - ref| / max(|ref|, abs_floor) in fp32 on the CPU (the float64 route of ``metrics`` would hold three
    1 GB arrays for the 117 M-element softmax)."""
    return ((got - ref).abs() / ref.abs().clamp_min(abs_floor)).max().item()


def test_softmax_full_config_whole_tensor_vs_oracle(ops):
    """[1,28,2048,2048] with 1 % of the entries at -inf: every one of the 117 440 512 outputs against the eager CPU
    module on the same seeded input."""
    x = inputs.softmax_inputs((1, 28, 2048, 2048))
    got = ops.softmax_lastdim(_dev(x)).cpu()
    ops.device_status()
    ref = cpu_ref.softmax(x)
    assert torch.equal(got == 0, ref == 0)
    assert torch.isfinite(got).all()
    assert _fp32_rel_err(got, ref, 1e-30) <= 1e-5


def test_sdpa_full_config_whole_tensor_vs_oracle(ops):
    """B4 Hq16 Hkv8 S2048 D128: all 64 heads against the eager CPU call (bf16) on the same seeded inputs."""
    q, k, v = inputs.sdpa_inputs(4, 16, 8, 2048)
    got = ops.sdpa_causal_gqa(_dev(q), _dev(k), _dev(v)).cpu()
    ops.device_status()
    ref = cpu_ref.sdpa_causal_gqa(q, k, v)
    assert torch.isfinite(got).all()
    err = (got.float() - ref.float()).abs().max().item()
    assert err <= max(2e-2, ref.float().abs().max().item() * 2.0 ** -7), err
    cos = torch.nn.functional.cosine_similarity(got.float(), ref.float(), dim=-1).min().item()
    assert cos >= 0.999, cos


@pytest.mark.parametrize("shape", [(64, 2048), (3, 5, 100), (7, 4096), (33, 1000), (2, 8192)])
def test_softmax_bf16(ops, shape):
    """bf16 rows: the eager CPU module computes in fp32 and rounds once; so does the kernel."""
    x = inputs.softmax_inputs(shape, mask_frac=0.05, seed=7).bfloat16()
    got = ops.softmax_lastdim(_dev(x)).cpu()
    ops.device_status()
    ref = cpu_ref.softmax(x)
    assert got.dtype == torch.bfloat16 and torch.equal(got == 0, ref == 0)
    # one rounding of the same fp32 value: at most one bf16 ulp apart
    assert ((got.float() - ref.float()).abs() <= ref.float().abs() * 2.0 ** -7 + 1e-30).all()
    assert (got != ref).float().mean().item() < 0.02


@pytest.mark.parametrize("M,K,N", [(128, 256, 512), (96, 128, 384), (64, 256, 128), (100, 64, 64), (300, 256, 128),
                                   (300, 128, 64)])
def test_row_sumsq_out_small_shapes(ops, M, K, N):
    """Partial row sums of squares from the shapes that do not take the 256-wide CTA-pair tiles: M <= 128 (single-CTA
    kernel) and N <= 128 (one slot per row, never split between two epilogue threads)."""
    g = torch.Generator().manual_seed(41)
    x = torch.randn(M, K, generator=g).bfloat16()
    w = (0.06 * torch.randn(N, K, generator=g)).bfloat16()
    res = torch.randn(M, N, generator=g).bfloat16()
    slots = (N + 127) // 128
    ss = torch.full((M, slots), -7.0, dtype=torch.float32, device="cuda")
    h = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    ops.gemm_fused(_dev(x), _dev(w), h, epilogue="residual", residual=_dev(res), row_sumsq_out=ss)
    ops.device_status()
    ref_h = cpu_ref.linear(x, w) + res
    metrics.assert_bf16_tensor_path(h.cpu(), ref_h, what="producer output")
    # every slot is overwritten (no stale -7), and the slots of a row add up to the row's sum of squares (a thread
    # puts its whole total into the first slot it covers and zeros into the rest: only the sum is defined)
    assert (ss >= 0).all()
    assert torch.allclose(ss.sum(1), h.float().pow(2).sum(-1), rtol=1e-4, atol=1e-3)
    # and against the oracle's rows (bf16 rounding of h is the only difference)
    assert torch.allclose(ss.sum(1).cpu(), ref_h.float().pow(2).sum(-1), rtol=2e-2, atol=1e-2)


# ------------------------------------------------------------------------------------------------------------
# Packed variable-length attention and pooling
# ------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("lens,Hq,Hkv", [([33, 128, 5], 4, 2), ([1, 127, 129, 0, 300, 256], 16, 8), ([512], 2, 2),
                                         ([130, 130, 130, 7], 3, 1)])
def test_sdpa_varlen_matches_per_sequence_oracle(ops, lens, Hq, Hkv):
    """Sequences packed back to back (no padding), one launch; every sequence against the eager CPU call on its own
    rows; an empty sequence and a trailing run of rows outside every sequence are left untouched."""
    g = torch.Generator().manual_seed(sum(lens) + Hq)
    tail = 9
    T = sum(lens) + tail
    qkv = torch.randn(T, (Hq + 2 * Hkv) * 128, generator=g).bfloat16()
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
    out = torch.full((T, Hq * 128), 7.0, dtype=torch.bfloat16, device="cuda")
    ops.sdpa_causal_gqa_varlen(_dev(qkv), _dev(cu), max(lens), Hq, Hkv, out)
    ops.device_status()
    got = out.cpu()
    off = 0
    for n in lens:
        if n:
            rows = qkv[off:off + n]
            q = rows[:, : Hq * 128].view(1, n, Hq, 128).transpose(1, 2)
            k = rows[:, Hq * 128: (Hq + Hkv) * 128].view(1, n, Hkv, 128).transpose(1, 2)
            v = rows[:, (Hq + Hkv) * 128:].view(1, n, Hkv, 128).transpose(1, 2)
            ref = cpu_ref.sdpa_causal_gqa(q, k, v).transpose(1, 2).reshape(n, Hq * 128)
            metrics.assert_bf16_tensor_path(got[off:off + n], ref, what=f"sequence of {n} at row {off}")
        off += n
    assert (got[off:] == 7.0).all(), "rows outside every sequence were written"


def test_sdpa_varlen_equals_fixed_length_kernel_bitwise(ops):
    """Equal lengths: the packed path must give the bits of the fixed-length token-major path (same blocks of keys,
    same per-row arithmetic; only the order in which work items are visited differs)."""
    B, S, Hq, Hkv = 5, 300, 4, 2
    qkv = torch.randn(B * S, (Hq + 2 * Hkv) * 128, generator=torch.Generator().manual_seed(3)).bfloat16().cuda()
    a = torch.empty(B * S, Hq * 128, dtype=torch.bfloat16, device="cuda")
    b = torch.empty_like(a)
    ops.sdpa_causal_gqa_tok(qkv, B, S, Hq, Hkv, a)
    cu = torch.arange(0, (B + 1) * S, S, dtype=torch.int32, device="cuda")
    ops.sdpa_causal_gqa_varlen(qkv, cu, S, Hq, Hkv, b)
    ops.device_status()
    assert torch.equal(a, b)


def test_sdpa_varlen_argument_checks(ops):
    qkv = torch.zeros(256, 4 * 128, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(256, 2 * 128, dtype=torch.bfloat16, device="cuda")
    cu = torch.tensor([0, 256], dtype=torch.int32, device="cuda")
    with pytest.raises(ValueError, match="workspace"):
        ops.sdpa_causal_gqa_varlen(qkv, cu, 256, 2, 1, out, workspace=torch.zeros(16, dtype=torch.uint8, device="cuda"))
    with pytest.raises(TypeError):
        ops.sdpa_causal_gqa_varlen(qkv, cu.long(), 256, 2, 1, out)
    with pytest.raises(ValueError):
        ops.sdpa_causal_gqa_varlen(qkv, cu, 1 << 20, 2, 1, out)   # longer than the query-block table admits


def test_pool_norm_l2_varlen(ops):
    H = 1024
    lens = [5, 0, 9, 1]
    g = torch.Generator().manual_seed(2)
    hs = torch.randn(sum(lens), H, generator=g).bfloat16()
    w = (1 + 0.1 * torch.randn(H, generator=g)).bfloat16()
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
    got = ops.pool_norm_l2_varlen(_dev(hs), _dev(w), _dev(cu)).cpu()
    ops.device_status()
    for b, n in enumerate(lens):
        if n == 0:
            assert float(got[b].abs().max()) == 0.0
            continue
        last = hs[int(cu[b + 1]) - 1]
        ref = torch.nn.functional.normalize(cpu_ref.rmsnorm_hf(last[None], w).float(), dim=-1)[0]
        assert (got[b] - ref).abs().max().item() < 2e-4


# ------------------------------------------------------------------------------------------------------------
# fp32 contraction on CUDA cores (register-tiled), both weight layouts, bias, ragged and unaligned shapes
# ------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("M,K,N", [(512, 1024, 2048), (32, 1024, 2048), (128, 3072, 1024), (100, 68, 132),
                                   (65, 16, 64), (1, 8, 4), (70, 36, 90), (33, 30, 50)])
@pytest.mark.parametrize("kn", [False, True])
def test_linear_f32_tiled_and_fallback(ops, M, K, N, kn):
    """K (and N for [K,N] weights) a multiple of 4 takes the register-tiled kernel, anything else the one-output-per
    thread kernel; both against a float64 product, and the tiled kernel bit-for-bit against the serial fmaf chain."""
    g = torch.Generator().manual_seed(M + K + N)
    x = torch.randn(M, K, generator=g)
    w = torch.randn(N, K, generator=g)
    bias = torch.randn(N, generator=g)
    wd = _dev(w.t().contiguous() if kn else w)
    got = ops.linear_f32(_dev(x), wd, _dev(bias), kn, route="simt").cpu()
    ops.device_status()
    want = x.double() @ w.double().t() + bias.double()
    scale = want.abs().max().item()
    assert (got.double() - want).abs().max().item() <= 1e-5 * scale
    if M * N <= 100 * 132:   # serial chain on the host: fmaf over k in ascending order, then + bias
        acc = np.zeros((M, N), dtype=np.float32)
        xn, wn = x.numpy(), w.numpy()
        for k in range(K):
            acc = np.asarray(np.float64(xn[:, k:k + 1]) * np.float64(wn[None, :, k]) + np.float64(acc), dtype=np.float32)
        ref = acc + bias.numpy()[None, :]
        assert np.array_equal(got.numpy(), ref), "not the serial fmaf chain"


@pytest.mark.parametrize("M,K,N", [(512, 1024, 2048), (256, 64, 8), (300, 136, 264), (1000, 3072, 1024), (40, 64, 96)])
@pytest.mark.parametrize("kn", [False, True])
def test_linear_f32_on_tensor_cores(ops, M, K, N, kn):
    """fp32 in, fp32 out, through one bf16 tcgen05 GEMM over exactly split operands: against a float64 product at the
    tolerance of an fp32 reduction, and against the CUDA-core kernel."""
    g = torch.Generator().manual_seed(M + 7 * K + N)
    x = torch.randn(M, K, generator=g) * torch.rand(M, 1, generator=g) * 4   # rows of different magnitude
    w = torch.randn(N, K, generator=g)
    w[::7] *= 1e-3
    bias = torch.randn(N, generator=g)
    wd = _dev(w.t().contiguous() if kn else w)
    got = ops.linear_f32(_dev(x), wd, _dev(bias), kn, route="tc").cpu()
    alt = ops.linear_f32(_dev(x), wd, _dev(bias), kn, route="simt").cpu()
    ops.device_status()
    want = x.double() @ w.double().t() + bias.double()
    # per output against the sum of |products| (what any fp32 accumulation order is held to): the CUDA-core kernel
    # rounds every step, the tensor core truncates its accumulator (see emk_linear_f32_tc) and lands within 2e-5;
    # element-wise the reference's own bound for fp32 matmul (rtol 5e-5, atol 2e-6 of the scale) holds with room
    mag = (x.double().abs() @ w.double().abs().t() + bias.double().abs())
    scale = want.abs().max().item()
    assert ((alt.double() - want).abs() <= 1e-5 * mag.clamp_min(1e-30)).all()
    assert ((got.double() - want).abs() <= 2e-5 * mag.clamp_min(1e-30)).all()
    assert ((got.double() - want).abs() <= 5e-5 * want.abs() + 2e-6 * scale).all()
    print(f"fp32 tc M{M} K{K} N{N}: max err / scale = {(got.double() - want).abs().max().item() / scale:.2e}")
    with pytest.raises(ValueError):
        ops.linear_f32(_dev(x[:, :4].contiguous()), _dev(w[:, :4].contiguous()), None, False, route="tc")
