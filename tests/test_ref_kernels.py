"""The hand-written kernels against the reference compiler's own emitted kernels, on the four kernel configurations at
their full sizes and on the same seeded inputs. ``oracle/_ref/`` holds those kernels (lowered for sm_100 by the
reference's pipeline and compiled with its nvcc flags by ``oracle/build_ref_kernels.py``); the tests are skipped where
it has not been built."""

from __future__ import annotations

import pytest
import torch

from oracle import cpu_ref, inputs, metrics, ref_kernels

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not ref_kernels.available(), reason="oracle/_ref not built")]


@pytest.fixture(scope="module")
def ops(libemk):
    from deplodock_b200 import ops as _ops

    assert torch.cuda.is_available()
    return _ops


def test_rmsnorm_matches_emitted_kernel(ops):
    x, w = inputs.rmsnorm_inputs()
    k = ref_kernels.RefKernel("rmsnorm")
    k.bind(x=x, p_weight=w)
    k.launch()
    ref = k.output.cpu()
    got = ops.rmsnorm(x.cuda(), w.cuda(), 1e-6).cpu()
    metrics.assert_fp32_reduction(got, ref, what="rmsnorm vs emitted kernel")
    metrics.assert_fp32_reduction(ref, cpu_ref.rmsnorm(x, w, 1e-6), what="emitted kernel vs eager CPU")


def test_softmax_matches_emitted_kernel(ops):
    x = inputs.softmax_inputs((1, 28, 2048, 2048))
    k = ref_kernels.RefKernel("softmax")
    k.bind(input=x)
    k.launch()
    ref = k.output
    got = ops.softmax_lastdim(x.cuda())
    # the emitted kernel is compiled with --use_fast_math (__expf, approximate division) and seeds the running maximum
    # with a soft -inf (-1e30), so it is itself a few 1e-6 away from the exact probabilities
    assert torch.isfinite(ref).all()
    diff = (got - ref).abs().max().item()
    assert diff <= 2e-5, diff
    assert torch.equal(got == 0, torch.isinf(x.cuda()) & (x.cuda() < 0)), "exact zeros exactly at the masked entries"


def test_linear_matches_emitted_kernel(ops):
    x, w = inputs.linear_inputs()
    k = ref_kernels.RefKernel("linear")
    k.bind(input=x, linear_wt=w.t().contiguous())   # the reference re-lays the weight as [K, N] at bind time
    k.launch()
    ref = k.output.cpu()
    got = ops.linear(x.cuda(), w.cuda()).cpu()
    metrics.assert_bf16_tensor_path(got, ref, what="linear vs emitted kernel")


def test_sdpa_matches_emitted_kernel(ops):
    q, kk, v = inputs.sdpa_inputs()
    k = ref_kernels.RefKernel("sdpa")
    k.bind(q=q, k=kk, v=v)
    k.launch()
    ref = k.output.cpu()
    got = ops.sdpa_causal_gqa(q.cuda(), kk.cuda(), v.cuda()).cpu()
    metrics.assert_bf16_tensor_path(got, ref, what="sdpa vs emitted kernel")


def test_fp32_matmul_matches_emitted_kernel(ops):
    """The fp32 tier: the q_proj shape of the reference's perf suite (512 x 1024 x 2048, B row-major [K, N])."""
    if "matmul_f32" not in __import__("json").loads((ref_kernels.REF_DIR / "manifest.json").read_text()):
        pytest.skip("oracle/_ref was built without the fp32 matmul configuration")
    g = torch.Generator().manual_seed(0)
    a = torch.randn(512, 1024, generator=g)
    b = torch.randn(1024, 2048, generator=g)
    k = ref_kernels.RefKernel("matmul_f32")
    k.bind(a=a, b=b)
    k.launch()
    ref = k.output.cpu()
    got = ops.linear_f32(a.cuda(), b.cuda(), None, True).cpu()
    want = torch.matmul(a.double(), b.double())
    scale = want.abs().max().item()
    # both sum 1024 fp32 products per output, in different orders: a few 1e-6 of the output scale apart
    assert (got.double() - want).abs().max().item() <= 2e-5 * scale
    assert (ref.double() - want).abs().max().item() <= 2e-5 * scale
    assert (got - ref).abs().max().item() <= 4e-5 * scale
