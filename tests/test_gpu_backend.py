"""``B200Backend`` through the reference's call surface (compile / run / benchmark_async) on traced graph records."""

from __future__ import annotations

import asyncio

import numpy as np
import pytest
import torch

from conftest import GOLDEN, load_golden
from oracle import cpu_ref, inputs, metrics

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def backend(libemk):
    from deplodock_b200.backend import B200Backend

    return B200Backend()


@pytest.mark.parametrize("case,rtol,atol", [
    ("rmsnorm_f32", 1e-5, 1e-6), ("rmsnorm_readme_shape", 1e-5, 1e-6), ("softmax_f32", 1e-5, 1e-7),
    ("linear_f32", 1e-4, 2e-6), ("linear_bias_f32", 1e-4, 2e-6), ("matmul_f32", 5e-5, 2e-6),
    ("sdpa_causal_gqa_f32", 5e-5, 2e-6), ("sdpa_full_f32", 5e-5, 2e-6), ("sdpa_causal_gqa_d128_f32", 5e-5, 2e-6),
    ("swiglu_f32", 1e-4, 1e-4)])
def test_run_matches_reference_fixture(backend, case, rtol, atol):
    """Tolerances are the reference's per-op ones (tests/compiler/e2e/test_ops_vs_torch.py:303-449) or tighter."""
    ins, outs = load_golden(case)
    compiled = backend.compile(GOLDEN / "graphs" / f"{case}.json")
    result, pre = backend.run(compiled, input_data=ins, pre_run=lambda: "pre")
    assert pre == "pre" and result.time_ms > 0
    assert set(result.outputs) == set(outs)
    for name, ref in outs.items():
        got = result.outputs[name]
        assert got.shape == ref.shape and got.dtype == ref.dtype
        np.testing.assert_allclose(got, ref, rtol=rtol, atol=atol)


def test_bf16_graph_uses_uint16_carriers_and_fp32_weights(backend):
    rec = {"inputs": ["x"], "outputs": ["linear"], "nodes": {
        "x": {"op": "InputOp", "op_fields": {}, "inputs": [], "output": {"name": "x", "shape": [200, 256], "dtype": "bf16"}},
        "p_weight": {"op": "ConstantOp", "op_fields": {"name": "p_weight", "value": None, "source_path": "weight"},
                     "inputs": [], "output": {"name": "p_weight", "shape": [520, 256], "dtype": "bf16"}},
        "linear": {"op": "LinearOp", "op_fields": {"has_bias": False}, "inputs": ["x", "p_weight"],
                   "output": {"name": "linear", "shape": [200, 520], "dtype": "bf16"}}}}
    x, w = inputs.linear_inputs(200, 256, 520)
    compiled = backend.compile(rec)
    assert compiled.steps[0].entry == "emk_linear_bf16"
    feed = {"x": x.view(torch.uint16).numpy(), "p_weight": w.float().numpy()}  # weights arrive as fp32 from HF modules
    result, _ = backend.run(compiled, input_data=feed)
    out = result.outputs["linear"]
    assert out.dtype == np.uint16
    got = torch.from_numpy(out.view(np.int16)).view(torch.bfloat16)
    metrics.assert_bf16_tensor_path(got, cpu_ref.linear(x, w), what="backend bf16 linear")


def test_missing_input_raises_keyerror(backend):
    compiled = backend.compile(GOLDEN / "graphs" / "rmsnorm_f32.json")
    ins, _ = load_golden("rmsnorm_f32")
    with pytest.raises(KeyError):
        backend.run(compiled, input_data={"p_weight": ins["p_weight"]})
    with pytest.raises(KeyError):
        backend.run(compiled, input_data={"x": ins["x"]})


def test_benchmark_async_result_shape(backend):
    compiled = backend.compile(GOLDEN / "graphs" / "rmsnorm_readme_shape.json")
    seen = []
    res = asyncio.run(backend.benchmark_async(compiled, warmup=2, num_iters=5, on_iter=seen.append))
    assert res.num_launches == 1 and res.captured and res.e2e_ms is None
    lt = res.per_launch[0]
    assert lt.kernel_name.startswith("k_rms_norm_") and len(lt.samples) == 5 and lt.time_ms > 0
    assert res.min_ms <= res.time_ms <= res.max_ms
    assert seen == list(range(5))
    assert lt.time_ms < 0.1  # a 0.5 MB rmsnorm is microseconds, not a host-timed call
