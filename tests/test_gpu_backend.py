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


def test_symbolic_sequence_length_one_compile_many_sizes(backend):
    """A graph traced with a symbolic axis is compiled once and run at several runtime sizes (one launch plan per
    size, weights uploaded once) — the reference's dynamic ``seq_len`` (``emmy/compiler/backend/cuda/program.py:770-958``)."""
    from deplodock_b200.trace import parse_dynamic_specs, trace_inline_code

    tr = trace_inline_code("nn.RMSNorm(2048, eps=1e-6)(torch.randn(1, 32, 2048))", parse_dynamic_specs(["seq_len@x:1"]))
    plan = backend.compile(tr.graph)
    assert plan.symbolic
    w = (1 + 0.02 * torch.randn(2048, generator=torch.Generator().manual_seed(1))).numpy()
    for S in (32, 7, 300):
        x = torch.randn(1, S, 2048, generator=torch.Generator().manual_seed(S))
        result, _ = backend.run(plan, input_data={"x": x.numpy(), "p_weight": w})
        out = result.outputs["rms_norm"]
        assert out.shape == (1, S, 2048)
        metrics.assert_fp32_reduction(out, cpu_ref.rmsnorm(x, torch.from_numpy(w), 1e-6), what=f"S={S}")
    assert len(plan.variants) == 3
    assert len({id(v.const_cache) for v in plan.variants.values()}) == 1 and "p_weight" in plan.const_cache
    # attention with the sequence axis symbolic on q, k and v
    code = ("q=torch.randn(1,4,48,128).bfloat16(); k=torch.randn(1,2,48,128).bfloat16(); "
            "v=torch.randn(1,2,48,128).bfloat16(); F.scaled_dot_product_attention(q,k,v,is_causal=True,enable_gqa=True)")
    tr = trace_inline_code(code, parse_dynamic_specs(["s@q:2", "s@k:2", "s@v:2"]))
    plan = backend.compile(tr.graph)
    for S in (48, 200):
        q, k, v = inputs.sdpa_inputs(1, 4, 2, S, seed=S)
        result, _ = backend.run(plan, input_data={"q": q, "k": k, "v": v})
        got = torch.from_numpy(result.outputs[plan.outputs[0]].view(np.int16)).view(torch.bfloat16)
        metrics.assert_bf16_tensor_path(got, cpu_ref.sdpa_causal_gqa(q, k, v), what=f"sdpa S={S}")
