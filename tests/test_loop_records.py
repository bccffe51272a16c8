"""The reference's shipped Loop-IR kernel records (``kernels/*.json``, copied to ``tests/golden/loop_records`` by
``tests/golden/make_golden.py``): recognition of the loop nests on CPU, and on the GPU each record run through
``B200Backend`` against the output of the reference's own LoopOp -> C++ renderer on the same seeded inputs (strided
samples and checksums stored beside the records)."""

from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import pytest

from deplodock_b200 import loopir
from deplodock_b200.backend import B200Backend, LoweringError
from deplodock_b200.graph import Graph
from oracle.inputs import loop_record_inputs

RECORDS = Path(__file__).parent / "golden" / "loop_records"
NAMES = sorted(p.stem for p in RECORDS.glob("*.json"))
EXPECTED = {
    "k_add_3_reduce": ("linear_residual", "emk_loop_linear_f32"),
    "k_add_5_reduce": ("linear_residual", "emk_loop_linear_f32"),
    "k_linear_1_reduce_reduce": ("linear", "emk_loop_linear_f32"),
    "k_linear_2_reduce_reduce": ("linear", "emk_loop_linear_f32"),
    "k_linear_4_reduce": ("linear", "emk_loop_linear_f32"),
    "k_linear_reduce_reduce": ("linear", "emk_loop_linear_f32"),
    "k_mul_1_reduce": ("rmsnorm", "emk_rmsnorm"),
    "k_mul_7_reduce": ("rmsnorm", "emk_rmsnorm"),
    "k_mul_8_reduce": ("silu_gate_linear", "emk_loop_linear_f32"),
    "k_scaled_dot_product_attention_masked_reduce": ("rope_scores", "emk_loop_rope_scores_f32"),
    "k_scaled_dot_product_attention_reduce_reduce": ("softmax_pv", "emk_loop_softmax_pv_f32"),
}


def _loop_node(g: Graph) -> str:
    return next(n for n, v in g.nodes.items() if v.op == "LoopOp")


def test_all_shipped_records_are_present():
    assert NAMES == sorted(EXPECTED)


@pytest.mark.parametrize("name", NAMES)
def test_record_is_recognised_verified_and_lowered(name):
    g = Graph.from_json(RECORDS / f"{name}.json")
    m = loopir.verify(g, _loop_node(g), loopir.classify(g, _loop_node(g)), points=3)
    assert m.kind == EXPECTED[name][0]
    plan = B200Backend().compile(g)
    assert [s.entry for s in plan.steps] == [EXPECTED[name][1]]
    assert plan.steps[0].kernel_name.startswith("k_")


def test_o_proj_record_reads_the_head_major_attention_output():
    g = Graph.from_json(RECORDS / "k_add_3_reduce.json")
    p = loopir.classify(g, _loop_node(g)).params
    # [1, 32, 128, 1, 64] read as x[m, k] = in[k // 64, m, k % 64]
    assert (p["x_inner"], p["x_stride_outer"], p["x_stride_m"]) == (64, 128 * 64, 64)
    assert p["residual"] == "hidden_states" and (p["M"], p["N"], p["K"]) == (128, 2048, 2048)


def test_rope_tables_are_told_apart_by_the_numbers():
    g = Graph.from_json(RECORDS / "k_scaled_dot_product_attention_masked_reduce.json")
    m = loopir.verify(g, _loop_node(g), loopir.classify(g, _loop_node(g)), points=2)
    assert (m.params["cos"], m.params["sin"]) == ("position_embeddings_0", "position_embeddings_1")
    assert m.params["scale"] == 0.125 and m.params["mask_fill"] == -1e9 and m.params["Hkv"] == 4


def _edited(name: str, old: str, new: str) -> Graph:
    rec = json.loads((RECORDS / f"{name}.json").read_text())
    node = next(v for v in rec["nodes"].values() if v["op"] == "LoopOp")
    body = [s.replace(old, new) for s in node["op_fields"]["body"]]
    assert body != node["op_fields"]["body"]
    node["op_fields"]["body"] = body
    return Graph.from_dict(rec)


def test_a_nest_that_only_looks_like_a_family_is_refused():
    # same structure as the RMSNorm record, but the reduction is a sum of x * w instead of x * x
    g = _edited("k_mul_1_reduce", "Load(name='in3', input='hidden_states', index=(Literal(value=0, dtype='int'), "
                "Var(name='a0'), Var(name='a1')))",
                "Load(name='in3', input='p_input_layernorm_weight', index=(Var(name='a1'),))")
    with pytest.raises(LoweringError):
        B200Backend().compile(g)
    # the linear record with the epilogue residual subtracted instead of added
    g = _edited("k_add_5_reduce", "Assign(name='v1', op=ElementwiseImpl('add')", "Assign(name='v1', op=ElementwiseImpl('subtract')")
    with pytest.raises(LoweringError):
        B200Backend().compile(g)
    # an activation read with a stride no kernel implements (every other k)
    g = _edited("k_linear_4_reduce", "input='merged_merged_merged_lift_mul_7', index=(Literal(value=0, dtype='int'), "
                "Var(name='a0'), Var(name='a2'))",
                "input='merged_merged_merged_lift_mul_7', index=(Literal(value=0, dtype='int'), Var(name='a0'), "
                "BinaryExpr(op='/', left=Var(name='a2'), right=Literal(value=2, dtype='int')))")
    with pytest.raises(LoweringError):
        B200Backend().compile(g)


def test_interpreter_executes_a_body_literally():
    g = Graph.from_json(RECORDS / "k_mul_1_reduce.json")
    node = g.nodes[_loop_node(g)]
    stmts = loopir.parse_body(node.op_fields["body"])
    rng = np.random.default_rng(1)
    x = rng.standard_normal((1, 128, 2048)).astype(np.float32)
    w = rng.standard_normal(2048).astype(np.float32)
    inputs = {"hidden_states": x, "p_input_layernorm_weight": w, "mean_count": np.float32([2048.0]),
              "add_c1": np.float32([1e-5])}
    writes = loopir.interpret_point(stmts, inputs, {"a0": 5})
    assert len(writes) == 2048 and writes[7][0] == (0, 5, 7)
    want = w * (x[0, 5] / np.sqrt((x[0, 5].astype(np.float64) ** 2).mean() + 1e-5))
    np.testing.assert_allclose([v for _, v in writes], want, rtol=2e-5, atol=2e-6)


# ------------------------------------------------------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("name", NAMES)
def test_record_runs_and_matches_the_reference_renderer(libemk, name):
    rec = json.loads((RECORDS / f"{name}.json").read_text())
    gold = np.load(RECORDS / f"{name}.npz")
    data = loop_record_inputs(rec, seed=int(gold["seed"]))
    backend = B200Backend()
    plan = backend.compile(Graph.from_dict(rec))
    result, _ = backend.run(plan, input_data=data)
    out = result.outputs[plan.outputs[0]].astype(np.float64).ravel()
    sample = gold["sample"].astype(np.float64)
    got = out[:: int(gold["stride"])]
    scale = max(1.0, float(np.abs(sample).max()))
    # fp32 reductions of up to 5632 terms in a different association order than the serial reference loop
    assert np.abs(got - sample).max() <= 2e-5 * scale, (name, float(np.abs(got - sample).max()), scale)
    assert abs(out.sum() - float(gold["sum"])) <= 1e-6 * float(gold["abs_sum"]) + 1e-3
