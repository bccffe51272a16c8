"""The traced decoder trunk through the backend interface: the reference tracer's record of a two-layer Qwen3-shaped
trunk (``tests/golden/graphs/qwen3_trunk_2layer_bf16.json``) and this package's own trace of the HF module are both
recognised and compiled to the fused five-launches-per-layer plan; anything else is refused. On the GPU the compiled
record runs through ``B200Backend.run`` and is held against the eager CPU trunk and the stored output of the
reference's wrapper module."""

from __future__ import annotations

import copy
import json

import numpy as np
import pytest
import torch

from conftest import GOLDEN
from oracle import cpu_ref, inputs

RECORD = GOLDEN / "graphs" / "qwen3_trunk_2layer_bf16.json"
SEMANTIC_OPS = ("CatOp", "ElementwiseOp", "GatherOp", "InputOp", "LinearOp", "MeanOp", "ReshapeOp", "SdpaOp", "SliceOp",
                "TransposeOp", "UnsqueezeOp")


def _record() -> dict:
    return json.loads(RECORD.read_text())


def test_reference_record_compiles_to_the_fused_plan():
    from deplodock_b200.backend import B200Backend
    from deplodock_b200.trunk import recognise_trunk
    from deplodock_b200.graph import Graph

    plan = B200Backend().compile(_record())
    assert plan.trunk is not None and plan.trunk.num_hidden_layers == 2
    names = [s.kernel_name for s in plan.steps]
    assert len(names) == 1 + 5 * 2 + 1            # gather, five launches per layer, final norm
    assert names[0] == "k_embed_gather_sumsq" and names[-1] == "k_rms_norm_final"
    assert [n.rsplit("_", 1)[0] for n in names[1:6]] == [
        "k_rmsnorm_linear_qkv_qknorm_rope", "k_scaled_dot_product_attention", "k_linear_o_proj_residual_sumsq",
        "k_rmsnorm_linear_gate_up_swiglu", "k_linear_down_residual_sumsq"]
    m = recognise_trunk(Graph.from_dict(_record()))
    assert (m.batch, m.seq, m.hidden_size, m.intermediate_size) == (1, 48, 1024, 3072)
    assert (m.num_attention_heads, m.num_key_value_heads, m.head_dim, m.vocab_size) == (16, 8, 128, 64)
    assert m.rms_norm_eps == pytest.approx(1e-6) and m.mask == "b_causal_mask"
    assert m.layers[1].wdown == "p_model_layers_1_mlp_down_proj_weight"
    assert m.layers[0].ln1 == "p_model_layers_0_input_layernorm_weight"
    # every compute node is claimed; the only unclaimed nodes are buffers no arithmetic reads
    g = Graph.from_dict(_record())
    assert {n.id for n in g.compute_nodes()} <= m.claimed
    assert plan.describe().count("\n") == len(names) - 1 and plan.outputs == g.outputs


@pytest.mark.parametrize("mutation", ["silu_to_add", "eps_differs", "f32_output", "extra_node", "mask_not_causal",
                                      "rope_slice_start"])
def test_near_misses_are_refused(mutation):
    from deplodock_b200.backend import B200Backend, LoweringError

    rec = copy.deepcopy(_record())
    nodes = rec["nodes"]
    if mutation == "silu_to_add":
        nid = next(k for k, n in nodes.items() if n["op"] == "ElementwiseOp" and n["op_fields"].get("op") == "silu")
        nodes[nid]["op_fields"]["op"] = "rsqrt"
    elif mutation == "eps_differs":
        nid = next(k for k, n in nodes.items() if n["op"] == "ConstantOp" and n["op_fields"].get("value") == 1e-06)
        nodes[nid]["op_fields"]["value"] = 1e-5
    elif mutation == "f32_output":
        nodes[rec["outputs"][0]]["output"]["dtype"] = "f32"
    elif mutation == "extra_node":
        out = rec["outputs"][0]
        nodes["extra"] = {"op": "SoftmaxOp", "op_fields": {"axis": -1}, "inputs": [out],
                          "output": dict(nodes[out]["output"], name="extra")}
        rec["outputs"] = ["extra"]
    elif mutation == "mask_not_causal":
        nodes["b_causal_mask"]["op_fields"]["source_path"] = "padding_mask"
        nodes["b_padding_mask"] = nodes.pop("b_causal_mask")
        for n in nodes.values():
            n["inputs"] = ["b_padding_mask" if i == "b_causal_mask" else i for i in n["inputs"]]
    elif mutation == "rope_slice_start":
        nid = next(k for k, n in nodes.items() if n["op"] == "SliceOp" and n["op_fields"].get("start") == 64)
        nodes[nid]["op_fields"]["start"] = 32
    with pytest.raises(LoweringError):
        B200Backend().compile(rec)


def test_own_tracer_yields_the_same_trunk():
    """``deplodock_b200.trace`` on the HF module behind its own wrapper: same semantic op counts as the reference
    tracer's one-layer record (``qwen3_layer_f32.ophist.json``) and the same recognised roles."""
    pytest.importorskip("transformers")
    from deplodock_b200.backend import B200Backend
    from deplodock_b200.trace import build_full_model_wrapper, trace_module

    cfg = inputs.EmbedModelConfig(vocab_size=64, num_hidden_layers=1)
    sd = inputs.embed_model_weights(cfg, seed=0)
    wrapper = build_full_model_wrapper(cpu_ref.build_hf_model(cfg, sd), 24, torch.bfloat16)
    ids = inputs.token_ids(1, 24, cfg.vocab_size, seed=3)
    graph, sources = trace_module(wrapper, (ids,))
    hist = graph.op_histogram()
    want = json.loads((GOLDEN / "graphs" / "qwen3_layer_f32.ophist.json").read_text())
    assert {k: hist.get(k, 0) for k in SEMANTIC_OPS} == {k: want[k] for k in SEMANTIC_OPS}
    assert sources["b_causal_mask"] == "causal_mask" and sources["b_model_rotary_emb_cos"] == "model.rotary_emb.cos"
    plan = B200Backend().compile(graph)
    assert plan.trunk is not None and len(plan.steps) == 1 + 5 + 1
    assert plan.trunk.layers[0].wq == "p_model_layers_0_self_attn_q_proj_weight"
    # the wrapper's buffers are what the eager module computes with: causal mask 0 / -inf, positions 0..S-1
    assert torch.equal(wrapper.position_ids, torch.arange(24)[None])
    assert wrapper.causal_mask[0, 0, 3, 4].item() == float("-inf") and wrapper.causal_mask[0, 0, 4, 3].item() == 0


def _input_data_for_record(rec: dict, sd: dict, ids: torch.Tensor, seq: int) -> dict:
    """What the reference's ``_bind_inputs`` hands ``Backend.run``: one array per graph input and per weight / buffer
    constant, found by ``source_path``; bf16 as uint16 bit patterns."""
    cos, sin = inputs.rope_tables(seq, 128, 1e6)
    mask = torch.triu(torch.full((seq, seq), float("-inf")), diagonal=1)[None, None]
    buffers = {"causal_mask": mask.bfloat16(), "position_ids": torch.arange(seq)[None],
               "model.rotary_emb.cos": cos.bfloat16()[None], "model.rotary_emb.sin": sin.bfloat16()[None]}
    data = {"input_ids": ids.numpy()}
    for nid, n in rec["nodes"].items():
        path = n["op_fields"].get("source_path") if n["op"] == "ConstantOp" else None
        if not path:
            continue
        t = buffers[path] if path in buffers else sd[path.removeprefix("model.")]
        data[nid] = t.view(torch.int16).numpy().view(np.uint16) if t.dtype == torch.bfloat16 else t.numpy()
    return data


@pytest.mark.gpu
def test_traced_trunk_runs_through_the_backend(libemk):
    from deplodock_b200.backend import B200Backend

    rec = _record()
    fixture = np.load(GOLDEN / "qwen3_trunk_2layer_bf16.npz")
    ids = torch.from_numpy(fixture["ids"])
    cfg = inputs.EmbedModelConfig(vocab_size=64, num_hidden_layers=2)
    sd = inputs.perturb_norm_weights(inputs.embed_model_weights(cfg, seed=0), seed=1)
    be = B200Backend()
    plan = be.compile(rec)
    data = _input_data_for_record(rec, sd, ids, 48)
    result, _ = be.run(plan, input_data=data)
    out = result.outputs[plan.outputs[0]]
    assert out.dtype == np.uint16 and out.shape == (1, 48, 1024)
    got = torch.from_numpy(out.view(np.int16)).view(torch.bfloat16).float()
    ref = cpu_ref.trunk_hidden_states(ids, cfg, sd).float()
    wrapper_out = torch.from_numpy(fixture["hidden"])
    for name, want in (("eager CPU trunk", ref), ("the reference wrapper's eager output", wrapper_out)):
        cos = torch.nn.functional.cosine_similarity(got, want, dim=-1).min().item()
        err = (got - want).abs().max().item()
        # un-normalised hidden states reach |x| ~ 30: the absolute bound scales with the largest magnitude, as in
        # the serving-runner tests (eight bf16 ulps of it)
        bound = 2.0 ** -4 * max(1.0, want.abs().max().item())
        assert cos >= 0.999 and err <= bound, f"vs {name}: cos {cos:.6f}, max abs {err:.3e} (bound {bound:.3e})"
    # weights stay on the device between runs with the same host arrays; new ids give new hidden states
    cached = {k: v[1].data_ptr() for k, v in plan.const_cache.items()}
    ids2 = inputs.token_ids(1, 48, 64, seed=9)
    data2 = dict(data, input_ids=ids2.numpy())
    result2, _ = be.run(plan, input_data=data2)
    assert {k: v[1].data_ptr() for k, v in plan.const_cache.items()} == cached
    got2 = torch.from_numpy(result2.outputs[plan.outputs[0]].view(np.int16)).view(torch.bfloat16).float()
    ref2 = cpu_ref.trunk_hidden_states(ids2, cfg, sd).float()
    assert torch.nn.functional.cosine_similarity(got2, ref2, dim=-1).min().item() >= 0.999
    assert not torch.equal(got, got2)


@pytest.mark.gpu
def test_own_trace_of_the_hf_module_runs_on_the_gpu(libemk):
    """nn.Module in, hidden states out: trace the wrapped HF trunk with this package's tracer, bind its parameters
    and buffers, run through the backend, compare with the module run eagerly on the CPU."""
    pytest.importorskip("transformers")
    from deplodock_b200.backend import B200Backend
    from deplodock_b200.trace import bind_inputs, build_full_model_wrapper, trace_module

    cfg = inputs.EmbedModelConfig(vocab_size=200, num_hidden_layers=3)
    sd = inputs.perturb_norm_weights(inputs.embed_model_weights(cfg, seed=0), seed=1)
    S = 130
    wrapper = build_full_model_wrapper(cpu_ref.build_hf_model(cfg, sd), S, torch.bfloat16)
    ids = inputs.token_ids(1, S, cfg.vocab_size, seed=11)
    with torch.no_grad():
        want = wrapper(ids).float()
    graph, sources = trace_module(wrapper, (ids,))
    be = B200Backend()
    plan = be.compile(graph)
    result, _ = be.run(plan, input_data=bind_inputs(graph, wrapper, (ids,), {}, sources))
    got = torch.from_numpy(result.outputs[plan.outputs[0]].view(np.int16)).view(torch.bfloat16).float()
    cos = torch.nn.functional.cosine_similarity(got, want, dim=-1).min().item()
    assert cos >= 0.999, cos
    assert (got - want).abs().max().item() <= 2.0 ** -4 * max(1.0, want.abs().max().item())
