"""The oracle against outputs of the reference itself (NumpyBackend, stored by tests/golden/make_golden.py).

``np_ref`` restates the reference ops' numpy ``forward`` methods and must match to float32 round-off; ``cpu_ref`` is
the eager PyTorch module and must match within the reference's own per-op test tolerances
(tests/compiler/e2e/test_ops_vs_torch.py:303-449 of the reference)."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import load_golden
from oracle import cpu_ref, inputs, np_ref


def _close(a, b, rtol, atol):
    np.testing.assert_allclose(np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64), rtol=rtol, atol=atol)


@pytest.mark.parametrize("case", ["rmsnorm_f32", "rmsnorm_readme_shape"])
def test_rmsnorm(case):
    ins, outs = load_golden(case)
    ref = outs["rms_norm"]
    _close(np_ref.rms_norm(ins["x"], ins["p_weight"], 1e-6), ref, 1e-6, 1e-6)
    got = cpu_ref.rmsnorm(torch.from_numpy(ins["x"]), torch.from_numpy(ins["p_weight"]), 1e-6)
    _close(got.numpy(), ref, 1e-4, 1e-5)
    got = cpu_ref.rmsnorm_hf(torch.from_numpy(ins["x"]), torch.from_numpy(ins["p_weight"]), 1e-6)
    _close(got.numpy(), ref, 1e-4, 1e-5)


def test_softmax():
    ins, outs = load_golden("softmax_f32")
    _close(np_ref.softmax(ins["input"]), outs["softmax"], 1e-6, 1e-7)
    _close(cpu_ref.softmax(torch.from_numpy(ins["input"])).numpy(), outs["softmax"], 2e-4, 1e-5)


def test_softmax_minus_inf_rows_match_torch():
    x = inputs.softmax_inputs((2, 4, 64), mask_frac=0.3, seed=5)
    assert torch.isinf(x).any()
    _close(np_ref.softmax(x.numpy()), cpu_ref.softmax(x).numpy(), 1e-5, 1e-7)


def test_linear_and_matmul():
    ins, outs = load_golden("linear_f32")
    _close(np_ref.linear(ins["input"], ins["p_weight"]), outs["linear"], 1e-6, 1e-6)
    _close(cpu_ref.linear(torch.from_numpy(ins["input"]), torch.from_numpy(ins["p_weight"])).numpy(), outs["linear"],
           1e-4, 2e-6)
    ins, outs = load_golden("linear_bias_f32")
    _close(np_ref.linear(ins["input"], ins["p_weight"], ins["p_bias"]), outs["linear"], 1e-6, 1e-6)
    ins, outs = load_golden("matmul_f32")
    _close(np_ref.matmul(ins["x0"], ins["x1"]), outs["matmul"], 1e-6, 1e-6)


@pytest.mark.parametrize("case", ["sdpa_causal_gqa_f32", "sdpa_causal_gqa_d128_f32"])
def test_sdpa_causal_gqa(case):
    ins, outs = load_golden(case)
    ref = outs["scaled_dot_product_attention"]
    _close(np_ref.sdpa(ins["q"], ins["k"], ins["v"], is_causal=True), ref, 1e-5, 1e-6)
    got = cpu_ref.sdpa_causal_gqa(*(torch.from_numpy(ins[n]) for n in "qkv"))
    _close(got.numpy(), ref, 5e-3, 1e-4)  # the reference's GQA tolerance


def test_sdpa_full():
    ins, outs = load_golden("sdpa_full_f32")
    _close(np_ref.sdpa(ins["q"], ins["k"], ins["v"]), outs["scaled_dot_product_attention"], 1e-5, 1e-6)


def test_swiglu_chain():
    ins, outs = load_golden("swiglu_f32")
    got = np_ref.silu(np_ref.matmul(ins["x"], ins["wg"])) * np_ref.matmul(ins["x"], ins["wu"])
    _close(got, outs["mul"], 1e-5, 1e-5)


def test_qwen3_layer_trunk_matches_reference_wrapper():
    """One Qwen3-shaped layer run through the reference's HF wrapper module (eager fp32) vs the numpy restatement and
    the eager functional trunk, with the weights regenerated from the seed."""
    from conftest import GOLDEN

    data = np.load(GOLDEN / "qwen3_layer_f32.npz")
    ids, ref = data["ids"], data["hidden"]
    cfg = inputs.EmbedModelConfig(vocab_size=64, num_hidden_layers=1)
    sd = inputs.perturb_norm_weights(inputs.embed_model_weights(cfg, seed=0, dtype=torch.float32), seed=1)
    sd_np = {k: v.numpy() for k, v in sd.items()}
    got = np_ref.trunk_hidden(ids, sd_np, cfg)
    _close(got, ref, 1e-3, 1e-3)  # the reference's whole-trunk tolerance (tests/compiler/ir/test_dynamic_shapes.py:388)
    assert np.max(np.abs(got - ref)) < 2e-4
    # pooled + normalised embedding of the eager functional trunk vs the same from the reference output
    emb = cpu_ref.embed_forward(torch.from_numpy(ids), cfg, sd).numpy()
    last = ref[:, -1]
    want = last / np.linalg.norm(last, axis=-1, keepdims=True)
    assert np.max(np.abs(emb - want)) < 2e-4


def test_functional_trunk_equals_hf_module_bf16():
    cfg = inputs.EmbedModelConfig().small(layers=2, vocab=300)
    sd = inputs.perturb_norm_weights(inputs.embed_model_weights(cfg))
    ids = inputs.token_ids(2, 40, cfg.vocab_size, seed=2)
    a = cpu_ref.embed_forward_hf(ids, cfg, sd)
    b = cpu_ref.embed_forward(ids, cfg, sd)
    cos = torch.nn.functional.cosine_similarity(a, b).min().item()
    assert cos > 0.9995 and (a - b).abs().max().item() < 5e-3


def test_w8_oracle_roundtrip():
    x, wq, s = inputs.linear_w8_inputs(8, 64, 32, seed=1)
    deq = wq.float() * s[:, None]
    # e4m3 with absmax/448 scaling keeps every channel's max exactly representable
    assert torch.allclose(deq.abs().amax(1), s * 448.0, rtol=1e-6)
    y = cpu_ref.linear_w8(x, wq, s)
    assert y.dtype == torch.bfloat16 and y.shape == (8, 32)
