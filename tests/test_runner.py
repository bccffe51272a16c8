"""The serving-side runner: span splitting (CPU) and per-sequence hidden states against the eager CPU trunk (GPU)."""

from __future__ import annotations

import pytest
import torch

from deplodock_b200.runner import split_spans
from oracle import cpu_ref, inputs


# ------------------------------------------------------------------------------------------------------------
# packed-batch span splitting (contract of emmy/serving/packed.py:6-34)
# ------------------------------------------------------------------------------------------------------------
def test_split_spans_at_position_zero():
    assert split_spans([0, 1, 2, 0, 1, 0], 16) == [(0, 3), (3, 5), (5, 6)]
    assert split_spans([], 16) == []
    assert split_spans([0], 16) == [(0, 1)]


def test_split_spans_garbage_first_position_and_chopping():
    # dummy-run batches: positions[0] != 0 still starts a span; over-long spans are cut into max_seq_len pieces
    assert split_spans([5, 6, 7, 8, 9], 2) == [(0, 2), (2, 4), (4, 5)]
    assert split_spans([3, 4, 0, 1, 2, 3, 4], 3) == [(0, 2), (2, 5), (5, 7)]


def test_split_spans_covers_every_token_once():
    import random

    rng = random.Random(0)
    for _ in range(50):
        lens = [rng.randint(1, 9) for _ in range(rng.randint(1, 8))]
        pos = [p for n in lens for p in range(n)]
        spans = split_spans(pos, 4)
        assert spans[0][0] == 0 and spans[-1][1] == len(pos)
        assert all(a < b and b - a <= 4 for a, b in spans)
        assert all(spans[i][1] == spans[i + 1][0] for i in range(len(spans) - 1))


def test_create_rejects_other_dtypes():
    from deplodock_b200.runner import EmbedForwardRunner

    with pytest.raises(ValueError, match="bf16"):
        EmbedForwardRunner.create({}, 128, dtype_str="float16", cfg=inputs.EmbedModelConfig())


# ------------------------------------------------------------------------------------------------------------
# GPU
# ------------------------------------------------------------------------------------------------------------
def _cos(a, b):
    return torch.nn.functional.cosine_similarity(a.double(), b.double(), dim=-1)


@pytest.fixture(scope="module")
def small_runner(libemk):
    from deplodock_b200.runner import EmbedForwardRunner

    cfg = inputs.EmbedModelConfig().small(layers=2, vocab=500)
    sd = inputs.perturb_norm_weights(inputs.embed_model_weights(cfg))
    return cfg, sd, EmbedForwardRunner.create(sd, 384, batch=4, cfg=cfg)


def _assert_hidden(got: torch.Tensor, ref: torch.Tensor, what: str):
    got, ref = got.float().cpu(), ref.float()
    assert got.shape == ref.shape, what
    assert torch.isfinite(got).all(), what
    # bf16 trunk output of O(1) magnitude after the final norm: one bf16 ulp at 4 is 2^-5
    assert _cos(got, ref).min().item() >= 0.998, what
    assert (got - ref).abs().max().item() <= 2.0 ** -4 * max(1.0, ref.abs().max().item()), what


@pytest.mark.gpu
@pytest.mark.parametrize("S", [1, 40, 128, 200, 384])
def test_single_sequence_hidden_states(small_runner, S):
    cfg, sd, runner = small_runner
    ids = inputs.token_ids(1, S, cfg.vocab_size, seed=S)
    got = runner.forward_hidden_states(ids[0].cuda())
    assert got.dtype == torch.bfloat16 and tuple(got.shape) == (S, cfg.hidden_size)
    _assert_hidden(got, cpu_ref.trunk_hidden_states(ids, cfg, sd)[0], f"S={S}")


@pytest.mark.gpu
def test_one_graph_per_sequence_length(small_runner):
    cfg, _, runner = small_runner
    a = inputs.token_ids(1, 77, cfg.vocab_size, seed=1)[0].cuda()
    b = inputs.token_ids(1, 77, cfg.vocab_size, seed=2)[0].cuda()
    before = runner.captures
    ra = runner.forward_hidden_states(a)
    assert runner.captures == before + 1
    rb = runner.forward_hidden_states(b)
    assert runner.captures == before + 1, "same S must reuse the captured graph"
    assert not torch.equal(ra, rb)
    assert torch.equal(runner.forward_hidden_states(a), ra), "replay over the shared buffers is deterministic"
    runner.forward_hidden_states(a[:50])
    assert runner.captures == before + 2


@pytest.mark.gpu
def test_batched_ragged_equals_per_sequence(small_runner):
    """Right padding is exact under the causal mask: every sequence of a padded group gets the result it gets alone."""
    cfg, sd, runner = small_runner
    lens = [40, 130, 7, 256, 384, 1, 90]
    seqs = [inputs.token_ids(1, n, cfg.vocab_size, seed=10 + i)[0].cuda() for i, n in enumerate(lens)]
    batched = runner.forward_hidden_states_batched(seqs)
    assert [tuple(t.shape) for t in batched] == [(n, cfg.hidden_size) for n in lens]
    for t, s, n in zip(batched, seqs, lens):
        alone = runner.forward_hidden_states(s)
        # same kernels, same per-row arithmetic; only the tile a row falls in differs
        assert _cos(t.float(), alone.float()).min().item() >= 0.9999
        _assert_hidden(t, cpu_ref.trunk_hidden_states(s.cpu()[None], cfg, sd)[0], f"len {n}")


@pytest.mark.gpu
def test_packed_forward_and_pooling(small_runner):
    cfg, sd, runner = small_runner
    lens = [33, 128, 5]
    seqs = [inputs.token_ids(1, n, cfg.vocab_size, seed=30 + i)[0] for i, n in enumerate(lens)]
    packed = torch.cat(seqs + [torch.zeros(6, dtype=torch.int64)]).cuda()     # vLLM pads num_tokens
    positions = torch.cat([torch.arange(n) for n in lens] + [torch.arange(6)]).cuda()
    out = runner.forward_packed(packed, positions)
    assert tuple(out.shape) == (sum(lens) + 6, cfg.hidden_size)
    off = 0
    for s, n in zip(seqs, lens):
        _assert_hidden(out[off:off + n], cpu_ref.trunk_hidden_states(s[None], cfg, sd)[0], f"span at {off}")
        off += n
    emb = runner.embed_packed(torch.cat(seqs).cuda(), torch.cat([torch.arange(n) for n in lens]).cuda()).cpu()
    assert tuple(emb.shape) == (3, cfg.hidden_size)
    for i, s in enumerate(seqs):
        ref = cpu_ref.embed_forward(s[None], cfg, sd)[0]
        assert _cos(emb[i], ref).item() >= 0.999 and (emb[i] - ref).abs().max().item() <= 2e-2


@pytest.mark.gpu
def test_packed_mixed_lengths_equal_per_sequence_runs(small_runner):
    """The variable-length forward (one launch of every kernel over the packed stream, no padding) against each
    sequence run alone through its own fixed-length plan: rows are independent in every kernel and the attention
    kernel visits the same blocks of keys, so the hidden states agree to the bit for sequences on the same GEMM
    kernel (more than 128 rows) and to rounding noise otherwise; and against the padded route."""
    cfg, sd, runner = small_runner
    lens = [200, 384, 130, 256, 7, 1, 129]
    seqs = [inputs.token_ids(1, n, cfg.vocab_size, seed=50 + i)[0] for i, n in enumerate(lens)]
    packed = torch.cat(seqs).cuda()
    positions = torch.cat([torch.arange(n) for n in lens]).cuda()
    before = runner.captures
    out = runner.forward_packed(packed, positions)
    assert runner.captures == before + 1            # one plan (one graph) for the whole stream
    assert tuple(out.shape) == (sum(lens), cfg.hidden_size)
    padded = runner.forward_packed_padded(packed, positions)
    off = 0
    for s, n in zip(seqs, lens):
        alone = runner.forward_hidden_states(s.cuda())
        if n > 128:
            assert torch.equal(out[off:off + n], alone), f"sequence of {n} tokens at row {off}"
        assert _cos(out[off:off + n].float(), alone.float()).min().item() >= 0.9999
        assert _cos(out[off:off + n].float(), padded[off:off + n].float()).min().item() >= 0.9999
        _assert_hidden(out[off:off + n], cpu_ref.trunk_hidden_states(s[None], cfg, sd)[0], f"len {n}")
        off += n
    # a second stream with other lengths in the same token budget replays the same graph
    lens2 = [384, 384, 300, 39]
    seqs2 = [inputs.token_ids(1, n, cfg.vocab_size, seed=70 + i)[0] for i, n in enumerate(lens2)]
    assert sum(lens2) == sum(lens)
    c0 = runner.captures
    out2 = runner.forward_packed(torch.cat(seqs2).cuda(), torch.cat([torch.arange(n) for n in lens2]).cuda())
    assert runner.captures == c0
    off = 0
    for s, n in zip(seqs2, lens2):
        _assert_hidden(out2[off:off + n], cpu_ref.trunk_hidden_states(s[None], cfg, sd)[0], f"second stream, len {n}")
        off += n


@pytest.mark.gpu
def test_limits(small_runner):
    cfg, _, runner = small_runner
    with pytest.raises(ValueError, match="exceeds max_seq_len"):
        runner.forward_hidden_states(torch.zeros(385, dtype=torch.int64, device="cuda"))
    assert runner.forward_hidden_states(torch.zeros(0, dtype=torch.int64, device="cuda")).shape == (0, cfg.hidden_size)
    # out-of-vocabulary ids of a dummy run are clamped, not read out of bounds
    out = runner.forward_packed(torch.full((9,), 10 ** 9, dtype=torch.int64, device="cuda"), list(range(9)))
    assert torch.isfinite(out.float()).all()


# ------------------------------------------------------------------------------------------------------------
# The vLLM model class (built against a stand-in for vLLM's config objects; vLLM itself is not imported)
# ------------------------------------------------------------------------------------------------------------
def _fake_vllm_config(cfg, dtype=torch.bfloat16, max_model_len=384, max_num_seqs=4, max_tokens=1024):
    from types import SimpleNamespace

    hf = SimpleNamespace(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size,
                         num_hidden_layers=cfg.num_hidden_layers, num_attention_heads=cfg.num_attention_heads,
                         num_key_value_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim,
                         rms_norm_eps=cfg.rms_norm_eps, rope_theta=cfg.rope_theta)
    mc = SimpleNamespace(dtype=dtype, max_model_len=max_model_len, hf_config=hf, pooler_config=None,
                         get_vocab_size=lambda: cfg.vocab_size, model="unused")
    return SimpleNamespace(model_config=mc, scheduler_config=SimpleNamespace(max_num_seqs=max_num_seqs,
                                                                             max_num_batched_tokens=max_tokens))


def test_vllm_model_class_surface(monkeypatch):
    """Class attributes and constructor of the reference's ``EmmyEmbedModel`` (``emmy/serving/vllm_model.py:48-69``)."""
    from deplodock_b200 import serving

    monkeypatch.setattr(serving.B200EmbedModel, "_make_pooler", staticmethod(lambda mc: None))
    cfg = inputs.EmbedModelConfig().small(layers=2, vocab=500)
    m = serving.B200EmbedModel(vllm_config=_fake_vllm_config(cfg), prefix="")
    assert m.is_pooling_model and m.default_seq_pooling_type == "LAST" and m.attn_type == "encoder_only"
    assert m.cfg.num_hidden_layers == 2 and m.cfg.head_dim == 128 and m.vocab_size == 500 and m.runner is None
    assert list(m.parameters()) == []      # weights live with the kernels, not in nn.Parameters
    assert tuple(m.embed_input_ids(torch.zeros(7, dtype=torch.int64)).shape) == (7, 0)
    with pytest.raises(RuntimeError, match="load_weights"):
        m.forward(torch.zeros(4, dtype=torch.int64), torch.arange(4))
    with pytest.raises(KeyError, match="lacks"):
        m.load_weights(iter([("model.norm.weight", torch.ones(1024))]))


@pytest.mark.gpu
def test_vllm_model_class_forward(libemk, monkeypatch):
    """``load_weights`` from a checkpoint-style stream (``model.`` prefixes, an LM head to skip), then a packed step
    with vLLM's padding: hidden states per request against the eager CPU trunk, zero rows past the last request."""
    from deplodock_b200 import serving

    monkeypatch.setattr(serving.B200EmbedModel, "_make_pooler", staticmethod(lambda mc: None))
    cfg = inputs.EmbedModelConfig().small(layers=2, vocab=500)
    sd = inputs.perturb_norm_weights(inputs.embed_model_weights(cfg))
    m = serving.B200EmbedModel(vllm_config=_fake_vllm_config(cfg, dtype=torch.float16))
    stream = [("model." + k, v) for k, v in sd.items()] + [("lm_head.weight", torch.zeros(4, 4))]
    taken = m.load_weights(iter(stream))
    assert "lm_head.weight" not in taken and len(taken) == len(sd)
    lens = [150, 1, 260]
    seqs = [inputs.token_ids(1, n, cfg.vocab_size, seed=90 + i)[0] for i, n in enumerate(lens)]
    ids = torch.cat(seqs + [torch.zeros(5, dtype=torch.int64)]).cuda()
    pos = torch.cat([torch.arange(n) for n in lens] + [torch.arange(5)]).cuda()
    out = m(ids, pos)
    assert out.dtype == torch.float16 and tuple(out.shape) == (sum(lens) + 5, cfg.hidden_size)
    off = 0
    for s, n in zip(seqs, lens):
        _assert_hidden(out[off:off + n], cpu_ref.trunk_hidden_states(s[None], cfg, sd)[0], f"request of {n} tokens")
        off += n
