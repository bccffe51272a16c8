"""The GEMM chain (``emk_gemm_bf16_chain``: several dependent projections as one persistent launch) against the same
GEMMs launched one by one. Both run the same tiles with the same arithmetic, so the outputs must be bit-equal; what the
chain adds is the hand-over of rows between phases inside one launch, which is what these cases exercise (many row
blocks, ragged last block, a single block, every phase count, repeated launches over one workspace)."""

from __future__ import annotations

import pytest
import torch

from oracle import cpu_ref, inputs, metrics

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops(libemk):
    from deplodock_b200 import ops as _ops

    assert torch.cuda.is_available()
    return _ops


def _layer_buffers(ops, M, S, seed=3):
    from deplodock_b200.model import rope_tables

    dev = "cuda"
    g = torch.Generator().manual_seed(seed)
    r = lambda *shape, scale=1.0: (scale * torch.randn(*shape, generator=g)).bfloat16().to(dev)  # noqa: E731
    cos, sin = rope_tables(S, 128, 1e6, dev)
    b = dict(attn=r(M, 2048), h0=r(M, 1024), wo=r(1024, 2048, scale=0.02), wgu=r(6144, 1024, scale=0.05),
             wd=r(1024, 3072, scale=0.02), wqkv=r(4096, 1024, scale=0.03),
             qn=(1 + 0.1 * torch.randn(128, generator=g)).bfloat16().to(dev),
             kn=(1 + 0.1 * torch.randn(128, generator=g)).bfloat16().to(dev), cm=ops.rope_chunk_major(cos, sin))
    b["h"] = b["h0"].clone()
    b["mlp"] = torch.empty(M, 3072, dtype=torch.bfloat16, device=dev)
    b["qkv"] = torch.empty(M, 4096, dtype=torch.bfloat16, device=dev)
    b["ss2"] = torch.empty(M, 8, device=dev)
    b["ss3"] = torch.empty(M, 8, device=dev)
    return b


def _phases(b, S, n, positions=None):
    ph = [dict(x=b["attn"], w=b["wo"], out=b["h"], epilogue="residual", residual=b["h"], row_sumsq_out=b["ss2"]),
          dict(x=b["h"], w=b["wgu"], out=b["mlp"], epilogue="swiglu", row_sumsq_in=b["ss2"], norm_dim=1024),
          dict(x=b["mlp"], w=b["wd"], out=b["h"], epilogue="residual", residual=b["h"], row_sumsq_out=b["ss3"]),
          dict(x=b["h"], w=b["wqkv"], out=b["qkv"], epilogue="qknorm_rope", row_sumsq_in=b["ss3"], norm_dim=1024,
               q_weight=b["qn"], k_weight=b["kn"], rope_cm=b["cm"], S=S, Hq=16, Hkv=8, positions=positions)]
    return ph[:n]


def _run_separately(ops, phases):
    for ph in phases:
        kw = dict(ph)
        ops.gemm_fused(kw.pop("x"), kw.pop("w"), kw.pop("out"), **kw)


def _reset(b):
    b["h"].copy_(b["h0"])
    for k in ("mlp", "qkv", "ss2", "ss3"):
        b[k].zero_()


@pytest.mark.parametrize("M,S,n", [(4096, 512, 4), (1024, 256, 4), (256, 256, 4), (96, 96, 4), (128, 128, 4), (2000, 500, 4),
                                   (8192, 512, 3), (768, 256, 2), (512, 512, 1)])
def test_chain_is_bit_equal_to_separate_launches(ops, M, S, n):
    b = _layer_buffers(ops, M, S)
    phases = _phases(b, S, n)
    _reset(b)
    _run_separately(ops, phases)
    torch.cuda.synchronize()
    want = {k: b[k].clone() for k in ("h", "mlp", "qkv", "ss2", "ss3")}
    ws = ops.gemm_chain_workspace(M, "cuda")
    for rep in range(3):   # the workspace is reused without clearing: every launch must leave it zero
        _reset(b)
        ops.gemm_chain(phases, ws)
        ops.device_status()
        for k, ref in want.items():
            if M > 128:
                assert torch.equal(b[k], ref), f"launch {rep}: {k} differs from the separate launches"
            elif k.startswith("ss"):
                # up to 128 rows a separate launch takes the single-CTA kernel, whose threads own other column ranges:
                # the partial sums land in other slots (only their sum is defined) and are added in another order
                torch.testing.assert_close(b[k].sum(1), ref.sum(1), rtol=1e-5, atol=0)
            else:
                assert (b[k] != ref).float().mean().item() < 0.005, k
                metrics.assert_bf16_tensor_path(b[k].cpu(), ref.cpu(), what=f"chain {k}")
        assert int(ws.abs().sum().item()) == 0, "counters not returned to zero"


def test_chain_matches_the_cpu_oracle(ops):
    """o_proj + residual -> RMSNorm-folded gate/up SwiGLU -> down + residual, against eager CPU arithmetic."""
    M, S = 512, 256
    b = _layer_buffers(ops, M, S, seed=11)
    ws = ops.gemm_chain_workspace(M, "cuda")
    _reset(b)
    ops.gemm_chain(_phases(b, S, 3), ws)
    ops.device_status()
    attn, h0 = b["attn"].cpu(), b["h0"].cpu()
    wo, wgu, wd = b["wo"].cpu(), b["wgu"].cpu(), b["wd"].cpu()
    h1 = (cpu_ref.linear(attn, wo).float() + h0.float()).bfloat16()
    # the chain folds the norm: rows scaled by rsqrt(mean(h1^2) + eps) after the product (norm weight = 1 here)
    rs = torch.rsqrt(h1.float().pow(2).mean(-1, keepdim=True) + 1e-6)
    gu = (torch.nn.functional.linear(h1.float(), wgu.float()) * rs).bfloat16().float()
    gate, up = gu[:, 0::2], gu[:, 1::2]
    mlp = (torch.nn.functional.silu(gate).bfloat16().float() * up).bfloat16()
    h2 = (cpu_ref.linear(mlp, wd).float() + h1.float()).bfloat16()
    metrics.assert_bf16_tensor_path(b["mlp"].cpu(), mlp, what="chain: gate/up SwiGLU")
    metrics.assert_bf16_tensor_path(b["h"].cpu(), h2, what="chain: hidden state after down + residual")


def test_chain_with_packed_positions(ops):
    """The QKV phase of a chain takes per-row rotary positions (packed sequences) like the single launch."""
    M, S = 700, 256
    b = _layer_buffers(ops, M, S)
    pos = (torch.arange(M, dtype=torch.int32) % 173).cuda()
    phases = _phases(b, S, 4, positions=pos)
    _reset(b)
    _run_separately(ops, phases)
    want = b["qkv"].clone()
    _reset(b)
    ops.gemm_chain(phases, ops.gemm_chain_workspace(M, "cuda"))
    ops.device_status()
    assert torch.equal(b["qkv"], want)


def test_chain_argument_checks(ops):
    M, S = 512, 256
    b = _layer_buffers(ops, M, S)
    ws = ops.gemm_chain_workspace(M, "cuda")
    ph = _phases(b, S, 2)
    broken = [dict(ph[0]), dict(ph[1])]
    broken[1]["x"] = b["h0"]                       # does not read the previous phase's output
    with pytest.raises(ValueError):
        ops.gemm_chain(broken, ws)
    with pytest.raises(ValueError):               # workspace too small
        ops.gemm_chain(ph, torch.zeros(2, dtype=torch.int32, device="cuda"))
    with pytest.raises(ValueError):
        ops.gemm_chain(_phases(b, S, 4) + _phases(b, S, 1), ws)   # five phases
    narrow = [dict(x=b["attn"], w=b["wo"][:128].contiguous(), out=torch.empty(M, 128, dtype=torch.bfloat16,
                                                                              device="cuda"))]
    with pytest.raises(ValueError):               # N <= 128 is not a CTA-pair tile
        ops.gemm_chain(narrow, ws)


def test_model_plans_with_and_without_the_chain_agree(libemk):
    from deplodock_b200.model import EmbedForward

    cfg = inputs.EmbedModelConfig(num_hidden_layers=3, vocab_size=1000)
    sd = inputs.embed_model_weights(cfg, seed=5)
    ids = inputs.token_ids(4, 160, cfg.vocab_size, seed=6)
    a = EmbedForward(cfg, sd, batch=4, seq=160, chain=True)
    c = EmbedForward(cfg, sd, batch=4, seq=160, chain=False)
    assert a.chain and not c.chain and a.num_launches == 1 + 1 + 2 * 3 + 1 and c.num_launches == 1 + 5 * 3 + 1
    ya = a(ids.cuda()).cpu().clone()
    ya2 = a(ids.cuda()).cpu().clone()          # graph replay over the same counter workspace
    yc = c(ids.cuda()).cpu().clone()
    assert torch.equal(ya, yc) and torch.equal(ya, ya2)


def test_packed_plan_with_and_without_the_chain_agree(libemk):
    """The variable-length plan (per-row rotary positions, cu_seqlens-driven attention) with chained projections."""
    from deplodock_b200.model import EmbedWeights, PackedForward

    cfg = inputs.EmbedModelConfig(num_hidden_layers=2, vocab_size=1000)
    w = EmbedWeights(cfg, inputs.embed_model_weights(cfg, seed=8))
    lens = [130, 64, 257, 5, 200]
    total = sum(lens)
    g = torch.Generator().manual_seed(9)
    ids = torch.randint(0, cfg.vocab_size, (total,), generator=g).cuda()
    pos = torch.cat([torch.arange(n, dtype=torch.int32) for n in lens]).cuda()
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32).cuda()
    outs = {}
    for chain in (False, True):
        plan = PackedForward(w, tokens=768, max_seqs=8, max_seq_len=384, chain=chain)
        assert plan.chain is chain
        plan.set_batch(ids, pos, cu)
        plan.replay()
        plan.replay()
        torch.cuda.synchronize()
        outs[chain] = (plan.hs[:total].clone(), plan.out[: len(lens)].clone())
    assert torch.equal(outs[False][0], outs[True][0])
    assert torch.equal(outs[False][1], outs[True][1])


def test_launch_overlap_setting_round_trip(ops):
    """``emk_set_launch_overlap`` returns the previous setting; a chained plan leaves the handle as it found it."""
    import os

    from deplodock_b200.model import EmbedForward

    h = ops.handle()
    default = os.environ.get("EMK_OVERLAP_LAUNCH", "1") != "0"
    assert h.set_launch_overlap(False) is default
    assert h.set_launch_overlap(True) is False
    assert h.set_launch_overlap(default) is True
    cfg = inputs.EmbedModelConfig(num_hidden_layers=1, vocab_size=500)
    plan = EmbedForward(cfg, inputs.embed_model_weights(cfg, seed=2), batch=2, seq=64, chain=True)
    plan(inputs.token_ids(2, 64, cfg.vocab_size, seed=3).cuda())
    assert h.set_launch_overlap(default) is default   # the plan restored it after capturing
