"""Seeded synthetic inputs for the five benchmark configurations (test infrastructure).

No public dataset or benchmark suite is involved on this path: the reference's own benches use ``randn`` tensors and
uniform-random token ids (``emmy/commands/run.py:1027-1056`` fills ``InputOp`` with ``standard_normal`` and weights
with ``standard_normal * 0.02``). Everything is generated on the CPU with ``torch.manual_seed(seed)`` so the CPU oracle
and the GPU kernels see the same bits. Every builder takes scale-down arguments so the tests can run small cases.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch


def rmsnorm_inputs(rows_shape=(1, 32), cols=2048, dtype=torch.float32, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(*rows_shape, cols, generator=g)
    w = 1.0 + 0.02 * torch.randn(cols, generator=g)
    return x.to(dtype), w.to(dtype)


def softmax_inputs(shape=(1, 28, 2048, 2048), mask_frac=0.01, seed=0):
    """N(0, 3) entries with ``mask_frac`` of them set to -inf; column 0 of a row is re-opened if the whole row were
    masked, so no row is fully masked."""
    g = torch.Generator().manual_seed(seed)
    x = 3.0 * torch.randn(*shape, generator=g)
    mask = torch.rand(*shape, generator=g) < mask_frac
    full = mask.all(dim=-1)
    if full.any():
        mask[..., 0] &= ~full
    x[mask] = float("-inf")
    return x


def linear_inputs(M=4096, K=2048, N=6144, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g).bfloat16()
    w = (0.02 * torch.randn(N, K, generator=g)).bfloat16()
    return x, w


def quantize_e4m3_per_channel(w32: torch.Tensor):
    """absmax/448 per output channel, weights rounded to e4m3."""
    s = w32.abs().amax(dim=1).clamp_min(1e-12) / 448.0
    wq = (w32 / s[:, None]).to(torch.float8_e4m3fn)
    return wq, s.float().contiguous()


def linear_w8_inputs(M=4096, K=2048, N=6144, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g).bfloat16()
    w32 = 0.02 * torch.randn(N, K, generator=g)
    wq, s = quantize_e4m3_per_channel(w32)
    return x, wq, s


def sdpa_inputs(B=4, Hq=16, Hkv=8, S=2048, D=128, dtype=torch.bfloat16, seed=0):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, Hq, S, D, generator=g).to(dtype)
    k = torch.randn(B, Hkv, S, D, generator=g).to(dtype)
    v = torch.randn(B, Hkv, S, D, generator=g).to(dtype)
    return q, k, v


@dataclass(frozen=True)
class EmbedModelConfig:
    """Shape of the Qwen3-Embedding-0.6B trunk (values of the benchmark configuration)."""

    vocab_size: int = 151669
    hidden_size: int = 1024
    intermediate_size: int = 3072
    num_hidden_layers: int = 28
    num_attention_heads: int = 16
    num_key_value_heads: int = 8
    head_dim: int = 128
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    initializer_range: float = 0.02

    def small(self, layers=2, vocab=1000):
        return EmbedModelConfig(vocab_size=vocab, num_hidden_layers=layers)


def embed_model_weights(cfg: EmbedModelConfig, seed=0, dtype=torch.bfloat16) -> dict[str, torch.Tensor]:
    """Random-init weights named like the HF ``Qwen3Model`` state dict: N(0, initializer_range) for embeddings and
    projections, ones for norm weights (HF default initialisation)."""
    g = torch.Generator().manual_seed(seed)
    H, I, D = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim
    nq, nkv = cfg.num_attention_heads, cfg.num_key_value_heads
    std = cfg.initializer_range

    def rnd(*shape):
        return (std * torch.randn(*shape, generator=g)).to(dtype)

    sd = {"embed_tokens.weight": rnd(cfg.vocab_size, H)}
    for i in range(cfg.num_hidden_layers):
        p = f"layers.{i}."
        sd[p + "input_layernorm.weight"] = torch.ones(H, dtype=dtype)
        sd[p + "self_attn.q_proj.weight"] = rnd(nq * D, H)
        sd[p + "self_attn.k_proj.weight"] = rnd(nkv * D, H)
        sd[p + "self_attn.v_proj.weight"] = rnd(nkv * D, H)
        sd[p + "self_attn.o_proj.weight"] = rnd(H, nq * D)
        sd[p + "self_attn.q_norm.weight"] = torch.ones(D, dtype=dtype)
        sd[p + "self_attn.k_norm.weight"] = torch.ones(D, dtype=dtype)
        sd[p + "post_attention_layernorm.weight"] = torch.ones(H, dtype=dtype)
        sd[p + "mlp.gate_proj.weight"] = rnd(I, H)
        sd[p + "mlp.up_proj.weight"] = rnd(I, H)
        sd[p + "mlp.down_proj.weight"] = rnd(H, I)
    sd["norm.weight"] = torch.ones(H, dtype=dtype)
    return sd


def perturb_norm_weights(sd: dict[str, torch.Tensor], seed=1) -> dict[str, torch.Tensor]:
    """Norm weights of 1 hide indexing mistakes; tests use 1 + N(0, 0.1) instead."""
    g = torch.Generator().manual_seed(seed)
    out = dict(sd)
    for k, v in sd.items():
        if "norm" in k:
            out[k] = (1.0 + 0.1 * torch.randn(v.shape, generator=g)).to(v.dtype)
    return out


def token_ids(batch=64, seq=512, vocab=151669, seed=0) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (batch, seq), generator=g, dtype=torch.int64)


def rope_tables(seq: int, head_dim: int = 128, theta: float = 1e6):
    """cos/sin ``[seq, head_dim]`` fp32 as HF's rotary embedding builds them (``cat(freqs, freqs)``)."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.int64).float() / head_dim))
    pos = torch.arange(seq, dtype=torch.float32)
    freqs = torch.outer(pos, inv_freq)
    emb = torch.cat([freqs, freqs], dim=-1)
    return emb.cos(), emb.sin()


def sdpa_scale(head_dim: int) -> float:
    return 1.0 / math.sqrt(head_dim)


def loop_record_inputs(record: dict, seed: int = 0) -> dict[str, "np.ndarray"]:
    """Seeded fp32 inputs for a Loop-IR kernel record (``kernels/*.json`` of the reference): scalar constants take their
    recorded value, weight constants (``value`` None) are N(0, 0.02) (1 + N(0, 0.02) for 1-D norm weights), rotary
    tables are uniform in [-1, 1], every other input is N(0, 1). One generator, node order of the record."""
    import numpy as np

    rng = np.random.default_rng(seed)
    out = {}
    for nid, node in record["nodes"].items():
        if node["op"] not in ("InputOp", "ConstantOp"):
            continue
        shape = tuple(int(d) for d in node["output"]["shape"])
        value = node.get("op_fields", {}).get("value")
        if node["op"] == "ConstantOp" and value not in (None, "None"):
            out[nid] = np.full(shape, float(value), dtype=np.float32)
        elif node["op"] == "ConstantOp":
            w = rng.standard_normal(shape).astype(np.float32) * np.float32(0.02)
            out[nid] = (w + np.float32(1.0)) if len(shape) == 1 else w
        elif "position_embeddings" in nid:
            out[nid] = rng.uniform(-1.0, 1.0, shape).astype(np.float32)
        else:
            out[nid] = rng.standard_normal(shape).astype(np.float32)
    return out
