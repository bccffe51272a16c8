"""The PyTorch-eager modules the reference traces, run on the CPU (test infrastructure; also the timed CPU baseline).

The reference's accuracy check runs the traced ``nn.Module`` eagerly and compares flat outputs
(``emmy/commands/run.py:1387-1397`` and ``:1423-1500``; it does so on CUDA, here the CPU is used as the benchmark
configuration asks). Each function below is the module of one benchmark configuration.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from oracle.inputs import EmbedModelConfig


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """``nn.RMSNorm(cols, eps)`` forward — the README example of the reference (``README.md:22``), traced to RmsNormOp
    (``emmy/compiler/trace/torch.py:758-771``)."""
    m = torch.nn.RMSNorm(x.shape[-1], eps=eps, dtype=x.dtype)
    with torch.no_grad():
        m.weight.copy_(w)
        return m(x)


def rmsnorm_hf(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """The HF Qwen3 RMSNorm module: statistics in fp32, normalised value cast back to the input dtype before the
    weight multiply (traced as pow/mean/add/rsqrt/multiply/multiply)."""
    xf = x.to(torch.float32)
    var = xf.pow(2).mean(-1, keepdim=True)
    return w * (xf * torch.rsqrt(var + eps)).to(x.dtype)


def softmax(x: torch.Tensor) -> torch.Tensor:
    """``torch.nn.Softmax(dim=-1)`` forward (SoftmaxOp, ``emmy/compiler/trace/torch.py:791-801``)."""
    with torch.no_grad():
        return torch.nn.Softmax(dim=-1)(x)


def linear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """``nn.Linear(K, N)`` forward in the operand dtype (LinearOp, ``emmy/compiler/trace/torch.py:526-535``); bf16 on
    the CPU accumulates in fp32 and rounds once."""
    with torch.no_grad():
        return F.linear(x, w, bias)


def linear_w8(x: torch.Tensor, wq: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """Oracle of the e4m3-weight linear: ``F.linear(x, (Wq.float() * s[:, None]).bfloat16())``. Not in the reference
    (parity unpinned); the kernel applies the scale after the sum instead of before the bf16 rounding of the weights."""
    with torch.no_grad():
        return F.linear(x, (wq.float() * scale[:, None]).to(x.dtype))


def sdpa_causal_gqa(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """``F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)`` (SdpaOp; the tracer reads
    ``is_causal`` from the first bool argument, ``emmy/compiler/trace/torch.py:559-583``)."""
    with torch.no_grad():
        return F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)


def sdpa_causal_gqa_fp32(q, k, v) -> torch.Tensor:
    """Same attention evaluated in fp32 from the bf16 inputs: separates the kernel's rounding from the oracle's."""
    with torch.no_grad():
        return F.scaled_dot_product_attention(q.float(), k.float(), v.float(), is_causal=True, enable_gqa=True)


def swiglu(x, w_gate, w_up) -> torch.Tensor:
    with torch.no_grad():
        return F.silu(F.linear(x, w_gate)) * F.linear(x, w_up)


# ---------------------------------------------------------------------------------------------------------------
# Qwen3-Embedding-shaped trunk
# ---------------------------------------------------------------------------------------------------------------
def build_hf_model(cfg: EmbedModelConfig, sd: dict[str, torch.Tensor], dtype=torch.bfloat16):
    """``transformers.Qwen3Model`` from a hand-written ``Qwen3Config`` (no checkpoint, no network) with ``sd`` loaded —
    the module ``emmy/compiler/trace/huggingface.py:17-186`` wraps and traces."""
    from transformers import Qwen3Config, Qwen3Model

    hf_cfg = Qwen3Config(
        vocab_size=cfg.vocab_size,
        hidden_size=cfg.hidden_size,
        intermediate_size=cfg.intermediate_size,
        num_hidden_layers=cfg.num_hidden_layers,
        num_attention_heads=cfg.num_attention_heads,
        num_key_value_heads=cfg.num_key_value_heads,
        head_dim=cfg.head_dim,
        rms_norm_eps=cfg.rms_norm_eps,
        rope_theta=cfg.rope_theta,
        max_position_embeddings=32768,
        tie_word_embeddings=True,
        attention_bias=False,
        attention_dropout=0.0,
        use_sliding_window=False,
        initializer_range=cfg.initializer_range,
    )
    hf_cfg._attn_implementation = "sdpa"
    model = Qwen3Model(hf_cfg).to(dtype)
    missing, unexpected = model.load_state_dict(sd, strict=False)
    if unexpected or any("rotary" not in m for m in missing):
        raise RuntimeError(f"state dict mismatch: missing={missing} unexpected={unexpected}")
    return model.eval()


def embed_forward_hf(ids: torch.Tensor, cfg: EmbedModelConfig, sd: dict[str, torch.Tensor]) -> torch.Tensor:
    """Eager HF trunk -> last-token pooling -> L2 normalise (the pooler the reference leaves to vLLM,
    ``emmy/serving/vllm_model.py:50-58``). Returns fp32 ``[B, hidden]``."""
    model = build_hf_model(cfg, sd)
    with torch.no_grad():
        hs = model(input_ids=ids).last_hidden_state
    return F.normalize(hs[:, -1].float(), p=2, dim=-1)


def embed_forward(ids: torch.Tensor, cfg: EmbedModelConfig, sd: dict[str, torch.Tensor]) -> torch.Tensor:
    """Last-token pooling + L2 normalisation of :func:`trunk_hidden_states`; fp32 ``[B, hidden]``."""
    return F.normalize(trunk_hidden_states(ids, cfg, sd)[:, -1].float(), p=2, dim=-1)


def trunk_hidden_states(ids: torch.Tensor, cfg: EmbedModelConfig, sd: dict[str, torch.Tensor]) -> torch.Tensor:
    """The trunk written out with torch functional ops in the module's own dtype and rounding order — the
    dataflow of the traced graph (GatherOp, RMSNorm chains, 7 LinearOps, RoPE chain, SdpaOp, SwiGLU per layer) — up to
    and including the final norm: ``[B, S, hidden]`` in the weights' dtype, i.e. what the reference's runner returns
    per sequence (``emmy/serving/runner.py:204-236``). Checked against :func:`embed_forward_hf` in the tests."""
    B, S = ids.shape
    D, nq, nkv = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads
    dt = sd["embed_tokens.weight"].dtype
    from oracle.inputs import rope_tables

    cos, sin = rope_tables(S, D, cfg.rope_theta)
    cos, sin = cos.to(dt)[None, None], sin.to(dt)[None, None]

    def rot(x):
        return torch.cat([-x[..., D // 2:], x[..., : D // 2]], dim=-1)

    with torch.no_grad():
        h = F.embedding(ids, sd["embed_tokens.weight"])
        for i in range(cfg.num_hidden_layers):
            p = f"layers.{i}."
            x = rmsnorm_hf(h, sd[p + "input_layernorm.weight"], cfg.rms_norm_eps)
            q = F.linear(x, sd[p + "self_attn.q_proj.weight"]).view(B, S, nq, D)
            k = F.linear(x, sd[p + "self_attn.k_proj.weight"]).view(B, S, nkv, D)
            v = F.linear(x, sd[p + "self_attn.v_proj.weight"]).view(B, S, nkv, D).transpose(1, 2)
            q = rmsnorm_hf(q, sd[p + "self_attn.q_norm.weight"], cfg.rms_norm_eps).transpose(1, 2)
            k = rmsnorm_hf(k, sd[p + "self_attn.k_norm.weight"], cfg.rms_norm_eps).transpose(1, 2)
            q = (q * cos) + (rot(q) * sin)
            k = (k * cos) + (rot(k) * sin)
            a = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
            a = a.transpose(1, 2).reshape(B, S, nq * D)
            h = h + F.linear(a, sd[p + "self_attn.o_proj.weight"])
            x = rmsnorm_hf(h, sd[p + "post_attention_layernorm.weight"], cfg.rms_norm_eps)
            m = F.silu(F.linear(x, sd[p + "mlp.gate_proj.weight"])) * F.linear(x, sd[p + "mlp.up_proj.weight"])
            h = h + F.linear(m, sd[p + "mlp.down_proj.weight"])
        return rmsnorm_hf(h, sd["norm.weight"], cfg.rms_norm_eps)
