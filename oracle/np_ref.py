"""Plain-numpy restatement of the math of the reference's Torch-IR ops (test infrastructure).

Each function follows the ``forward`` of the op class it names in ``emmy/compiler/ir/frontend/ir.py`` and the
decomposition rule that lowers it; fp32 throughout (the reference's NumpyBackend evaluates graphs in the node dtype,
``emmy/compiler/backend/base.py:139-205``). Pinned against NumpyBackend outputs stored in ``tests/golden/*.npz``.
"""

from __future__ import annotations

import numpy as np


def linear(x, w, bias=None):
    """LinearOp.forward — ``x @ w.T (+ bias)`` (``ir/frontend/ir.py:202-217``; decomposition
    ``passes/frontend/decomposition/040_linear.py:16-43``)."""
    y = x @ np.swapaxes(w, -1, -2)
    return y if bias is None else y + bias


def matmul(a, b, bias=None):
    """MatmulOp.forward — ``a @ b (+ bias)`` with b row-major ``[K,N]`` (``ir/frontend/ir.py:221-237``)."""
    y = a @ b
    return y if bias is None else y + bias


def rms_norm(x, weight, eps=1e-6):
    """RmsNormOp.forward — ``(x / sqrt(mean(x*x, -1) + eps)) * weight`` (``ir/frontend/ir.py:296-312``; decomposition
    ``080_rms_norm.py:17-60`` computes the same value as ``x * rsqrt(sum(x*x) * (1/N) + eps) * w``)."""
    rms = np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)
    return (x / rms) * weight


def softmax(x, axis=-1):
    """SoftmaxOp.forward — ``exp(x - max) / sum(exp(x - max))`` (``ir/frontend/ir.py:343-358``)."""
    m = np.max(x, axis=axis, keepdims=True)
    with np.errstate(invalid="ignore"):
        e = np.exp(x - m)
    return e / np.sum(e, axis=axis, keepdims=True)


def sdpa(q, k, v, is_causal=False, mask=None):
    """SdpaOp.forward (``ir/frontend/ir.py:241-275``): K/V heads repeated ``Hq // Hkv`` times for GQA, scores scaled
    by ``1/sqrt(head_dim)``, causal entries lowered by 1e9 (``010_sdpa.py:101-131`` uses the same soft -inf; an additive
    mask input is added instead, ``:93-99``), softmax, ``attn @ v``."""
    while k.ndim < q.ndim:
        k = k[None]
    while v.ndim < q.ndim:
        v = v[None]
    if q.ndim >= 3 and k.shape[-3] != q.shape[-3]:
        group = q.shape[-3] // k.shape[-3]
        k = np.repeat(k, group, axis=-3)
        v = np.repeat(v, group, axis=-3)
    scores = q @ np.swapaxes(k, -2, -1) / np.sqrt(q.shape[-1])
    if is_causal:
        tri = np.triu(np.ones((scores.shape[-2], scores.shape[-1]), dtype=scores.dtype), k=1)
        scores = scores - tri * 1e9
    if mask is not None:
        scores = scores + mask
    return softmax(scores, -1) @ v


def silu(x):
    """``x * recip(1 + exp(-x))`` (``passes/frontend/decomposition/020_silu.py:11-36``)."""
    return x * (1.0 / (1.0 + np.exp(-x)))


def rotate_half(x):
    """``cat(-x[..., D/2:], x[..., :D/2])`` — the slice/negative/cat chain of the traced HF rotary embedding."""
    h = x.shape[-1] // 2
    return np.concatenate([-x[..., h:], x[..., :h]], axis=-1)


def rope(x, cos, sin):
    """``x * cos + rotate_half(x) * sin`` — the multiply/add chain following the cat."""
    return x * cos + rotate_half(x) * sin


def swiglu_mlp(x, w_gate, w_up, w_down):
    """``down(silu(gate(x)) * up(x))`` — the traced Qwen3 MLP: three LinearOps, silu, multiply."""
    return linear(silu(linear(x, w_gate)) * linear(x, w_up), w_down)


def trunk_hidden(ids, sd, cfg):
    """fp32 numpy forward of the Qwen3-shaped trunk as the traced graph computes it (GatherOp, RMSNorm chains,
    LinearOps, RoPE chain, SdpaOp with the additive causal mask, SwiGLU): the final-norm hidden states ``[B,S,H]``,
    the output of the graph ``build_full_model_wrapper`` traces (``emmy/compiler/trace/huggingface.py:17-186``).
    ``sd`` maps HF parameter names to float32 arrays. Small configurations only (pure numpy)."""
    B, S = ids.shape
    D, nq, nkv = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads
    inv_freq = 1.0 / (cfg.rope_theta ** (np.arange(0, D, 2, dtype=np.float32) / D))
    freqs = np.outer(np.arange(S, dtype=np.float32), inv_freq)
    emb = np.concatenate([freqs, freqs], -1)
    cos, sin = np.cos(emb)[None, None], np.sin(emb)[None, None]
    h = sd["embed_tokens.weight"][ids]
    for i in range(cfg.num_hidden_layers):
        p = f"layers.{i}."
        x = rms_norm(h, sd[p + "input_layernorm.weight"], cfg.rms_norm_eps)
        q = linear(x, sd[p + "self_attn.q_proj.weight"]).reshape(B, S, nq, D)
        k = linear(x, sd[p + "self_attn.k_proj.weight"]).reshape(B, S, nkv, D)
        v = linear(x, sd[p + "self_attn.v_proj.weight"]).reshape(B, S, nkv, D)
        q = rms_norm(q, sd[p + "self_attn.q_norm.weight"], cfg.rms_norm_eps).transpose(0, 2, 1, 3)
        k = rms_norm(k, sd[p + "self_attn.k_norm.weight"], cfg.rms_norm_eps).transpose(0, 2, 1, 3)
        v = v.transpose(0, 2, 1, 3)
        q, k = rope(q, cos, sin), rope(k, cos, sin)
        a = sdpa(q, k, v, is_causal=True).transpose(0, 2, 1, 3).reshape(B, S, nq * D)
        h = h + linear(a, sd[p + "self_attn.o_proj.weight"])
        x = rms_norm(h, sd[p + "post_attention_layernorm.weight"], cfg.rms_norm_eps)
        h = h + swiglu_mlp(x, sd[p + "mlp.gate_proj.weight"], sd[p + "mlp.up_proj.weight"],
                           sd[p + "mlp.down_proj.weight"])
    return rms_norm(h, sd["norm.weight"], cfg.rms_norm_eps)


def embed_forward(ids, sd, cfg):
    """Trunk, then last-token pooling and L2 normalise (the pooler the reference leaves to vLLM,
    ``emmy/serving/vllm_model.py:50-58``)."""
    last = trunk_hidden(ids, sd, cfg)[:, -1]
    return last / np.maximum(np.linalg.norm(last, axis=-1, keepdims=True), 1e-12)
