"""``B200EmbedModel`` — the out-of-tree vLLM pooling model class on the hand-written kernels.

Counterpart of the reference's ``EmmyEmbedModel`` (``emmy/serving/vllm_model.py:48-103``): the class vLLM instantiates
when a causal-trunk embedding model is served with ``--hf-overrides '{"architectures": ["B200EmbedModel"]}'``
(``--runner pooling --enforce-eager``). Same surface — ``is_pooling_model``, ``default_seq_pooling_type = "LAST"``,
``attn_type = "encoder_only"`` (whole-sequence prefills: every request reaches ``forward`` whole and
``positions == 0`` marks a sequence start), ``forward(input_ids, positions, ...)`` over vLLM's packed
``(num_tokens_padded,)`` tensors returning ``(num_tokens_padded, hidden)`` hidden states that vLLM's pooler then
last-token-pools and L2-normalises, ``embed_input_ids`` and ``load_weights``.

Two differences from the reference class. It computes in bf16 (the reference's runner carries fp16 / fp32 only and
downcasts bf16 requests to fp16, ``vllm_model.py:34-45``). And it takes its weights from vLLM: ``load_weights``
consumes the ``(name, tensor)`` stream vLLM reads from the checkpoint and prepares the kernels' weight layout from it,
where the reference ignores the stream and has its runner load the checkpoint a second time by model id.

``forward`` runs the whole packed step as one variable-length forward (``EmbedForwardRunner.forward_packed``): no
per-sequence loop, no padding to a static batch.

vLLM is imported only when it is needed (its pooler, its registry), so the class can be built and tested without it.
"""

from __future__ import annotations

import logging
from collections.abc import Iterable

import torch
import torch.nn as nn

from deplodock_b200.model import EmbedConfig, EmbedWeights
from deplodock_b200.runner import EmbedForwardRunner

logger = logging.getLogger(__name__)

ARCHITECTURE = "B200EmbedModel"


def _embed_config_from_hf(hf_config) -> EmbedConfig:
    """Trunk shape from an HF config object (``Qwen3Config`` and relatives)."""
    head_dim = getattr(hf_config, "head_dim", None) or hf_config.hidden_size // hf_config.num_attention_heads
    theta = getattr(hf_config, "rope_theta", None)
    if theta is None:   # newer configs keep it under rope_parameters
        theta = (getattr(hf_config, "rope_parameters", None) or {}).get("rope_theta", 1e6)
    return EmbedConfig(vocab_size=hf_config.vocab_size, hidden_size=hf_config.hidden_size,
                       intermediate_size=hf_config.intermediate_size,
                       num_hidden_layers=hf_config.num_hidden_layers,
                       num_attention_heads=hf_config.num_attention_heads,
                       num_key_value_heads=getattr(hf_config, "num_key_value_heads", hf_config.num_attention_heads),
                       head_dim=head_dim, rms_norm_eps=hf_config.rms_norm_eps, rope_theta=float(theta))


class B200EmbedModel(nn.Module):
    is_pooling_model = True
    default_seq_pooling_type = "LAST"
    attn_type = "encoder_only"  # whole-sequence prefills only (disables chunked prefill)

    def __init__(self, *, vllm_config, prefix: str = "") -> None:
        super().__init__()
        mc = vllm_config.model_config
        self.out_dtype = mc.dtype
        self.vocab_size = mc.get_vocab_size()
        self.max_seq_len = int(mc.max_model_len)
        self.cfg = _embed_config_from_hf(mc.hf_config)
        sched = getattr(vllm_config, "scheduler_config", None)
        #: sequences and tokens one step can carry: vLLM's own limits size the runner's buffers
        self.max_num_seqs = int(getattr(sched, "max_num_seqs", 1) or 1)
        self.max_num_tokens = int(getattr(sched, "max_num_batched_tokens", 0) or 0) or self.max_seq_len
        self.pooler = self._make_pooler(mc)
        self.runner: EmbedForwardRunner | None = None   # built by load_weights
        if mc.dtype not in (torch.bfloat16, torch.float16, torch.float32):
            raise ValueError(f"unsupported --dtype {mc.dtype}")
        if mc.dtype != torch.bfloat16:
            logger.warning("[serving] the trunk computes in bfloat16; hidden states are returned as %s", mc.dtype)

    @staticmethod
    def _make_pooler(model_config):
        try:
            from vllm.model_executor.layers.pooler import DispatchPooler
        except Exception:  # noqa: BLE001 - vLLM absent or not importable here: the class still runs stand-alone
            return None
        return DispatchPooler.for_embedding(model_config.pooler_config)

    # -- vLLM model protocol -----------------------------------------------------------------------------------
    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        """Consume vLLM's checkpoint stream and prepare the kernels' weight layout. Names may carry a ``model.``
        prefix; the LM head of a causal-LM checkpoint and rotary buffers are skipped. Returns the names taken."""
        state: dict[str, torch.Tensor] = {}
        taken: set[str] = set()
        for name, tensor in weights:
            key = name[len("model."):] if name.startswith("model.") else name
            if key.startswith("lm_head.") or "rotary_emb" in key:
                continue
            state[key] = tensor
            taken.add(name)
        need = ["embed_tokens.weight", "norm.weight"] + [
            f"layers.{i}.{leaf}" for i in range(self.cfg.num_hidden_layers) for leaf in (
                "input_layernorm.weight", "self_attn.q_proj.weight", "self_attn.k_proj.weight",
                "self_attn.v_proj.weight", "self_attn.o_proj.weight", "self_attn.q_norm.weight",
                "self_attn.k_norm.weight", "post_attention_layernorm.weight", "mlp.gate_proj.weight",
                "mlp.up_proj.weight", "mlp.down_proj.weight")]
        missing = [n for n in need if n not in state]
        if missing:
            raise KeyError(f"checkpoint stream lacks {len(missing)} trunk weights, e.g. {missing[:3]}")
        # buffers sized by vLLM's own step limits: at most max_num_batched_tokens tokens in max_num_seqs sequences
        pad = -(-self.max_seq_len // 128) * 128
        tokens = max(pad, min(self.max_num_tokens, self.max_num_seqs * pad))
        self.runner = EmbedForwardRunner(EmbedWeights(self.cfg, state), self.max_seq_len, self.max_num_seqs,
                                         max_tokens=tokens)
        return taken

    def forward(self, input_ids, positions, intermediate_tensors=None, inputs_embeds=None, **kwargs):
        """Packed ``(num_tokens_padded,)`` ids and 0-based per-request positions in, ``(num_tokens_padded, hidden)``
        hidden states out. vLLM pads ``num_tokens``; padding tokens whose positions restart at 0 form one more span,
        exactly as in the reference's split (their rows are computed and ignored by the pooler)."""
        if self.runner is None:
            raise RuntimeError("load_weights has not been called")
        out = self.runner.forward_packed(input_ids, positions)
        return out.to(device=input_ids.device, dtype=self.out_dtype)

    def embed_input_ids(self, input_ids):
        # protocol stub, as in the reference: the embedding table lives with the kernels
        return torch.empty((input_ids.shape[0], 0), device=input_ids.device, dtype=self.out_dtype)


def vllm_model_class():
    """``B200EmbedModel`` with vLLM's ``IsAttentionFree`` marker mixed in (no KV cache is allocated for it) — what
    gets registered with vLLM. Imports vLLM."""
    from vllm.model_executor.models.interfaces import IsAttentionFree

    return type(ARCHITECTURE, (B200EmbedModel, IsAttentionFree), {"__module__": __name__})


def register() -> None:
    """Register the architecture with vLLM's model registry (call from a vLLM plugin entry point, or before building
    the engine): ``vllm serve <model> --runner pooling --enforce-eager --hf-overrides
    '{"architectures": ["B200EmbedModel"]}'``."""
    from vllm import ModelRegistry

    if ARCHITECTURE not in ModelRegistry.get_supported_archs():
        ModelRegistry.register_model(ARCHITECTURE, vllm_model_class())
