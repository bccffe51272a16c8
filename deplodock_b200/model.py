"""Qwen3-Embedding-shaped forward on the emk kernels: token ids -> pooled, L2-normalised embeddings.

The reference serves this model one sequence per forward: ``EmmyForwardRunner`` traces the HF trunk with
``build_full_model_wrapper`` (``emmy/compiler/trace/huggingface.py:17-186``), compiles it into one program and replays
a captured CUDA graph per sequence (``emmy/serving/runner.py:204-236``); vLLM then pools the last token and normalises
(``emmy/serving/vllm_model.py:50-58``). The traced layer is GatherOp, five RMSNorm chains, seven LinearOps, a RoPE
chain, repeat_kv, SdpaOp with an additive causal mask, and a SwiGLU — 18 generated kernels per layer.

Here the same dataflow is a fixed plan of five launches per layer over a whole batch of sequences, with the two
RMSNorms of a layer folded around the GEMMs (the producer's epilogue writes partial row sums of squares, the consumer
scales its accumulator rows; the norm weight is folded into the projection):

    GEMM(Wqkv * ln1) + rmsnorm-in + q/k-norm + RoPE (epilogue) -> causal GQA flash attention (token-major, no transposes)
        -> GEMM(Wo) + residual + row sums of squares -> GEMM((Wgate|Wup interleaved) * ln2) + rmsnorm-in + SwiGLU
        -> GEMM(Wdown) + residual + row sums of squares

preceded by the embedding gather (which also writes the first row sums of squares) and followed by a last-token
RMSNorm + L2 kernel (``fold_rmsnorm=False`` keeps the two stand-alone RMSNorm kernels: seven launches per layer). The
whole forward is captured once in a CUDA graph and replayed. Sequences are independent, so a batch can be processed in
chunks (``chunk_seqs``). Weights are prepared once (:class:`EmbedWeights`) and shared by plans of different shapes,
which take prefixes of one activation workspace (:class:`EmbedWorkspace`): q/k/v projections concatenated, gate/up
rows interleaved, cos/sin tables rounded to bf16 as the eager module does.
"""

from __future__ import annotations

import os

from dataclasses import dataclass

import torch

from deplodock_b200 import ops


@dataclass(frozen=True)
class EmbedConfig:
    """Trunk shape; defaults are Qwen3-Embedding-0.6B."""

    vocab_size: int = 151669
    hidden_size: int = 1024
    intermediate_size: int = 3072
    num_hidden_layers: int = 28
    num_attention_heads: int = 16
    num_key_value_heads: int = 8
    head_dim: int = 128
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6

    @classmethod
    def from_any(cls, cfg) -> "EmbedConfig":
        """Accepts any object with these attribute names (an HF ``Qwen3Config`` included)."""
        return cls(**{f: getattr(cfg, f) for f in cls.__dataclass_fields__})  # type: ignore[attr-defined]

    def linear_flops_per_token(self) -> int:
        H, I, D = self.hidden_size, self.intermediate_size, self.head_dim
        nq, nkv = self.num_attention_heads, self.num_key_value_heads
        per_layer = H * (nq + 2 * nkv) * D + nq * D * H + 3 * H * I
        return 2 * per_layer * self.num_hidden_layers

    def attention_flops(self, batch: int, seq: int) -> int:
        """Causal-useful flops: 4 * B * Hq * D * S(S+1)/2 per layer."""
        return self.num_hidden_layers * 4 * batch * self.num_attention_heads * self.head_dim * (seq * (seq + 1) // 2)


def rope_tables(seq: int, head_dim: int, theta: float, device) -> tuple[torch.Tensor, torch.Tensor]:
    """cos/sin ``[seq, head_dim]`` bf16 as HF builds them for a bf16 module (``cat(freqs, freqs)``, cast to bf16)."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.int64).float() / head_dim))
    freqs = torch.outer(torch.arange(seq, dtype=torch.float32), inv_freq)
    emb = torch.cat([freqs, freqs], dim=-1)
    cos = emb.cos().to(torch.bfloat16).contiguous().to(device)
    sin = emb.sin().to(torch.bfloat16).contiguous().to(device)
    return cos, sin


#: a rank with this many token rows runs the projections between two attention launches as one GEMM chain
#: (``emk_gemm_bf16_chain``): the whole forward measured 1.5-3 % faster at 8192 and 16384 rows, 2-3 % slower at 4096
#: (the chain's dependency latencies outweigh the launches it saves) and 1-2 % slower at 32768 (nothing left to hide)
CHAIN_MIN_TOKENS = 8192
CHAIN_MAX_TOKENS = 16384


def launch_names(num_layers: int, fold_rmsnorm: bool = True, hidden_states: bool = False,
                 pool: bool = True, chain: bool = False) -> list[tuple[str, str]]:
    """``(kernel name, C-ABI entry)`` of every launch of one chunk of the plan, in order — what
    :meth:`EmbedForward.launch_list` launches, computable without a device (the backend shim lists a compiled trunk
    with it). ``chain``: o_proj, gate/up, down and the next layer's QKV projection as one launch."""
    L: list[tuple[str, str]] = []
    if fold_rmsnorm and chain:
        L.append(("k_embed_gather_sumsq", "emk_embed_gather_sumsq"))
        L.append(("k_rmsnorm_linear_qkv_qknorm_rope_0", "emk_gemm_bf16_fused"))
        for i in range(num_layers):
            L.append((f"k_scaled_dot_product_attention_{i}", "emk_sdpa_causal_gqa_bf16_tok"))
            tail = f"_qkv_{i + 1}" if i + 1 < num_layers else ""
            L.append((f"k_linear_chain_o_proj_gate_up_down_{i}{tail}", "emk_gemm_bf16_chain"))
    elif fold_rmsnorm:
        L.append(("k_embed_gather_sumsq", "emk_embed_gather_sumsq"))
        for i in range(num_layers):
            L += [(f"k_rmsnorm_linear_qkv_qknorm_rope_{i}", "emk_gemm_bf16_fused"),
                  (f"k_scaled_dot_product_attention_{i}", "emk_sdpa_causal_gqa_bf16_tok"),
                  (f"k_linear_o_proj_residual_sumsq_{i}", "emk_gemm_bf16_fused"),
                  (f"k_rmsnorm_linear_gate_up_swiglu_{i}", "emk_gemm_bf16_fused"),
                  (f"k_linear_down_residual_sumsq_{i}", "emk_gemm_bf16_fused")]
    else:
        L.append(("k_embed_gather", "emk_embed_gather"))
        for i in range(num_layers):
            L += [(f"k_rms_norm_input_{i}", "emk_rmsnorm"),
                  (f"k_linear_qkv_qknorm_rope_{i}", "emk_linear_bf16_qknorm_rope"),
                  (f"k_scaled_dot_product_attention_{i}", "emk_sdpa_causal_gqa_bf16_tok"),
                  (f"k_linear_o_proj_residual_{i}", "emk_linear_bf16"),
                  (f"k_rms_norm_post_attention_{i}", "emk_rmsnorm"),
                  (f"k_linear_gate_up_swiglu_{i}", "emk_linear_bf16"),
                  (f"k_linear_down_residual_{i}", "emk_linear_bf16")]
    if hidden_states:
        L.append(("k_rms_norm_final", "emk_rmsnorm"))
    if pool:
        L.append(("k_pool_norm_l2", "emk_pool_norm_l2"))
    return L


class _LayerWeights:
    __slots__ = ("ln1", "wqkv", "qn", "kn", "wo", "ln2", "wgu", "wdown")


class EmbedWeights:
    """The trunk's weights in the layout the kernels read, prepared once and shared by every plan: q/k/v projections
    concatenated, gate/up rows interleaved, and (``fold_rmsnorm``) the two per-layer RMSNorm weights multiplied into
    the projection that follows them. ``state_dict`` uses the HF ``Qwen3Model`` parameter names."""

    def __init__(self, cfg, state_dict: dict[str, torch.Tensor], *, device=None, fold_rmsnorm: bool = True) -> None:
        self.cfg = c = EmbedConfig.from_any(cfg)
        self.fold_rmsnorm = bool(fold_rmsnorm)
        if c.head_dim != 128:
            raise ValueError("the attention kernel is built for head_dim 128")
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        dev, bf = self.device, torch.bfloat16

        def w(name: str) -> torch.Tensor:
            t = state_dict[name]
            return t.to(device=dev, dtype=bf).contiguous()

        self.embed = w("embed_tokens.weight")
        self.final_norm = w("norm.weight")
        self.layers: list[_LayerWeights] = []
        for i in range(c.num_hidden_layers):
            p = f"layers.{i}."
            lw = _LayerWeights()
            lw.ln1 = w(p + "input_layernorm.weight")
            lw.wqkv = torch.cat([w(p + "self_attn.q_proj.weight"), w(p + "self_attn.k_proj.weight"),
                                 w(p + "self_attn.v_proj.weight")], dim=0).contiguous()
            lw.qn = w(p + "self_attn.q_norm.weight")
            lw.kn = w(p + "self_attn.k_norm.weight")
            lw.wo = w(p + "self_attn.o_proj.weight")
            lw.ln2 = w(p + "post_attention_layernorm.weight")
            gate, up = w(p + "mlp.gate_proj.weight"), w(p + "mlp.up_proj.weight")
            # rows interleaved (gate_0, up_0, gate_1, up_1, ...) so one accumulator row holds both halves of a pair
            lw.wgu = torch.stack([gate, up], dim=1).reshape(2 * c.intermediate_size, c.hidden_size).contiguous()
            lw.wdown = w(p + "mlp.down_proj.weight")
            if self.fold_rmsnorm:
                # RMSNorm folded around the GEMMs: y = rsqrt(mean(h^2)+eps) * (h @ (W * w_norm)^T)
                lw.wqkv = (lw.wqkv.float() * lw.ln1.float()[None, :]).to(bf).contiguous()
                lw.wgu = (lw.wgu.float() * lw.ln2.float()[None, :]).to(bf).contiguous()
            self.layers.append(lw)


class EmbedWorkspace:
    """Activation buffers sized for ``max_tokens`` tokens / ``max_batch`` sequences. Plans of different (batch, seq)
    take prefixes of the same buffers, so each captured CUDA graph replays over memory that stays put — the scheme of
    the reference's shared buffer set sized at ``max_seq_len`` (``emmy/serving/runner.py:160-170``)."""

    def __init__(self, cfg, max_tokens: int, max_batch: int, device) -> None:
        c = EmbedConfig.from_any(cfg)
        nq, nkv, D = c.num_attention_heads, c.num_key_value_heads, c.head_dim
        dev, bf = torch.device(device), torch.bfloat16
        self.max_tokens, self.max_batch = int(max_tokens), int(max_batch)
        T = self.max_tokens
        self.ids = torch.zeros(T, dtype=torch.int64, device=dev)
        self.h = torch.empty(T, c.hidden_size, dtype=bf, device=dev)
        self.x = torch.empty(T, c.hidden_size, dtype=bf, device=dev)
        self.hs = torch.empty(T, c.hidden_size, dtype=bf, device=dev)
        self.qkv = torch.empty(T, (nq + 2 * nkv) * D, dtype=bf, device=dev)
        self.attn = torch.empty(T, nq * D, dtype=bf, device=dev)
        self.mlp = torch.empty(T, c.intermediate_size, dtype=bf, device=dev)
        self.out = torch.empty(self.max_batch, c.hidden_size, dtype=torch.float32, device=dev)
        # scratch of the two folded RMSNorms: partial row sums of squares, one slot per 128 hidden columns, fully
        # overwritten by every producer (no clearing, no atomics)
        self.ss1 = torch.zeros(T, c.hidden_size // 128, dtype=torch.float32, device=dev)
        self.ss2 = torch.zeros(T, c.hidden_size // 128, dtype=torch.float32, device=dev)


class EmbedForward:
    """Batch forward of the trunk on one GPU. ``state_dict`` uses the HF ``Qwen3Model`` parameter names; pass
    ``weights=`` (an :class:`EmbedWeights`) and ``workspace=`` to share them between plans of different shapes.
    With ``hidden_states=True`` the plan also writes the final-norm hidden states of every token to ``self.hs``
    (``[batch * seq, hidden]`` bf16), which is what the reference's runner returns."""

    #: kernel launches per layer / outside the layers, for launch accounting in the bench
    @property
    def LAUNCHES_FIXED(self) -> int:
        return 1 + int(self.hidden_states) + int(self.pool)

    @property
    def LAUNCHES_PER_LAYER(self) -> int:
        if self.chain:
            return 2
        return 5 if self.fold_rmsnorm else 7

    def __init__(self, cfg, state_dict: dict[str, torch.Tensor] | None = None, *, batch: int, seq: int, device=None,
                 chunk_seqs: int | None = None, fold_rmsnorm: bool = True, weights: EmbedWeights | None = None,
                 workspace: EmbedWorkspace | None = None, hidden_states: bool = False,
                 rope: tuple[torch.Tensor, torch.Tensor] | None = None, pool: bool = True,
                 chain: bool | None = None) -> None:
        if weights is None:
            if state_dict is None:
                raise ValueError("give a state_dict or prepared weights")
            weights = EmbedWeights(cfg, state_dict, device=device, fold_rmsnorm=fold_rmsnorm)
        self.weights = weights
        self.cfg = c = weights.cfg
        self.fold_rmsnorm = weights.fold_rmsnorm
        self.device = dev = weights.device
        self.batch, self.seq = int(batch), int(seq)
        self.chunk_seqs = self.batch if not chunk_seqs else min(int(chunk_seqs), self.batch)
        if self.batch % self.chunk_seqs != 0:
            raise ValueError("chunk_seqs must divide the batch")
        self.hidden_states = bool(hidden_states)
        self.pool = bool(pool)   # False: stop at the final-norm hidden states (what a traced trunk returns)
        if not self.pool and not self.hidden_states:
            raise ValueError("a plan without pooling must produce hidden states")
        if self.hidden_states and self.chunk_seqs != self.batch:
            raise ValueError("hidden_states=True needs the whole batch in one chunk")
        self.embed, self.final_norm, self.layers = weights.embed, weights.final_norm, weights.layers
        if rope is None:
            self.cos, self.sin = rope_tables(self.seq, c.head_dim, c.rope_theta, dev)
        else:   # cos/sin buffers of a traced module ([seq, head_dim] or [1, seq, head_dim]) instead of theta
            self.cos, self.sin = (t.reshape(-1, c.head_dim).to(device=dev, dtype=torch.bfloat16).contiguous()
                                  for t in rope)
            if self.cos.shape[0] != self.seq or self.sin.shape[0] != self.seq:
                raise ValueError("rotary tables do not match the sequence length")
        self.rope_cm = ops.rope_chunk_major(self.cos, self.sin)

        T = self.chunk_seqs * self.seq
        if workspace is None:
            workspace = EmbedWorkspace(c, T, self.batch, dev)
            if self.batch * self.seq > T:   # chunked plan: the id buffer still holds the whole batch
                workspace.ids = torch.zeros(self.batch * self.seq, dtype=torch.int64, device=dev)
        if workspace.max_tokens < T or workspace.max_batch < self.batch or workspace.ids.numel() < self.batch * self.seq:
            raise ValueError("workspace too small for this plan")
        self.workspace = ws = workspace
        self.ids = ws.ids[: self.batch * self.seq].view(self.batch, self.seq)
        self.h, self.x, self.hs = ws.h[:T], ws.x[:T], ws.hs[:T]
        self.qkv, self.attn, self.mlp = ws.qkv[:T], ws.attn[:T], ws.mlp[:T]
        self.out = ws.out[: self.batch]
        self.ss1, self.ss2 = ws.ss1[:T], ws.ss2[:T]
        #: the GEMMs between two attention launches as one chained launch (None: by size; EMK_GEMM_CHAIN=0/1 forces)
        if chain is None:
            env = os.environ.get("EMK_GEMM_CHAIN")
            chain = (env != "0") and (env == "1" or CHAIN_MIN_TOKENS <= T <= CHAIN_MAX_TOKENS)
        self.chain = bool(chain) and self.fold_rmsnorm
        self.chain_ws = ops.gemm_chain_workspace(T, dev) if self.chain else None
        self._graph: torch.cuda.CUDAGraph | None = None

    # -----------------------------------------------------------------------------------------------------------
    @property
    def num_launches(self) -> int:
        chunks = self.batch // self.chunk_seqs
        per_layer = self.LAUNCHES_PER_LAYER
        return chunks * (per_layer * self.cfg.num_hidden_layers + self.LAUNCHES_FIXED + int(self.chain))

    def flops(self) -> int:
        return self.cfg.linear_flops_per_token() * self.batch * self.seq + self.cfg.attention_flops(self.batch,
                                                                                                     self.seq)

    def launch_list(self, ids: torch.Tensor, out: torch.Tensor) -> list[tuple[str, str, object]]:
        """The plan of one chunk as ``(kernel name, C-ABI entry, thunk)`` per launch, in launch order. Calling the
        thunks one after the other is the forward; the backend shim lists and times them one by one."""
        c = self.cfg
        B, S = ids.shape
        nq, nkv = c.num_attention_heads, c.num_key_value_heads
        eps = c.rms_norm_eps
        H = c.hidden_size
        L: list[tuple[str, str, object]] = []

        def add(name: str, entry: str, fn) -> None:
            L.append((name, entry, fn))

        def qkv_phase(lw) -> dict:
            return dict(x=self.h, w=lw.wqkv, out=self.qkv, epilogue="qknorm_rope", row_sumsq_in=self.ss1, norm_dim=H,
                        norm_eps=eps, q_weight=lw.qn, k_weight=lw.kn, rope_cm=self.rope_cm, S=S, Hq=nq, Hkv=nkv,
                        qk_eps=eps)

        def mlp_phases(lw) -> list[dict]:
            return [dict(x=self.attn, w=lw.wo, out=self.h, epilogue="residual", residual=self.h,
                         row_sumsq_out=self.ss2),
                    dict(x=self.h, w=lw.wgu, out=self.mlp, epilogue="swiglu", row_sumsq_in=self.ss2, norm_dim=H,
                         norm_eps=eps),
                    dict(x=self.mlp, w=lw.wdown, out=self.h, epilogue="residual", residual=self.h,
                         row_sumsq_out=self.ss1)]

        if self.fold_rmsnorm and self.chain:
            add("k_embed_gather_sumsq", "emk_embed_gather_sumsq",
                lambda: ops.embed_gather(self.embed, ids, out=self.h, row_sumsq=self.ss1))
            first = dict(qkv_phase(self.layers[0]))
            add("k_rmsnorm_linear_qkv_qknorm_rope_0", "emk_gemm_bf16_fused",
                lambda first=first: ops.gemm_fused(first["x"], first["w"], first["out"],
                                                   **{k: v for k, v in first.items() if k not in ("x", "w", "out")}))
            for i, lw in enumerate(self.layers):
                add(f"k_scaled_dot_product_attention_{i}", "emk_sdpa_causal_gqa_bf16_tok",
                    lambda: ops.sdpa_causal_gqa_tok(self.qkv, B, S, nq, nkv, self.attn))
                phases = mlp_phases(lw)
                tail = ""
                if i + 1 < len(self.layers):
                    phases.append(qkv_phase(self.layers[i + 1]))
                    tail = f"_qkv_{i + 1}"
                add(f"k_linear_chain_o_proj_gate_up_down_{i}{tail}", "emk_gemm_bf16_chain",
                    lambda phases=phases: ops.gemm_chain(phases, self.chain_ws))
        elif self.fold_rmsnorm:
            add("k_embed_gather_sumsq", "emk_embed_gather_sumsq",
                lambda: ops.embed_gather(self.embed, ids, out=self.h, row_sumsq=self.ss1))
            for i, lw in enumerate(self.layers):
                add(f"k_rmsnorm_linear_qkv_qknorm_rope_{i}", "emk_gemm_bf16_fused",
                    lambda lw=lw: ops.gemm_fused(self.h, lw.wqkv, self.qkv, epilogue="qknorm_rope",
                                                 row_sumsq_in=self.ss1, norm_dim=H, norm_eps=eps, q_weight=lw.qn,
                                                 k_weight=lw.kn, rope_cm=self.rope_cm, S=S, Hq=nq, Hkv=nkv, qk_eps=eps))
                add(f"k_scaled_dot_product_attention_{i}", "emk_sdpa_causal_gqa_bf16_tok",
                    lambda: ops.sdpa_causal_gqa_tok(self.qkv, B, S, nq, nkv, self.attn))
                add(f"k_linear_o_proj_residual_sumsq_{i}", "emk_gemm_bf16_fused",
                    lambda lw=lw: ops.gemm_fused(self.attn, lw.wo, self.h, epilogue="residual", residual=self.h,
                                                 row_sumsq_out=self.ss2))
                add(f"k_rmsnorm_linear_gate_up_swiglu_{i}", "emk_gemm_bf16_fused",
                    lambda lw=lw: ops.gemm_fused(self.h, lw.wgu, self.mlp, epilogue="swiglu", row_sumsq_in=self.ss2,
                                                 norm_dim=H, norm_eps=eps))
                add(f"k_linear_down_residual_sumsq_{i}", "emk_gemm_bf16_fused",
                    lambda lw=lw: ops.gemm_fused(self.mlp, lw.wdown, self.h, epilogue="residual", residual=self.h,
                                                 row_sumsq_out=self.ss1))
        else:
            add("k_embed_gather", "emk_embed_gather", lambda: ops.embed_gather(self.embed, ids, out=self.h))
            for i, lw in enumerate(self.layers):
                add(f"k_rms_norm_input_{i}", "emk_rmsnorm", lambda lw=lw: ops.rmsnorm(self.h, lw.ln1, eps, out=self.x))
                add(f"k_linear_qkv_qknorm_rope_{i}", "emk_linear_bf16_qknorm_rope",
                    lambda lw=lw: ops.linear_qknorm_rope(self.x, lw.wqkv, lw.qn, lw.kn, self.rope_cm, S, nq, nkv, eps,
                                                         out=self.qkv))
                add(f"k_scaled_dot_product_attention_{i}", "emk_sdpa_causal_gqa_bf16_tok",
                    lambda: ops.sdpa_causal_gqa_tok(self.qkv, B, S, nq, nkv, self.attn))
                add(f"k_linear_o_proj_residual_{i}", "emk_linear_bf16",
                    lambda lw=lw: ops.linear(self.attn, lw.wo, residual=self.h, out=self.h))
                add(f"k_rms_norm_post_attention_{i}", "emk_rmsnorm",
                    lambda lw=lw: ops.rmsnorm(self.h, lw.ln2, eps, out=self.x))
                add(f"k_linear_gate_up_swiglu_{i}", "emk_linear_bf16",
                    lambda lw=lw: ops.linear(self.x, lw.wgu, swiglu=True, out=self.mlp))
                add(f"k_linear_down_residual_{i}", "emk_linear_bf16",
                    lambda lw=lw: ops.linear(self.mlp, lw.wdown, residual=self.h, out=self.h))
        if self.hidden_states:
            add("k_rms_norm_final", "emk_rmsnorm", lambda: ops.rmsnorm(self.h, self.final_norm, eps, out=self.hs))
        if self.pool:
            add("k_pool_norm_l2", "emk_pool_norm_l2",
                lambda: ops.pool_norm_l2(self.h, self.final_norm, B, S, eps, out=out))
        assert [(n, e) for n, e, _ in L] == launch_names(c.num_hidden_layers, self.fold_rmsnorm, self.hidden_states,
                                                         self.pool, self.chain)
        return L

    def _forward_chunk(self, ids: torch.Tensor, out: torch.Tensor) -> None:
        # a chained plan launches everything the ordinary way: kernels that become resident early only spin next to
        # the chain's long-lived CTAs (measured 1.5-2 % on the 16 x 512 forward); the setting is per launch, so it is
        # in force while the plan is launched or captured and restored afterwards
        h = ops.handle()
        prev = h.set_launch_overlap(False) if self.chain else None
        try:
            for _, _, fn in self.launch_list(ids, out):
                fn()
        finally:
            if prev is not None:
                h.set_launch_overlap(prev)

    def forward_eager(self) -> torch.Tensor:
        """Launch the plan on the current stream from ``self.ids``; returns ``self.out`` ``[batch, hidden]`` fp32."""
        cs = self.chunk_seqs
        for b0 in range(0, self.batch, cs):
            self._forward_chunk(self.ids[b0:b0 + cs], self.out[b0:b0 + cs])
        return self.out

    def capture(self) -> None:
        """Capture the whole forward in one CUDA graph (after one eager warm-up run)."""
        self.forward_eager()
        torch.cuda.synchronize(self.device)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self.forward_eager()
        self._graph = g

    def replay(self) -> torch.Tensor:
        if self._graph is None:
            self.capture()
        self._graph.replay()
        return self.out

    def __call__(self, ids: torch.Tensor) -> torch.Tensor:
        """Copy ``ids`` (host or device, ``[batch, seq]`` int64) into the static input buffer and run the graph."""
        if tuple(ids.shape) != (self.batch, self.seq):
            raise ValueError(f"expected ids of shape {(self.batch, self.seq)}, got {tuple(ids.shape)}")
        self.ids.copy_(ids, non_blocking=True)
        return self.replay()


class PackedForward:
    """The same trunk over a PACKED stream of sequences of different lengths: ``tokens`` rows in all, up to
    ``max_seqs`` sequences, none longer than ``max_seq_len`` — the wire format of the reference's vLLM plugin
    (``emmy/serving/vllm_model.py:70-91``: packed ``(num_tokens,)`` ids and 0-based per-request positions), run the way
    its serving notes ask for as follow-up #1 (``emmy/serving/ARCHITECTURE.md:133-137``): one forward at mixed lengths,
    no padding between sequences. The GEMMs run over the token rows as they are (rows are independent); the fused
    QKV epilogue takes each row's rotary position from ``positions``; attention walks a table of 128-row query blocks
    built on the device from ``cu_seqlens``; pooling reads each sequence's last row.

    Everything that varies between requests lives in device buffers (``ids``, ``positions``, ``cu_seqlens``), so one
    captured CUDA graph per token budget serves any mix of lengths. Rows past the last sequence are computed from
    token 0 and ignored."""

    def __init__(self, weights: EmbedWeights, *, tokens: int, max_seqs: int, max_seq_len: int,
                 workspace: EmbedWorkspace | None = None, hidden_states: bool = True, pool: bool = True,
                 chain: bool | None = None) -> None:
        self.weights = weights
        self.cfg = c = weights.cfg
        if not weights.fold_rmsnorm:
            raise ValueError("the packed plan uses the folded-RMSNorm weights")
        self.device = dev = weights.device
        self.tokens, self.max_seqs, self.max_seq_len = int(tokens), int(max_seqs), int(max_seq_len)
        self.hidden_states, self.pool = bool(hidden_states), bool(pool)
        T = self.tokens
        if workspace is None:
            workspace = EmbedWorkspace(c, T, self.max_seqs, dev)
        if workspace.max_tokens < T or workspace.max_batch < self.max_seqs:
            raise ValueError("workspace too small for this plan")
        ws = self.workspace = workspace
        self.ids = ws.ids[:T]
        self.h, self.hs = ws.h[:T], ws.hs[:T]
        self.qkv, self.attn, self.mlp = ws.qkv[:T], ws.attn[:T], ws.mlp[:T]
        self.ss1, self.ss2 = ws.ss1[:T], ws.ss2[:T]
        self.out = ws.out[: self.max_seqs]
        self.attn.zero_()   # rows outside every sequence are never written by the attention kernel
        self.positions = torch.zeros(T, dtype=torch.int32, device=dev)
        self.cu_seqlens = torch.zeros(self.max_seqs + 1, dtype=torch.int32, device=dev)
        self.vl_ws = ops.sdpa_varlen_workspace(self.max_seqs, T, dev)
        cos, sin = rope_tables(self.max_seq_len, c.head_dim, c.rope_theta, dev)
        self.rope_cm = ops.rope_chunk_major(cos, sin)
        if chain is None:   # as in EmbedForward
            env = os.environ.get("EMK_GEMM_CHAIN")
            chain = (env != "0") and (env == "1" or CHAIN_MIN_TOKENS <= T <= CHAIN_MAX_TOKENS)
        self.chain = bool(chain)
        self.chain_ws = ops.gemm_chain_workspace(T, dev) if self.chain else None
        self._graph: torch.cuda.CUDAGraph | None = None

    @property
    def num_launches(self) -> int:
        per_layer = 3 if self.chain else 6   # the variable-length attention is two launches (item table + kernel)
        return 1 + int(self.chain) + per_layer * self.cfg.num_hidden_layers + int(self.hidden_states) + int(self.pool)

    def set_batch(self, ids: torch.Tensor, positions: torch.Tensor, cu_seqlens: torch.Tensor) -> None:
        """Copy a packed batch into the static buffers: ``ids`` / ``positions`` ``(n,)`` with ``n <= tokens``,
        ``cu_seqlens`` ``(b + 1,)`` with ``b <= max_seqs`` (unused sequence slots become empty sequences)."""
        n, b = int(ids.shape[0]), int(cu_seqlens.shape[0]) - 1
        if n > self.tokens or b > self.max_seqs:
            raise ValueError(f"batch of {n} tokens / {b} sequences exceeds the plan ({self.tokens} / {self.max_seqs})")
        self.ids[:n].copy_(ids, non_blocking=True)
        self.positions[:n].copy_(positions, non_blocking=True)
        if n < self.tokens:
            self.ids[n:].zero_()
            self.positions[n:].zero_()
        self.cu_seqlens[: b + 1].copy_(cu_seqlens, non_blocking=True)
        if b < self.max_seqs:
            self.cu_seqlens[b + 1:].fill_(n)

    def forward_eager(self) -> None:
        c = self.cfg
        nq, nkv, H, eps = c.num_attention_heads, c.num_key_value_heads, c.hidden_size, c.rms_norm_eps
        ops.embed_gather(self.weights.embed, self.ids, out=self.h, row_sumsq=self.ss1)

        def qkv_phase(lw) -> dict:
            return dict(x=self.h, w=lw.wqkv, out=self.qkv, epilogue="qknorm_rope", row_sumsq_in=self.ss1, norm_dim=H,
                        norm_eps=eps, q_weight=lw.qn, k_weight=lw.kn, rope_cm=self.rope_cm, S=self.max_seq_len,
                        Hq=nq, Hkv=nkv, qk_eps=eps, positions=self.positions)

        def run(ph: dict) -> None:
            ops.gemm_fused(ph["x"], ph["w"], ph["out"], **{k: v for k, v in ph.items() if k not in ("x", "w", "out")})

        layers = self.weights.layers
        h = ops.handle()
        prev = h.set_launch_overlap(False) if self.chain else None   # see EmbedForward._forward_chunk
        try:
            self._layers_and_head(layers, run, qkv_phase, nq, nkv, H, eps)
        finally:
            if prev is not None:
                h.set_launch_overlap(prev)

    def _layers_and_head(self, layers, run, qkv_phase, nq, nkv, H, eps) -> None:
        if self.chain:
            run(qkv_phase(layers[0]))
        for i, lw in enumerate(layers):
            if not self.chain:
                run(qkv_phase(lw))
            ops.sdpa_causal_gqa_varlen(self.qkv, self.cu_seqlens, self.max_seq_len, nq, nkv, self.attn,
                                       workspace=self.vl_ws)
            phases = [dict(x=self.attn, w=lw.wo, out=self.h, epilogue="residual", residual=self.h,
                           row_sumsq_out=self.ss2),
                      dict(x=self.h, w=lw.wgu, out=self.mlp, epilogue="swiglu", row_sumsq_in=self.ss2, norm_dim=H,
                           norm_eps=eps),
                      dict(x=self.mlp, w=lw.wdown, out=self.h, epilogue="residual", residual=self.h,
                           row_sumsq_out=self.ss1)]
            if self.chain:
                if i + 1 < len(layers):
                    phases.append(qkv_phase(layers[i + 1]))
                ops.gemm_chain(phases, self.chain_ws)
            else:
                for ph in phases:
                    run(ph)
        if self.hidden_states:
            ops.rmsnorm(self.h, self.weights.final_norm, eps, out=self.hs)
        if self.pool:
            ops.pool_norm_l2_varlen(self.h, self.weights.final_norm, self.cu_seqlens, eps, out=self.out)

    def replay(self) -> None:
        if self._graph is None:
            self.forward_eager()
            torch.cuda.synchronize(self.device)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self.forward_eager()
            self._graph = g
        self._graph.replay()
