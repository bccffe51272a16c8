"""Serving-side runner: hidden states of whole sequences, one or many per forward, from a packed token stream.

Mirror of the reference's ``EmmyForwardRunner`` (``emmy/serving/runner.py:47-271``) and of the packed-batch seam of
its vLLM model (``emmy/serving/vllm_model.py:70-91``, ``emmy/serving/packed.py:6-34``), on the hand-written kernels:

* ``forward_hidden_states(token_ids)`` — one sequence ``(S,)`` -> ``(S, hidden)``; one CUDA graph per sequence length,
  captured on first sight of that S and kept in an LRU cache, all graphs replaying over one shared buffer set sized for
  ``max_seq_len`` (the reference's per-S graph cache over prefix-occupied buffers, ``runner.py:204-236``).
* ``forward_hidden_states_batched(list)`` — the reference pads every step to a static ``(batch_cap, max_seq_len)``
  program (``runner.py:238-271``). Here a group is padded to its own longest sequence rounded up to 128 tokens, one plan
  (and graph) per ``(group size, padded length)``; right padding is exact under the causal mask (a token attends only to
  earlier positions), and padded rows are not read out.
* ``forward_packed(input_ids, positions)`` — vLLM's packed ``(num_tokens,)`` ids with 0-based per-request positions,
  split at ``positions == 0`` (``split_spans``), run batched, concatenated back; the tail is zero-padded to
  ``num_tokens`` like ``EmmyEmbedModel.forward``.
* ``embed_packed`` — last-token pooling + L2 normalisation of each span (what vLLM's pooler does after the reference's
  forward, ``vllm_model.py:50-58``).

The trunk dtype is bf16 (the reference's runner supports fp16 / fp32 only, ``vllm_model.py:34-45``).
"""

from __future__ import annotations

from collections import OrderedDict

import torch

from deplodock_b200.model import EmbedConfig, EmbedForward, EmbedWeights, EmbedWorkspace

#: plans (CUDA graphs) kept per runner before the least recently used one is dropped
PLAN_CACHE_MAX = 64
#: sequences of a batched group are padded to a multiple of this many tokens (the attention kernel's query block)
PAD_TO = 128


def split_spans(positions, max_seq_len: int) -> list[tuple[int, int]]:
    """Per-sequence ``(start, end)`` spans of a packed batch: a sequence starts wherever ``positions[i] == 0``; index
    0 always starts one (dummy-run batches carry garbage positions), and spans longer than ``max_seq_len`` are cut
    into ``max_seq_len`` pieces. Same contract as ``emmy/serving/packed.py:6-34``."""
    n = len(positions)
    if n == 0:
        return []
    cuts = [0] + [i for i in range(1, n) if positions[i] == 0] + [n]
    spans: list[tuple[int, int]] = []
    for a, b in zip(cuts[:-1], cuts[1:]):
        while b - a > max_seq_len:
            spans.append((a, a + max_seq_len))
            a += max_seq_len
        spans.append((a, b))
    return spans


class EmbedForwardRunner:
    """One set of prepared weights + a cache of per-shape plans over a shared workspace."""

    def __init__(self, weights: EmbedWeights, max_seq_len: int, batch_cap: int = 1, max_tokens: int | None = None) -> None:
        if max_seq_len <= 0 or batch_cap <= 0:
            raise ValueError("max_seq_len and batch_cap must be positive")
        self.weights = weights
        self.cfg: EmbedConfig = weights.cfg
        self.max_seq_len = int(max_seq_len)
        self.batch_cap = int(batch_cap)
        pad_len = -(-self.max_seq_len // PAD_TO) * PAD_TO
        #: token budget of one forward (a padded group never exceeds it)
        self.max_tokens = int(max_tokens) if max_tokens else self.batch_cap * pad_len
        if self.max_tokens < pad_len:
            raise ValueError("max_tokens is smaller than one padded sequence")
        self.workspace = EmbedWorkspace(self.cfg, self.max_tokens, self.batch_cap, weights.device)
        self._plans: OrderedDict[tuple[int, int], EmbedForward] = OrderedDict()
        self.captures = 0   # plans built so far (each one captures a CUDA graph on first use)

    @classmethod
    def create(cls, model, max_seq_len: int, dtype_str: str = "bfloat16", batch: int = 1, *, cfg=None,
               device=None) -> "EmbedForwardRunner":
        """``model``: an HF ``Qwen3Model`` (its ``config`` and ``state_dict()`` are used) or a state dict together with
        ``cfg``. Keyword names follow ``EmmyForwardRunner.create`` (``runner.py:72``); loading from a model id is left
        to the caller (no network access is assumed here)."""
        if dtype_str not in ("bfloat16", "bf16"):
            raise ValueError(f"trunk dtype {dtype_str!r} is not supported: the kernels are bf16")
        if hasattr(model, "state_dict") and not isinstance(model, dict):
            cfg = cfg or model.config
            state = model.state_dict()
        else:
            if cfg is None:
                raise ValueError("cfg is required with a bare state dict")
            state = model
        return cls(EmbedWeights(cfg, state, device=device), max_seq_len=max_seq_len, batch_cap=batch)

    @property
    def hidden_size(self) -> int:
        return self.cfg.hidden_size

    # -----------------------------------------------------------------------------------------------------------
    def _plan(self, batch: int, seq: int) -> EmbedForward:
        key = (batch, seq)
        plan = self._plans.get(key)
        if plan is not None:
            self._plans.move_to_end(key)
            return plan
        plan = EmbedForward(self.cfg, batch=batch, seq=seq, weights=self.weights, workspace=self.workspace,
                            hidden_states=True)
        self.captures += 1
        self._plans[key] = plan
        if len(self._plans) > PLAN_CACHE_MAX:
            self._plans.popitem(last=False)
        return plan

    def forward_hidden_states(self, token_ids: torch.Tensor) -> torch.Tensor:
        """One sequence: ``token_ids`` a 1-D integer CUDA tensor of length ``S <= max_seq_len``; returns ``(S, hidden)``
        bf16 (cloned: the shared buffer is reused by the next request)."""
        s = int(token_ids.shape[0])
        if s > self.max_seq_len:
            raise ValueError(f"seq_len {s} exceeds max_seq_len {self.max_seq_len}")
        if s == 0:
            return torch.empty(0, self.hidden_size, dtype=torch.bfloat16, device=self.weights.device)
        plan = self._plan(1, s)
        plan.ids.copy_(token_ids.reshape(1, s), non_blocking=True)
        plan.replay()
        return plan.hs[:s].clone()

    def forward_hidden_states_batched(self, token_ids_list: list[torch.Tensor]) -> list[torch.Tensor]:
        """Any number of sequences, in groups of at most ``batch_cap`` sequences and ``max_tokens`` padded tokens;
        returns ``(S_i, hidden)`` tensors in the order given."""
        lens = [int(t.shape[0]) for t in token_ids_list]
        if lens and max(lens) > self.max_seq_len:
            raise ValueError(f"seq_len {max(lens)} exceeds max_seq_len {self.max_seq_len}")
        results: list[torch.Tensor | None] = [None] * len(lens)
        start = 0
        while start < len(lens):
            end, longest = start, 0
            while end < len(lens) and end - start < self.batch_cap:
                cand = -(-max(longest, lens[end], 1) // PAD_TO) * PAD_TO
                if (end - start + 1) * cand > self.max_tokens:
                    break
                longest = max(longest, lens[end])
                end += 1
            group = range(start, end)
            B = len(group)
            S = -(-max(longest, 1) // PAD_TO) * PAD_TO
            plan = self._plan(B, S)
            plan.ids.zero_()
            for row, i in enumerate(group):
                if lens[i]:
                    plan.ids[row, : lens[i]].copy_(token_ids_list[i], non_blocking=True)
            plan.replay()
            hs = plan.hs.view(B, S, self.hidden_size)
            for row, i in enumerate(group):
                results[i] = hs[row, : lens[i]].clone()
            start = end
        return results  # type: ignore[return-value]

    # -- the packed seam of the vLLM plugin ------------------------------------------------------------------------
    def forward_packed(self, input_ids: torch.Tensor, positions) -> torch.Tensor:
        """``input_ids`` ``(num_tokens,)`` packed sequences, ``positions`` their 0-based per-request positions (tensor or
        sequence); returns ``(num_tokens, hidden)`` bf16, zero rows where the spans do not cover the tail."""
        n = int(input_ids.shape[0])
        ids = input_ids.clamp(0, self.cfg.vocab_size - 1).to(torch.int64)
        pos = positions.detach().cpu().reshape(-1).tolist() if isinstance(positions, torch.Tensor) else list(positions)
        spans = split_spans(pos, self.max_seq_len)
        chunks = self.forward_hidden_states_batched([ids[a:b] for a, b in spans]) if spans else []
        if chunks:
            out = torch.cat(chunks, dim=0)
        else:
            out = torch.zeros(0, self.hidden_size, dtype=torch.bfloat16, device=input_ids.device)
        if out.shape[0] < n:
            out = torch.nn.functional.pad(out, (0, 0, 0, n - out.shape[0]))
        return out

    def embed_packed(self, input_ids: torch.Tensor, positions) -> torch.Tensor:
        """Last-token pooling and L2 normalisation per span: ``(num_sequences, hidden)`` fp32."""
        pos = positions.detach().cpu().reshape(-1).tolist() if isinstance(positions, torch.Tensor) else list(positions)
        spans = split_spans(pos, self.max_seq_len)
        hidden = self.forward_packed(input_ids, pos)
        last = torch.tensor([b - 1 for _, b in spans], dtype=torch.int64, device=hidden.device)
        return torch.nn.functional.normalize(hidden.index_select(0, last).float(), p=2.0, dim=-1)
