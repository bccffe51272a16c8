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
  split at ``positions == 0`` (``split_spans``) and run as ONE variable-length forward over the stream as it is
  (``deplodock_b200.model.PackedForward``: rotary positions per row, attention over a ``cu_seqlens`` table, no padding
  between sequences; one captured graph per token budget of 128-token steps) — the reference's stated follow-up for
  this seam (``emmy/serving/ARCHITECTURE.md:133-137``); the result covers ``num_tokens`` rows like
  ``EmmyEmbedModel.forward``. ``forward_packed_padded`` keeps the earlier route (groups padded to their longest
  sequence) for comparison.
* ``embed_packed`` — last-token pooling + L2 normalisation of each span (what vLLM's pooler does after the reference's
  forward, ``vllm_model.py:50-58``), from the same variable-length forward.

The trunk dtype is bf16 (the reference's runner supports fp16 / fp32 only, ``vllm_model.py:34-45``).
"""

from __future__ import annotations

from collections import OrderedDict

import torch

from deplodock_b200.model import EmbedConfig, EmbedForward, EmbedWeights, EmbedWorkspace, PackedForward

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
        self._packed: OrderedDict[int, PackedForward] = OrderedDict()
        #: sequences one packed forward admits (a packed stream of max_tokens one-token requests at the extreme)
        self.packed_max_seqs = max(self.batch_cap, min(self.max_tokens, 1024))
        if self.workspace.out.shape[0] < self.packed_max_seqs:
            self.workspace.out = torch.empty(self.packed_max_seqs, self.cfg.hidden_size, dtype=torch.float32,
                                             device=weights.device)
            self.workspace.max_batch = self.packed_max_seqs
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
    def _packed_plan(self, tokens: int) -> PackedForward:
        bucket = min(-(-max(tokens, 1) // PAD_TO) * PAD_TO, -(-self.max_tokens // PAD_TO) * PAD_TO)
        plan = self._packed.get(bucket)
        if plan is not None:
            self._packed.move_to_end(bucket)
            return plan
        plan = PackedForward(self.weights, tokens=bucket, max_seqs=self.packed_max_seqs, max_seq_len=self.max_seq_len,
                             workspace=self.workspace if bucket <= self.workspace.max_tokens else None)
        self.captures += 1
        self._packed[bucket] = plan
        if len(self._packed) > PLAN_CACHE_MAX:
            self._packed.popitem(last=False)
        return plan

    def _run_packed(self, input_ids: torch.Tensor, positions):
        """One variable-length forward per ``max_tokens`` worth of whole spans. Yields ``(plan, first row of the
        chunk in the stream, rows, spans of the chunk relative to it)`` after each replay; the plan's buffers are
        valid until the next one."""
        n = int(input_ids.shape[0])
        dev = self.weights.device
        ids = input_ids.to(device=dev).clamp(0, self.cfg.vocab_size - 1).to(torch.int64)
        pos = positions.detach().cpu().reshape(-1).tolist() if isinstance(positions, torch.Tensor) else list(positions)
        spans = split_spans(pos, self.max_seq_len)
        i = 0
        while i < len(spans):
            j, start = i, spans[i][0]
            while j < len(spans) and spans[j][1] - start <= self.max_tokens and j - i < self.packed_max_seqs:
                j += 1
            end = spans[j - 1][1]
            rel = [(a - start, b - start) for a, b in spans[i:j]]
            plan = self._packed_plan(end - start)
            # positions restart at 0 in every span (a span cut at max_seq_len continues a request: it is a new
            # sequence for the trunk, as in the reference's split)
            p = torch.cat([torch.arange(b - a, dtype=torch.int32) for a, b in rel]).to(dev, non_blocking=True)
            cu = torch.tensor([0] + [b for _, b in rel], dtype=torch.int32).to(dev, non_blocking=True)
            plan.set_batch(ids[start:end], p, cu)
            plan.replay()
            yield plan, start, end - start, rel
            i = j
        if not spans and n:
            return

    def forward_packed(self, input_ids: torch.Tensor, positions) -> torch.Tensor:
        """``input_ids`` ``(num_tokens,)`` packed sequences, ``positions`` their 0-based per-request positions (tensor or
        sequence); returns ``(num_tokens, hidden)`` bf16 final-norm hidden states."""
        n = int(input_ids.shape[0])
        out = torch.zeros(n, self.hidden_size, dtype=torch.bfloat16, device=self.weights.device)
        for plan, start, rows, _ in self._run_packed(input_ids, positions):
            out[start:start + rows].copy_(plan.hs[:rows])
        return out

    def forward_packed_padded(self, input_ids: torch.Tensor, positions) -> torch.Tensor:
        """The same result by the padded route: spans run as batched groups, each padded to its longest sequence."""
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
        rows = [plan.out[: len(rel)].clone() for plan, _, _, rel in self._run_packed(input_ids, positions)]
        if not rows:
            return torch.zeros(0, self.hidden_size, dtype=torch.float32, device=self.weights.device)
        return torch.cat(rows, dim=0)
