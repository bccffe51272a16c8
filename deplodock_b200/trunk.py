"""Recogniser for the traced Qwen3-shaped decoder trunk: Torch-IR graph in, fused launch plan out.

The reference serves a model by tracing the HF module behind ``build_full_model_wrapper``
(``emmy/compiler/trace/huggingface.py:17-186``) and handing the graph to ``Backend.compile``
(``emmy/serving/runner.py:75-167``). The traced layer is not made of the ops the kernels are named after: RMSNorm
arrives as ``pow -> MeanOp -> add eps -> rsqrt -> multiply -> multiply(weight)`` with broadcasts spelled as
``IndexMapOp`` nodes, RoPE as ``multiply(cos) + multiply(CatOp(negative(SliceOp), SliceOp), sin)``, grouped KV heads as
``UnsqueezeOp -> IndexMapOp -> ReshapeOp`` (``repeat_kv``), attention as ``SdpaOp`` with an additive ``causal_mask``
buffer, and SwiGLU as ``silu(LinearOp) * LinearOp``. The reference's pipeline fuses that by rewriting; here the graph is
matched, structurally and from the output backwards, against the one dataflow the hand-written plan implements:

    GatherOp -> [ rmsnorm -> q/k/v LinearOp -> per-head rmsnorm(q, k) -> RoPE(q, k) -> repeat_kv -> SdpaOp(causal)
                  -> o_proj LinearOp + residual -> rmsnorm -> silu(gate) * up -> down LinearOp + residual ] x L
             -> rmsnorm

A match yields the shape of the trunk and which graph constant plays which role; ``deplodock_b200.model.EmbedForward``
then runs it as five launches per layer. Every compute node of the graph must be claimed by the match — a graph that
contains anything else (another op, another wiring, other dtypes) is refused with :class:`TrunkMismatch`, which the
backend turns into ``LoweringError``. Both the reference tracer's records and the records of
``deplodock_b200.trace`` (which keeps casts as ``ToOp`` and does not spell broadcasts out) are accepted.
"""

from __future__ import annotations

from dataclasses import dataclass, field

from deplodock_b200.graph import Graph, Node

_CASTS = {"ToOp", "ContiguousOp", "CloneOp", "TypeAsOp", "DetachOp", "AliasOp"}
_VIEWS = {"ReshapeOp", "ViewOp", "UnsqueezeOp", "SqueezeOp", "FlattenOp"}


class TrunkMismatch(ValueError):
    """The graph is not the decoder trunk the fused plan implements; the message says where the match stopped."""


@dataclass
class LayerRoles:
    """Graph constant ids of one decoder layer."""

    ln1: str
    wq: str
    wk: str
    wv: str
    qn: str
    kn: str
    wo: str
    ln2: str
    wgate: str
    wup: str
    wdown: str


@dataclass
class TrunkMatch:
    ids: str                      # the int64 token-id graph input
    output: str                   # the final-norm hidden states [B, S, hidden]
    embed: str
    final_norm: str
    cos: str
    sin: str
    mask: str | None              # additive causal-mask constant (implied by the kernel, never read), if any
    layers: list[LayerRoles]
    batch: int
    seq: int
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    claimed: set[str] = field(default_factory=set)

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    def state_dict_names(self) -> dict[str, str]:
        """HF ``Qwen3Model`` parameter name -> graph constant id (the naming ``EmbedWeights`` reads)."""
        names = {"embed_tokens.weight": self.embed, "norm.weight": self.final_norm}
        for i, lr in enumerate(self.layers):
            p = f"layers.{i}."
            names.update({
                p + "input_layernorm.weight": lr.ln1, p + "self_attn.q_proj.weight": lr.wq,
                p + "self_attn.k_proj.weight": lr.wk, p + "self_attn.v_proj.weight": lr.wv,
                p + "self_attn.q_norm.weight": lr.qn, p + "self_attn.k_norm.weight": lr.kn,
                p + "self_attn.o_proj.weight": lr.wo, p + "post_attention_layernorm.weight": lr.ln2,
                p + "mlp.gate_proj.weight": lr.wgate, p + "mlp.up_proj.weight": lr.wup,
                p + "mlp.down_proj.weight": lr.wdown})
        return names


class _Matcher:
    def __init__(self, g: Graph) -> None:
        self.g = g
        self.claimed: set[str] = set()

    # -- primitives --------------------------------------------------------------------------------------------
    def node(self, nid: str) -> Node:
        return self.g.nodes[nid]

    def claim(self, *nids: str) -> None:
        self.claimed.update(nids)

    def fail(self, nid: str, what: str):
        n = self.g.nodes.get(nid)
        desc = f"{nid} ({n.op} {n.op_fields.get('op', '')} {list(n.output.shape)} {n.output.dtype})" if n else nid
        raise TrunkMismatch(f"expected {what} at {desc}")

    def through_casts(self, nid: str) -> str:
        """Follow dtype casts / copies (the reference's tracer drops them, this package's keeps them as ToOp)."""
        while self.node(nid).op in _CASTS:
            self.claim(nid)
            nid = self.node(nid).inputs[0]
        return nid

    def through_broadcast(self, nid: str) -> str:
        """Follow casts, broadcasts spelled as IndexMapOp, and the views in front of a broadcast constant."""
        while True:
            n = self.node(nid)
            if n.op in _CASTS or n.op == "IndexMapOp" or (n.op in _VIEWS and self._leads_to_constant(nid)):
                self.claim(nid)
                nid = n.inputs[0]
                continue
            return nid

    def _leads_to_constant(self, nid: str) -> bool:
        n = self.node(nid)
        while n.op in _CASTS or n.op in _VIEWS or n.op == "IndexMapOp":
            n = self.node(n.inputs[0])
        return n.op == "ConstantOp"

    def elementwise(self, nid: str, name: str, what: str) -> list[str]:
        nid = self.through_casts(nid)
        n = self.node(nid)
        if n.op != "ElementwiseOp" or n.op_fields.get("op") != name:
            self.fail(nid, what)
        self.claim(nid)
        return [i for i in n.inputs]

    def is_elementwise(self, nid: str, name: str) -> bool:
        n = self.node(self.through_casts(nid))
        return n.op == "ElementwiseOp" and n.op_fields.get("op") == name

    def scalar_const(self, nid: str, what: str) -> float:
        src = self.through_broadcast(nid)
        n = self.node(src)
        if n.op != "ConstantOp" or n.op_fields.get("value") is None:
            self.fail(src, what)
        self.claim(src)
        return float(n.op_fields["value"])

    def weight_const(self, nid: str, what: str, shape: tuple[int, ...] | None = None) -> str:
        src = self.through_broadcast(nid)
        n = self.node(src)
        if n.op != "ConstantOp" or n.op_fields.get("value") is not None:
            self.fail(src, what)
        if shape is not None and tuple(n.output.shape) != tuple(shape):
            self.fail(src, f"{what} of shape {list(shape)}")
        self.claim(src)
        return src

    def same_value(self, a: str, b: str) -> bool:
        return self.through_casts(a) == self.through_casts(b)

    def view_chain(self, nid: str, allowed: set[str]) -> str:
        """Follow casts and the named view ops; returns the first node that is neither."""
        while True:
            nid = self.through_casts(nid)
            n = self.node(nid)
            if n.op in allowed:
                self.claim(nid)
                # the reference records the arguments of transpose / unsqueeze / slice as extra scalar constants
                nid = n.inputs[0]
                continue
            return nid

    def claim_arg_constants(self) -> None:
        """Scalar ConstantOps the reference's tracer records for ``dim`` / ``start`` / ``end`` arguments: they feed no
        arithmetic (some are not even wired to a node); claim those that only views, slices and cats read."""
        readers: dict[str, list[Node]] = {}
        for n in self.g.nodes.values():
            for i in n.inputs:
                readers.setdefault(i, []).append(n)
        for nid, n in self.g.nodes.items():
            if n.op == "ConstantOp" and n.op_fields.get("value") is not None:
                if all(r.op in ("SliceOp", "CatOp", "TransposeOp", "UnsqueezeOp") for r in readers.get(nid, [])):
                    self.claim(nid)

    # -- patterns ----------------------------------------------------------------------------------------------
    def rmsnorm(self, nid: str, what: str) -> tuple[str, str, float]:
        """``weight * (x * rsqrt(mean(x^2, -1) + eps))`` -> (x, weight constant, eps)."""
        a, b = self.elementwise(nid, "multiply", f"the weight multiply of {what}")
        if self.node(self.through_broadcast(a)).op != "ConstantOp":
            a, b = b, a
        n_out = self.node(self.through_casts(nid))
        w = self.weight_const(a, f"the weight of {what}", (n_out.output.shape[-1],))
        x, rs = self.elementwise(b, "multiply", f"x * rsqrt(...) of {what}")
        if not self.is_elementwise(self.through_broadcast(rs), "rsqrt"):
            x, rs = rs, x
        (var_eps,) = self.elementwise(self.through_broadcast(rs), "rsqrt", f"rsqrt of {what}")
        m, e = self.elementwise(var_eps, "add", f"mean + eps of {what}")
        if self.node(self.through_casts(m)).op != "MeanOp":
            m, e = e, m
        eps = self.scalar_const(e, f"eps of {what}")
        mean = self.node(self.through_casts(m))
        if mean.op != "MeanOp" or mean.op_fields.get("axis", -1) not in (-1, len(mean.output.shape) - 1):
            self.fail(mean.id, f"mean over the last axis of {what}")
        self.claim(mean.id)
        px, pe = self.elementwise(mean.inputs[0], "pow", f"x^2 of {what}")
        if self.scalar_const(pe, f"exponent of {what}") != 2.0:
            self.fail(pe, "exponent 2")
        if not self.same_value(px, x):
            self.fail(px, f"the normalised operand of {what} ({self.through_casts(x)})")
        return self.through_casts(x), w, eps

    def rope(self, nid: str, what: str) -> tuple[str, str, str]:
        """``t * cos + cat(-t[..., D/2:], t[..., :D/2]) * sin`` -> (t, cos constant, sin constant)."""
        a, b = self.elementwise(nid, "add", f"the sum of {what}")
        ta, ca = self.elementwise(a, "multiply", f"t * cos of {what}")
        tb, cb = self.elementwise(b, "multiply", f"rotate_half(t) * sin of {what}")
        if self.node(self.through_casts(ta)).op == "CatOp":   # the rotated branch came first
            (ta, ca), (tb, cb) = (tb, cb), (ta, ca)
        cat = self.node(self.through_casts(tb))
        if cat.op != "CatOp":
            self.fail(cat.id, f"the rotate_half concatenation of {what}")
        self.claim(cat.id)
        parts = [i for i in cat.inputs if self.node(i).op != "ConstantOp" or self.node(i).op_fields.get("value") is None]
        if len(parts) != 2:
            self.fail(cat.id, "a concatenation of two halves")
        (hi_neg,) = self.elementwise(parts[0], "negative", f"-t[..., D/2:] of {what}")
        hi = self.node(self.through_casts(hi_neg))
        lo = self.node(self.through_casts(parts[1]))
        t = self.through_casts(ta)
        D = self.node(t).output.shape[-1]
        for sl, start in ((hi, D // 2), (lo, 0)):
            if sl.op != "SliceOp" or int(sl.op_fields.get("start", -1)) != start or sl.output.shape[-1] != D // 2 \
                    or sl.op_fields.get("dim", -1) not in (-1, len(sl.output.shape) - 1):
                self.fail(sl.id, f"a half-width slice starting at {start} of {what}")
            if not self.same_value(sl.inputs[0], t):
                self.fail(sl.id, f"a slice of {t}")
            self.claim(sl.id)
        cos = self.weight_const(ca, f"cos table of {what}")
        sin = self.weight_const(cb, f"sin table of {what}")
        return t, cos, sin

    def repeat_kv(self, nid: str, heads: int) -> str:
        """``unsqueeze(2) -> broadcast x g -> reshape [B, Hkv*g, S, D]`` (or nothing when g == 1) -> the KV tensor."""
        nid = self.through_casts(nid)
        n = self.node(nid)
        if n.op in ("ReshapeOp", "ViewOp") and n.output.shape[1] == heads:
            b = self.node(self.through_casts(n.inputs[0]))
            if b.op == "IndexMapOp" and len(b.output.shape) == 5:
                u = self.node(self.through_casts(b.inputs[0]))
                if u.op in ("UnsqueezeOp", "ReshapeOp") and len(u.output.shape) == 5 and u.output.shape[2] == 1:
                    self.claim(n.id, b.id, u.id)
                    return self.through_casts(u.inputs[0])
        return nid

    def linear(self, nid: str, what: str) -> tuple[str, str]:
        nid = self.through_casts(nid)
        n = self.node(nid)
        if n.op != "LinearOp" or n.op_fields.get("has_bias"):
            self.fail(nid, f"the bias-free LinearOp of {what}")
        self.claim(nid)
        return n.inputs[0], self.weight_const(n.inputs[1], f"the weight of {what}")

    def head_split(self, nid: str, what: str) -> str:
        """``transpose(1, 2)`` of a ``[B, S, H, D]`` view -> the node under the transpose (still 4-D)."""
        nid = self.through_casts(nid)
        n = self.node(nid)
        if n.op != "TransposeOp" or sorted(int(a) % 4 for a in n.op_fields.get("axes", [])) != [1, 2]:
            self.fail(nid, f"transpose(1, 2) of {what}")
        self.claim(nid)
        return self.through_casts(n.inputs[0])

    def flat_view(self, nid: str, what: str) -> str:
        nid = self.through_casts(nid)
        n = self.node(nid)
        if n.op not in ("ReshapeOp", "ViewOp"):
            self.fail(nid, f"the view of {what}")
        self.claim(nid)
        return self.through_casts(n.inputs[0])


def recognise_trunk(g: Graph) -> TrunkMatch:
    """Match ``g`` against the decoder trunk (see the module docstring); raises :class:`TrunkMismatch`."""
    if len(g.outputs) != 1 or len(g.inputs) != 1:
        raise TrunkMismatch("the trunk has one graph input (token ids) and one output (hidden states)")
    m = _Matcher(g)
    out = g.outputs[0]
    out_info = g.nodes[out].output
    if out_info.dtype != "bf16" or len(out_info.shape) != 3:
        raise TrunkMismatch(f"the fused plan computes in bf16 on [B, S, hidden]; the graph output is "
                            f"{list(out_info.shape)} {out_info.dtype}")
    B, S, H = out_info.shape
    h, final_norm, eps = m.rmsnorm(out, "the final norm")
    layers: list[LayerRoles] = []
    cos = sin = mask = None
    nq = nkv = D = inter = None
    while m.node(h).op != "GatherOp":
        # h = h_mid + down(silu(gate(x2)) * up(x2)),  x2 = rmsnorm(h_mid)
        a, b = m.elementwise(h, "add", "the MLP residual add")
        if m.node(m.through_casts(a)).op == "LinearOp":
            a, b = b, a
        h_mid = m.through_casts(a)
        mlp, wdown = m.linear(b, "down_proj")
        ga, up = m.elementwise(mlp, "multiply", "silu(gate) * up")
        if not m.is_elementwise(ga, "silu"):
            ga, up = up, ga
        (gate,) = m.elementwise(ga, "silu", "silu(gate)")
        x2g, wgate = m.linear(gate, "gate_proj")
        x2u, wup = m.linear(up, "up_proj")
        if not m.same_value(x2g, x2u):
            m.fail(x2u, "gate_proj and up_proj reading the same normalised activations")
        hx, ln2, e2 = m.rmsnorm(x2g, "the post-attention norm")
        if hx != h_mid:
            m.fail(hx, f"the post-attention norm of {h_mid}")
        # h_mid = h_prev + o_proj(flatten(transpose(sdpa(q, k, v))))
        a, b = m.elementwise(h_mid, "add", "the attention residual add")
        if m.node(m.through_casts(a)).op == "LinearOp":
            a, b = b, a
        h_prev = m.through_casts(a)
        attn_flat, wo = m.linear(b, "o_proj")
        sd = m.node(m.head_split(m.flat_view(attn_flat, "the attention output"), "the attention output"))
        if sd.op != "SdpaOp":
            m.fail(sd.id, "SdpaOp")
        m.claim(sd.id)
        if len(sd.inputs) > 3:
            mk = m.node(m.through_broadcast(sd.inputs[3]))
            if mk.op != "ConstantOp" or "causal_mask" not in str(mk.op_fields.get("source_path") or mk.id):
                m.fail(mk.id, "the additive causal-mask buffer (a general mask has no kernel)")
            m.claim(mk.id)
            mask = mk.id
        elif not sd.op_fields.get("is_causal"):
            m.fail(sd.id, "causal attention")
        _, hq, s_, d_ = sd.output.shape
        # q = rope(transpose(rmsnorm(view(q_proj(x1)))))
        tq, cq, sq = m.rope(sd.inputs[0], "RoPE of q")
        xq, qn, eq = m.rmsnorm(m.head_split(tq, "q"), "q_norm")
        x1q, wq = m.linear(m.flat_view(xq, "q heads"), "q_proj")
        # k = repeat_kv(rope(transpose(rmsnorm(view(k_proj(x1))))))
        kt = m.repeat_kv(sd.inputs[1], hq)
        tk, ck, sk = m.rope(kt, "RoPE of k")
        hkv = m.node(tk).output.shape[1]
        xk, kn, ek = m.rmsnorm(m.head_split(tk, "k"), "k_norm")
        x1k, wk = m.linear(m.flat_view(xk, "k heads"), "k_proj")
        # v = repeat_kv(transpose(view(v_proj(x1))))
        vt = m.repeat_kv(sd.inputs[2], hq)
        x1v, wv = m.linear(m.flat_view(m.head_split(vt, "v"), "v heads"), "v_proj")
        if not (m.same_value(x1q, x1k) and m.same_value(x1q, x1v)):
            m.fail(x1k, "q/k/v projections reading the same normalised activations")
        hx, ln1, e1 = m.rmsnorm(x1q, "the input norm")
        if hx != h_prev:
            m.fail(hx, f"the input norm of {h_prev}")
        if (cq, sq) != (ck, sk) or (cos is not None and (cos, sin) != (cq, sq)):
            m.fail(cq, "one pair of rotary tables shared by q, k and all layers")
        cos, sin = cq, sq
        if len({eps, e1, e2, eq, ek}) != 1:
            m.fail(out, f"one RMSNorm eps throughout (found {sorted({eps, e1, e2, eq, ek})})")
        shape = (hq, hkv, d_, g.nodes[wgate].output.shape[0])
        if nq is None:
            nq, nkv, D, inter = shape
        elif shape != (nq, nkv, D, inter):
            m.fail(sd.id, "the same head counts and widths in every layer")
        if s_ != S or d_ != 128 or hq % hkv != 0:
            m.fail(sd.id, "head_dim 128, Hq a multiple of Hkv, and the graph's sequence length")
        for wid, want in ((wq, (nq * D, H)), (wk, (nkv * D, H)), (wv, (nkv * D, H)), (wo, (H, nq * D)),
                          (wgate, (inter, H)), (wup, (inter, H)), (wdown, (H, inter))):
            if tuple(g.nodes[wid].output.shape) != want:
                m.fail(wid, f"a projection weight of shape {list(want)}")
        layers.append(LayerRoles(ln1, wq, wk, wv, qn, kn, wo, ln2, wgate, wup, wdown))
        h = h_prev
    if not layers:
        raise TrunkMismatch("no decoder layer between the embedding gather and the final norm")
    layers.reverse()
    gather = m.node(h)
    m.claim(gather.id)
    embed = m.weight_const(gather.inputs[0], "the embedding table")
    ids = m.through_casts(gather.inputs[1])
    if ids not in g.inputs or g.nodes[ids].output.dtype != "i64" or tuple(g.nodes[ids].output.shape) != (B, S):
        m.fail(ids, f"the int64 token-id input of shape {[B, S]}")
    m.claim(ids)
    vocab, He = g.nodes[embed].output.shape
    if He != H or H % 128 != 0:
        m.fail(embed, f"an embedding table of width {H} (a multiple of 128)")
    for t in (cos, sin):
        if g.nodes[t].output.shape[-2:] != (S, D):
            m.fail(t, f"a rotary table ending in {[S, D]}")
    m.claim_arg_constants()
    # position ids and other buffers no arithmetic node reads stay unclaimed without harm; compute nodes must not
    stray = [n.id for n in g.compute_nodes() if n.id not in m.claimed]
    if stray:
        raise TrunkMismatch(f"{len(stray)} nodes are not part of the decoder-trunk dataflow, e.g. "
                            + ", ".join(f"{s} ({g.nodes[s].op})" for s in stray[:4]))
    return TrunkMatch(ids=ids, output=out, embed=embed, final_norm=final_norm, cos=cos, sin=sin, mask=mask,
                      layers=layers, batch=B, seq=S, vocab_size=vocab, hidden_size=H, intermediate_size=inter,
                      num_attention_heads=nq, num_key_value_heads=nkv, head_dim=D, rms_norm_eps=eps,
                      claimed=m.claimed)


def looks_like_trunk(g: Graph) -> bool:
    """Cheap test used by the dispatcher: an embedding gather and attention in one graph."""
    ops = {n.op for n in g.nodes.values()}
    return "GatherOp" in ops and "SdpaOp" in ops
