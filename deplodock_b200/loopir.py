"""Loop-IR kernel records (``kernels/*.json`` of the reference) -> hand-written kernels.

The records the reference ships are Loop-IR sub-graphs: one ``LoopOp`` node whose ``op_fields.body`` is a list of
``repr`` strings of frozen dataclasses (``emmy/compiler/graph.py:143-247``) — ``Loop(axis=Axis(name, extent), body)``,
``Load(name, input, index)``, ``Assign(name, op=ElementwiseImpl(..), args)``, ``Accum(name, value, op)``,
``Write(output, index, value)``, ``Select`` / ``SelectBranch``, and index expressions ``Var`` / ``Literal`` /
``BinaryExpr`` with ``/`` as integer division (``emmy/compiler/ir/stmt/leaves.py:96-469``, ``emmy/compiler/ir/expr.py``).
The reference re-``eval``s those strings and lowers the loop nest to generated CUDA; here the nest is *recognised*:
``classify`` parses the body into a small tree, reads off its reduction structure and operand addressing, and names one
of the kernel families below with the parameters the kernel needs. Index expressions are not pattern-matched
textually: they are evaluated numerically over the whole iteration space (numpy), and the resulting offsets are
checked against the addressing the kernel implements, so an unexpected layout is refused instead of mis-read.

    rmsnorm            y = w * (x * rsqrt(sum(x^2) / count + eps))                      -> emk_rmsnorm
    linear             y[m,n] = sum_k x[m,k] * W[n,k]                                   -> emk_loop_linear_f32
    linear_residual    ... + r[m,n]  (x possibly read through a [K/D, M, D] permutation) -> emk_loop_linear_f32
    silu_gate_linear   y[m,n] = silu(g[m,n]) * sum_k x[m,k] * W[n,k]                    -> emk_loop_linear_f32
    rope_scores        s[h,i,j] = scale * sum_d rope(q)[i,h,d] * rope(k)[j,h/g,d] + (j <= i ? zero : fill)
                                                                                        -> emk_loop_rope_scores_f32
    softmax_pv         o[h,i,d] = sum_j softmax_j(s[h,i,:]) * v[j,h/g,d]                -> emk_loop_softmax_pv_f32

``interpret_point`` executes a body literally (scalar Python) for fixed outer loop indices; ``verify`` uses it to check
a classification on a few random output points against ``reference_formula`` — the numpy statement of what the chosen
kernel computes — so a nest that merely looks like a family is refused.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import numpy as np


# ------------------------------------------------------------------------------------------------------------
# parsing: the repr strings are evaluated against stand-in classes that only record their arguments
# ------------------------------------------------------------------------------------------------------------
class _Node:
    _fields: tuple[str, ...] = ()

    def __init__(self, *args, **kw):
        for name, val in zip(self._fields, args):
            setattr(self, name, val)
        for name, val in kw.items():
            setattr(self, name, val)

    def __repr__(self):
        return f"{type(self).__name__}({', '.join(f'{k}={v!r}' for k, v in self.__dict__.items())})"


def _cls(name: str, fields: tuple[str, ...]):
    return type(name, (_Node,), {"_fields": fields})


Axis = _cls("Axis", ("name", "extent"))
Loop = _cls("Loop", ("axis", "body"))
Load = _cls("Load", ("name", "input", "index"))
Assign = _cls("Assign", ("name", "op", "args"))
Accum = _cls("Accum", ("name", "value", "op"))
Write = _cls("Write", ("output", "index", "value"))
Select = _cls("Select", ("name", "branches"))
SelectBranch = _cls("SelectBranch", ("value", "select"))
Cond = _cls("Cond", ("cond", "body"))
Var = _cls("Var", ("name",))
Literal = _cls("Literal", ("value", "dtype"))
BinaryExpr = _cls("BinaryExpr", ("op", "left", "right"))


class ElementwiseImpl(str):
    def __new__(cls, name):
        return super().__new__(cls, name)


_NAMESPACE = {c.__name__: c for c in (Axis, Loop, Load, Assign, Accum, Write, Select, SelectBranch, Cond, Var, Literal,
                                      BinaryExpr)}
_NAMESPACE["ElementwiseImpl"] = ElementwiseImpl


def parse_body(body: list[str]) -> list[_Node]:
    """Statements of a ``LoopOp`` body. The strings come from a record file: they are evaluated with no builtins and
    only the stand-in classes in scope."""
    return [eval(stmt, {"__builtins__": {}}, dict(_NAMESPACE)) for stmt in body]  # noqa: S307


def eval_index(expr, env: dict[str, np.ndarray]):
    """Numeric value of an index expression for (broadcastable) arrays of axis values."""
    if isinstance(expr, Var):
        return env[expr.name]
    if isinstance(expr, Literal):
        return np.int64(expr.value)
    if isinstance(expr, BinaryExpr):
        a, b = eval_index(expr.left, env), eval_index(expr.right, env)
        op = expr.op
        if op == "+":
            return a + b
        if op == "-":
            return a - b
        if op == "*":
            return a * b
        if op == "/":
            return a // b
        if op == "%":
            return a % b
        if op == "<":
            return a < b
        if op == "<=":
            return a <= b
        if op == ">":
            return a > b
        if op == ">=":
            return a >= b
        if op == "==":
            return a == b
        raise ValueError(f"index operator {op!r} is not understood")
    raise ValueError(f"index expression {expr!r} is not understood")


# ------------------------------------------------------------------------------------------------------------
# classification
# ------------------------------------------------------------------------------------------------------------
@dataclass
class LoopMatch:
    kind: str                       # see the module docstring
    output: str
    out_shape: tuple[int, ...]
    params: dict[str, Any] = field(default_factory=dict)


class LoopRecordError(ValueError):
    """The loop nest is not one of the recognised families (or reads its operands in a layout no kernel implements)."""


def _walk(stmts, loops, acc):
    """Flatten the nest: ``acc`` gets (statement, tuple of enclosing Loop axes)."""
    for s in stmts:
        if isinstance(s, Loop):
            _walk(s.body, loops + (s.axis,), acc)
        else:
            acc.append((s, loops))


def _flat_offset(shape, index, env):
    strides = np.cumprod((1,) + tuple(reversed(shape[1:])))[::-1]
    off = 0
    for stride, e in zip(strides, index):
        off = off + np.int64(stride) * eval_index(e, env)
    return off


def classify(graph, node_id: str) -> LoopMatch:
    """``graph``: a :class:`deplodock_b200.graph.Graph`; ``node_id``: its ``LoopOp`` node."""
    node = graph.nodes[node_id]
    stmts = parse_body(list(node.op_fields["body"]))
    flat: list[tuple[_Node, tuple]] = []
    _walk(stmts, (), flat)
    loads = {s.name: (s, lp) for s, lp in flat if isinstance(s, Load)}
    assigns = {s.name: s for s, _ in flat if isinstance(s, Assign)}
    accums = [(s, lp) for s, lp in flat if isinstance(s, Accum)]
    writes = [(s, lp) for s, lp in flat if isinstance(s, Write)]
    selects = [s for s, _ in flat if isinstance(s, Select)]
    if len(writes) != 1:
        raise LoopRecordError(f"{node_id}: expected one Write, found {len(writes)}")
    write, write_loops = writes[0]
    out_shape = tuple(node.output.shape)
    shape_of = lambda buf: tuple(graph.nodes[buf].output.shape)  # noqa: E731
    const_value = lambda buf: graph.nodes[buf].op_fields.get("value")  # noqa: E731

    def scalar_const(name):
        ld = loads.get(name)
        if ld is None:
            return None
        v = const_value(ld[0].input)
        return None if v in (None, "None") else float(v)

    acc_ops = [str(a.op) for a, _ in accums]
    assign_ops = sorted(str(a.op) for a in assigns.values())

    # -- attention halves of the reference's unfused lowering: recognised by structure, no kernel ---------------
    if selects and len(accums) == 1 and len(out_shape) == 4 and out_shape[-1] == out_shape[-2]:
        H, S = int(out_shape[1]), int(out_shape[2])
        D = int(accums[0][1][-1].extent)
        bufs = [s.input for s, lp in loads.values() if lp]          # loads inside the nest, in order of appearance
        proj = [b for b in dict.fromkeys(bufs) if len(shape_of(b)) == 4]
        tabs = [b for b in dict.fromkeys(bufs) if len(shape_of(b)) == 3]
        consts = {n: scalar_const(n) for n, (s, lp) in loads.items() if not lp}
        if len(proj) != 2 or len(tabs) != 2 or len(consts) != 3:
            raise LoopRecordError(f"{node_id}: attention-score nest with unexpected operands {proj} {tabs}")
        q_buf = next(b for b in proj if shape_of(b)[-1] == H * D)
        k_buf = next(b for b in proj if b != q_buf)
        # which table multiplies the rotated half: sin; the other: cos (decided by verify() on the numbers)
        post_mul = next(a for a in assigns.values() if str(a.op) == "multiply" and accums[0][0].name in a.args)
        scale = scalar_const(next(a for a in post_mul.args if a != accums[0][0].name))
        mask_sel = next(sel for sel in selects if all(b.value in consts for b in sel.branches))
        zero, fill = (scalar_const(b.value) for b in mask_sel.branches)
        return LoopMatch("rope_scores", write.output, out_shape,
                         {"q": q_buf, "k": k_buf, "tables": tabs, "S": S, "H": H, "Hkv": shape_of(k_buf)[-1] // D, "D": D,
                          "scale": scale, "mask_zero": zero, "mask_fill": fill})
    if acc_ops == ["maximum", "add", "add"] and "exp" in assign_ops:
        H, S, D = int(out_shape[1]), int(out_shape[2]), int(out_shape[-1])
        bufs = list(dict.fromkeys(s.input for s, lp in loads.values() if lp))
        sc_buf = next(b for b in bufs if shape_of(b)[-2:] == (S, S))
        v_buf = next(b for b in bufs if b != sc_buf)
        return LoopMatch("softmax_pv", write.output, out_shape,
                         {"scores": sc_buf, "v": v_buf, "S": S, "H": H, "Hkv": shape_of(v_buf)[-1] // D, "D": D})

    # -- RMSNorm -------------------------------------------------------------------------------------------------
    if acc_ops == ["add"] and "rsqrt" in assign_ops:
        acc, acc_loops = accums[0]
        sq = assigns.get(acc.value)
        if sq is None or str(sq.op) != "multiply" or len(set(loads[a][0].input for a in sq.args)) != 1:
            raise LoopRecordError(f"{node_id}: rsqrt nest whose reduction is not a sum of squares")
        x_buf = loads[sq.args[0]][0].input
        cols = int(acc_loops[-1].extent)
        div = next(a for a in assigns.values() if str(a.op) == "divide")
        add = next(a for a in assigns.values() if str(a.op) == "add")
        count = next((scalar_const(n) for n in div.args if scalar_const(n) is not None), None)
        eps = next((scalar_const(n) for n in add.args if scalar_const(n) is not None), None)
        weight = next((s.input for s, _ in loads.values() if len(shape_of(s.input)) == 1 and shape_of(s.input)[0] == cols
                       and graph.nodes[s.input].op == "ConstantOp"), None)
        if count != float(cols) or eps is None or weight is None or shape_of(x_buf)[-1] != cols:
            raise LoopRecordError(f"{node_id}: RMSNorm nest with unexpected constants (count={count}, eps={eps})")
        return LoopMatch("rmsnorm", write.output, out_shape, {"x": x_buf, "weight": weight, "eps": eps, "cols": cols})

    # -- linear family -------------------------------------------------------------------------------------------
    if acc_ops == ["add"]:
        acc, acc_loops = accums[0]
        prod = assigns.get(acc.value)
        if prod is None or str(prod.op) != "multiply" or len(prod.args) != 2:
            raise LoopRecordError(f"{node_id}: reduction is not a sum of products")
        (la, _), (lb, _) = loads[prod.args[0]], loads[prod.args[1]]
        w_ld, x_ld = (la, lb) if graph.nodes[la.input].op == "ConstantOp" and len(shape_of(la.input)) == 2 else (lb, la)
        if graph.nodes[w_ld.input].op != "ConstantOp" or len(shape_of(w_ld.input)) != 2:
            raise LoopRecordError(f"{node_id}: no 2-D weight operand in the contraction")
        axes = {ax.name: int(ax.extent) for ax in acc_loops}
        k_ax = acc_loops[-1].name
        # W[n, k]: which axes index its two dimensions
        w_idx = w_ld.index
        if not (isinstance(w_idx[0], Var) and isinstance(w_idx[1], Var) and w_idx[1].name == k_ax):
            raise LoopRecordError(f"{node_id}: weight is not read as W[n, k]")
        n_ax = w_idx[0].name
        m_axes = [ax.name for ax in acc_loops if ax.name not in (n_ax, k_ax)]
        if len(m_axes) != 1:
            raise LoopRecordError(f"{node_id}: expected one row axis, found {m_axes}")
        m_ax = m_axes[0]
        M, N, K = axes[m_ax], axes[n_ax], axes[k_ax]
        if shape_of(w_ld.input) != (N, K):
            raise LoopRecordError(f"{node_id}: weight shape {shape_of(w_ld.input)} does not match [{N}, {K}]")
        grid = {m_ax: np.arange(M, dtype=np.int64)[:, None], k_ax: np.arange(K, dtype=np.int64)[None, :],
                n_ax: np.int64(0)}
        x_off = np.broadcast_to(_flat_offset(shape_of(x_ld.input), x_ld.index, grid), (M, K))
        x_inner, x_so, x_sm = _blocked_layout(x_off, M, K)
        if x_inner is None:
            raise LoopRecordError(f"{node_id}: activation operand {x_ld.input} is read in a layout no kernel implements")
        # the output and any [M, N] epilogue operand must be plain row-major
        mn = {m_ax: np.arange(M, dtype=np.int64)[:, None], n_ax: np.arange(N, dtype=np.int64)[None, :], k_ax: np.int64(0)}
        plain = np.arange(M, dtype=np.int64)[:, None] * N + np.arange(N, dtype=np.int64)[None, :]
        if not np.array_equal(np.broadcast_to(_flat_offset(out_shape, write.index, mn), (M, N)), plain):
            raise LoopRecordError(f"{node_id}: output is not written as a row-major [M, N] matrix")
        params = {"x": x_ld.input, "w": w_ld.input, "M": M, "N": N, "K": K, "x_inner": x_inner, "x_stride_outer": x_so,
                  "x_stride_m": x_sm, "residual": None, "gate": None}
        post = assigns.get(write.value) if write.value != acc.name else None
        kind = "linear"
        if post is not None:
            other = [a for a in post.args if a != acc.name]
            if str(post.op) == "add" and len(other) == 1 and other[0] in loads:
                kind, key, ld = "linear_residual", "residual", loads[other[0]][0]
            elif str(post.op) == "multiply" and len(other) == 1 and _is_silu_of_load(other[0], assigns, loads, scalar_const):
                kind, key, ld = "silu_gate_linear", "gate", _is_silu_of_load(other[0], assigns, loads, scalar_const)
            else:
                raise LoopRecordError(f"{node_id}: epilogue {post.op}({post.args}) after the contraction is not understood")
            if not np.array_equal(np.broadcast_to(_flat_offset(shape_of(ld.input), ld.index, mn), (M, N)), plain):
                raise LoopRecordError(f"{node_id}: epilogue operand {ld.input} is not a row-major [M, N] matrix")
            params[key] = ld.input
        return LoopMatch(kind, write.output, out_shape, params)

    raise LoopRecordError(f"{node_id}: loop nest with reductions {acc_ops} and ops {assign_ops} matches no kernel family")


def _blocked_layout(off: np.ndarray, M: int, K: int):
    """Solve ``off[m, k] == (k // D) * so + m * sm + k % D`` for (D, so, sm); plain row-major is (K, 0, K)."""
    row0 = off[0]
    breaks = np.nonzero(np.diff(row0) != 1)[0]
    D = int(breaks[0]) + 1 if len(breaks) else K
    if K % D != 0:
        return None, None, None
    so = int(row0[D] - row0[0]) if D < K else 0
    sm = int(off[1, 0] - off[0, 0]) if M > 1 else K
    k = np.arange(K, dtype=np.int64)[None, :]
    m = np.arange(M, dtype=np.int64)[:, None]
    want = (k // D) * so + m * sm + k % D + int(off[0, 0])
    if int(off[0, 0]) != 0 or not np.array_equal(off, want):
        return None, None, None
    return D, so, sm


def _is_silu_of_load(name, assigns, loads, scalar_const):
    """``name`` = x * reciprocal(1 + exp(-x)) for a loaded x (``020_silu.py:11-36`` of the reference's decomposition);
    returns that Load or None."""
    mul = assigns.get(name)
    if mul is None or str(mul.op) != "multiply" or len(mul.args) != 2:
        return None
    for x_name, r_name in (mul.args, mul.args[::-1]):
        rec = assigns.get(r_name)
        if x_name not in loads or rec is None or str(rec.op) != "reciprocal":
            continue
        add = assigns.get(rec.args[0])
        if add is None or str(add.op) != "add":
            continue
        one = [a for a in add.args if scalar_const(a) == 1.0]
        ex = [assigns.get(a) for a in add.args if a in assigns]
        if not one or not ex or str(ex[0].op) != "exp":
            continue
        neg = assigns.get(ex[0].args[0])
        if neg is None or str(neg.op) != "negative" or neg.args[0] not in loads:
            continue
        if loads[neg.args[0]][0].input == loads[x_name][0].input:
            return loads[x_name][0]
    return None


# ------------------------------------------------------------------------------------------------------------
# literal execution of a body at chosen points, and verification of a classification against it
# ------------------------------------------------------------------------------------------------------------
_IDENTITY = {"add": 0.0, "maximum": -np.inf, "multiply": 1.0, "minimum": np.inf}
_UNARY = {"negative": lambda a: -a, "exp": lambda a: np.exp(np.float32(a)), "reciprocal": lambda a: np.float32(1.0) / a,
          "rsqrt": lambda a: np.float32(1.0) / np.sqrt(np.float32(a))}
_BINARY = {"multiply": lambda a, b: a * b, "add": lambda a, b: a + b, "subtract": lambda a, b: a - b,
           "divide": lambda a, b: a / b, "maximum": max, "minimum": min}


def interpret_point(stmts, inputs: dict[str, np.ndarray], fixed: dict[str, int]) -> list[tuple[tuple[int, ...], float]]:
    """Execute the body in fp32 with the loop axes named in ``fixed`` pinned to one value and every other loop run in
    full; returns the (index, value) pairs it writes. Loads whose index falls outside the buffer (the unselected side
    of a rotate-half ``Select``) read 0."""
    env: dict[str, Any] = {}
    axes: dict[str, np.int64] = {}
    writes: list[tuple[tuple[int, ...], float]] = []

    def load(s):
        buf = inputs[s.input]
        idx = tuple(int(eval_index(e, axes)) for e in s.index)
        if any(i < 0 or i >= n for i, n in zip(idx, buf.shape)):
            return np.float32(0.0)
        return np.float32(buf[idx])

    def run(block):
        for s in block:
            if isinstance(s, Loop):
                for inner in s.body:
                    if isinstance(inner, Accum):
                        env[inner.name] = np.float32(_IDENTITY[str(inner.op)])
                rng = [fixed[s.axis.name]] if s.axis.name in fixed else range(int(s.axis.extent))
                for v in rng:
                    axes[s.axis.name] = np.int64(v)
                    run(s.body)
            elif isinstance(s, Load):
                env[s.name] = load(s)
            elif isinstance(s, Assign):
                a = [env[n] for n in s.args]
                op = str(s.op)
                env[s.name] = np.float32(_UNARY[op](*a) if op in _UNARY else _BINARY[op](*a))
            elif isinstance(s, Accum):
                env[s.name] = np.float32(_BINARY[str(s.op)](env[s.name], env[s.value]))
            elif isinstance(s, Select):
                env[s.name] = next(env[b.value] for b in s.branches if bool(eval_index(b.select, axes)))
            elif isinstance(s, Write):
                writes.append((tuple(int(eval_index(e, axes)) for e in s.index), float(env[s.value])))
            else:
                raise LoopRecordError(f"statement {type(s).__name__} is not understood")

    run(stmts)
    return writes


def reference_formula(match: LoopMatch, inputs: dict[str, np.ndarray]):
    """What the kernel chosen for ``match`` computes, as a function ``index -> value`` in float64 numpy."""
    p = match.params
    f64 = lambda name: inputs[name].astype(np.float64)  # noqa: E731
    if match.kind == "rmsnorm":
        x, w = f64(p["x"]).reshape(-1, p["cols"]), f64(p["weight"])

        def f(idx):
            row = int(np.ravel_multi_index(idx[:-1], match.out_shape[:-1]))
            return w[idx[-1]] * (x[row, idx[-1]] / np.sqrt((x[row] ** 2).sum() / p["cols"] + p["eps"]))
        return f
    if match.kind in ("linear", "linear_residual", "silu_gate_linear"):
        x, w = f64(p["x"]).ravel(), f64(p["w"])
        k = np.arange(p["K"])
        koff = (k // p["x_inner"]) * p["x_stride_outer"] + k % p["x_inner"]

        def f(idx):
            flat = int(np.ravel_multi_index(idx, match.out_shape))
            m, n = divmod(flat, p["N"])
            acc = float((x[koff + m * p["x_stride_m"]] * w[n]).sum())
            if p["residual"] is not None:
                acc += float(f64(p["residual"]).ravel()[flat])
            if p["gate"] is not None:
                g = float(f64(p["gate"]).ravel()[flat])
                acc *= g / (1.0 + np.exp(-g))
            return acc
        return f
    if match.kind == "rope_scores":
        S, H, D, g = p["S"], p["H"], p["D"], p["H"] // p["Hkv"]
        q, kk = f64(p["q"]).reshape(S, H, D), f64(p["k"]).reshape(S, p["Hkv"], D)
        cos, sin = f64(p["cos"]).reshape(S, D), f64(p["sin"]).reshape(S, D)
        rot = lambda t: np.concatenate([-t[..., D // 2:], t[..., : D // 2]], axis=-1)  # noqa: E731

        def f(idx):
            _, h, i, j = idx
            a = q[i, h] * cos[i] + rot(q[i, h]) * sin[i]
            b = kk[j, h // g] * cos[j] + rot(kk[j, h // g]) * sin[j]
            return p["scale"] * float((a * b).sum()) + (p["mask_zero"] if j <= i else p["mask_fill"])
        return f
    if match.kind == "softmax_pv":
        S, H, D, g = p["S"], p["H"], p["D"], p["H"] // p["Hkv"]
        sc, v = f64(p["scores"]).reshape(H, S, S), f64(p["v"]).reshape(S, p["Hkv"], D)

        def f(idx):
            h, i, d = idx[1], idx[2], idx[-1]
            e = np.exp(sc[h, i] - sc[h, i].max())
            return float(((e / e.sum()) * v[:, h // g, d]).sum())
        return f
    raise LoopRecordError(f"no formula for {match.kind}")


def verify(graph, node_id: str, match: LoopMatch, points: int = 6, seed: int = 0) -> LoopMatch:
    """Check ``match`` on random inputs at a few random output points against the literal execution of the body;
    for ``rope_scores`` this also decides which of the two tables is the cosine. Raises ``LoopRecordError``."""
    node = graph.nodes[node_id]
    stmts = parse_body(list(node.op_fields["body"]))
    rng = np.random.default_rng(seed)
    inputs = {}
    for nid in node.inputs:
        src = graph.nodes[nid]
        val = src.op_fields.get("value") if src.op == "ConstantOp" else None
        shape = tuple(src.output.shape)
        inputs[nid] = (np.full(shape, float(val), dtype=np.float32) if val is not None
                       else rng.standard_normal(shape).astype(np.float32) * np.float32(0.5))
    top = [s for s in stmts if isinstance(s, Loop)]
    if len(top) != 1:
        raise LoopRecordError(f"{node_id}: expected one top-level loop nest")
    # outer (non-reduce) axes down to the Write: the loops on the path to the Write statement
    path: list[Axis] = []

    def find(block, acc):
        for s in block:
            if isinstance(s, Write):
                path.extend(acc)
                return True
            if isinstance(s, Loop) and find(s.body, acc + [s.axis]):
                return True
        return False

    find(top, [])
    candidates = [match]
    if match.kind == "rope_scores":
        a, b = match.params["tables"]
        candidates = [LoopMatch(match.kind, match.output, match.out_shape, {**match.params, "cos": c, "sin": s_})
                      for c, s_ in ((a, b), (b, a))]
    last_err = None
    for cand in candidates:
        f = reference_formula(cand, inputs)
        ok = True
        for _ in range(points):
            fixed = {ax.name: int(rng.integers(0, int(ax.extent))) for ax in path}
            for idx, val in interpret_point(stmts, inputs, fixed):
                want = f(idx)
                if not np.isclose(val, want, rtol=2e-4, atol=2e-4 * max(1.0, abs(want))):
                    ok, last_err = False, f"{node_id}: body gives {val} at {idx}, the {cand.kind} kernel would give {want}"
                    break
            if not ok:
                break
        if ok:
            return cand
    raise LoopRecordError(last_err or f"{node_id}: classification {match.kind} failed verification")
