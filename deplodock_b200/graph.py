"""Minimal container for Torch-IR graph records — the ``kernels/*.json`` / ``Graph.to_dict`` format of the reference
(``emmy/compiler/graph.py:875-997``): ``{"inputs": [...], "outputs": [...], "nodes": {id: {"op", "op_fields",
"inputs", "output": {"name", "shape", "dtype"}}}}``.

Only what the backend needs is modelled: node ids, op class name and fields, operand ids, output shape and dtype
token. A live reference ``Graph`` object (when the reference package is importable) is accepted through its own
``to_dict``.

Symbolic dimensions: the reference writes an atomic symbolic dim as its name (``"seq_len"``) and a composite one as its
pretty-printed expression (``emmy/compiler/graph.py:953-1007``); both are kept here as strings.
:meth:`Graph.symbolic_env` reads the runtime value of every atomic name off the supplied input arrays (first-seen
position wins, as ``emmy/compiler/graph.py:686-706``) and :meth:`Graph.resolve` substitutes it, evaluating composite
expressions (``+ - * // %``, ``min``, ``max``, ``round_up``, ``ceildiv``), which gives the static graph a kernel
plan is built for. Kernels are always launched with concrete sizes: one plan per binding of the symbols.
"""

from __future__ import annotations

import ast
import json
import operator
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any

import numpy as np

#: dtype token -> (numpy carrier dtype, bytes). bf16 travels as uint16 bit patterns, as in the reference
#: (``emmy/compiler/dtype.py:61-69``).
DTYPES: dict[str, tuple[np.dtype, int]] = {
    "f32": (np.dtype(np.float32), 4),
    "f16": (np.dtype(np.float16), 2),
    "bf16": (np.dtype(np.uint16), 2),
    "i64": (np.dtype(np.int64), 8),
    "i32": (np.dtype(np.int32), 4),
    "bool": (np.dtype(np.bool_), 1),
}


_DTYPE_ALIASES = {"float32": "f32", "float16": "f16", "bfloat16": "bf16", "int64": "i64", "int32": "i32"}


_BIN = {ast.Add: operator.add, ast.Sub: operator.sub, ast.Mult: operator.mul, ast.FloorDiv: operator.floordiv,
        ast.Div: operator.floordiv, ast.Mod: operator.mod}
_FUNCS = {"min": min, "max": max, "round_up": lambda a, b: -(-a // b) * b, "ceildiv": lambda a, b: -(-a // b)}


def eval_dim(expr, env: dict[str, int]) -> int:
    """A dimension under ``env``: ints pass through, a name is looked up, an expression string is evaluated with
    integer arithmetic (``/`` is integer division, as in the reference's index expressions)."""
    if isinstance(expr, int):
        return expr

    def ev(n: ast.AST) -> int:
        if isinstance(n, ast.Constant) and isinstance(n.value, int):
            return n.value
        if isinstance(n, ast.Name):
            if n.id not in env:
                raise KeyError(f"symbolic dimension {n.id!r} has no runtime value (known: {sorted(env)})")
            return int(env[n.id])
        if isinstance(n, ast.BinOp) and type(n.op) in _BIN:
            return int(_BIN[type(n.op)](ev(n.left), ev(n.right)))
        if isinstance(n, ast.UnaryOp) and isinstance(n.op, ast.USub):
            return -ev(n.operand)
        if isinstance(n, ast.Call) and isinstance(n.func, ast.Name) and n.func.id in _FUNCS and not n.keywords:
            return int(_FUNCS[n.func.id](*[ev(a) for a in n.args]))
        raise ValueError(f"unsupported dimension expression {expr!r}")

    return ev(ast.parse(str(expr), mode="eval").body)


def dim_symbols(expr) -> set[str]:
    if isinstance(expr, int):
        return set()
    return {n.id for n in ast.walk(ast.parse(str(expr), mode="eval")) if isinstance(n, ast.Name) and n.id not in _FUNCS}


@dataclass(frozen=True)
class TensorInfo:
    name: str
    shape: tuple  # ints, or strings for symbolic dimensions (a name or an expression over names)
    dtype: str

    @property
    def is_static(self) -> bool:
        return all(isinstance(d, int) for d in self.shape)

    @property
    def np_dtype(self) -> np.dtype:
        return DTYPES[self.dtype][0]


@dataclass
class Node:
    id: str
    op: str
    op_fields: dict[str, Any]
    inputs: list[str]
    output: TensorInfo


@dataclass
class Graph:
    inputs: list[str]
    outputs: list[str]
    nodes: dict[str, Node] = field(default_factory=dict)

    # -- construction ------------------------------------------------------------------------------------------
    @classmethod
    def from_dict(cls, d: dict) -> "Graph":
        nodes: dict[str, Node] = {}
        for nid, nd in d["nodes"].items():
            out = nd["output"]
            shape = []
            for dim in out["shape"]:
                if isinstance(dim, bool) or not isinstance(dim, (int, str)):
                    raise ValueError(f"node {nid!r}: dimension {dim!r} is neither an int nor a symbolic name")
                if isinstance(dim, str):
                    try:
                        dim_symbols(dim)
                    except SyntaxError as exc:
                        raise ValueError(f"node {nid!r}: cannot parse symbolic dimension {dim!r}") from exc
                shape.append(dim)
            dtype = _DTYPE_ALIASES.get(out["dtype"], out["dtype"])   # older records spell the numpy name
            if dtype not in DTYPES:
                raise TypeError(f"node {nid!r}: unknown dtype token {dtype!r}")
            fields = dict(nd.get("op_fields") or {})
            if nd["op"] == "ConstantOp" and isinstance(fields.get("value"), str):
                # Loop-IR records carry constant values as strings ('None', '1e-05')
                fields["value"] = None if fields["value"] == "None" else float(fields["value"])
            nodes[nid] = Node(nid, nd["op"], fields, list(nd.get("inputs") or []),
                              TensorInfo(out.get("name", nid), tuple(shape), dtype))
        g = cls(list(d["inputs"]), list(d["outputs"]), nodes)
        for nid in g.inputs + g.outputs:
            if nid not in nodes:
                raise KeyError(f"graph boundary names unknown node {nid!r}")
        for n in nodes.values():
            for i in n.inputs:
                if i not in nodes:
                    raise KeyError(f"node {n.id!r} reads unknown node {i!r}")
        return g

    @classmethod
    def from_json(cls, path: str | Path) -> "Graph":
        return cls.from_dict(json.loads(Path(path).read_text()))

    @classmethod
    def coerce(cls, obj: Any) -> "Graph":
        """Accept this class, a record dict, a JSON path, or a reference ``Graph`` (anything with ``to_dict``)."""
        if isinstance(obj, cls):
            return obj
        if isinstance(obj, dict):
            return cls.from_dict(obj)
        if isinstance(obj, (str, Path)):
            return cls.from_json(obj)
        if hasattr(obj, "to_dict"):
            return cls.from_dict(obj.to_dict())
        raise TypeError(f"cannot build a Graph from {type(obj).__name__}")

    def to_dict(self) -> dict:
        return {"inputs": list(self.inputs), "outputs": list(self.outputs),
                "nodes": {nid: {"op": n.op, "op_fields": dict(n.op_fields), "inputs": list(n.inputs),
                                "output": {"name": n.output.name, "shape": list(n.output.shape),
                                           "dtype": n.output.dtype}} for nid, n in self.nodes.items()}}

    # -- queries -----------------------------------------------------------------------------------------------
    def topological_order(self) -> list[str]:
        order: list[str] = []
        state: dict[str, int] = {}

        def visit(nid: str) -> None:
            st = state.get(nid, 0)
            if st == 2:
                return
            if st == 1:
                raise ValueError(f"cycle through node {nid!r}")
            state[nid] = 1
            for i in self.nodes[nid].inputs:
                visit(i)
            state[nid] = 2
            order.append(nid)

        for nid in self.nodes:
            visit(nid)
        return order

    def node_role(self, nid: str) -> str:
        """'input' / 'constant' / 'output' / 'scratch' (same classes as ``emmy/compiler/graph.py:673-684``)."""
        if nid in self.inputs:
            return "input"
        if self.nodes[nid].op == "ConstantOp":
            return "constant"
        if nid in self.outputs:
            return "output"
        return "scratch"

    @property
    def is_symbolic(self) -> bool:
        return any(not n.output.is_static for n in self.nodes.values())

    def symbols(self) -> set[str]:
        out: set[str] = set()
        for n in self.nodes.values():
            for d in n.output.shape:
                out |= dim_symbols(d)
        return out

    def symbolic_env(self, input_data: dict | None = None) -> dict[str, int]:
        """Runtime value of every atomic symbolic input dim, read off the supplied input arrays (first-seen position
        wins; inputs that are absent or have fewer dims than declared are skipped) — ``emmy/compiler/graph.py:686-706``."""
        env: dict[str, int] = {}
        for nid in self.inputs:
            if not input_data or nid not in input_data:
                continue
            arr_shape = tuple(getattr(input_data[nid], "shape", None) or np.asarray(input_data[nid]).shape)
            for i, d in enumerate(self.nodes[nid].output.shape):
                if isinstance(d, str) and d.isidentifier() and i < len(arr_shape):
                    env.setdefault(d, int(arr_shape[i]))
        return env

    def resolve(self, env: dict[str, int]) -> "Graph":
        """The static graph under ``env``: every symbolic dimension replaced by its value (``shape`` op fields that
        name symbols included). Raises ``KeyError`` for a symbol without a value."""
        if not self.is_symbolic:
            return self
        nodes: dict[str, Node] = {}
        for nid, n in self.nodes.items():
            fields = dict(n.op_fields)
            for key in ("shape", "out_shape", "source_shape"):
                if isinstance(fields.get(key), (list, tuple)):
                    fields[key] = [eval_dim(d, env) if isinstance(d, str) else d for d in fields[key]]
            shape = tuple(eval_dim(d, env) for d in n.output.shape)
            nodes[nid] = Node(nid, n.op, fields, list(n.inputs), TensorInfo(n.output.name, shape, n.output.dtype))
        return Graph(list(self.inputs), list(self.outputs), nodes)

    def compute_nodes(self) -> list[Node]:
        return [self.nodes[n] for n in self.topological_order()
                if self.nodes[n].op not in ("InputOp", "ConstantOp")]

    def single_node_graph(self, nid: str, operands: list[str] | None = None) -> "Graph":
        """The node ``nid`` as a stand-alone graph: the node itself, its scalar / weight ``ConstantOp`` producers as
        they are, and every other operand turned into an ``InputOp`` of the same name, shape and dtype — the
        per-kernel reproducer sub-graph of the reference (``emmy/compiler/pipeline/dump.py:135-180``). ``operands``
        replaces the node's own input ids (a plan step reads through views and casts)."""
        node = self.nodes[nid]
        ins = list(node.inputs if operands is None else operands)
        nodes: dict[str, Node] = {}
        inputs: list[str] = []
        for i in ins:
            src = self.nodes[i]
            if src.op == "ConstantOp":
                nodes[i] = Node(i, src.op, dict(src.op_fields), [], src.output)
            else:
                nodes[i] = Node(i, "InputOp", {}, [], src.output)
                if i not in inputs:
                    inputs.append(i)
        nodes[nid] = Node(nid, node.op, dict(node.op_fields), ins, node.output)
        return Graph(inputs, [nid], nodes)

    def op_histogram(self) -> dict[str, int]:
        h: dict[str, int] = {}
        for n in self.nodes.values():
            h[n.op] = h.get(n.op, 0) + 1
        return h
