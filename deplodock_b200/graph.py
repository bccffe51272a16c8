"""Minimal container for Torch-IR graph records — the ``kernels/*.json`` / ``Graph.to_dict`` format of the reference
(``emmy/compiler/graph.py:875-997``): ``{"inputs": [...], "outputs": [...], "nodes": {id: {"op", "op_fields",
"inputs", "output": {"name", "shape", "dtype"}}}}``.

Only what the backend needs is modelled: node ids, op class name and fields, operand ids, output shape and dtype
token. A live reference ``Graph`` object (when the reference package is importable) is accepted through its own
``to_dict``. Symbolic dimensions are not supported: every kernel here is launched with concrete sizes.
"""

from __future__ import annotations

import json
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


@dataclass(frozen=True)
class TensorInfo:
    name: str
    shape: tuple[int, ...]
    dtype: str

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
                if not isinstance(dim, int):
                    raise ValueError(f"node {nid!r}: symbolic dimension {dim!r} is not supported by this backend")
                shape.append(int(dim))
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

    def symbolic_env(self, input_data: dict | None = None) -> dict[str, int]:
        """Always empty: shapes are static here (the reference resolves symbolic dims, ``graph.py:686-706``)."""
        return {}

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
