"""Tracing of inline PyTorch expressions and modules into Torch-IR graph records.

Mirrors the behaviour of the reference's ``--code`` entry (``emmy/commands/trace.py:114-223``: the last statement must
be an expression; statements before it are a preamble run with ``torch``, ``nn`` and ``F`` in scope; a call of an
``nn.Module`` instance is traced as that module, anything else becomes the ``forward`` of a wrapper whose tensor
inputs are the tensor names of the preamble and inline tensor-constructor calls) and of its FX walk
(``emmy/compiler/trace/torch.py:71-135``: ``torch.export.export``, parameters/buffers become ``ConstantOp`` with a
``source_path``, other placeholders ``InputOp``, casts and ``contiguous``/``clone`` pass their input through,
``:698-701``). The ops this backend has kernels for, and the ops the HF decoder trunk is traced into (embedding gather,
the pow / mean / rsqrt RMSNorm chain, slice / negative / cat RoPE, transposes, ``expand`` as ``IndexMapOp``), get the
reference's Torch-IR op names; anything else is recorded under its ATen name and rejected later by
``B200Backend.compile`` with a ``LoweringError``. :func:`build_full_model_wrapper` makes an HF model traceable the way
the reference's wrapper does (``emmy/compiler/trace/huggingface.py:17-186``).

When the reference package is importable its tracer can be used instead: ``B200Backend.compile`` accepts its ``Graph``
objects directly.
"""

from __future__ import annotations

import ast
import re
from dataclasses import dataclass
from typing import Any

import torch
import torch.nn.functional as F

from deplodock_b200.graph import Graph

_DTYPE_TOKENS = {torch.float32: "f32", torch.float16: "f16", torch.bfloat16: "bf16", torch.int64: "i64",
                 torch.int32: "i32", torch.bool: "bool"}
_TENSOR_CTORS = frozenset({"randn", "rand", "zeros", "ones", "empty", "full", "arange", "linspace", "tensor",
                           "randint", "eye"})


@dataclass
class TraceResult:
    graph: Graph
    slug: str
    module: torch.nn.Module
    args: tuple
    kwargs: dict
    const_sources: dict[str, str]  # ConstantOp node id -> attribute path on the module


def _slugify(text: str) -> str:
    return re.sub(r"[^a-z0-9]+", "_", text.lower()).strip("_")[:48] or "expr"


def _token(dtype: torch.dtype) -> str:
    try:
        return _DTYPE_TOKENS[dtype]
    except KeyError:
        raise TypeError(f"dtype {dtype} has no graph token") from None


class _InputLifter(ast.NodeTransformer):
    """Replaces tensor names of the preamble and inline tensor-constructor calls by fresh parameter names."""

    def __init__(self, scope: dict) -> None:
        self.scope = scope
        self.params: dict[str, torch.Tensor] = {}
        self._synth = 0

    def visit_Name(self, node: ast.Name):
        val = self.scope.get(node.id)
        if isinstance(val, torch.Tensor) and isinstance(node.ctx, ast.Load):
            self.params.setdefault(node.id, val)
        return node

    def visit_Call(self, node: ast.Call):
        f = node.func
        if (isinstance(f, ast.Attribute) and isinstance(f.value, ast.Name) and f.value.id == "torch"
                and f.attr in _TENSOR_CTORS):
            value = eval(compile(ast.Expression(node), "<--code>", "eval"), self.scope)  # noqa: S307 - local CLI input
            if isinstance(value, torch.Tensor):
                name = f"_x{self._synth}"
                self._synth += 1
                self.params[name] = value
                return ast.copy_location(ast.Name(id=name, ctx=ast.Load()), node)
        return self.generic_visit(node)


def trace_inline_code(code: str, dynamic: list[tuple[str, str, int]] | None = None) -> TraceResult:
    """Trace ``"<preamble>; <final expression>"`` (see the module docstring for the grammar). ``dynamic``: symbolic
    axes, by input name as it appears in the record (``x`` for a single inline tensor, else the preamble's names)."""
    tree = ast.parse(code)
    if not tree.body or not isinstance(tree.body[-1], ast.Expr):
        raise ValueError('--code must end with an expression (e.g. "torch.nn.Softmax(dim=-1)(torch.randn(4, 8))")')
    final = tree.body[-1].value
    scope: dict[str, Any] = {"torch": torch, "nn": torch.nn, "F": F}
    exec(compile(ast.Module(body=tree.body[:-1], type_ignores=[]), "<--code>", "exec"), scope)  # noqa: S102

    if isinstance(final, ast.Call):
        try:
            callee = eval(compile(ast.Expression(final.func), "<--code>", "eval"), scope)  # noqa: S307
        except Exception:  # noqa: BLE001
            callee = None
        if isinstance(callee, torch.nn.Module):
            args = tuple(eval(compile(ast.Expression(a), "<--code>", "eval"), scope) for a in final.args)  # noqa: S307
            kwargs = {k.arg: eval(compile(ast.Expression(k.value), "<--code>", "eval"), scope)  # noqa: S307
                      for k in final.keywords if k.arg}
            graph, sources = trace_module(callee, args, kwargs, dynamic)
            return TraceResult(graph, _slugify(ast.unparse(final.func)), callee, args, kwargs, sources)

    lifter = _InputLifter(scope)
    rewritten = ast.fix_missing_locations(lifter.visit(final))
    params = lifter.params
    if not params:
        raise ValueError("--code expression has no tensor inputs to trace")
    synth = [k for k in params if k.startswith("_x")]
    rename = {synth[0]: "x"} if len(synth) == 1 else {old: f"x{i}" for i, old in enumerate(synth)}
    taken = set(params) - set(synth)
    rename = {old: (new if new not in taken else f"{new}_") for old, new in rename.items()}
    params = {rename.get(k, k): v for k, v in params.items()}
    for node in ast.walk(rewritten):
        if isinstance(node, ast.Name) and node.id in rename:
            node.id = rename[node.id]
    sig = ", ".join(["self", *params])
    src = f"class _Wrapper(torch.nn.Module):\n    def forward({sig}):\n        return {ast.unparse(rewritten)}\n"
    exec(src, scope)  # noqa: S102
    module = scope["_Wrapper"]()
    args = tuple(params.values())
    graph, sources = trace_module(module, args, {}, dynamic)
    return TraceResult(graph, _slugify(ast.unparse(final)), module, args, {}, sources)


def graph_from_code(code: str):
    """``(graph, slug, (module, args, kwargs))`` — the return shape of the reference's ``graph_from_code``."""
    r = trace_inline_code(code)
    return r.graph, r.slug, (r.module, r.args, r.kwargs)


# ------------------------------------------------------------------------------------------------------------
# FX walk
# ------------------------------------------------------------------------------------------------------------
_PASSTHROUGH_TARGETS = ("aten.to.", "aten._to_copy.", "aten.contiguous.", "aten.clone.", "aten.alias.", "aten.detach.",
                        "aten.type_as.", "aten.lift_fresh_copy.", "aten.dropout.")
_VIEW_TARGETS = ("aten.view.", "aten.reshape.", "aten._unsafe_view.", "aten.squeeze.", "aten.flatten.")


DYNAMIC_DIM_MAX = 4096   # upper bound of every dynamic axis, as in the reference (emmy/compiler/trace/dynamic.py:19)


def parse_dynamic_specs(specs: list[str] | None) -> list[tuple[str, str, int]]:
    """``--dynamic NAME@INPUT:AXIS`` strings -> ``(name, input, axis)`` triples; several specs may share a NAME (the
    same symbolic size on several inputs), an ``(INPUT, AXIS)`` position may appear once. The grammar and its errors
    are the reference's (``emmy/compiler/trace/dynamic.py:22-65``)."""
    out: list[tuple[str, str, int]] = []
    seen: set[tuple[str, int]] = set()
    for raw in specs or []:
        name, at, locator = raw.partition("@")
        inp, colon, axis_s = locator.rpartition(":")
        if not at or not colon:
            raise ValueError(f"--dynamic {raw!r}: expected NAME@INPUT:AXIS form (e.g. seq_len@x:1)")
        name, inp = name.strip(), inp.strip()
        if not name or not name.isidentifier():
            raise ValueError(f"--dynamic {raw!r}: NAME must be an identifier")
        if not inp:
            raise ValueError(f"--dynamic {raw!r}: INPUT name is empty")
        try:
            axis = int(axis_s)
        except ValueError:
            raise ValueError(f"--dynamic {raw!r}: AXIS must be an int, got {axis_s!r}") from None
        if axis < 0:
            raise ValueError(f"--dynamic {raw!r}: AXIS must be >= 0, got {axis}")
        if (inp, axis) in seen:
            raise ValueError(f"--dynamic {raw!r}: ({inp}, axis {axis}) appears more than once")
        seen.add((inp, axis))
        out.append((name, inp, axis))
    return out


def _dim_token(d, symbols: dict[str, str]):
    """An FX shape entry as a record dimension: an int, or for a symbolic size its expression with torch's symbol
    names (``s0``, ``s77``) replaced by the user's dimension names."""
    if isinstance(d, int):
        return int(d)
    text = str(d)
    for sym, name in sorted(symbols.items(), key=lambda kv: -len(kv[0])):
        text = re.sub(rf"\b{re.escape(sym)}\b", name, text)
    try:
        return int(text)
    except ValueError:
        return text


def _shape_dtype(node, symbols: dict[str, str] | None = None) -> tuple[list, str]:
    val = node.meta.get("val")
    if val is None or not isinstance(val, torch.Tensor):
        raise ValueError(f"FX node {node.name} carries no tensor value")
    return [_dim_token(d, symbols or {}) for d in val.shape], _token(val.dtype)


def trace_module(module: torch.nn.Module, args: tuple, kwargs: dict | None = None,
                 dynamic: list[tuple[str, str, int]] | None = None) -> tuple[Graph, dict[str, str]]:
    """``torch.export.export`` the module and convert its FX graph to a Torch-IR record. ``dynamic`` marks axes of
    inputs as symbolic (``(name, input, axis)``, see :func:`parse_dynamic_specs`): the record then carries the name
    in every shape the axis flows into (``emmy/compiler/trace/dynamic.py:68-88`` builds the same ``dynamic_shapes``)."""
    dynamic_shapes = None
    if dynamic:
        import inspect

        params = [p for p in inspect.signature(module.forward).parameters]
        dims: dict[str, Any] = {}
        dynamic_shapes = {p: None for p in params[: len(args)]}
        dynamic_shapes.update({k: None for k in (kwargs or {})})
        for name, inp, axis in dynamic:
            if inp not in dynamic_shapes:
                raise ValueError(f"--dynamic: the traced call has no input named {inp!r} (inputs: {list(dynamic_shapes)})")
            dims.setdefault(name, torch.export.Dim(name, min=2, max=DYNAMIC_DIM_MAX))
            dynamic_shapes[inp] = {**(dynamic_shapes[inp] or {}), axis: dims[name]}
    exported = torch.export.export(module, args, kwargs=kwargs or None, dynamic_shapes=dynamic_shapes)
    symbols: dict[str, str] = {}
    if dynamic:
        by_input = {}
        for name, inp, axis in dynamic:
            by_input.setdefault(inp, []).append((axis, name))
        user_inputs = [n for n in exported.graph.nodes if n.op == "placeholder"
                       and n.name not in exported.graph_signature.inputs_to_parameters
                       and n.name not in exported.graph_signature.inputs_to_buffers]
        for ph, pname in zip(user_inputs, list(dynamic_shapes)):
            for axis, name in by_input.get(pname, []):
                d = ph.meta["val"].shape[axis]
                if not isinstance(d, int):
                    symbols[str(d)] = name
    sig = exported.graph_signature
    param_paths = dict(sig.inputs_to_parameters)
    param_paths.update(sig.inputs_to_buffers)
    nodes: dict[str, dict] = {}
    inputs: list[str] = []
    outputs: list[str] = []
    sources: dict[str, str] = {}

    def add(nid, op, fields, ins, shape, dtype):
        nodes[nid] = {"op": op, "op_fields": fields, "inputs": ins,
                      "output": {"name": nid, "shape": shape, "dtype": dtype}}

    def const_scalar(base: str, idx: int, value: float) -> str:
        nid = f"{base}_c{idx}"
        add(nid, "ConstantOp", {"name": nid, "value": float(value), "source_path": None}, [], [1], "f32")
        return nid

    for node in exported.graph.nodes:
        if node.op == "placeholder":
            shape, dtype = _shape_dtype(node, symbols)
            if node.name in param_paths:
                path = param_paths[node.name]
                sources[node.name] = path
                add(node.name, "ConstantOp", {"name": node.name, "value": None, "source_path": path,
                                              "source_shape": shape, "source_dtype": str(node.meta["val"].dtype)},
                    [], shape, dtype)
            else:
                add(node.name, "InputOp", {}, [], shape, dtype)
                inputs.append(node.name)
        elif node.op == "call_function":
            target = str(node.target)
            if not isinstance(node.meta.get("val"), torch.Tensor):
                continue  # metadata assertions and other value-less bookkeeping nodes
            shape, dtype = _shape_dtype(node, symbols)
            a = list(node.args)
            kw = dict(node.kwargs)
            tin = [x.name for x in a if hasattr(x, "name")]
            if target.startswith("aten.rms_norm."):
                eps = a[3] if len(a) > 3 and a[3] is not None else kw.get("eps")
                eps = 1e-6 if eps is None else float(eps)
                if len(a) < 3 or a[2] is None:
                    raise ValueError("rms_norm without a weight is not supported")
                const_scalar(node.name, 2, eps)
                add(node.name, "RmsNormOp", {"eps": eps}, [a[0].name, a[2].name], shape, dtype)
            elif target.startswith("aten.softmax.") or target.startswith("aten._softmax."):
                add(node.name, "SoftmaxOp", {"axis": int(a[1])}, [a[0].name], shape, dtype)
            elif target.startswith("aten.linear."):
                has_bias = len(a) > 2 and a[2] is not None
                add(node.name, "LinearOp", {"has_bias": has_bias}, [x.name for x in a[:3] if x is not None], shape,
                    dtype)
            elif target.startswith(("aten.mm.", "aten.matmul.", "aten.bmm.")):
                add(node.name, "MatmulOp", {"has_bias": False}, tin[:2], shape, dtype)
            elif target.startswith("aten.addmm."):
                add(node.name, "MatmulOp", {"has_bias": True}, [a[1].name, a[2].name, a[0].name], shape, dtype)
            elif target.startswith("aten.scaled_dot_product_attention."):
                # the reference reads is_causal from the first bool argument (emmy/compiler/trace/torch.py:567-571)
                bools = [v for v in list(a[3:]) + list(kw.values()) if isinstance(v, bool)]
                is_causal = bool(kw.get("is_causal", bools[0] if bools else False))
                mask = kw.get("attn_mask", a[3] if len(a) > 3 and hasattr(a[3], "name") else None)
                ins = [a[0].name, a[1].name, a[2].name] + ([mask.name] if mask is not None else [])
                const_scalar(node.name, 3, 0.0)
                add(node.name, "SdpaOp", {"is_causal": is_causal}, ins, shape, dtype)
            elif target.startswith(("aten.add.Tensor", "aten.mul.Tensor", "aten.silu.")) and all(
                    hasattr(x, "name") for x in a[:1 if "silu" in target else 2]):
                # same names as the reference's ElementwiseOp (emmy/compiler/trace/torch.py:506-523)
                name = "silu" if "silu" in target else ("add" if "add" in target else "multiply")
                add(node.name, "ElementwiseOp", {"op": name}, tin[:1 if name == "silu" else 2], shape, dtype)
            elif target.startswith(("aten.add.Tensor", "aten.mul.Tensor", "aten.pow.Tensor_Scalar")) and hasattr(
                    a[0], "name") and isinstance(a[1], (int, float)):
                # tensor (op) python scalar: the scalar becomes a one-element ConstantOp, as in the reference's records
                name = "pow" if "pow" in target else ("add" if "add" in target else "multiply")
                add(node.name, "ElementwiseOp", {"op": name}, [a[0].name, const_scalar(node.name, 1, a[1])], shape, dtype)
            elif target.startswith(("aten.rsqrt.", "aten.neg.")):
                add(node.name, "ElementwiseOp", {"op": "rsqrt" if "rsqrt" in target else "negative"}, tin[:1], shape,
                    dtype)
            elif target.startswith("aten.embedding."):
                add(node.name, "GatherOp", {"axis": 0}, [a[0].name, a[1].name], shape, dtype)
            elif target.startswith("aten.mean.dim"):
                dims = a[1] if isinstance(a[1], (list, tuple)) else [a[1]]
                if len(dims) != 1:
                    raise ValueError("mean over several axes is not supported")
                add(node.name, "MeanOp", {"axis": int(dims[0]), "keepdim": bool(a[2]) if len(a) > 2 else False},
                    [a[0].name], shape, dtype)
            elif target.startswith("aten.slice.Tensor"):
                dim = int(a[1]) if len(a) > 1 else 0
                start = int(a[2]) if len(a) > 2 and a[2] is not None else 0
                add(node.name, "SliceOp", {"shape": shape, "dim": dim, "start": start}, [a[0].name], shape, dtype)
            elif target.startswith("aten.cat."):
                axis = int(a[1]) if len(a) > 1 else int(kw.get("dim", 0))
                add(node.name, "CatOp", {"axis": axis}, [x.name for x in a[0]], shape, dtype)
            elif target.startswith("aten.transpose.int"):
                add(node.name, "TransposeOp", {"axes": [int(a[1]), int(a[2])]}, [a[0].name], shape, dtype)
            elif target.startswith("aten.unsqueeze."):
                add(node.name, "UnsqueezeOp", {"dim": int(a[1])}, [a[0].name], shape, dtype)
            elif target.startswith("aten.expand."):
                add(node.name, "IndexMapOp", {"out_shape": shape}, [a[0].name], shape, dtype)
            elif target.startswith(_PASSTHROUGH_TARGETS):
                add(node.name, "ToOp", {}, tin[:1], shape, dtype)
            elif target.startswith(_VIEW_TARGETS):
                add(node.name, "ReshapeOp", {"shape": shape}, tin[:1], shape, dtype)
            else:
                add(node.name, "Aten:" + target, {}, tin, shape, dtype)
        elif node.op == "output":
            for out in node.args[0] if isinstance(node.args[0], (tuple, list)) else [node.args[0]]:
                if hasattr(out, "name"):
                    outputs.append(out.name)
    return Graph.from_dict({"inputs": inputs, "outputs": outputs, "nodes": nodes}), sources


def bind_inputs(graph: Graph, module: torch.nn.Module, args: tuple, kwargs: dict, sources: dict[str, str]):
    """``input_data`` for ``Backend.run``: example tensors for the graph inputs, module parameters / buffers for the
    weight constants (the reference's ``_bind_inputs``, ``emmy/commands/run.py:1227-1278``). Tensors are passed as
    torch tensors (the backend accepts them), which also carries bf16, unlike the reference's ``tensor.numpy()``."""
    flat: list[torch.Tensor] = []
    for v in list(args) + list(kwargs.values()):
        if isinstance(v, torch.Tensor):
            flat.append(v)
        elif isinstance(v, (list, tuple)):
            flat.extend(t for t in v if isinstance(t, torch.Tensor))
    if len(flat) != len(graph.inputs):
        raise ValueError(f"graph has {len(graph.inputs)} inputs, the call provided {len(flat)} tensors")
    data: dict[str, Any] = {nid: t.detach() for nid, t in zip(graph.inputs, flat)}
    named = dict(module.named_parameters(remove_duplicate=False))
    named.update(dict(module.named_buffers(remove_duplicate=False)))
    for nid, path in sources.items():
        if path not in named:
            raise KeyError(f"Could not bind constant {nid} (source_path={path!r})")
        data[nid] = named[path].detach()
    return data


# ------------------------------------------------------------------------------------------------------------
# HF model wrapper
# ------------------------------------------------------------------------------------------------------------
class _FixedRotary(torch.nn.Module):
    """Stands in for the model's rotary-embedding submodule and returns tables computed once, eagerly. Under
    ``torch.export`` the original submodule's non-persistent ``inv_freq`` buffer loses its value, which would trace
    RoPE as the identity."""

    def __init__(self, cos: torch.Tensor, sin: torch.Tensor) -> None:
        super().__init__()
        self.register_buffer("cos", cos)
        self.register_buffer("sin", sin)

    def forward(self, *args, **kwargs):
        return self.cos, self.sin


class FullModelWrapper(torch.nn.Module):
    """``forward(input_ids) -> hidden states`` (logits for a causal-LM head model) of an HF decoder with everything
    that depends on the sequence length precomputed as buffers: the additive causal mask ``causal_mask``
    ``[1, 1, S, S]`` (0 / -inf), ``position_ids`` ``[1, S]`` and the rotary tables ``model.rotary_emb.cos`` / ``.sin``
    ``[1, S, head_dim]``. The traced graph then holds no mask- or position-construction ops, and the buffers appear
    as ``ConstantOp`` nodes under those source paths — the same record the reference's wrapper yields."""

    def __init__(self, model: torch.nn.Module, seq_len: int, dtype: torch.dtype) -> None:
        super().__init__()
        self.model = model
        neg = torch.full((seq_len, seq_len), float("-inf"), dtype=dtype)
        self.register_buffer("causal_mask", torch.triu(neg, diagonal=1)[None, None])
        self.register_buffer("position_ids", torch.arange(seq_len, dtype=torch.long)[None])
        trunk = getattr(model, "model", model)
        rotary = getattr(trunk, "rotary_emb", None)
        if rotary is not None:
            with torch.no_grad():
                probe = torch.zeros(1, seq_len, model.config.hidden_size, dtype=dtype)
                cos, sin = rotary(probe, self.position_ids)
            trunk.rotary_emb = _FixedRotary(cos.clone(), sin.clone())

    def forward(self, input_ids):
        return self.model(input_ids=input_ids, attention_mask=self.causal_mask, position_ids=self.position_ids,
                          use_cache=False, return_dict=False)[0]


def build_full_model_wrapper(model: torch.nn.Module, seq_len: int, dtype: torch.dtype) -> torch.nn.Module:
    """Static-shape wrapper of an HF decoder for tracing (the reference's ``build_full_model_wrapper`` in its default
    mode; its ``dynamic=True`` mode has no counterpart here: plans are built per sequence length)."""
    return FullModelWrapper(model, seq_len, dtype)
