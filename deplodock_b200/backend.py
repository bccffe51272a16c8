"""``B200Backend``: the reference's ``Backend`` call surface over the hand-written sm_100a kernels.

Mirrors ``emmy/compiler/backend/base.py:45-205`` (``RunResult``, ``LaunchTime``, ``BenchmarkResult``, ``Backend``) and
``emmy/compiler/backend/cuda/backend.py:61-237`` (``CudaBackend``: constructor keywords, ``compile``, ``run``,
``benchmark_async``, ``close_async_worker``). Where the reference lowers a Torch-IR graph through its rewrite pipeline
to generated CUDA (``Pipeline.build(CUDA_PASSES).run``, ``backend.py:135-142``), ``compile`` here dispatches each
Torch-IR op to one C-ABI kernel and returns a plan; nothing is generated or compiled at run time.

    compiled = backend.compile(graph)                 # Graph | record dict | JSON path | reference Graph object
    result, pre = backend.run(compiled, input_data={node_id: ndarray, ...})
    bench = await backend.benchmark_async(compiled, warmup=5, num_iters=20)

Conventions kept from the reference: ``input_data`` holds one numpy array per graph input and per weight
``ConstantOp``; bf16 travels as ``uint16`` bit patterns (``emmy/compiler/dtype.py:69``); weights may arrive as fp32 and
are cast to the node dtype (``emmy/commands/run.py:1264-1267``); scalar ``ConstantOp``s are materialised from
``op.value`` (``backend/base.py:184-191``); a missing input raises ``KeyError``; kernel names keep the ``k_`` prefix.
Ops without a hand-written kernel raise :class:`LoweringError` — there is no interpreter fallback.
"""

from __future__ import annotations

import asyncio
import statistics
import zlib
from abc import ABC, abstractmethod
from collections.abc import Callable
from dataclasses import dataclass, field
from typing import Any

import numpy as np

from deplodock_b200.graph import Graph, Node


# ------------------------------------------------------------------------------------------------------------
# Result types and the abstract base (emmy/compiler/backend/base.py:45-205)
# ------------------------------------------------------------------------------------------------------------
class LoweringError(RuntimeError):
    """No hand-written kernel covers a node (the reference raises ``LoweringError`` from its pipeline)."""


try:
    # Inside the reference's process the reference's own types are used, so that its callers' isinstance checks and
    # dataclass handling see exactly what CudaBackend would hand them.
    from emmy.compiler.backend.base import Backend, BenchmarkResult, LaunchTime, RunResult

    USES_REFERENCE_TYPES = True
except Exception:  # noqa: BLE001 - the reference package is absent (the usual case): same fields, defined here
    USES_REFERENCE_TYPES = False

    @dataclass
    class RunResult:
        outputs: dict[str, Any]
        time_ms: float | None = None

    @dataclass
    class LaunchTime:
        idx: int
        kernel_name: str
        time_ms: float
        samples: tuple[float, ...] | None = None

    @dataclass
    class BenchmarkResult:
        time_ms: float
        min_ms: float | None = None
        max_ms: float | None = None
        num_launches: int = 0
        per_launch: list[LaunchTime] | None = None
        captured: bool = False
        e2e_ms: float | None = None
        e2e_min_ms: float | None = None

    class Backend(ABC):
        """Abstract backend: Graph -> compiled artifact -> run (``emmy/compiler/backend/base.py:94-205``)."""

        name: str = "stub"
        bench_compile_timeout_s: float = 30.0
        bench_run_timeout_s: float = 10.0
        bench_wall_timeout_s: float | None = None

        @abstractmethod
        def compile(self, graph: Any) -> Any: ...

        @abstractmethod
        def run(self, compiled: Any, *, input_data: dict[str, np.ndarray] | None = None,
                pre_run: Callable[[], Any] | None = None) -> tuple[RunResult, Any]: ...


# ------------------------------------------------------------------------------------------------------------
# Plan
# ------------------------------------------------------------------------------------------------------------
@dataclass
class PlanStep:
    """One kernel launch: reads ``args`` (node ids) from the value table and writes ``out``."""

    kernel_name: str
    entry: str          # C-ABI entry point
    out: str
    args: list[str]
    attrs: dict[str, Any] = field(default_factory=dict)


@dataclass
class CompiledPlan:
    """What ``compile`` returns. Exposes ``inputs/outputs/nodes/symbolic_env`` because the reference's callers read
    them off the compiled artifact (``emmy/commands/run.py:214,254,1249-1256``; ``backend/cuda/backend.py:172-176``)."""

    graph: Graph
    steps: list[PlanStep]
    aliases: dict[str, str]   # view-like nodes (reshape/contiguous/to) -> the node whose buffer they share
    trunk: Any = None         # a ``trunk.TrunkMatch`` when the graph was recognised as a whole decoder trunk
    # device copies of the weight constants, kept between runs while the caller passes the same host objects
    # (host -> device once per compiled plan, not once per run)
    const_cache: dict[str, tuple[Any, Any]] = field(default_factory=dict, repr=False)
    executor: Any = field(default=None, repr=False)   # the trunk's EmbedForward, built at the first run
    # A graph with symbolic dimensions: ``steps`` is the plan at the hint size (what ``describe`` prints); every
    # binding of the symbols met at run time gets its own static plan, kept here (one plan per sequence length, as
    # the serving runner keeps one captured graph per length). Variants share the parent's constant cache.
    symbolic: bool = False
    variants: dict[tuple, "CompiledPlan"] = field(default_factory=dict, repr=False)

    def variant_for(self, input_data: dict | None) -> "CompiledPlan":
        """The static plan for the shapes of ``input_data`` (the plan itself when the graph has no symbols)."""
        if not self.symbolic:
            return self
        env = self.graph.symbolic_env(input_data)
        missing = self.graph.symbols() - set(env)
        if missing:
            raise KeyError(f"cannot resolve symbolic dimension(s) {sorted(missing)}: supply the inputs that carry them")
        key = tuple(sorted(env.items()))
        v = self.variants.get(key)
        if v is None:
            v = lower(self.graph.resolve(env))
            v.const_cache = self.const_cache
            self.variants[key] = v
        return v

    @property
    def inputs(self) -> list[str]:
        return self.graph.inputs

    @property
    def outputs(self) -> list[str]:
        return self.graph.outputs

    @property
    def nodes(self) -> dict[str, Node]:
        return self.graph.nodes

    def symbolic_env(self, input_data=None) -> dict[str, int]:
        return self.graph.symbolic_env(input_data)

    #: size assumed for every symbolic dimension when a plan is built without inputs (compile-time validation,
    #: ``describe``, benchmarks without data) — the role of the reference's ``Dim.hint``
    SYMBOL_HINT = 128

    def describe(self) -> str:
        """The dispatch plan as text: one line per launch (what ``emmy compile --ir cuda`` prints for this backend)."""
        lines = []
        for i, s in enumerate(self.steps):
            n = self.graph.nodes[s.out]
            lines.append(f"{i:3d} {s.kernel_name:<44} {s.entry:<32} out={s.out} {list(n.output.shape)} {n.output.dtype}"
                         f" args={s.args} {s.attrs if s.attrs else ''}")
        return "\n".join(lines)


_PASSTHROUGH = {"ContiguousOp", "CloneOp", "ToOp", "TypeAsOp", "DetachOp", "AliasOp"}
_VIEWS = {"ReshapeOp", "ViewOp", "UnsqueezeOp", "SqueezeOp", "FlattenOp"}


def _name(prefix: str, node: Node) -> str:
    tag = zlib.crc32(f"{node.id}:{node.output.shape}:{node.output.dtype}".encode()) & 0xFFFFFF
    return f"k_{prefix}_{tag:06x}"


def _is_causal_mask_const(g: Graph, nid: str) -> bool:
    n = g.nodes[nid]
    return n.op == "ConstantOp" and "causal_mask" in str(n.op_fields.get("source_path") or n.id)


def _consumers(g: Graph, nid: str) -> list[str]:
    return [n.id for n in g.nodes.values() if nid in n.inputs]


def _sole_consumer_is_multiply(g: Graph, nid: str) -> bool:
    cons = _consumers(g, nid)
    if len(cons) != 1 or nid in g.outputs:
        return False
    c = g.nodes[cons[0]]
    return c.op == "ElementwiseOp" and c.op_fields.get("op") == "multiply" and all(
        g.nodes[i].output.shape == c.output.shape for i in c.inputs)


def _lower_trunk(graph: Graph) -> CompiledPlan:
    """A traced decoder trunk (embedding gather + attention in one graph): matched as a whole against the fused
    five-launches-per-layer plan (``deplodock_b200.trunk``); anything that does not match is refused."""
    from deplodock_b200 import trunk as _trunk
    from deplodock_b200.model import launch_names

    try:
        m = _trunk.recognise_trunk(graph)
    except _trunk.TrunkMismatch as exc:
        raise LoweringError(f"the graph holds an embedding gather and attention but is not the decoder trunk the "
                            f"fused plan implements: {exc}") from exc
    roles: list[list[str]] = [[m.embed, m.ids]]
    for lr in m.layers:
        roles += [[lr.wq, lr.wk, lr.wv, lr.ln1, lr.qn, lr.kn, m.cos, m.sin], [], [lr.wo], [lr.wgate, lr.wup, lr.ln2],
                  [lr.wdown]]
    roles.append([m.final_norm])
    names = launch_names(m.num_hidden_layers, True, True, False)
    assert len(names) == len(roles)
    steps = [PlanStep(name, entry, m.output, args, {"launch": i}) for i, ((name, entry), args) in
             enumerate(zip(names, roles))]
    return CompiledPlan(graph, steps, {}, trunk=m)


def lower(graph: Graph) -> CompiledPlan:
    """Op-by-op dispatch of a Torch-IR graph onto C-ABI entry points; a whole traced decoder trunk is matched onto
    the fused model plan instead."""
    from deplodock_b200 import trunk as _trunk

    if _trunk.looks_like_trunk(graph):
        return _lower_trunk(graph)
    steps: list[PlanStep] = []
    aliases: dict[str, str] = {}
    silu_of: dict[str, str] = {}   # silu nodes folded into their consuming multiply -> their operand

    def src(nid: str) -> str:
        while nid in aliases:
            nid = aliases[nid]
        return nid

    for node in graph.compute_nodes():
        op, f = node.op, node.op_fields
        ins = [src(i) for i in node.inputs]
        dt = node.output.dtype
        if op in _PASSTHROUGH or op in _VIEWS:
            aliases[node.id] = ins[0]
        elif op == "RmsNormOp":
            if dt not in ("f32", "bf16"):
                raise LoweringError(f"{node.id}: RmsNormOp in {dt} has no kernel")
            steps.append(PlanStep(_name("rms_norm", node), "emk_rmsnorm", node.id, ins[:2], {"eps": float(f.get("eps", 1e-6))}))
        elif op == "SoftmaxOp":
            axis = f.get("axis", -1)
            rank = len(node.output.shape)
            if axis not in (-1, rank - 1):
                raise LoweringError(f"{node.id}: softmax over axis {axis} has no kernel (last axis only)")
            steps.append(PlanStep(_name("softmax", node), "emk_softmax_lastdim", node.id, ins[:1]))
        elif op in ("LinearOp", "MatmulOp"):
            kn = op == "MatmulOp"
            w_shape = graph.nodes[ins[1]].output.shape
            if len(w_shape) != 2:
                raise LoweringError(f"{node.id}: batched second operand {w_shape} has no kernel")
            has_bias = bool(f.get("has_bias"))
            if dt == "bf16":
                K = w_shape[0] if kn else w_shape[1]
                N = w_shape[1] if kn else w_shape[0]
                entry = "emk_linear_bf16" if (K % 8 == 0 and N % 8 == 0) else "emk_linear_bf16_simt"
            elif dt == "f32":
                # fp32 graphs: tensor cores on exactly split bf16 operands from 256 rows on, the register-tiled
                # CUDA-core kernel below that (and for K or N not a multiple of 8)
                from deplodock_b200.ops import F32_TC_MIN_ROWS

                K = w_shape[0] if kn else w_shape[1]
                N = w_shape[1] if kn else w_shape[0]
                rows = int(np.prod(node.output.shape[:-1])) if len(node.output.shape) > 1 else 1
                entry = "emk_linear_f32_tc" if (K % 8 == 0 and N % 8 == 0 and rows >= F32_TC_MIN_ROWS) \
                    else "emk_linear_f32_simt"
            else:
                raise LoweringError(f"{node.id}: {op} in {dt} has no kernel")
            steps.append(PlanStep(_name("linear", node), entry, node.id, ins[: 3 if has_bias else 2],
                                  {"kn": kn, "has_bias": has_bias}))
        elif op == "ElementwiseOp":
            name = str(f.get("op"))
            shapes = [graph.nodes[i].output.shape for i in ins]
            if dt not in ("f32", "bf16") or name not in ("add", "multiply", "silu") or any(
                    sh != node.output.shape for sh in shapes):
                raise LoweringError(f"{node.id}: ElementwiseOp {name!r} on shapes {shapes} ({dt}) has no kernel "
                                    "(same-shape add / multiply / silu only)")
            if name == "silu" and _sole_consumer_is_multiply(graph, node.id):
                silu_of[node.id] = ins[0]   # folded into the multiply that consumes it
                continue
            if name == "multiply":
                folded = [i for i in dict.fromkeys(node.inputs) if i in silu_of]
                # silu(a) * silu(b) and silu(a) * silu(a): only one silu can ride in the multiply, so every other
                # folded operand (and a silu that is both operands) gets its own launch first
                keep = folded[0] if folded and len(set(node.inputs)) == 2 else None
                for sid in folded:
                    if sid != keep:
                        steps.append(PlanStep(_name("silu", graph.nodes[sid]), "emk_elementwise", sid,
                                              [silu_of.pop(sid)], {"op": "silu"}))
                if keep is not None:
                    other = next(i for i in node.inputs if i != keep)
                    steps.append(PlanStep(_name("silu_mul", node), "emk_elementwise", node.id,
                                          [silu_of[keep], src(other)], {"op": "silu_multiply"}))
                    continue
            # y = matmul(...) + r in bf16: the add becomes the GEMM's residual epilogue when the product has no other
            # use (not a graph output either) and r already exists when the GEMM runs: a graph input, a constant, or
            # the output of an earlier launch
            if name == "add" and dt == "bf16" and ins[0] != ins[1]:
                produced: dict[str, int] = {st.out: k for k, st in enumerate(steps)}
                for k, st in enumerate(steps):
                    if not (st.out in ins and st.entry == "emk_linear_bf16" and not st.attrs["has_bias"]
                            and "residual" not in st.attrs and _consumers(graph, st.out) == [node.id]
                            and st.out not in graph.outputs
                            and all(src(o) != st.out for o in graph.outputs)):
                        continue
                    other = next(i for i in ins if i != st.out)
                    ready = graph.node_role(other) in ("input", "constant") or produced.get(other, len(steps)) < k
                    if not ready:
                        continue
                    st.args.append(other)
                    st.attrs["residual"] = True
                    aliases[node.id] = st.out
                    break
                if node.id in aliases:
                    continue
            steps.append(PlanStep(_name(name, node), "emk_elementwise", node.id, ins[: 1 if name == "silu" else 2],
                                  {"op": name}))
        elif op == "LoopOp":
            # a Loop-IR kernel record of the reference (kernels/*.json): recognise the loop nest
            from deplodock_b200 import loopir

            try:
                m = loopir.verify(graph, node.id, loopir.classify(graph, node.id))
            except loopir.LoopRecordError as exc:
                raise LoweringError(str(exc)) from exc
            kname = f"k_{node.output.name}"
            p = m.params
            if m.kind == "rmsnorm":
                steps.append(PlanStep(kname, "emk_rmsnorm", node.id, [src(p["x"]), src(p["weight"])],
                                      {"eps": float(p["eps"])}))
            elif m.kind in ("linear", "linear_residual", "silu_gate_linear"):
                extra = [src(p[k]) for k in ("residual", "gate") if p[k] is not None]
                steps.append(PlanStep(kname, "emk_loop_linear_f32", node.id, [src(p["x"]), src(p["w"]), *extra],
                                      {"kind": m.kind, "M": p["M"], "N": p["N"], "K": p["K"], "x_inner": p["x_inner"],
                                       "x_stride_outer": p["x_stride_outer"], "x_stride_m": p["x_stride_m"]}))
            elif m.kind == "rope_scores":
                steps.append(PlanStep(kname, "emk_loop_rope_scores_f32", node.id,
                                      [src(p["q"]), src(p["k"]), src(p["cos"]), src(p["sin"])],
                                      {k: p[k] for k in ("S", "H", "Hkv", "D", "scale", "mask_zero", "mask_fill")}))
            else:  # softmax_pv
                steps.append(PlanStep(kname, "emk_loop_softmax_pv_f32", node.id, [src(p["scores"]), src(p["v"])],
                                      {k: p[k] for k in ("S", "H", "Hkv", "D")}))
        elif op == "SdpaOp":
            causal = bool(f.get("is_causal"))
            if len(ins) > 3:
                if _is_causal_mask_const(graph, ins[3]):
                    causal = True   # the HF wrapper's additive 0/-inf causal buffer: implied, never read
                else:
                    raise LoweringError(f"{node.id}: SdpaOp with a general additive mask has no kernel")
            q_shape = graph.nodes[ins[0]].output.shape
            k_shape = graph.nodes[ins[1]].output.shape
            if len(q_shape) != 4:
                raise LoweringError(f"{node.id}: SdpaOp expects [B,H,S,D] operands, got {q_shape}")
            fast = dt == "bf16" and causal and q_shape[-1] == 128 and q_shape[2] == k_shape[2]
            steps.append(PlanStep(_name("scaled_dot_product_attention", node),
                                  "emk_sdpa_causal_gqa_bf16" if fast else "emk_sdpa_simt", node.id, ins[:3],
                                  {"causal": causal}))
        else:
            raise LoweringError(
                f"{node.id}: Torch-IR op {op} has no hand-written kernel in this backend (whole Qwen3-shaped trunks go "
                "through deplodock_b200.model.EmbedForward)")
    return CompiledPlan(graph, steps, aliases)


def dump_plan(plan: CompiledPlan, dump_dir) -> None:
    """Write the compilation artefacts the reference's dumper writes for the stages this backend has
    (``emmy/compiler/pipeline/dump.py:125-206``): ``00_torch.json`` (the input graph), ``50_cuda.kernels.txt`` (the
    launch plan) and per launch ``50_cuda.kernels/<kname>.torch.json`` — the Torch op behind that launch as a
    stand-alone sub-graph that ``python -m deplodock_b200 run --ir <file> --bench`` re-runs — with a
    ``<kname>.torch.txt`` header giving its origin node and ``i/N`` coverage (always ``1/1 — full`` here: one launch
    per Torch op, nothing is split or fused at this level)."""
    import json
    from pathlib import Path

    d = Path(dump_dir)
    (d / "50_cuda.kernels").mkdir(parents=True, exist_ok=True)
    (d / "00_torch.json").write_text(json.dumps(plan.graph.to_dict(), indent=1))
    (d / "50_cuda.kernels.txt").write_text(plan.describe() + "\n")
    if plan.trunk is not None:
        return   # the launches of a fused trunk are not single Torch ops: no per-kernel sub-graph records
    for s in plan.steps:
        node = plan.graph.nodes[s.out]
        sub = plan.graph.single_node_graph(s.out, operands=list(s.args) + [i for i in node.inputs[len(s.args):]
                                                                          if plan.graph.nodes[i].op == "ConstantOp"])
        (d / "50_cuda.kernels" / f"{s.kernel_name}.torch.json").write_text(json.dumps(sub.to_dict(), indent=1))
        (d / "50_cuda.kernels" / f"{s.kernel_name}.torch.txt").write_text(
            f"# matching torch ops for kernel '{s.kernel_name}' ({s.entry})\n"
            f"#   {s.out} ({node.op}): 1/1 — full\n")


# ------------------------------------------------------------------------------------------------------------
# Backend
# ------------------------------------------------------------------------------------------------------------
class B200Backend(Backend):
    """Drop-in for ``CudaBackend`` on B200. Constructor keywords match ``CudaBackend.__init__``
    (``backend/cuda/backend.py:70-112``); ``dump``, ``tune_db`` and the bench budgets are accepted and unused (there are
    no variants to tune and nothing to compile)."""

    name = "b200"

    def __init__(self, *, debug: bool | None = None, dump=None, bench_wall_timeout_s: float | None = None,
                 bench_compile_timeout_s: float = 30.0, bench_run_timeout_s: float = 10.0, tune_db=None,
                 device_id: int | None = None) -> None:
        self.debug = bool(debug)
        self.dump = dump
        self.bench_wall_timeout_s = bench_wall_timeout_s
        self.bench_compile_timeout_s = bench_compile_timeout_s
        self.bench_run_timeout_s = bench_run_timeout_s
        self.tune_db = tune_db
        self.device_id = device_id
        self.last_debug_result = None

    def close_async_worker(self) -> None:
        """The reference kills its bench subprocess here; this backend benches in-process (every wait is bounded)."""

    async def aclose_async_worker(self) -> None:
        return None

    # -- compile -----------------------------------------------------------------------------------------------
    def compile(self, graph: Any) -> CompiledPlan:
        if isinstance(graph, CompiledPlan):
            return graph
        g = Graph.coerce(graph)
        if g.is_symbolic:
            # validated (and listed) at the hint size; the launch plan proper is built per binding at run time
            hint = lower(g.resolve({name: CompiledPlan.SYMBOL_HINT for name in g.symbols()}))
            plan = CompiledPlan(g, hint.steps, hint.aliases, trunk=hint.trunk, symbolic=True)
        else:
            plan = lower(g)
        if self.dump:
            dump_plan(plan, self.dump)
        return plan

    # -- run ---------------------------------------------------------------------------------------------------
    def _device(self):
        import torch

        return torch.device("cuda", self.device_id if self.device_id is not None else torch.cuda.current_device())

    def _upload(self, plan: CompiledPlan, input_data: dict[str, Any]) -> dict[str, Any]:
        """Host arrays -> device tensors for inputs and constants (cast to the node dtype). The device copy of a
        weight constant is kept on the plan and reused while the caller passes the same host object again."""
        import torch

        dev = self._device()
        vals: dict[str, torch.Tensor] = {}
        g = plan.graph
        want_dtype = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16, "i64": torch.int64,
                      "i32": torch.int32, "bool": torch.bool}
        fresh_constants = False
        for nid, node in g.nodes.items():
            role = g.node_role(nid)
            if role not in ("input", "constant"):
                continue
            info = node.output
            if nid in input_data:
                arr = input_data[nid]
                cached = plan.const_cache.get(nid) if role == "constant" else None
                if cached is not None and cached[0] is arr and cached[1].device == dev:
                    vals[nid] = cached[1]
                    continue
                if isinstance(arr, torch.Tensor):
                    t = arr
                else:
                    a = np.ascontiguousarray(np.asarray(arr))
                    if info.dtype == "bf16" and a.dtype == np.uint16:
                        t = torch.from_numpy(a.view(np.int16)).view(torch.bfloat16)
                    else:
                        t = torch.from_numpy(a)
                t = t.to(device=dev, dtype=want_dtype[info.dtype]).reshape(info.shape).contiguous()
                vals[nid] = t
                if role == "constant":
                    plan.const_cache[nid] = (arr, t)
                    fresh_constants = True
            elif role == "input":
                raise KeyError(f"Missing input for node {nid!r}")
            elif node.op_fields.get("value") is not None:
                vals[nid] = torch.tensor([float(node.op_fields["value"])], device=dev)
            else:
                used = any(nid in s.args for s in plan.steps)
                if used:
                    raise KeyError(f"ConstantOp {nid!r} has no value and was not supplied in input_data")
        if plan.trunk is not None:
            if plan.executor is None or fresh_constants:
                plan.executor = self._build_trunk_executor(plan, vals, dev)
            vals["__executor__"] = plan.executor
        return vals

    @staticmethod
    def _build_trunk_executor(plan: CompiledPlan, vals: dict[str, Any], dev):
        """The fused model plan for a recognised trunk: weights re-laid out once (q/k/v concatenated, gate/up
        interleaved, norm weights folded), rotary tables taken from the graph's own cos/sin buffers."""
        from deplodock_b200.model import EmbedConfig, EmbedForward

        m = plan.trunk
        cfg = EmbedConfig(vocab_size=m.vocab_size, hidden_size=m.hidden_size, intermediate_size=m.intermediate_size,
                          num_hidden_layers=m.num_hidden_layers, num_attention_heads=m.num_attention_heads,
                          num_key_value_heads=m.num_key_value_heads, head_dim=m.head_dim,
                          rms_norm_eps=m.rms_norm_eps, rope_theta=0.0)
        sd = {name: vals[nid] for name, nid in m.state_dict_names().items()}
        ex = EmbedForward(cfg, sd, batch=m.batch, seq=m.seq, device=dev, hidden_states=True, pool=False,
                          rope=(vals[m.cos], vals[m.sin]), chain=False)   # one launch per listed kernel
        ex.launches = ex.launch_list(ex.ids, ex.out)
        return ex

    def _execute(self, plan: CompiledPlan, vals: dict[str, Any], step_idx: int | None = None) -> None:
        from deplodock_b200 import ops

        steps = plan.steps if step_idx is None else [plan.steps[step_idx]]
        g = plan.graph
        if plan.trunk is not None:
            ex, m = vals["__executor__"], plan.trunk
            if step_idx is None or step_idx == 0:
                ex.ids.copy_(vals[m.ids].reshape(ex.ids.shape))
            for s in steps:
                ex.launches[s.attrs["launch"]][2]()
            vals[m.output] = ex.hs.view(m.batch, m.seq, m.hidden_size)
            return
        for s in steps:
            a = [vals[i] for i in s.args]
            shape = g.nodes[s.out].output.shape
            if s.entry == "emk_rmsnorm":
                y = ops.rmsnorm(a[0], a[1].reshape(-1), s.attrs["eps"])
            elif s.entry == "emk_softmax_lastdim":
                y = ops.softmax_lastdim(a[0])
            elif s.entry in ("emk_linear_bf16", "emk_linear_bf16_simt"):
                fn = ops.linear if s.entry == "emk_linear_bf16" else ops.linear_simt
                if s.attrs.get("residual"):
                    y = fn(a[0], a[1], residual=a[2].reshape(-1, a[1].shape[1 if s.attrs["kn"] else 0]).contiguous(),
                           w_is_kn=s.attrs["kn"])
                else:
                    y = fn(a[0], a[1], bias=a[2].reshape(-1) if s.attrs["has_bias"] else None, w_is_kn=s.attrs["kn"])
            elif s.entry in ("emk_linear_f32_simt", "emk_linear_f32_tc"):
                y = ops.linear_f32(a[0], a[1], a[2].reshape(-1) if s.attrs["has_bias"] else None, s.attrs["kn"],
                                   route="tc" if s.entry == "emk_linear_f32_tc" else "simt")
            elif s.entry == "emk_loop_linear_f32":
                at = s.attrs
                extra = a[2] if len(a) > 2 else None
                y = ops.loop_linear_f32(a[0].reshape(-1), a[1], at["M"], at["N"], at["K"], x_inner=at["x_inner"],
                                        x_stride_outer=at["x_stride_outer"], x_stride_m=at["x_stride_m"],
                                        residual=extra if at["kind"] == "linear_residual" else None,
                                        gate=extra if at["kind"] == "silu_gate_linear" else None)
            elif s.entry == "emk_elementwise":
                y = ops.elementwise(s.attrs["op"], a[0].contiguous(), a[1].contiguous() if len(a) > 1 else None)
            elif s.entry == "emk_loop_rope_scores_f32":
                at = s.attrs
                y = ops.loop_rope_scores_f32(a[0], a[1], a[2], a[3], at["S"], at["H"], at["Hkv"], at["D"], at["scale"],
                                             at["mask_zero"], at["mask_fill"])
            elif s.entry == "emk_loop_softmax_pv_f32":
                at = s.attrs
                y = ops.loop_softmax_pv_f32(a[0], a[1], at["S"], at["H"], at["Hkv"], at["D"])
            elif s.entry == "emk_sdpa_causal_gqa_bf16":
                y = ops.sdpa_causal_gqa(a[0], a[1], a[2])
            elif s.entry == "emk_sdpa_simt":
                y = ops.sdpa_simt(a[0], a[1], a[2], s.attrs["causal"])
            else:  # pragma: no cover - lower() only emits the entries above
                raise LoweringError(f"no executor for {s.entry}")
            vals[s.out] = y.reshape(shape)
        for alias, target in plan.aliases.items():
            if target in vals and (step_idx is None):
                vals[alias] = vals[target].reshape(g.nodes[alias].output.shape)

    def _download(self, plan: CompiledPlan, vals: dict[str, Any]) -> dict[str, np.ndarray]:
        import torch

        outs: dict[str, np.ndarray] = {}
        for name in plan.outputs:
            t = vals[name] if name in vals else vals[plan.aliases[name]]
            info = plan.graph.nodes[name].output
            t = t.reshape(info.shape).contiguous()
            if info.dtype == "bf16":
                outs[name] = t.view(torch.int16).cpu().numpy().view(np.uint16)
            else:
                outs[name] = t.cpu().numpy().astype(info.np_dtype, copy=False)
        return outs

    def run(self, compiled: Any, *, input_data: dict[str, np.ndarray] | None = None,
            pre_run: Callable[[], Any] | None = None) -> tuple[RunResult, Any]:
        import torch

        from deplodock_b200 import ops

        from deplodock_b200.gpu_lock import gpu_lock

        plan = self.compile(compiled).variant_for(input_data)
        with gpu_lock():   # the reference runs pre_run (its eager check) inside the same lock window, base.py:143-157
            pre_result = pre_run() if pre_run is not None else None
            vals = self._upload(plan, input_data or {})
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            self._execute(plan, vals)
            stop.record()
            ops.device_status()  # synchronises; raises HungKernelError / RuntimeError on device-side failure
            elapsed = start.elapsed_time(stop)
            if plan.steps and elapsed <= 0.0:
                raise RuntimeError("zero elapsed time for a non-empty program")  # reference: program.py:1027-1031
            return RunResult(outputs=self._download(plan, vals), time_ms=elapsed), pre_result

    # -- benchmark ---------------------------------------------------------------------------------------------
    async def benchmark_async(self, compiled: Any, *, warmup: int = 5, num_iters: int | str = 20, on_iter=None,
                              nvcc_flags: str | None = None, capture_graphs: bool = True,
                              input_data: dict[str, np.ndarray] | None = None) -> BenchmarkResult:
        """Per-launch median/min over CUDA-graph-captured windows and a whole-program window — the reference's
        protocol (``backend/cuda/program.py:1152-1374``). Inputs not supplied are filled with the reference's
        deterministic pattern ``0.01 * ((7 i + 13) mod 101 - 50)`` (``program.py:265-276``)."""
        await asyncio.sleep(0)
        return self._benchmark(self.compile(compiled), warmup, num_iters, on_iter, capture_graphs, input_data)

    def benchmark(self, compiled: Any, **kw) -> BenchmarkResult:
        """Synchronous form of :meth:`benchmark_async`."""
        kw.pop("nvcc_flags", None)
        return self._benchmark(self.compile(compiled), kw.get("warmup", 5), kw.get("num_iters", 20), kw.get("on_iter"),
                               kw.get("capture_graphs", True), kw.get("input_data"))

    @staticmethod
    def _default_fill(shape: tuple[int, ...], dtype: str) -> np.ndarray:
        n = int(np.prod(shape)) if shape else 1
        i = np.arange(n, dtype=np.int64)
        base = (0.01 * (((7 * i + 13) % 101) - 50)).astype(np.float32).reshape(shape)
        if dtype in ("i64", "i32"):
            return np.zeros(shape, dtype=np.int64)
        return base

    def _benchmark(self, plan: CompiledPlan, warmup, num_iters, on_iter, capture_graphs, input_data) -> BenchmarkResult:
        import torch

        from deplodock_b200 import ops

        from deplodock_b200.gpu_lock import gpu_lock

        if plan.symbolic:
            if input_data and plan.graph.symbols() <= set(plan.graph.symbolic_env(input_data)):
                plan = plan.variant_for(input_data)
            else:   # no inputs to read the sizes from: bench at the hint size
                plan = lower(plan.graph.resolve({n: CompiledPlan.SYMBOL_HINT for n in plan.graph.symbols()}))
        with gpu_lock():
            return self._benchmark_locked(plan, warmup, num_iters, on_iter, capture_graphs, input_data)

    def _benchmark_locked(self, plan: CompiledPlan, warmup, num_iters, on_iter, capture_graphs,
                          input_data) -> BenchmarkResult:
        import torch

        from deplodock_b200 import ops

        iters = 20 if num_iters == "auto" else int(num_iters)
        data = dict(input_data or {})
        for nid, node in plan.graph.nodes.items():
            if plan.graph.node_role(nid) in ("input", "constant") and nid not in data \
                    and node.op_fields.get("value") is None:
                data[nid] = self._default_fill(node.output.shape, node.output.dtype)
        vals = self._upload(plan, data)
        for _ in range(max(1, warmup)):
            self._execute(plan, vals)
        ops.device_status()

        def window(fn, reps: int) -> list[float]:
            """``iters`` samples of ms per call, each a replay of ``reps`` captured back-to-back launches."""
            graph = None
            if capture_graphs:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    for _ in range(reps):
                        fn()
            samples = []
            for it in range(iters):
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record()
                if graph is not None:
                    graph.replay()
                else:
                    for _ in range(reps):
                        fn()
                e.record()
                torch.cuda.synchronize()
                samples.append(s.elapsed_time(e) / reps)
                if on_iter is not None:
                    on_iter(it)
            return samples

        per_launch: list[LaunchTime] = []
        for idx, step in enumerate(plan.steps):
            s0, e0 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s0.record()
            self._execute(plan, vals, idx)
            e0.record()
            torch.cuda.synchronize()
            one = max(s0.elapsed_time(e0), 1e-3)
            reps = int(min(512, max(1, round(1.0 / one))))  # ~1 ms windows, as the reference calibrates
            samples = window(lambda i=idx: self._execute(plan, vals, i), reps)
            per_launch.append(LaunchTime(idx, step.kernel_name, statistics.median(samples), tuple(samples)))
        e2e = e2e_min = None
        if len(plan.steps) > 1:
            samples = window(lambda: self._execute(plan, vals), 1)
            e2e, e2e_min = statistics.median(samples), min(samples)
        ops.device_status()
        return BenchmarkResult(
            time_ms=sum(lt.time_ms for lt in per_launch),
            min_ms=sum(min(lt.samples) for lt in per_launch),
            max_ms=sum(max(lt.samples) for lt in per_launch),
            num_launches=len(per_launch), per_launch=per_launch, captured=bool(capture_graphs),
            e2e_ms=e2e, e2e_min_ms=e2e_min)
