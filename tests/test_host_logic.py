"""Host-side logic that needs no GPU: record loading, op dispatch, status mapping, sharding, gather (gloo ranks)."""

from __future__ import annotations

import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from conftest import GOLDEN

ROOT = Path(__file__).resolve().parent.parent


# ---------------------------------------------------------------------------------------------------- graph records
def test_graph_records_load_and_dispatch():
    from deplodock_b200.backend import B200Backend
    from deplodock_b200.graph import Graph

    be = B200Backend()
    expect = {
        "cfg1_rmsnorm": ["emk_rmsnorm"],
        "cfg2_softmax": ["emk_softmax_lastdim"],
        "cfg3_linear_bf16": ["emk_linear_bf16"],
        "cfg4_sdpa_bf16": ["emk_sdpa_causal_gqa_bf16"],
        "linear_f32": ["emk_linear_f32_simt"],
        "linear_bias_f32": ["emk_linear_f32_simt"],
        "matmul_f32": ["emk_linear_f32_simt"],
        "sdpa_causal_gqa_f32": ["emk_sdpa_simt"],
        "sdpa_full_f32": ["emk_sdpa_simt"],
    }
    for name, entries in expect.items():
        g = Graph.from_json(GOLDEN / "graphs" / f"{name}.json")
        plan = be.compile(g)
        assert [s.entry for s in plan.steps] == entries, name
        assert all(s.kernel_name.startswith("k_") for s in plan.steps)
        assert plan.inputs == g.inputs and plan.outputs == g.outputs and plan.symbolic_env({}) == {}
        assert plan.describe()
    plan = be.compile(GOLDEN / "graphs" / "cfg4_sdpa_bf16.json")
    assert plan.steps[0].attrs["causal"] is True
    assert be.compile(plan) is plan


def test_kernel_names_are_stable_across_processes():
    from deplodock_b200.backend import B200Backend

    a = B200Backend().compile(GOLDEN / "graphs" / "cfg1_rmsnorm.json").steps[0].kernel_name
    b = B200Backend().compile(GOLDEN / "graphs" / "cfg1_rmsnorm.json").steps[0].kernel_name
    assert a == b and a.startswith("k_rms_norm_")


def test_unsupported_ops_raise_lowering_error():
    from deplodock_b200.backend import B200Backend, LoweringError

    plan = B200Backend().compile(GOLDEN / "graphs" / "swiglu_f32.json")   # silu folded into the multiply
    assert [s.entry for s in plan.steps] == ["emk_linear_f32_simt", "emk_linear_f32_simt", "emk_elementwise"]
    assert plan.steps[2].attrs == {"op": "silu_multiply"} and plan.steps[2].args == ["matmul", "matmul_1"]
    rec = {"inputs": ["x"], "outputs": ["s"], "nodes": {
        "x": {"op": "InputOp", "op_fields": {}, "inputs": [], "output": {"name": "x", "shape": [4, 8], "dtype": "f32"}},
        "s": {"op": "SoftmaxOp", "op_fields": {"axis": 0}, "inputs": ["x"],
              "output": {"name": "s", "shape": [4, 8], "dtype": "f32"}}}}
    with pytest.raises(LoweringError):
        B200Backend().compile(rec)


def test_graph_validation_errors():
    from deplodock_b200.graph import Graph

    base = {"inputs": ["x"], "outputs": ["y"], "nodes": {
        "x": {"op": "InputOp", "op_fields": {}, "inputs": [], "output": {"name": "x", "shape": [2], "dtype": "f32"}}}}
    with pytest.raises(KeyError):
        Graph.from_dict(base)
    bad = {"inputs": ["x"], "outputs": ["x"], "nodes": {
        "x": {"op": "InputOp", "op_fields": {}, "inputs": [], "output": {"name": "x", "shape": ["seq len ("], "dtype": "f32"}}}}
    with pytest.raises(ValueError):
        Graph.from_dict(bad)
    bad["nodes"]["x"]["output"] = {"name": "x", "shape": [2.5], "dtype": "f32"}
    with pytest.raises(ValueError):
        Graph.from_dict(bad)
    bad["nodes"]["x"]["output"] = {"name": "x", "shape": [2], "dtype": "q4"}
    with pytest.raises(TypeError):
        Graph.from_dict(bad)


def test_backend_constructor_matches_reference_keywords():
    from deplodock_b200.backend import B200Backend, Backend

    be = B200Backend(debug=False, dump=None, bench_wall_timeout_s=5.0, bench_compile_timeout_s=1.0,
                     bench_run_timeout_s=2.0, tune_db="auto", device_id=0)
    assert isinstance(be, Backend) and be.name == "b200"
    assert be.bench_run_timeout_s == 2.0 and be.device_id == 0
    be.close_async_worker()


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from deplodock_b200 import cabi

    monkeypatch.setattr(cabi, "_lib", None)
    monkeypatch.setattr(cabi, "LIB_PATH", tmp_path / "libemk.so")
    with pytest.raises(cabi.EmkLibraryMissing):
        cabi.load_library()


def test_ops_refuse_to_run_without_cuda(libemk):
    from deplodock_b200 import ops

    if torch.cuda.is_available():
        pytest.skip("CUDA present")
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        ops.rmsnorm(torch.zeros(2, 8), torch.ones(8))


def test_status_codes_map_to_reference_exception_types(libemk):
    from deplodock_b200 import cabi

    class FakeHandle(cabi.Handle):
        def __init__(self):  # no device
            self.lib = cabi.load_library()
            self.ptr = None

        def last_error(self):
            return "detail"

    h = FakeHandle()
    h.check(cabi.EMK_OK, "ok")
    for rc, exc in [(cabi.EMK_ERR_SHAPE, ValueError), (cabi.EMK_ERR_ALIGN, ValueError), (cabi.EMK_ERR_LIMIT, ValueError),
                    (cabi.EMK_ERR_DTYPE, TypeError), (cabi.EMK_ERR_TIMEOUT, cabi.HungKernelError),
                    (cabi.EMK_ERR_CUDA, RuntimeError)]:
        with pytest.raises(exc):
            h.check(rc, "call")
    assert issubclass(cabi.HungKernelError, RuntimeError)


# ---------------------------------------------------------------------------------------------------- model config
def test_model_flop_accounting_matches_the_benchmark_figures():
    from deplodock_b200.model import EmbedConfig

    cfg = EmbedConfig()
    lin = cfg.linear_flops_per_token() * 64 * 512
    att = cfg.attention_flops(64, 512)
    assert lin == 2 * 32768 * 440401920
    assert att == 28 * 4 * 64 * 16 * 128 * 131328
    assert abs((lin + att) / 3.079e13 - 1) < 2e-3


# ---------------------------------------------------------------------------------------------------- sharding
def test_shard_batch_covers_everything_once():
    from deplodock_b200.dist import shard_batch

    for total in (0, 1, 7, 64, 65):
        for world in (1, 2, 3, 4, 8):
            shards = [shard_batch(total, r, world) for r in range(world)]
            assert shards[0].start == 0 and shards[-1].stop == total
            assert all(a.stop == b.start for a, b in zip(shards, shards[1:]))
            assert max(s.size for s in shards) - min(s.size for s in shards) <= 1
    with pytest.raises(ValueError):
        shard_batch(8, 2, 2)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _gather_worker(rank: int, world: int, port: int, total: int, q) -> None:
    sys.path.insert(0, str(ROOT))
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    import torch.distributed as dist

    from deplodock_b200.dist import gather_embeddings, init_process_group, shard_batch

    r, _, w = init_process_group("gloo")
    sh = shard_batch(total, r, w)
    full = torch.arange(total * 4, dtype=torch.float32).reshape(total, 4)
    got = gather_embeddings(full[sh.start:sh.stop].clone(), total)
    q.put((rank, torch.equal(got, full)))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("total", [8, 7])
def test_gather_embeddings_two_gloo_ranks(total):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_gather_worker, args=(r, 2, port, total, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert results == [(0, True), (1, True)]


def _failing_rank_worker(rank: int, world: int, port: int, q) -> None:
    """Rank 1 never joins the collective; rank 0's gather must end with an error within the group timeout."""
    sys.path.insert(0, str(ROOT))
    import datetime

    import torch.distributed as dist

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=5))
    if rank == 1:
        q.put((1, "left"))
        q.close()
        q.join_thread()
        os._exit(0)  # leaves between steps, no collective in flight
    try:
        t = torch.zeros(4, 4)
        out = torch.empty(8, 4)
        dist.all_gather_into_tensor(out, t)
        q.put((0, "completed"))
    except Exception as ex:  # noqa: BLE001
        q.put((0, "error:" + type(ex).__name__))
    q.close()
    q.join_thread()
    os._exit(0)


def test_rank_that_leaves_is_detected_by_group_timeout():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_failing_rank_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
    assert results[1] == "left"
    assert results[0].startswith("error:"), results


# ---------------------------------------------------------------------------------------------------- bench contract
def test_bench_reference_arm_prints_contract_line(monkeypatch, capsys):
    """The CPU arm of bench.py on a tiny stand-in model: one JSON line with the contract's keys."""
    import json

    sys.path.insert(0, str(ROOT))
    import bench
    from oracle import inputs

    small = inputs.EmbedModelConfig().small(layers=1, vocab=128)
    monkeypatch.setattr(inputs, "EmbedModelConfig", lambda: small)
    monkeypatch.setattr(bench, "SEQ", 64)

    class A:
        gpus, steps, warmup = 1, 1, 0

    bench.run_reference_arm(A())
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better",
                "scaling", "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in line
    assert line["impl"] == "reference" and line["value"] > 0 and line["e2e"]["h2d_bytes_per_step"] == 0


# ------------------------------------------------------------------------------------------- folds keep launch order
def _rec(nodes: dict, inputs: list[str], outputs: list[str]) -> dict:
    out = {}
    for nid, (op, ins, shape, dtype, fields) in nodes.items():
        out[nid] = {"op": op, "op_fields": dict(fields), "inputs": list(ins),
                    "output": {"name": nid, "shape": list(shape), "dtype": dtype}}
    return {"inputs": inputs, "outputs": outputs, "nodes": out}


def _assert_args_produced_before_use(plan):
    ready = {nid for nid in plan.graph.nodes if plan.graph.node_role(nid) in ("input", "constant")}
    for st in plan.steps:
        for a in st.args:
            assert a in ready, f"{st.kernel_name} reads {a!r} before any launch wrote it"
        ready.add(st.out)
    for o in plan.outputs:
        t = o
        while t in plan.aliases:
            t = plan.aliases[t]
        assert t in ready


def test_residual_fold_waits_for_its_addend():
    """``matmul(x, w) + rms_norm(x)``: the addend is computed after the product, so the add cannot ride in the GEMM
    that was already placed; ``matmul(x, w) + r`` with r a graph input still folds."""
    from deplodock_b200.backend import lower
    from deplodock_b200.graph import Graph

    bf = "bf16"
    late = _rec({
        "x": ("InputOp", [], [64, 256], bf, {}), "w": ("ConstantOp", [], [256, 256], bf, {}),
        "g": ("ConstantOp", [], [256], bf, {}),
        "mm": ("MatmulOp", ["x", "w"], [64, 256], bf, {}),
        "rn": ("RmsNormOp", ["x", "g"], [64, 256], bf, {"eps": 1e-6}),
        "add": ("ElementwiseOp", ["mm", "rn"], [64, 256], bf, {"op": "add"})}, ["x"], ["add"])
    plan = lower(Graph.from_dict(late))
    _assert_args_produced_before_use(plan)
    assert [s.entry for s in plan.steps] == ["emk_linear_bf16", "emk_rmsnorm", "emk_elementwise"]
    early = _rec({
        "x": ("InputOp", [], [64, 256], bf, {}), "r": ("InputOp", [], [64, 256], bf, {}),
        "w": ("ConstantOp", [], [256, 256], bf, {}),
        "mm": ("MatmulOp", ["x", "w"], [64, 256], bf, {}),
        "add": ("ElementwiseOp", ["mm", "r"], [64, 256], bf, {"op": "add"})}, ["x", "r"], ["add"])
    plan = lower(Graph.from_dict(early))
    _assert_args_produced_before_use(plan)
    assert [s.entry for s in plan.steps] == ["emk_linear_bf16"] and plan.steps[0].attrs["residual"] is True
    # the bare product is a graph output too: folding would return the sum in its place
    both = dict(early)
    both["outputs"] = ["add", "mm"]
    plan = lower(Graph.from_dict(both))
    _assert_args_produced_before_use(plan)
    assert [s.entry for s in plan.steps] == ["emk_linear_bf16", "emk_elementwise"]
    # p + p
    twice = _rec({
        "x": ("InputOp", [], [64, 256], bf, {}), "w": ("ConstantOp", [], [256, 256], bf, {}),
        "mm": ("MatmulOp", ["x", "w"], [64, 256], bf, {}),
        "add": ("ElementwiseOp", ["mm", "mm"], [64, 256], bf, {"op": "add"})}, ["x"], ["add"])
    plan = lower(Graph.from_dict(twice))
    _assert_args_produced_before_use(plan)
    assert [s.entry for s in plan.steps] == ["emk_linear_bf16", "emk_elementwise"]


def test_silu_fold_with_two_silu_operands():
    from deplodock_b200.backend import lower
    from deplodock_b200.graph import Graph

    f = "f32"
    two = _rec({
        "a": ("InputOp", [], [8, 32], f, {}), "b": ("InputOp", [], [8, 32], f, {}),
        "sa": ("ElementwiseOp", ["a"], [8, 32], f, {"op": "silu"}),
        "sb": ("ElementwiseOp", ["b"], [8, 32], f, {"op": "silu"}),
        "m": ("ElementwiseOp", ["sa", "sb"], [8, 32], f, {"op": "multiply"})}, ["a", "b"], ["m"])
    plan = lower(Graph.from_dict(two))
    _assert_args_produced_before_use(plan)
    assert [s.attrs["op"] for s in plan.steps] == ["silu", "silu_multiply"]
    assert plan.steps[1].args == ["a", "sb"]
    same = _rec({
        "a": ("InputOp", [], [8, 32], f, {}),
        "sa": ("ElementwiseOp", ["a"], [8, 32], f, {"op": "silu"}),
        "m": ("ElementwiseOp", ["sa", "sa"], [8, 32], f, {"op": "multiply"})}, ["a"], ["m"])
    plan = lower(Graph.from_dict(same))
    _assert_args_produced_before_use(plan)
    assert [s.attrs["op"] for s in plan.steps] == ["silu", "multiply"] and plan.steps[1].args == ["sa", "sa"]


def test_ops_check_buffer_sizes_before_the_call():
    """Caller-provided buffers reach the library as raw pointers: a short or mistyped one must be a Python error."""
    from deplodock_b200 import ops

    with pytest.raises(ValueError, match="holds 8 elements"):
        ops._check_buffer("row_sumsq_out", torch.zeros(8), 16, torch.float32)
    with pytest.raises(TypeError):
        ops._check_buffer("out", torch.zeros(16), 16, torch.bfloat16)
    ops._check_buffer("out", None, 16, torch.bfloat16)


# ------------------------------------------------------------------------------------------------ symbolic dimensions
def _symbolic_record():
    return _rec({
        "x": ("InputOp", [], [2, "seq_len", 256], "f32", {}),
        "w": ("ConstantOp", [], [256], "f32", {}),
        "y": ("RmsNormOp", ["x", "w"], [2, "seq_len", 256], "f32", {"eps": 1e-6}),
        "flat": ("ReshapeOp", ["y"], ["(seq_len * 2)", 256], "f32", {"shape": ["(seq_len * 2)", 256]})}, ["x"], ["flat"])


def test_symbolic_dims_resolve_from_input_shapes():
    """Records carry atomic symbolic dims as names and composite ones as expressions (``emmy/compiler/graph.py:953-1007``);
    the values come from the input arrays (``graph.py:686-706``)."""
    from deplodock_b200.graph import Graph, eval_dim

    g = Graph.from_dict(_symbolic_record())
    assert g.is_symbolic and g.symbols() == {"seq_len"}
    assert g.symbolic_env(None) == {} and g.symbolic_env({"w": np.zeros(256)}) == {}
    env = g.symbolic_env({"x": np.zeros((2, 37, 256), dtype=np.float32)})
    assert env == {"seq_len": 37}
    r = g.resolve(env)
    assert not r.is_symbolic and r.nodes["flat"].output.shape == (74, 256) and r.nodes["flat"].op_fields["shape"] == [74, 256]
    assert g.nodes["x"].output.shape == (2, "seq_len", 256)   # the record itself is unchanged
    assert g.to_dict()["nodes"]["x"]["output"]["shape"] == [2, "seq_len", 256]
    assert eval_dim("round_up(seq_len, 64) // 2 + min(seq_len, 8)", {"seq_len": 100}) == 72
    with pytest.raises(KeyError):
        g.resolve({})
    with pytest.raises(ValueError):
        eval_dim("seq_len ** 2", {"seq_len": 3})


def test_symbolic_graph_compiles_to_one_plan_per_binding():
    from deplodock_b200.backend import B200Backend

    plan = B200Backend().compile(_symbolic_record())
    assert plan.symbolic and [s.entry for s in plan.steps] == ["emk_rmsnorm"] and "seq_len" in plan.describe()
    assert plan.symbolic_env({"x": np.zeros((2, 5, 256))}) == {"seq_len": 5}
    a = plan.variant_for({"x": np.zeros((2, 5, 256))})
    b = plan.variant_for({"x": np.zeros((2, 9, 256))})
    assert a is not b and a is plan.variant_for({"x": np.zeros((2, 5, 256))}) and len(plan.variants) == 2
    assert a.graph.nodes["flat"].output.shape == (10, 256) and b.graph.nodes["y"].output.shape == (2, 9, 256)
    assert a.const_cache is plan.const_cache          # weights are uploaded once for all bindings
    with pytest.raises(KeyError):
        plan.variant_for({})


def test_dynamic_spec_grammar_and_tracing():
    from deplodock_b200.trace import parse_dynamic_specs, trace_inline_code

    assert parse_dynamic_specs(["seq_len@x:1", "seq_len@mask:2"]) == [("seq_len", "x", 1), ("seq_len", "mask", 2)]
    for bad in ("seq_len", "seq_len@x", "@x:1", "s@:1", "s@x:one", "s@x:-1"):
        with pytest.raises(ValueError):
            parse_dynamic_specs([bad])
    with pytest.raises(ValueError):
        parse_dynamic_specs(["a@x:1", "b@x:1"])
    tr = trace_inline_code("nn.RMSNorm(256, eps=1e-6)(torch.randn(2, 5, 256))", parse_dynamic_specs(["seq_len@x:1"]))
    assert tr.graph.nodes["x"].output.shape == (2, "seq_len", 256)
    assert tr.graph.nodes["rms_norm"].output.shape == (2, "seq_len", 256)
    with pytest.raises(ValueError, match="no input named"):
        trace_inline_code("nn.RMSNorm(256)(torch.randn(2, 5, 256))", [("s", "nope", 1)])


def test_backend_subclasses_the_reference_base_when_it_is_importable():
    """Inside the reference's process ``B200Backend`` must BE a reference ``Backend`` (its callers check with
    isinstance) and hand back the reference's own result dataclasses. Needs the reference checkout: skipped without."""
    import subprocess

    from oracle import build_ref_kernels

    ref = build_ref_kernels.find_reference()
    if ref is None:
        pytest.skip("reference checkout not present")
    code = (
        "import sys; sys.path.insert(0, %r)\n"
        "from deplodock_b200 import backend\n"
        "from emmy.compiler.backend.base import Backend, RunResult, BenchmarkResult, LaunchTime\n"
        "b = backend.B200Backend(device_id=0)\n"
        "assert backend.USES_REFERENCE_TYPES and isinstance(b, Backend)\n"
        "assert backend.RunResult is RunResult and backend.BenchmarkResult is BenchmarkResult\n"
        "assert backend.LaunchTime is LaunchTime\n"
        "print('OK', len(b.compile(%r).steps))\n") % (str(ROOT), str(GOLDEN / "graphs" / "cfg1_rmsnorm.json"))
    res = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300,
                         env=dict(os.environ, PYTHONPATH=ref))
    assert res.returncode == 0 and "OK 1" in res.stdout, res.stderr[-2000:]
    from deplodock_b200 import backend

    assert not backend.USES_REFERENCE_TYPES   # and stand-alone it defines the same types itself
    assert [f for f in backend.BenchmarkResult.__dataclass_fields__] == [
        "time_ms", "min_ms", "max_ms", "num_launches", "per_launch", "captured", "e2e_ms", "e2e_min_ms"]


def test_launch_names_of_the_chained_plan():
    """With the GEMM chain the plan is: gather, the first layer's QKV, then attention + one chain per layer (the
    chain of the last layer has no next QKV)."""
    from deplodock_b200.model import launch_names

    names = launch_names(3, chain=True)
    assert [e for _, e in names] == ["emk_embed_gather_sumsq", "emk_gemm_bf16_fused"] + [
        "emk_sdpa_causal_gqa_bf16_tok", "emk_gemm_bf16_chain"] * 3 + ["emk_pool_norm_l2"]
    assert names[3][0] == "k_linear_chain_o_proj_gate_up_down_0_qkv_1"
    assert names[-2][0] == "k_linear_chain_o_proj_gate_up_down_2"
    assert len(launch_names(3, chain=False)) == 1 + 5 * 3 + 1


def _pipelined_gather_worker(rank: int, world: int, port: int, q) -> None:
    sys.path.insert(0, str(ROOT))
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    import torch.distributed as dist

    from deplodock_b200.dist import PipelinedGather, init_process_group, shard_batch

    r, _, w = init_process_group("gloo")
    total, hidden = 8, 4
    sh = shard_batch(total, r, w)
    pipe = PipelinedGather(sh.size, total, hidden, "cpu")
    ok = True
    local = torch.empty(sh.size, hidden)
    for step in range(5):   # more steps than buffers: every staging / output pair is reused
        full = torch.arange(total * hidden, dtype=torch.float32).reshape(total, hidden) + 100 * step
        local.copy_(full[sh.start:sh.stop])      # the same tensor object every step, as a plan's output buffer is
        pipe.submit(local)
        if step % 2 == 1:
            ok = ok and torch.equal(pipe.result(), full)
    pipe.flush()
    ok = ok and torch.equal(pipe.result(), full)
    try:
        PipelinedGather(sh.size + 1, total, hidden, "cpu")
        ok = False
    except ValueError:
        pass
    q.put((rank, ok))
    dist.barrier()
    dist.destroy_process_group()


def test_pipelined_gather_two_gloo_ranks():
    """The gather that runs beside the next forward: staged copies, asynchronous collectives, buffers reused only
    after their gather completed; results in shard order at every step."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_pipelined_gather_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert results == [(0, True), (1, True)]


def test_pipelined_gather_single_process():
    from deplodock_b200.dist import PipelinedGather

    pipe = PipelinedGather(3, 3, 2, "cpu")
    x = torch.arange(6, dtype=torch.float32).reshape(3, 2)
    pipe.submit(x)
    assert torch.equal(pipe.result(), x)
    with pytest.raises(RuntimeError):
        PipelinedGather(3, 3, 2, "cpu").result()
