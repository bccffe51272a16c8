"""Command line: ``python -m deplodock_b200 {compile,run} ...``.

The two verbs of the reference's CLI that sit on the kernel path (``emmy/cli.py:17-47``, ``emmy/commands/run.py:23-140``,
``emmy/commands/compile.py:66-290``), with the same input grammar (``-c/--code`` inline expression, ``--ir`` or a
positional ``.json`` record: Torch-IR, or one of the reference's Loop-IR kernel records, ``kernels/*.json``), the same accuracy rule against eager PyTorch (``run.py:1440-1500``), the same
bench table rows (``Eager PyTorch`` / ``Emmy`` / ``vs Eager``, ``run.py:1715-1730``) and the same
``60_bench_compare.json`` artefact under ``--dump-dir`` / ``EMMY_DUMP_DIR`` (``run.py:375-394``). Exit code 0 iff the
accuracy verdict is PASS (or no eager reference exists, for ``--ir``).

``run --profile`` re-invokes the command under ``ncu`` and prints the per-kernel counter table with roofline columns
(``deplodock_b200.profile``; ``61_ncu_metrics.json``), ``--bench`` also writes ``60_benchmark.json`` (the per-launch
record the reference's dumper writes, ``emmy/compiler/pipeline/dump.py:311-323``), ``compile --ir`` takes the reference's
stage names (``torch | tensor | loop | tile | kernel | cuda``: the first three print the Torch-IR record, the stage
this backend starts from; the last three print the dispatch plan, the stage it ends at). GPU work is done under the
``EMMY_GPU_LOCK`` file lock when that variable is set. A traced decoder trunk (a ``.json`` record of the wrapped HF
module) compiles to the fused model plan. Model ids, ``--layer``, ``--golden``, ``--ab``, ``--dynamic`` and the tuner
verbs are not provided: there is nothing to tune or generate and no checkpoint store to resolve ids against. ``--dynamic NAME@INPUT:AXIS`` (with ``--code``) traces an axis as a
symbolic dimension; records with symbolic dimensions get one launch plan per runtime size.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

import numpy as np


def _add_common(p: argparse.ArgumentParser) -> None:
    p.add_argument("input", nargs="?", help=".json Torch-IR record (same as --ir)")
    p.add_argument("--code", "-c", help="inline expression, e.g. 'torch.nn.RMSNorm(2048)(torch.randn(1,32,2048))'")
    p.add_argument("--dump-dir", default=None)
    p.add_argument("--dynamic", action="append", default=None, metavar="NAME@INPUT:AXIS",
                   help="with --code: trace axis AXIS of input INPUT as the symbolic dimension NAME (repeatable)")
    p.add_argument("-v", "--verbose", action="count", default=0)


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="deplodock_b200", description=__doc__.split("\n\n")[0])
    sub = parser.add_subparsers(dest="command", required=True)
    c = sub.add_parser("compile", help="lower a Torch-IR graph to a launch plan and print it")
    _add_common(c)
    c.add_argument("--ir", choices=["torch", "tensor", "loop", "tile", "kernel", "cuda"], default="cuda",
                   help="stage to print (the reference's stage names): torch / tensor / loop -> the Torch-IR record "
                        "(this backend has no IR between the traced graph and its kernels); tile / kernel / cuda -> "
                        "the dispatch plan, one line per launch (default)")
    c.add_argument("--output", "-o", default=None)
    r = sub.add_parser("run", help="compile + run on the B200 backend, check against eager PyTorch")
    _add_common(r)
    r.add_argument("--ir", default=None, help="path to a Torch-IR .json record (random inputs, no accuracy check)")
    r.add_argument("--bench", "-b", action="store_true")
    r.add_argument("--warmup", type=int, default=10)
    r.add_argument("--iters", type=int, default=100)
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--debug", action="store_true")
    r.add_argument("--profile", action="store_true",
                   help="re-run this command under ncu (bounded number of launches, --clock-control none) and print "
                        "the per-kernel counter table with roofline columns")
    r.add_argument("--profile-launches", type=int, default=24, help="launches ncu captures at most (default 24)")
    r.add_argument("--profile-kernels", default=None, help="regex: capture only kernels whose name matches")
    return parser


def _fail(msg: str) -> None:
    print(f"Error: {msg}", file=sys.stderr)
    raise SystemExit(1)


def _load(args):
    """Returns ``(graph, slug, TraceResult | None)``."""
    from deplodock_b200.graph import Graph

    ir_path = getattr(args, "ir", None) if args.command == "run" else None
    given = [x for x in (args.code, args.input, ir_path) if x]
    if len(given) != 1:
        _fail("give exactly one of --code, --ir, or a positional .json record")
    if args.code:
        from deplodock_b200.trace import parse_dynamic_specs, trace_inline_code

        try:
            dynamic = parse_dynamic_specs(args.dynamic)
        except ValueError as exc:
            print(f"Error: {exc}", file=sys.stderr)
            raise SystemExit(2) from None
        tr = trace_inline_code(args.code, dynamic or None)
        return tr.graph, tr.slug, tr
    path = Path(ir_path or args.input)
    if path.suffix != ".json":
        _fail(f"{path}: only .json Torch-IR records are accepted (model ids are not traced by this backend)")
    return Graph.from_json(path), path.stem, None


def accuracy_verdict(values: np.ndarray, eager: np.ndarray, is_fp16: bool) -> tuple[bool, float, float, float]:
    """The reference's dual rule (``emmy/commands/run.py:1452-1491``): PASS when ``max_diff <= max(abs_tol, rel *
    peak)`` or ``mean_diff <= max(abs_tol, mean_rel * peak)``; (rel, mean_rel, abs_tol) = (0.08, 0.005, 1e-3), or
    (1.0, 1.0, 1e-1) for fp16 outputs."""
    values = np.asarray(values, dtype=np.float64).ravel()
    eager = np.asarray(eager, dtype=np.float64).ravel()
    diff = np.abs(values - eager)
    max_diff, mean_diff = float(diff.max(initial=0.0)), float(diff.mean()) if diff.size else 0.0
    rel, mean_rel, abs_tol = (1.0, 1.0, 1e-1) if is_fp16 else (0.08, 0.005, 1e-3)
    peak = float(np.abs(eager).max(initial=0.0))
    tol, mean_tol = max(abs_tol, rel * peak), max(abs_tol, mean_rel * peak)
    return (max_diff <= tol or mean_diff <= mean_tol), max_diff, mean_diff, tol


def _to_f32(arr: np.ndarray, dtype_token: str) -> np.ndarray:
    if dtype_token == "bf16" and arr.dtype == np.uint16:
        return (arr.astype(np.uint32) << 16).view(np.float32)
    return arr.astype(np.float32)


def render_table(results: dict[str, float]) -> list[str]:
    eager = results.get("Eager PyTorch", 0.0)
    rows = [("Backend", "Latency (us)", "vs Eager")]
    rows += [(n, f"{us:.0f}", f"{eager / us:.2f}x" if us > 0 and eager else "-") for n, us in results.items()]
    w = [max(len(r[i]) for r in rows) for i in range(3)]
    fmt = lambda r: f"{r[0]:<{w[0]}}  {r[1]:>{w[1]}}  {r[2]:>{w[2]}}"  # noqa: E731
    return [fmt(rows[0]), "-" * (sum(w) + 4)] + [fmt(r) for r in rows[1:]]


def _time_eager_us(fn, warmup: int, iters: int) -> float:
    import torch

    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) * 1e3 / iters


def cmd_compile(args) -> int:
    from deplodock_b200.backend import B200Backend

    graph, _slug, _ = _load(args)
    if args.ir in ("torch", "tensor", "loop"):
        text = json.dumps(graph.to_dict(), indent=2)
    else:
        text = B200Backend(dump=args.dump_dir or os.environ.get("EMMY_DUMP_DIR")).compile(graph).describe()
    if args.output:
        Path(args.output).write_text(text + "\n")
    else:
        print(text)
    return 0


def cmd_run(args) -> int:
    import torch

    from deplodock_b200 import profile as _profile
    from deplodock_b200.backend import B200Backend
    from deplodock_b200.gpu_lock import gpu_lock
    from deplodock_b200.trace import bind_inputs

    graph, slug, tr = _load(args)
    in_ncu_child = bool(os.environ.get(_profile.NCU_CHILD_ENV))
    dump_dir = args.dump_dir or os.environ.get("EMMY_DUMP_DIR")
    backend = B200Backend(debug=args.debug, dump=dump_dir)
    plan = backend.compile(graph)
    if args.verbose:
        print(plan.describe())
    if not torch.cuda.is_available():
        _fail("no CUDA device: this backend has no CPU path")

    ok = True
    eager_fn = None
    if tr is not None:
        data = bind_inputs(graph, tr.module, tr.args, tr.kwargs, tr.const_sources)
        with torch.no_grad():
            eager = tr.module(*tr.args, **tr.kwargs)
        with gpu_lock():
            result, _ = backend.run(plan, input_data=data)
            if in_ncu_child:
                # under the profiler the eager module runs once on the GPU too: its kernels are the table's ref side
                dev = torch.device("cuda")
                with torch.no_grad():
                    tr.module.to(dev)(*(a.to(dev) if isinstance(a, torch.Tensor) else a for a in tr.args),
                                      **{k: v.to(dev) if isinstance(v, torch.Tensor) else v
                                         for k, v in tr.kwargs.items()})
                torch.cuda.synchronize()
                tr.module.to("cpu")
        eager_list = [eager] if isinstance(eager, torch.Tensor) else [e for e in eager if isinstance(e, torch.Tensor)]
        for name, e in zip(plan.outputs, eager_list):
            token = graph.nodes[name].output.dtype
            got = _to_f32(result.outputs[name], token)
            if np.isnan(got).any():
                print(f"CORRECTNESS FAIL: output {name} contains NaN")
                ok = False
                continue
            passed, max_diff, mean_diff, tol = accuracy_verdict(got, e.detach().float().cpu().numpy(), token == "f16")
            print(f"Accuracy vs eager: max_diff={max_diff:.6f} mean_diff={mean_diff:.6f} tol={tol:.6f} "
                  f"{'PASS' if passed else 'FAIL'}")
            ok = ok and passed
        if args.bench:
            dev = torch.device("cuda")
            mod = tr.module.to(dev)
            cargs = tuple(a.to(dev) if isinstance(a, torch.Tensor) else a for a in tr.args)
            ckw = {k: v.to(dev) if isinstance(v, torch.Tensor) else v for k, v in tr.kwargs.items()}

            def eager_fn():
                with torch.no_grad():
                    return mod(*cargs, **ckw)
    else:
        rng = np.random.default_rng(args.seed)
        data = {}
        for nid in graph.inputs:
            info = graph.nodes[nid].output
            vals = rng.standard_normal(info.shape).astype(np.float32)
            data[nid] = torch.from_numpy(vals)
        for nid, node in graph.nodes.items():
            if node.op == "ConstantOp" and node.op_fields.get("value") is None and nid not in data:
                info = node.output
                data[nid] = torch.from_numpy((rng.standard_normal(info.shape) * 0.05 + (1.0 if len(info.shape) == 1
                                                                                         else 0.0)).astype(np.float32))
        with gpu_lock():
            result, _ = backend.run(plan, input_data=data)
        print(f"Ran {len(plan.steps)} launch(es) in {result.time_ms:.3f} ms (no eager reference for a .json record)")

    if args.bench:
        results: dict[str, float] = {}
        with gpu_lock():
            if eager_fn is not None:
                results["Eager PyTorch"] = _time_eager_us(eager_fn, args.warmup, args.iters)
            bench = backend.benchmark(plan, warmup=args.warmup, num_iters=args.iters, input_data=data)
        results["Emmy"] = bench.time_ms * 1e3
        print()
        for line in render_table(results):
            print(line)
        if bench.per_launch:
            print()
            for lt in bench.per_launch:
                print(f"  [{lt.idx}] {lt.kernel_name:<48} {lt.time_ms * 1e3:9.1f} us")
        if dump_dir:
            Path(dump_dir).mkdir(parents=True, exist_ok=True)
            eager_us = results.get("Eager PyTorch")
            payload = {"warmup": args.warmup, "iters": args.iters, "slug": slug,
                       "backends": {n: {"latency_us": us} for n, us in results.items()}}
            if eager_us:
                for n, us in results.items():
                    payload["backends"][n]["speedup_vs_eager"] = (eager_us / us) if us else 0.0
            (Path(dump_dir) / "60_bench_compare.json").write_text(json.dumps(payload, indent=2))
            record = {"time_ms": bench.time_ms, "min_ms": bench.min_ms, "max_ms": bench.max_ms,
                      "num_launches": bench.num_launches,
                      "per_launch": [{"idx": lt.idx, "kernel_name": lt.kernel_name, "time_ms": lt.time_ms}
                                     for lt in bench.per_launch or []]}
            if bench.e2e_ms is not None:
                record["e2e_ms"] = bench.e2e_ms
            (Path(dump_dir) / "60_benchmark.json").write_text(json.dumps(record, indent=2))
    if args.profile and ok:
        with gpu_lock():
            _profile.run_profile(args, dump_dir)
    return 0 if ok else 1


def main(argv: list[str] | None = None) -> int:
    from deplodock_b200.backend import LoweringError

    args = build_parser().parse_args(argv)
    try:
        return cmd_compile(args) if args.command == "compile" else cmd_run(args)
    except LoweringError as e:
        print(f"LoweringError: {e}", file=sys.stderr)
        return 1
    except SystemExit as e:
        return int(e.code or 0)


if __name__ == "__main__":
    sys.exit(main())
