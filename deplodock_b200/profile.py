"""``run --profile``: hardware counters of the launches of one ``run`` invocation, as a per-kernel table.

Same contract as the reference's ``emmy run --profile`` (``emmy/commands/run.py:670-928``): the command line re-invokes
itself under ``ncu --csv`` with a curated metric list, an environment flag keeps the profiled child from spawning
``ncu`` again, the launch-by-launch CSV is reduced to one metric dict per kernel (``.sum`` counters summed, the rest
averaged), the kernels of this backend are listed first and the kernels of the eager PyTorch module (which the child
also runs once, on the GPU) after them as the ``ref`` side, and ``61_ncu_metrics.csv`` / ``61_ncu_metrics.json`` land in
the dump directory. Added here: the tensor-pipe counter and DRAM bytes, from which the table derives achieved GB/s
and the fraction of the measured HBM copy bandwidth — the roofline columns.

Differences forced by running on shared B200 machines: ``--clock-control none`` is always given (``ncu`` must not lock
the GPU's clocks); the child first runs once WITHOUT ``ncu`` and is profiled only if that run exits 0 (profiling a
faulting program has left GPUs unusable); the number of captured launches is bounded (``--profile-launches``), and
nothing but the small program given on the command line is ever captured — never a whole model forward.
"""

from __future__ import annotations

import csv
import io
import json
import os
import re
import shutil
import subprocess
import sys
from pathlib import Path

#: set in the environment of the profiled child: it runs the plan (and the eager module) once and does not spawn ncu
NCU_CHILD_ENV = "EMK_NCU_CHILD"

NCU_METRICS = (
    "gpu__time_duration.sum",
    "sm__warps_active.avg.pct_of_peak_sustained_active",
    "sm__throughput.avg.pct_of_peak_sustained_elapsed",
    "dram__throughput.avg.pct_of_peak_sustained_elapsed",
    "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active",
    "sm__pipe_fma_cycles_active.avg.pct_of_peak_sustained_active",
    "dram__bytes_read.sum",
    "dram__bytes_write.sum",
    "smsp__inst_executed_pipe_lsu.sum",
    "l1tex__data_bank_conflicts_pipe_lsu_mem_shared_op_ld.sum",
    "l1tex__data_bank_conflicts_pipe_lsu_mem_shared_op_st.sum",
    "launch__registers_per_thread",
)

#: table columns: (metric, label)
COMPARE_COLS = (
    ("gpu__time_duration.sum", "dur"),
    ("sm__warps_active.avg.pct_of_peak_sustained_active", "occ%"),
    ("sm__throughput.avg.pct_of_peak_sustained_elapsed", "sm%"),
    ("dram__throughput.avg.pct_of_peak_sustained_elapsed", "dram%"),
    ("sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active", "tensor%"),
    ("sm__pipe_fma_cycles_active.avg.pct_of_peak_sustained_active", "fma%"),
    ("smsp__inst_executed_pipe_lsu.sum", "lsu.inst"),
    ("l1tex__data_bank_conflicts_pipe_lsu_mem_shared_op_ld.sum", "ld.cnflct"),
    ("l1tex__data_bank_conflicts_pipe_lsu_mem_shared_op_st.sum", "st.cnflct"),
    ("launch__registers_per_thread", "regs"),
)
REF_ROWS_MAX = 12

#: CUDA function names of this library's kernels. The reference's emitted kernels are literally called ``k_*`` and
#: its table splits the two sides on that prefix; the hand-written kernels have ordinary names (ncu prints them as
#: ``void <unnamed>::name<...>(...)``, as it prints PyTorch's own anonymous-namespace kernels), so they are told apart
#: by this list. ``tests/test_profile_cli.py`` checks it against the ``__global__`` definitions under ``csrc/``.
OWN_KERNELS = frozenset({
    "elementwise_kernel", "embed_gather_kernel", "emk_wait_expiry_kernel", "expand_e4m3_bf16_kernel",
    "fmha_causal_kernel", "gemm2_bf16_kernel", "gemm2_chain_kernel", "gemm_bf16_kernel", "gemm_f32_simt_kernel", "gemm_f32_tiled_kernel",
    "gemm_simt_kernel", "gemm_w8_kernel", "loop_linear_f32_kernel", "loop_rope_scores_f32_kernel",
    "loop_softmax_pv_f32_kernel", "pool_norm_l2_kernel", "qknorm_rope_kernel", "rmsnorm_cta_kernel",
    "rmsnorm_from_partials_kernel", "rmsnorm_generic_kernel", "rmsnorm_warp_kernel", "sdpa_simt_kernel",
    "softmax_generic_kernel", "softmax_multiwarp_kernel", "softmax_warp_kernel", "split6_bf16_kernel",
    "varlen_items_kernel"})
_BASE_NAME_RE = re.compile(r"^(?:void\s+)?(?:[A-Za-z_][A-Za-z_0-9]*::|\(anonymous namespace\)::|<unnamed>::)*"
                           r"([A-Za-z_][A-Za-z_0-9]*)")


def kernel_base_name(name: str) -> str:
    """``void <unnamed>::gemm2_bf16_kernel<256, 3, 0, 2>(CUtensorMap_st, ...)`` -> ``gemm2_bf16_kernel``."""
    m = _BASE_NAME_RE.match(name.strip())
    return m.group(1) if m else name.strip()


def is_own_kernel(name: str) -> bool:
    """This library's kernels live in anonymous namespaces (or ``emk::``); a listed base name under a NAMED namespace
    (``at::native::elementwise_kernel``) is somebody else's."""
    base = kernel_base_name(name)
    if base.startswith("k_"):
        return True
    if base not in OWN_KERNELS:
        return False
    head = name.strip()
    head = head[5:] if head.startswith("void ") else head
    prefix = head[: head.index(base)]
    scopes = [p for p in prefix.split("::") if p]
    return all(p in ("<unnamed>", "(anonymous namespace)", "emk") for p in scopes)


def load_hbm_peak_gbs() -> float | None:
    """Measured HBM copy bandwidth of this pool's GPUs when the peaks file sits beside the package, else ``None``."""
    p = Path(__file__).resolve().parent.parent / "MEASURED_PEAKS.json"
    try:
        return float(json.loads(p.read_text())["hbm_gbs"])
    except Exception:  # noqa: BLE001 - the column is simply left out
        return None


def child_argv(args) -> list[str]:
    """The ``run`` invocation the profiler (and the plain run before it) executes: same input, minimal iterations."""
    cmd = [sys.executable, "-m", "deplodock_b200", "run"]
    if args.code is not None:
        cmd += ["--code", args.code]
    elif getattr(args, "ir", None):
        cmd += ["--ir", str(args.ir)]
    else:
        cmd.append(str(args.input))
    cmd += ["--seed", str(args.seed)]
    return cmd


def ncu_argv(ncu: str, child: list[str], launches: int, kernel_regex: str | None) -> list[str]:
    cmd = [ncu, "--csv", "--clock-control", "none", "--target-processes", "all", "--metrics", ",".join(NCU_METRICS),
           "-c", str(int(launches))]
    if kernel_regex:
        cmd += ["-k", f"regex:{kernel_regex}"]
    return cmd + child


def split_ncu_output(stdout: str) -> tuple[str, str]:
    """``(status lines, csv text)``: ncu prints ``==PROF==`` lines first, the table starts at the ``"ID"`` header."""
    lines = stdout.splitlines()
    for i, line in enumerate(lines):
        if line.startswith('"ID"'):
            return "\n".join(lines[:i]), "\n".join(lines[i:]) + "\n"
    return stdout, ""


def parse_ncu_csv(csv_text: str) -> dict[str, dict[str, float]]:
    """Launch-by-launch CSV -> ``{kernel name: {metric: value}}``; ``.sum`` and ``smsp__`` counters are summed over
    the launches of a kernel, everything else averaged; ``launches`` counts them."""
    per: dict[str, dict[str, list[float]]] = {}
    for row in csv.DictReader(io.StringIO(csv_text)):
        k, m = row.get("Kernel Name", ""), row.get("Metric Name", "")
        raw = (row.get("Metric Value", "") or "").replace(",", "")
        if not (k and m and raw):
            continue
        try:
            per.setdefault(k, {}).setdefault(m, []).append(float(raw))
        except ValueError:
            continue
    out: dict[str, dict[str, float]] = {}
    for k, metrics in per.items():
        red = {m: (sum(v) if m.endswith(".sum") or m.startswith("smsp__") else sum(v) / len(v))
               for m, v in metrics.items()}
        red["launches"] = float(max(len(v) for v in metrics.values()))
        out[k] = red
    return out


def ncu_units(csv_text: str) -> dict[str, str]:
    units: dict[str, str] = {}
    for row in csv.DictReader(io.StringIO(csv_text)):
        m, u = row.get("Metric Name", ""), row.get("Metric Unit", "")
        if m and u and m not in units:
            units[m] = u
    return units


_TO_SECONDS = {"nsecond": 1e-9, "ns": 1e-9, "usecond": 1e-6, "us": 1e-6, "msecond": 1e-3, "ms": 1e-3, "second": 1.0,
               "s": 1.0}
_TO_BYTES = {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9}


def add_roofline(parsed: dict[str, dict[str, float]], units: dict[str, str], hbm_peak_gbs: float | None) -> None:
    """Adds ``dram_gbs`` (DRAM read + write bytes / duration) and ``hbm_frac`` (of the measured copy bandwidth) to
    every kernel that has the three counters."""
    t_unit = _TO_SECONDS.get(units.get("gpu__time_duration.sum", "nsecond"), 1e-9)
    for m in parsed.values():
        dur = m.get("gpu__time_duration.sum")
        rd, wr = m.get("dram__bytes_read.sum"), m.get("dram__bytes_write.sum")
        if not dur or rd is None or wr is None:
            continue
        nbytes = rd * _TO_BYTES.get(units.get("dram__bytes_read.sum", "byte"), 1.0) + \
            wr * _TO_BYTES.get(units.get("dram__bytes_write.sum", "byte"), 1.0)
        m["dram_bytes"] = nbytes
        m["dram_gbs"] = nbytes / (dur * t_unit) / 1e9
        if hbm_peak_gbs:
            m["hbm_frac"] = m["dram_gbs"] / hbm_peak_gbs


def render_compare(parsed: dict[str, dict[str, float]], units: dict[str, str] | None = None) -> list[str]:
    """One aligned table: this backend's kernels (side ``dep``) sorted by duration, then the eager module's kernels
    (side ``ref``, the slowest ``REF_ROWS_MAX``), with the counters as columns plus ``GB/s`` and ``hbm`` (fraction of
    the measured HBM peak) where known."""
    if not parsed:
        return []
    dur_key = COMPARE_COLS[0][0]
    own = sorted((k for k in parsed if is_own_kernel(k)), key=lambda k: -parsed[k].get(dur_key, 0.0))
    ref = sorted((k for k in parsed if not is_own_kernel(k)), key=lambda k: -parsed[k].get(dur_key, 0.0))
    hidden = max(0, len(ref) - REF_ROWS_MAX)
    ref = ref[:REF_ROWS_MAX]

    def fmt(v) -> str:
        if v is None:
            return "-"
        return f"{v:,.0f}" if abs(v) >= 100 or v == int(v) else f"{v:.1f}"

    unit = (units or {}).get(dur_key, "")
    head = ["side", "kernel", "n"] + [f"dur ({unit})" if lab == "dur" and unit else lab for _, lab in COMPARE_COLS] + [
        "GB/s", "hbm"]
    rows = [head]
    for side, names in (("dep", own), ("ref", ref)):
        for k in names:
            m = parsed[k]
            shown = k if len(k) <= 60 else k[:57] + "..."
            rows.append([side, shown, fmt(m.get("launches"))] + [fmt(m.get(metric)) for metric, _ in COMPARE_COLS] + [
                fmt(m.get("dram_gbs")), "-" if m.get("hbm_frac") is None else f"{m['hbm_frac']:.2f}"])
    widths = [max(len(r[i]) for r in rows) for i in range(len(head))]
    lines = ["ncu compare — this backend's kernels (dep) and the eager PyTorch module's (ref), same counters:"]
    for i, r in enumerate(rows):
        lines.append("  ".join(c.ljust(w) if j < 2 else c.rjust(w) for j, (c, w) in enumerate(zip(r, widths))))
        if i == 0:
            lines.append("-" * (sum(widths) + 2 * (len(widths) - 1)))
    if hidden:
        lines.append(f"  … {hidden} more reference kernel(s) below the duration cut")
    return lines


def run_profile(args, dump_dir: str | None = None, *, runner=subprocess.run) -> dict | None:
    """Profile the invocation described by ``args`` (see the module docstring). Returns the parsed per-kernel dict, or
    ``None`` when nothing was profiled (inside the child, without ``ncu``, or when the plain run failed)."""
    if os.environ.get(NCU_CHILD_ENV):
        return None
    ncu = shutil.which("ncu")
    if ncu is None:
        print("ncu not found on PATH; skipping --profile output")
        return None
    env = dict(os.environ)
    env[NCU_CHILD_ENV] = "1"
    env.pop("EMMY_DUMP_DIR", None)   # the child must not overwrite the parent's dump artefacts
    child = child_argv(args)
    plain = runner(child, capture_output=True, text=True, env=env, timeout=300)
    if plain.returncode != 0:
        print(f"not profiled: the plain run of the same command exited {plain.returncode}", file=sys.stderr)
        if plain.stderr.strip():
            print(plain.stderr.strip()[-2000:], file=sys.stderr)
        return None
    cmd = ncu_argv(ncu, child, getattr(args, "profile_launches", 24), getattr(args, "profile_kernels", None))
    print()
    print("=" * 80)
    print("ncu --csv --clock-control none (curated hardware metrics)")
    print("=" * 80)
    try:
        res = runner(cmd, capture_output=True, text=True, env=env, timeout=600)
    except subprocess.TimeoutExpired:
        print("ncu profiling timed out", file=sys.stderr)
        return None
    status, csv_text = split_ncu_output(res.stdout)
    if not csv_text:
        if res.stdout.strip():
            print(res.stdout)
        if res.returncode != 0 and res.stderr.strip():
            print(res.stderr, file=sys.stderr)
        return None
    parsed = parse_ncu_csv(csv_text)
    units = ncu_units(csv_text)
    add_roofline(parsed, units, load_hbm_peak_gbs())
    for line in render_compare(parsed, units):
        print(line)
    if dump_dir is not None:
        out = Path(dump_dir)
        out.mkdir(parents=True, exist_ok=True)
        (out / "61_ncu_metrics.csv").write_text(csv_text)
        (out / "61_ncu_metrics.json").write_text(json.dumps(parsed, indent=2, default=str))
        print(f"ncu metrics → {out / '61_ncu_metrics.csv'}")
        print(f"ncu metrics → {out / '61_ncu_metrics.json'}")
    elif status.strip():
        print(status)
    if res.returncode != 0 and res.stderr.strip():
        print(res.stderr, file=sys.stderr)
    return parsed
