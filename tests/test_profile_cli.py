"""``run --profile`` (ncu re-invocation, counter table, artefacts), the GPU file lock and the stage names of ``compile``.

CPU part: the CSV reduction and the table on a canned ncu output, the child command line, the recursion guard, the
refusal to profile when the plain run fails. GPU part: ``run --profile`` on the ``[1, 32, 2048]`` RMSNorm (one small
kernel, a handful of launches)."""

from __future__ import annotations

import json
import os
import shutil
import subprocess
import sys
import threading
import time
from pathlib import Path
from types import SimpleNamespace

import pytest

from deplodock_b200 import profile
from deplodock_b200.__main__ import build_parser, main

CANNED = '''==PROF== Connected to process 4242
==PROF== Profiling "rmsnorm_cta_kernel" - 0: 0%....50%....100% - 4 passes
"ID","Process ID","Process Name","Host Name","Kernel Name","Context","Stream","Block Size","Grid Size","Device","CC","Section Name","Metric Name","Metric Unit","Metric Value"
"0","4242","python","box","void (anonymous namespace)::rmsnorm_cta_kernel<float>(const float *, const float *, float *, int, int, float)","1","7","(256, 1, 1)","(32, 1, 1)","0","10.0","Command line profiler metrics","gpu__time_duration.sum","nsecond","2,400"
"0","4242","python","box","void (anonymous namespace)::rmsnorm_cta_kernel<float>(const float *, const float *, float *, int, int, float)","1","7","(256, 1, 1)","(32, 1, 1)","0","10.0","Command line profiler metrics","dram__bytes_read.sum","byte","270,336"
"0","4242","python","box","void (anonymous namespace)::rmsnorm_cta_kernel<float>(const float *, const float *, float *, int, int, float)","1","7","(256, 1, 1)","(32, 1, 1)","0","10.0","Command line profiler metrics","dram__bytes_write.sum","byte","0"
"0","4242","python","box","void (anonymous namespace)::rmsnorm_cta_kernel<float>(const float *, const float *, float *, int, int, float)","1","7","(256, 1, 1)","(32, 1, 1)","0","10.0","Command line profiler metrics","launch__registers_per_thread","register/thread","40"
"0","4242","python","box","void (anonymous namespace)::rmsnorm_cta_kernel<float>(const float *, const float *, float *, int, int, float)","1","7","(256, 1, 1)","(32, 1, 1)","0","10.0","Command line profiler metrics","sm__warps_active.avg.pct_of_peak_sustained_active","%","11.5"
"1","4242","python","box","void (anonymous namespace)::rmsnorm_cta_kernel<float>(const float *, const float *, float *, int, int, float)","1","7","(256, 1, 1)","(32, 1, 1)","0","10.0","Command line profiler metrics","gpu__time_duration.sum","nsecond","2,600"
"1","4242","python","box","void (anonymous namespace)::rmsnorm_cta_kernel<float>(const float *, const float *, float *, int, int, float)","1","7","(256, 1, 1)","(32, 1, 1)","0","10.0","Command line profiler metrics","sm__warps_active.avg.pct_of_peak_sustained_active","%","12.5"
"2","4242","python","box","void at::native::vectorized_elementwise_kernel<4, at::native::MulFunctor<float>>(int, float *)","1","7","(128, 1, 1)","(64, 1, 1)","0","10.0","Command line profiler metrics","gpu__time_duration.sum","nsecond","3,100"
'''


def test_csv_reduction_sides_and_roofline_columns():
    status, csv_text = profile.split_ncu_output(CANNED)
    assert status.startswith("==PROF==") and csv_text.startswith('"ID"')
    parsed = profile.parse_ncu_csv(csv_text)
    own = next(k for k in parsed if "rmsnorm_cta_kernel" in k)
    ref = next(k for k in parsed if "vectorized_elementwise" in k)
    assert parsed[own]["gpu__time_duration.sum"] == 5000.0          # .sum counters add up over launches
    assert parsed[own]["sm__warps_active.avg.pct_of_peak_sustained_active"] == 12.0   # everything else is averaged
    assert parsed[own]["launches"] == 2 and parsed[ref]["launches"] == 1
    assert profile.is_own_kernel(own) and not profile.is_own_kernel(ref)
    # ncu's own spelling of an anonymous namespace, with and without a return type
    assert profile.is_own_kernel("void <unnamed>::gemm2_bf16_kernel<256, 3, 1, 2>(CUtensorMap_st, CUtensorMap_st, GemmArgs)")
    assert profile.is_own_kernel("<unnamed>::gemm_w8_kernel(CUtensorMap_st, CUtensorMap_st, W8Args)")
    units = profile.ncu_units(csv_text)
    assert units["gpu__time_duration.sum"] == "nsecond"
    profile.add_roofline(parsed, units, 6454.9)
    assert parsed[own]["dram_gbs"] == pytest.approx(270336 / 5000e-9 / 1e9)
    assert parsed[own]["hbm_frac"] == pytest.approx(parsed[own]["dram_gbs"] / 6454.9)
    lines = profile.render_compare(parsed, units)
    body = [l for l in lines if l.startswith(("dep", "ref"))]
    assert len(body) == 2 and body[0].startswith("dep") and "rmsnorm_cta_kernel" in body[0] and body[1].startswith("ref")
    assert "dur (nsecond)" in lines[1] and "tensor%" in lines[1] and "hbm" in lines[1]


def test_own_kernel_list_matches_the_sources():
    import re

    found = set()
    for path in (Path(__file__).resolve().parent.parent / "deplodock_b200" / "csrc").glob("*.cu*"):
        for m in re.finditer(r"__global__\s+void\s+(?:__cluster_dims__\([^)]*\)\s*)?(?:__launch_bounds__\([^)]*\)\s*)?"
                             r"([A-Za-z_][A-Za-z_0-9]*)\s*\(", path.read_text(), flags=re.S):
            found.add(m.group(1))
    assert found == set(profile.OWN_KERNELS)
    # PyTorch's own anonymous-namespace kernels are printed the same way by ncu and must stay on the ref side
    assert not profile.is_own_kernel("void <unnamed>::softmax_warp_forward<float, float, float, 11, 0, 0>(T2 *, const T1 *)")
    assert profile.is_own_kernel("void <unnamed>::split6_bf16_kernel<1, 1>(const float *, __nv_bfloat16 *, long, long)")
    assert profile.is_own_kernel("k_rms_norm_239c6c") and not profile.is_own_kernel("void at::native::elementwise_kernel<128>()")
    assert profile.kernel_base_name("<unnamed>::fmha_causal_kernel(CUtensorMap_st, FmhaArgs)") == "fmha_causal_kernel"


def _args(argv):
    return build_parser().parse_args(argv)


def test_profile_command_lines_and_guards(monkeypatch, tmp_path, capsys):
    args = _args(["run", "-c", "torch.nn.RMSNorm(64)(torch.randn(2, 64))", "--profile", "--profile-launches", "5",
                  "--profile-kernels", "rmsnorm"])
    child = profile.child_argv(args)
    assert child[1:4] == ["-m", "deplodock_b200", "run"] and "--profile" not in child and "--code" in child
    cmd = profile.ncu_argv("/usr/bin/ncu", child, 5, "rmsnorm")
    assert cmd[:4] == ["/usr/bin/ncu", "--csv", "--clock-control", "none"]
    assert cmd[cmd.index("-c") + 1] == "5" and cmd[cmd.index("-k") + 1] == "regex:rmsnorm"
    assert cmd[cmd.index("--metrics") + 1].split(",")[0] == "gpu__time_duration.sum" and cmd[-len(child):] == child

    calls = []

    def fake_runner(cmd, **kw):
        calls.append((cmd, kw["env"].get(profile.NCU_CHILD_ENV), kw["env"].get("EMMY_DUMP_DIR")))
        return SimpleNamespace(returncode=0, stdout=CANNED if "--csv" in cmd else "ok", stderr="")

    monkeypatch.setattr(shutil, "which", lambda name: "/usr/bin/ncu")
    monkeypatch.setenv("EMMY_DUMP_DIR", str(tmp_path / "parent"))
    parsed = profile.run_profile(args, str(tmp_path), runner=fake_runner)
    # the plain run comes first, then the same command under ncu; both are marked as children; the child does not
    # inherit the dump directory
    assert len(calls) == 2 and "--csv" not in calls[0][0] and "--csv" in calls[1][0]
    assert all(c[1] == "1" and c[2] is None for c in calls)
    assert parsed and json.loads((tmp_path / "61_ncu_metrics.json").read_text()).keys() == parsed.keys()
    assert (tmp_path / "61_ncu_metrics.csv").read_text().startswith('"ID"')
    assert "ncu compare" in capsys.readouterr().out
    # a failing plain run: nothing is profiled
    calls.clear()
    failing = lambda cmd, **kw: (calls.append(cmd), SimpleNamespace(returncode=3, stdout="", stderr="boom"))[1]  # noqa: E731
    assert profile.run_profile(args, None, runner=failing) is None and len(calls) == 1
    # inside the profiled child nothing is spawned
    monkeypatch.setenv(profile.NCU_CHILD_ENV, "1")
    calls.clear()
    assert profile.run_profile(args, None, runner=fake_runner) is None and not calls


def test_gpu_lock_serialises_processes_and_nests(tmp_path, monkeypatch):
    from deplodock_b200.gpu_lock import gpu_lock

    with gpu_lock():   # unset: a no-op
        pass
    lock = tmp_path / "sub" / "gpu.lock"
    monkeypatch.setenv("EMMY_GPU_LOCK", str(lock))
    holder = subprocess.Popen([sys.executable, "-c", (
        "import sys, time; sys.path.insert(0, %r)\n"
        "from deplodock_b200.gpu_lock import gpu_lock\n"
        "with gpu_lock():\n"
        "    print('held', flush=True); time.sleep(1.0)\n") % str(Path(__file__).resolve().parent.parent)],
        stdout=subprocess.PIPE, text=True, env=dict(os.environ))
    assert holder.stdout.readline().strip() == "held"
    t0 = time.perf_counter()
    with gpu_lock():
        waited = time.perf_counter() - t0
        with gpu_lock():   # nested in the same thread
            pass
    holder.wait()
    assert waited > 0.5, "the lock was not exclusive across processes"


def test_compile_accepts_the_reference_stage_names(capsys):
    code = "torch.nn.RMSNorm(64)(torch.randn(2, 64))"
    for stage in ("torch", "tensor", "loop"):
        assert main(["compile", "-c", code, "--ir", stage]) == 0
        assert json.loads(capsys.readouterr().out)["outputs"] == ["rms_norm"]
    for stage in ("tile", "kernel", "cuda"):
        assert main(["compile", "-c", code, "--ir", stage]) == 0
        assert "emk_rmsnorm" in capsys.readouterr().out


@pytest.mark.gpu
def test_run_profile_on_the_readme_rmsnorm(tmp_path, capsys, libemk):
    if shutil.which("ncu") is None:
        pytest.skip("ncu not on PATH")
    rc = main(["run", "-c", "torch.nn.RMSNorm(2048, eps=1e-6)(torch.randn(1, 32, 2048))", "--bench", "--warmup", "3",
               "--iters", "5", "--profile", "--profile-launches", "6", "--dump-dir", str(tmp_path)])
    out = capsys.readouterr().out
    assert rc == 0 and "PASS" in out
    bench = json.loads((tmp_path / "60_benchmark.json").read_text())
    assert bench["num_launches"] == 1 and bench["per_launch"][0]["kernel_name"].startswith("k_rms_norm")
    assert {"time_ms", "min_ms", "max_ms"} <= bench.keys()
    metrics_file = tmp_path / "61_ncu_metrics.json"
    if not metrics_file.exists():
        pytest.skip("ncu produced no counters here (profiling closed or not permitted): " + out[-300:])
    parsed = json.loads(metrics_file.read_text())
    own = [k for k in parsed if profile.is_own_kernel(k)]
    assert own and "rmsnorm" in own[0]
    assert parsed[own[0]]["gpu__time_duration.sum"] > 0 and "dep" in out and "ncu compare" in out
