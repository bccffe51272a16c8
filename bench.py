"""Benchmark of the hot path on B200: the Qwen3-Embedding-0.6B-shaped forward (64 sequences x 512 tokens, bf16,
random-init weights, uniform-random token ids), batch-sharded over N GPUs, plus the four per-kernel configurations.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--no-kernels]

Prints ONE JSON line on rank 0. A step is one forward of the whole 64-sequence batch: every rank replays its captured
CUDA graph on its shard (64/N sequences) and the pooled embeddings are all-gathered. ``value`` is sequences/s with the
ids already resident on the device; ``e2e`` repeats the measurement through the public call with pinned host ids
(host->device copy of the ids and device->host copy of the gathered embeddings inside the timed region).
``roofline`` describes the dominant kernel of the step (the tcgen05 GEMM), timed with CUDA events around every
launch of it in extra eager passes of the same plan that follow a second of graph replays without a pause (so they
run at the sustained clock of the timed region; the clock is sampled and reported); ``kernels`` lists the four named
kernel configurations with their own roofline fractions. Weights and ids are the seeded CPU-generated inputs of the
benchmark configuration; ``parity`` holds the gathered embeddings of the timed run against the CPU oracle (the
PyTorch-eager trunk) on the same weights and ids, and the process exits 1 when they are outside the tolerance.
``cpu_baseline`` is that oracle's time. ``--impl reference`` runs only the CPU arm, with all host threads.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
BATCH, SEQ = 64, 512
METRIC, UNIT = "embed_forward_seqs_per_s", "seq/s"


def load_peaks() -> tuple[dict, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return {k: float(d[k]) for k in FALLBACK_PEAKS}, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int) -> None:
        self.gpu_index = gpu_index
        self.rows: list[list[str]] = []
        self.proc = None
        self.thread = None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return

        def pump():
            for line in self.proc.stdout:
                parts = [x.strip() for x in line.split(",")]
                if len(parts) >= 9:
                    self.rows.append(parts)

        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()

    def stop(self) -> dict:
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=3)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        busy = [c for c in sm if c > 0]
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------------------------
# CPU arm (the oracle, timed)
# ------------------------------------------------------------------------------------------------------------
def cpu_reference_sample(sd_cpu, cfg, n_seqs: int, repeats: int = 1) -> dict:
    """Times the eager CPU trunk on the first ``n_seqs`` sequences of the benchmark batch; ``embeddings`` holds its
    output (the checker's answer for those sequences)."""
    import torch

    from oracle import cpu_ref, inputs

    torch.set_num_threads(os.cpu_count() or 1)
    ids = inputs.token_ids(BATCH, SEQ, cfg.vocab_size, seed=0)[:n_seqs]
    cpu_ref.embed_forward(ids[:1, :64], cfg, sd_cpu)  # warm-up of the thread pool / kernels
    best = math.inf
    out = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        out = cpu_ref.embed_forward(ids, cfg, sd_cpu)
        best = min(best, time.perf_counter() - t0)
    return {"value": n_seqs / best, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{n_seqs} of {BATCH} sequences x {SEQ} tokens, eager CPU trunk, {best:.2f} s",
            "seconds": best, "embeddings": out}


def run_reference_arm(args) -> None:
    """The reference's own CPU path for this workload: the PyTorch-eager trunk on the host cores."""
    import torch

    from oracle import inputs

    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return
    cfg = inputs.EmbedModelConfig()
    sd = inputs.embed_model_weights(cfg, seed=0)
    per_step = 16   # 16 of the 64 sequences per step: about 1.7 s of work on 16 cores
    times = []
    res = None
    for i in range(args.warmup + args.steps):
        res = cpu_reference_sample(sd, cfg, per_step)
        res.pop("embeddings", None)
        if i >= args.warmup:
            times.append(res["seconds"])
    avg = sum(times) / len(times)
    value = per_step / avg
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": avg * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "qwen3-embedding-0.6b-shaped forward, 64x512 tokens, last-token pool + L2",
                   "sample_per_step": f"{per_step} sequences x {SEQ} tokens", "threads": torch.get_num_threads()},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                         "sample": f"{per_step} sequences x {SEQ} tokens per step, eager CPU trunk (the module the "
                                   "reference traces and checks against)"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    emitted = reference_emitted_kernels()
    if emitted is not None:
        line["emitted_kernels_on_this_gpu"] = emitted
    print(json.dumps(line), flush=True)


def reference_emitted_kernels():
    """The reference compiler's own emitted kernels for the four kernel configurations (``oracle/_ref``, lowered for
    sm_100 by its pipeline and compiled with its nvcc flags), timed on this GPU on the seeded inputs with the protocol
    used for the hand-written kernels (CUDA graph of back-to-back launches). ``None`` without a GPU or without the
    prebuilt files."""
    try:
        import torch

        from oracle import inputs, ref_kernels

        if not torch.cuda.is_available() or not ref_kernels.available():
            return None
        rows = []
        import json as _json

        built = _json.loads((ref_kernels.REF_DIR / "manifest.json").read_text())
        for name in ("rmsnorm", "softmax", "linear", "sdpa", "matmul_f32"):
            if name not in built:
                continue
            k = ref_kernels.RefKernel(name)
            if name == "rmsnorm":
                x, w = inputs.rmsnorm_inputs()
                k.bind(x=x, p_weight=w)
            elif name == "softmax":
                k.bind(input=inputs.softmax_inputs((1, 28, 2048, 2048)))
            elif name == "linear":
                x, w = inputs.linear_inputs()
                k.bind(input=x, linear_wt=w.t().contiguous())
            elif name == "matmul_f32":
                g = torch.Generator().manual_seed(0)
                k.bind(a=torch.randn(512, 1024, generator=g), b=torch.randn(1024, 2048, generator=g))
            else:
                q, kk, v = inputs.sdpa_inputs()
                k.bind(q=q, k=kk, v=v)
            rows.append({"config": name, "kernel": k.meta["kernel_name"], "grid": k.meta["grid"][0],
                         "block": k.meta["block"][0], "us": round(k.time_us(10 if name == "rmsnorm" else 3, 3), 1)})
            del k
            torch.cuda.empty_cache()
        return rows
    except Exception as exc:  # noqa: BLE001 - an informational table must not fail the arm
        return {"unavailable": f"{type(exc).__name__}: {exc}"[:200]}


# ------------------------------------------------------------------------------------------------------------
# Per-kernel configurations (rank 0, one GPU)
# ------------------------------------------------------------------------------------------------------------
def _graph_time_us(fn, reps: int, iters: int = 5) -> tuple[float, float]:
    """Median and min microseconds per call of ``fn`` measured as a CUDA graph of ``reps`` back-to-back launches."""
    import torch

    fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(reps):
            fn()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    samples = []
    for _ in range(iters):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        g.replay()
        e.record()
        torch.cuda.synchronize()
        samples.append(s.elapsed_time(e) * 1e3 / reps)
    return statistics.median(samples), min(samples)


def serving_table(weights) -> list[dict]:
    """Requests per second of the serving-side runner (``deplodock_b200.runner``): the two workloads the reference
    quotes for its vLLM plugin (64 requests x 256 tokens; uniform 512 tokens) through the per-length and padded-group
    routes, and the packed variable-length route (one forward over the concatenated stream, no padding) on the same
    uniform workloads and on 64 requests of mixed lengths 64..512 — next to the padded route on that mix. Ids resident
    on the device, hidden states of every token produced, all requests submitted at once."""
    import time

    import torch

    from deplodock_b200.runner import EmbedForwardRunner

    rows = []
    cfg = weights.cfg
    gen = torch.Generator().manual_seed(0)

    def best_of(serve, n=3):
        serve()   # captures the graph(s)
        torch.cuda.synchronize()
        best = float("inf")
        for _ in range(n):
            t0 = time.perf_counter()
            out = serve()
            torch.cuda.synchronize()
            best = min(best, time.perf_counter() - t0)
        return best, out

    for tokens, batch_cap in ((256, 1), (256, 8), (256, 32), (512, 32)):
        runner = EmbedForwardRunner(weights, max_seq_len=tokens, batch_cap=batch_cap)
        reqs = [torch.randint(0, cfg.vocab_size, (tokens,), generator=gen).cuda() for _ in range(64)]

        def serve():
            if batch_cap == 1:
                return [runner.forward_hidden_states(r) for r in reqs]
            return runner.forward_hidden_states_batched(reqs)

        best, out = best_of(serve)
        assert len(out) == 64 and tuple(out[0].shape) == (tokens, cfg.hidden_size)
        rows.append({"route": "one graph per length" if batch_cap == 1 else "padded groups", "requests": 64,
                     "tokens_per_request": tokens, "batch_cap": batch_cap, "req_per_s": round(64 / best, 1),
                     "ms_total": round(best * 1e3, 2)})
        del runner
        torch.cuda.empty_cache()
    mixed = [int(x) for x in torch.randint(64, 513, (64,), generator=gen)]
    for label, lens in (("64 x 256", [256] * 64), ("64 x 512", [512] * 64), ("64 x mixed 64..512", mixed)):
        runner = EmbedForwardRunner(weights, max_seq_len=512, batch_cap=64)
        ids = torch.cat([torch.randint(0, cfg.vocab_size, (n,), generator=gen) for n in lens]).cuda()
        pos = torch.cat([torch.arange(n) for n in lens])
        for route, fn in (("packed variable-length", runner.forward_packed),
                          ("padded groups", runner.forward_packed_padded)):
            best, out = best_of(lambda fn=fn: fn(ids, pos))
            assert tuple(out.shape) == (sum(lens), cfg.hidden_size)
            rows.append({"route": route, "requests": 64, "tokens_per_request": label, "tokens": sum(lens),
                         "req_per_s": round(64 / best, 1), "ms_total": round(best * 1e3, 2)})
        del runner
        torch.cuda.empty_cache()
    return rows


def loop_record_table() -> list[dict]:
    """The reference's eleven shipped Loop-IR kernel records (``kernels/*.json``, held as fixtures under
    ``tests/golden/loop_records``) through ``B200Backend.benchmark``: recognised, lowered to one launch each, timed
    with the backend's own protocol (CUDA-graph windows, median)."""
    from deplodock_b200.backend import B200Backend

    rows = []
    be = B200Backend()
    for path in sorted((ROOT / "tests" / "golden" / "loop_records").glob("k_*.json")):
        plan = be.compile(path)
        res = be.benchmark(plan, warmup=3, num_iters=10)
        rows.append({"record": path.stem, "entry": plan.steps[0].entry, "us": round(res.time_ms * 1e3, 2),
                     "us_min": round((res.min_ms or 0.0) * 1e3, 2)})
    return rows


def kernel_cases() -> dict:
    """The named kernel configurations: ``name -> builder``; a builder allocates the seeded device inputs and returns
    ``(launch thunk, bound, algorithmic work per launch, unit scale, peak key, note, launches per timing graph)``."""
    import torch

    from deplodock_b200 import ops

    dev = "cuda"

    def gen():
        return torch.Generator(device=dev).manual_seed(0)

    def rms_small():
        g = gen()
        x = torch.randn(1, 32, 2048, device=dev, generator=g)
        w = 1 + 0.02 * torch.randn(2048, device=dev, generator=g)
        y = torch.empty_like(x)
        return (lambda: ops.rmsnorm(x, w, 1e-6, out=y), "hbm", 532480, 1e9, "hbm_gbs",
                "0.5 MB, L2-resident, latency-bound", 200)

    def rms_big():
        g = gen()
        xs = [torch.randn(32768, 1024, device=dev, generator=g).bfloat16() for _ in range(3)]
        ws = torch.ones(1024, device=dev, dtype=torch.bfloat16)
        ys = [torch.empty_like(t) for t in xs]
        state = {"i": 0}

        def fn():
            i = state["i"] = (state["i"] + 1) % 3
            ops.rmsnorm(xs[i], ws, 1e-6, out=ys[i])

        return fn, "hbm", 2 * 32768 * 1024 * 2 + 2048, 1e9, "hbm_gbs", "3 rotating 64 MB buffer pairs (> L2)", 30

    def softmax():
        g = gen()
        x = 3 * torch.randn(28 * 2048, 2048, device=dev, generator=g)
        m = torch.rand(x.shape, device=dev, generator=g) < 0.01
        m[:, 0] = False
        x[m] = float("-inf")
        del m
        y = torch.empty_like(x)
        return (lambda: ops.softmax_lastdim(x, out=y), "hbm", 939524096, 1e9, "hbm_gbs",
                "470 MB in + 470 MB out (> L2)", 10)

    def linear_inputs(M=4096):
        g = gen()
        x = torch.randn(M, 2048, device=dev, generator=g).bfloat16()
        w32 = 0.02 * torch.randn(6144, 2048, device=dev, generator=g)
        y = torch.empty(M, 6144, device=dev, dtype=torch.bfloat16)
        return x, w32, y

    def linear():
        x, w32, y = linear_inputs()
        w = w32.bfloat16()
        return lambda: ops.linear(x, w, out=y), "tensor", 103079215104, 1e12, "bf16_tflops", "burst peak", 20

    def w8(workspace, M=4096):
        def build():
            x, w32, y = linear_inputs(M)
            s = (w32.abs().amax(1) / 448.0).contiguous()
            wq = (w32 / s[:, None]).to(torch.float8_e4m3fn)
            if workspace:
                fn = lambda: ops.linear_w8(x, wq, s, out=y)  # noqa: E731
                note = ("burst peak; weight expanded to bf16 once into a 25 MB scratch, then the bf16 CTA-pair GEMM "
                        "(M > 256 route)")
            else:
                fn = lambda: ops.linear_w8(x, wq, s, out=y, workspace=None)  # noqa: E731
                note = "burst peak; no scratch: every 128-row tile converts its weight tiles again"
            if M <= 256:
                # few rows: the launch is bound by reading W (12.6 MB as e4m3 bytes + x + y), not by the tensor core
                nbytes = 6144 * 2048 + M * 2048 * 2 + M * 6144 * 2 + 6144 * 4
                return fn, "hbm", nbytes, 1e9, "hbm_gbs", f"M = {M}: weight-read bound; W stays e4m3 in HBM", 50
            return fn, "tensor", 2 * M * 2048 * 6144, 1e12, "bf16_tflops", note, 20
        return build

    def sdpa():
        g = gen()
        q = torch.randn(4, 16, 2048, 128, device=dev, generator=g).bfloat16()
        k = torch.randn(4, 8, 2048, 128, device=dev, generator=g).bfloat16()
        v = torch.randn(4, 8, 2048, 128, device=dev, generator=g).bfloat16()
        o = torch.empty_like(q)
        return (lambda: ops.sdpa_causal_gqa(q, k, v, out=o), "tensor", 68753031168, 1e12, "bf16_tflops",
                "causal-useful flops, burst peak", 20)

    def sdpa_model(B):
        def build():
            g = gen()
            qkv = torch.randn(B * 512, 4096, device=dev, generator=g).bfloat16()
            o = torch.empty(B * 512, 2048, device=dev, dtype=torch.bfloat16)
            return (lambda: ops.sdpa_causal_gqa_tok(qkv, B, 512, 16, 8, o), "tensor",
                    4 * B * 16 * 128 * (512 * 513 // 2), 1e12, "bf16_tflops",
                    f"the attention launch of the model plan at {B} sequences: token-major fused QKV buffer", 20)
        return build

    def matmul_f32(M, K, N, extra=None):
        """The fp32 tier of the reference's perf suite (tests/perf/cases.py:60-74): Qwen3 projection shapes as
        torch.matmul (B row-major [K, N]), torch.matmul + r and silu(x @ wg) * (x @ wu)."""
        def build():
            g = gen()
            a = torch.randn(M, K, device=dev, generator=g)
            b = torch.randn(K, N, device=dev, generator=g)
            flops = 2 * M * K * N
            note = ("fp32 in / fp32 out; 256 rows and up run on the tensor cores over exactly split bf16 operands "
                    "(6x the flops at bf16 rate), fewer rows on CUDA cores; the fraction is of the nominal fp32 "
                    "CUDA-core rate (72 TFLOP/s = 148 SMs x 128 lanes x 2 x 1.9 GHz), which the split route can exceed")
            if extra == "add":
                r = torch.randn(M, N, device=dev, generator=g)
                fn = lambda: ops.elementwise("add", ops.linear_f32(a, b, None, True), r)  # noqa: E731
            elif extra == "gated":
                b2 = torch.randn(K, N, device=dev, generator=g)
                fn = lambda: ops.elementwise("silu_multiply", ops.linear_f32(a, b, None, True),  # noqa: E731
                                             ops.linear_f32(a, b2, None, True))
                flops *= 2
            else:
                fn = lambda: ops.linear_f32(a, b, None, True)  # noqa: E731
            return fn, "fma", flops, 1e12, "f32_tflops_nominal", note, 20
        return build

    def layer_gemms(M, chained):
        """The four projections between two attention launches of the model plan (o_proj + residual, gate/up SwiGLU,
        down + residual, next layer's QKV with q/k-norm + RoPE) at one rank's rows: as one chained launch or as four."""
        def build():
            from deplodock_b200.model import rope_tables

            g = gen()
            r = lambda *sh, sc=1.0: (sc * torch.randn(*sh, device=dev, generator=g)).bfloat16()  # noqa: E731
            attn, h = r(M, 2048), r(M, 1024)
            wo, wgu, wd, wqkv = r(1024, 2048, sc=0.02), r(6144, 1024, sc=0.05), r(1024, 3072, sc=0.02), r(4096, 1024, sc=0.03)
            mlp = torch.empty(M, 3072, device=dev, dtype=torch.bfloat16)
            qkv = torch.empty(M, 4096, device=dev, dtype=torch.bfloat16)
            ss2, ss3 = torch.empty(M, 8, device=dev), torch.empty(M, 8, device=dev)
            qn = torch.ones(128, device=dev, dtype=torch.bfloat16)
            cm = ops.rope_chunk_major(*rope_tables(512, 128, 1e6, dev))
            phases = [dict(x=attn, w=wo, out=h, epilogue="residual", residual=h, row_sumsq_out=ss2),
                      dict(x=h, w=wgu, out=mlp, epilogue="swiglu", row_sumsq_in=ss2, norm_dim=1024),
                      dict(x=mlp, w=wd, out=h, epilogue="residual", residual=h, row_sumsq_out=ss3),
                      dict(x=h, w=wqkv, out=qkv, epilogue="qknorm_rope", row_sumsq_in=ss3, norm_dim=1024, q_weight=qn,
                           k_weight=qn, rope_cm=cm, S=512, Hq=16, Hkv=8)]
            flops = 2 * M * (1024 * 2048 + 6144 * 1024 + 1024 * 3072 + 4096 * 1024)
            if chained:
                ws = ops.gemm_chain_workspace(M, dev)
                fn = lambda: ops.gemm_chain(phases, ws)  # noqa: E731
                note = "one persistent launch, tiles of a phase wait for their 256-row block of the phase before"
            else:
                def fn():
                    for ph in phases:
                        ops.gemm_fused(ph["x"], ph["w"], ph["out"],
                                       **{k: v for k, v in ph.items() if k not in ("x", "w", "out")})
                note = "four launches (the time is of all four)"
            return fn, "tensor", flops, 1e12, "bf16_tflops", note + "; burst peak", 10
        return build

    return {
        "k_linear chain o_proj>gate_up>down>qkv 4096 rows (8-GPU shard), one launch": layer_gemms(4096, True),
        "k_linear o_proj, gate_up, down, qkv 4096 rows (8-GPU shard), four launches": layer_gemms(4096, False),
        "k_matmul f32 512x1024x2048 (q_proj s512)": matmul_f32(512, 1024, 2048),
        "k_matmul f32 128x1024x2048 (q_proj s128)": matmul_f32(128, 1024, 2048),
        "k_matmul f32 32x1024x2048 (q_proj s32)": matmul_f32(32, 1024, 2048),
        "k_matmul_add f32 512x3072x1024 (down_proj + r s512)": matmul_f32(512, 3072, 1024, "add"),
        "k_gated_mlp f32 512x1024x3072 (silu(x@wg)*(x@wu) s512)": matmul_f32(512, 1024, 3072, "gated"),
        "k_rms_norm [1,32,2048] f32": rms_small,
        "k_rms_norm [32768,1024] bf16": rms_big,
        "k_softmax [1,28,2048,2048] f32": softmax,
        "k_linear 4096x2048x6144 bf16": linear,
        "k_linear 4096x2048x6144 e4m3 weights": w8(True),
        "k_linear 4096x2048x6144 e4m3 weights, converted inside the main loop": w8(False),
        "k_linear 256x2048x6144 e4m3 weights, converted inside the main loop": w8(False, 256),
        "k_linear 128x2048x6144 e4m3 weights, converted inside the main loop": w8(False, 128),
        "k_scaled_dot_product_attention B4 Hq16 Hkv8 S2048 D128": sdpa,
        "k_scaled_dot_product_attention 64x512 token-major (model shape)": sdpa_model(64),
        "k_scaled_dot_product_attention 8x512 token-major (8-GPU shard)": sdpa_model(8),
    }


def kernel_table(peaks: dict, only: str | None = None, launches: int = 0) -> list[dict]:
    """One row per named kernel configuration, timed as a CUDA graph of back-to-back launches (median, min). With
    ``launches`` > 0 the matching cases are instead launched eagerly that many times and not timed by graph — the
    small, self-ending program a profiler is pointed at (``bench.py --only-kernel <substring> --launches 2``)."""
    import torch

    from deplodock_b200 import ops

    rows = []
    for name, build in kernel_cases().items():
        if only and only not in name:
            continue
        fn, bound, work, unit_scale, peak_key, note, reps = build()
        if launches > 0:
            fn()
            torch.cuda.synchronize()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(launches):
                fn()
            e.record()
            torch.cuda.synchronize()
            us = mn = s.elapsed_time(e) * 1e3 / launches
            note = f"{note}; {launches} eager launches"
        else:
            us, mn = _graph_time_us(fn, reps)
        achieved = work / (us * 1e-6) / unit_scale
        peak = peaks.get(peak_key, 72.0)   # fp32 CUDA-core rows: nominal 148 SMs x 128 FMA lanes x 2 x 1.9 GHz
        rows.append({"kernel": name, "us": round(us, 2), "us_min": round(mn, 2), "bound": bound,
                     "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s" if bound == "hbm" else "TFLOP/s",
                     "frac": round(achieved / peak, 4), "note": note})
        del fn
        torch.cuda.empty_cache()
    ops.device_status()
    return rows


# ------------------------------------------------------------------------------------------------------------
# Main arm
# ------------------------------------------------------------------------------------------------------------
def gemm_event_pass(model, passes: int = 8, heat=None, gpu_index: int = 0) -> dict:
    """Eager passes of the plan with CUDA events around every kernel launch (on the launching stream): time per
    kernel family, and for the tcgen05 GEMM the flops and time per operand shape. ``heat()`` (about a second of graph
    replays) runs first and the ``passes`` instrumented passes follow it back to back without a synchronisation in
    between, so the launches are timed at the sustained, power-capped clock of the timed region and not at the
    burst clock of an idle GPU; the SM clock is sampled while they run. Returns per-forward averages."""
    import torch

    from deplodock_b200 import ops

    names = ["embed_gather", "rmsnorm", "linear", "linear_qknorm_rope", "gemm_fused", "gemm_chain",
             "sdpa_causal_gqa_tok", "pool_norm_l2"]
    originals = {n: getattr(ops, n) for n in names}
    events = []

    def wrap(name, fn):
        def timed(*args, **kw):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            r = fn(*args, **kw)
            e.record()
            fam, key, fl = name, name, 0
            if name == "gemm_chain":   # several projections in one persistent launch: flops summed over its phases
                phases = args[0]
                M = phases[0]["x"].numel() // phases[0]["x"].shape[-1]
                fl = sum(2 * M * ph["x"].shape[-1] * ph["w"].shape[0] for ph in phases)
                key = f"chain[{M} rows: " + " -> ".join(f"{ph['w'].shape[0]}x{ph['x'].shape[-1]}+{ph['epilogue']}"
                                                       for ph in phases) + "]"
                fam = "linear"
            elif name in ("linear", "linear_qknorm_rope", "gemm_fused"):
                x, w = args[0], args[1]
                M = x.numel() // x.shape[-1]
                fl = 2 * M * x.shape[-1] * w.shape[0]
                if name == "gemm_fused":
                    epi = kw.get("epilogue", "none") + ("+rmsnorm_in" if kw.get("row_sumsq_in") is not None else "") + (
                        "+sumsq_out" if kw.get("row_sumsq_out") is not None else "")
                else:
                    epi = "qknorm_rope" if name != "linear" else (
                        "residual" if kw.get("residual") is not None else ("swiglu" if kw.get("swiglu") else "none"))
                key = f"{M}x{w.shape[0]}x{x.shape[-1]}+{epi}"
                fam = "linear"
            events.append((s, e, fam, key, fl))
            return r
        return timed

    for n in names:
        setattr(ops, n, wrap(n, originals[n]))
    sampler = ClockSampler(gpu_index)
    try:
        model.forward_eager()
        torch.cuda.synchronize()
        events.clear()
        if heat is not None:
            heat()
        sampler.start()
        for _ in range(passes):
            model.forward_eager()
        torch.cuda.synchronize()
    finally:
        clocks = sampler.stop()
        for n in names:
            setattr(ops, n, originals[n])
    families: dict[str, list] = {}
    by_shape: dict[str, list] = {}
    for s, e, name, key, fl in events:
        ms = s.elapsed_time(e)
        f = families.setdefault(name, [0, 0.0])
        f[0] += 1
        f[1] += ms
        if name == "linear":
            acc = by_shape.setdefault(key, [0, 0.0, 0])
            acc[0] += 1
            acc[1] += ms
            acc[2] += fl
    shapes = {k: {"launches": n // passes, "avg_us": round(ms * 1e3 / n, 1), "tflops": round(fl / (ms * 1e-3) / 1e12, 1)}
              for k, (n, ms, fl) in by_shape.items()}
    fam = {k: {"launches": n // passes, "ms": round(ms / passes, 3)} for k, (n, ms) in families.items()}
    lin = families.get("linear", [0, 0.0])
    return {"launches": lin[0] // passes, "ms": lin[1] / passes, "flops": sum(v[2] for v in by_shape.values()) // passes,
            "by_shape": shapes, "families": fam, "all_kernels_ms": sum(ms for _, ms in families.values()) / passes,
            "passes": passes, "sm_mhz": clocks.get("sm_mhz"), "reasons": clocks.get("reasons")}


# DRAM read + write bytes of ONE gemm2_bf16_kernel launch from an ncu capture of the model's down projection at the
# full row count of a one-GPU shard (32768 x 3072 -> 1024 with the residual epilogue; 201 MB activations + 67 MB
# residual in, 67 MB out: together they do not fit the 126 MB L2, so the figure is not flattered by a resident
# output): 292.3 MB read + 52.3 MB written = 344.6 MB against 341.8 MB algorithmic. The summary with the command is
# profiles/gemm2_bf16_down_proj_32768x3072x1024.md. Rows scale the figure for a smaller shard.
GEMM_TRAFFIC_CAPTURE = {"bytes": 344595712, "rows": 32768, "algorithmic_bytes": 32768 * (3072 + 1024 + 1024) * 2 + 1024 * 3072 * 2,
                        "kernel": "gemm2_bf16_kernel, down projection + residual of one rank's shard",
                        "source": "profiles/gemm2_bf16_down_proj_32768x3072x1024.md"}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-kernels", action="store_true", help="skip the per-kernel table")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU oracle pass (no parity check, no CPU baseline)")
    ap.add_argument("--chunk-seqs", type=int, default=0, help="sequences per activation chunk (0 = whole shard)")
    ap.add_argument("--only-kernel", default=None, metavar="SUBSTR",
                    help="run only the named kernel configurations whose name contains SUBSTR and print their rows")
    ap.add_argument("--launches", type=int, default=0,
                    help="with --only-kernel: launch eagerly this many times (a small program for a profiler)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    if args.impl == "reference":
        run_reference_arm(args)
        return

    import torch
    import torch.distributed as dist

    from deplodock_b200 import cabi, ops
    from deplodock_b200.dist import PipelinedGather, gather_embeddings, init_process_group, shard_batch
    from deplodock_b200.model import EmbedConfig, EmbedForward

    cabi.load_library()  # fail loudly when the CUDA extension is missing
    if args.only_kernel:
        peaks, _ = load_peaks()
        torch.cuda.set_device(0)
        print(json.dumps({"kernels": kernel_table(peaks, args.only_kernel, args.launches)}), flush=True)
        return
    rank, local_rank, world = init_process_group()
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    peaks, peak_src = load_peaks()

    cfg = EmbedConfig()
    shard = shard_batch(BATCH, rank, world)

    # Weights and ids: the seeded synthetic inputs of the benchmark configuration, generated on the CPU (N(0, 0.02)
    # projections and embeddings, norm weights 1, uniform-random ids; identical on every rank = replicated weights).
    # The CPU oracle below is run on these same tensors, so the timed outputs are the ones that get checked.
    from oracle import inputs as oin

    ocfg = oin.EmbedModelConfig()
    sd_cpu = oin.embed_model_weights(ocfg, seed=0)
    H = cfg.hidden_size
    model = EmbedForward(cfg, sd_cpu, batch=shard.size, seq=SEQ, device=dev, chunk_seqs=args.chunk_seqs or None)
    check = rank == 0 and not args.no_cpu
    if not check:
        del sd_cpu
    ids_all = oin.token_ids(BATCH, SEQ, cfg.vocab_size, seed=0)
    ids_host = ids_all[shard.start:shard.stop].contiguous().pin_memory()
    model.ids.copy_(ids_host)
    model.capture()
    gathered = torch.empty(BATCH, H, dtype=torch.float32, device=dev)
    out_host = torch.empty(BATCH, H, dtype=torch.float32).pin_memory()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # device-timed steps: the all-gather of step i runs beside the forward of step i + 1 (PipelinedGather); every
    # gather still in flight is waited for before the closing event of the timed region
    pipe = PipelinedGather(shard.size, BATCH, H, dev) if shard.size * world == BATCH else None

    def step_device():
        model.replay()
        if pipe is not None:
            pipe.submit(model.out)
        else:
            gather_embeddings(model.out, BATCH, out=gathered)

    def finish_device():
        if pipe is not None:
            gathered.copy_(pipe.result())
            pipe.flush()

    def step_e2e():
        model(ids_host)
        gather_embeddings(model.out, BATCH, out=gathered)
        out_host.copy_(gathered, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def timed(fn, steps, finish=None):
        barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(steps):
            fn()
        if finish is not None:
            finish()
        e.record()
        barrier()
        ms = torch.tensor([s.elapsed_time(e)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item()

    for _ in range(args.warmup):
        step_device()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    total_ms = timed(step_device, args.steps, finish_device)
    clocks = sampler.stop() if sampler else None
    for _ in range(2):
        step_e2e()
    e2e_ms = timed(step_e2e, args.steps)
    ops.device_status()
    finite = bool(torch.isfinite(gathered).all().item())
    got_all = out_host.clone()   # the gathered embeddings of the last end-to-end step

    ms_per_step = total_ms / args.steps
    value = BATCH / (ms_per_step * 1e-3)
    e2e_value = BATCH / (e2e_ms / args.steps * 1e-3)

    if rank == 0:
        def heat():   # about a second of graph replays: the instrumented passes start at the sustained clock
            for _ in range(max(3, int(1000.0 / max(ms_per_step, 1e-3)))):
                model.replay()

        gp = gemm_event_pass(model, passes=8 if world == 1 else 16, heat=heat, gpu_index=local_rank)
        gemm_tflops = gp["flops"] / (gp["ms"] * 1e-3) / 1e12
        peak = peaks["bf16_tflops_sustained"]
        cap = GEMM_TRAFFIC_CAPTURE
        roofline = {
            "bound": "tensor",
            "kernel": ("gemm2_chain_kernel + gemm2_bf16_kernel (tcgen05 cta_group::2; o_proj, gate/up, down and the "
                       "next layer's QKV of every layer as one persistent launch)" if model.chain else
                       "gemm2_bf16_kernel (tcgen05 cta_group::2, all four projections of every layer)"),
            "achieved": round(gemm_tflops, 1), "peak": peak, "peak_source": f"{peak_src} (sustained cuBLAS bf16)",
            "unit": "TFLOP/s", "frac": round(gemm_tflops / peak, 4),
            "frac_of_burst_peak": round(gemm_tflops / peaks["bf16_tflops"], 4),
            "launches_per_step": gp["launches"], "avg_launch_us": round(gp["ms"] * 1e3 / gp["launches"], 2),
            "gemm_share_of_step": round(gp["ms"] / gp["all_kernels_ms"], 4),
            # the instrumented passes follow ~1 s of replays without a pause: their clock and their kernel-time sum
            # are reported so that the fraction can be read against the peak that matches the clock
            "event_pass": {"passes": gp["passes"], "all_kernels_ms": round(gp["all_kernels_ms"], 3),
                           "vs_ms_per_step": round(gp["all_kernels_ms"] / ms_per_step, 4),
                           "sm_mhz": gp["sm_mhz"], "reasons": gp["reasons"]},
            "by_shape": gp["by_shape"],
            "traffic": None if cap["bytes"] is None else cap["bytes"] * shard.size * SEQ / cap["rows"],
            "traffic_algorithmic": cap["algorithmic_bytes"] * shard.size * SEQ / cap["rows"],
            "traffic_kernel": cap["kernel"], "traffic_source": cap["source"],
        }
        step_flops = cfg.linear_flops_per_token() * BATCH * SEQ + cfg.attention_flops(BATCH, SEQ)
        line = {
            "metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "qwen3-embedding-0.6b-shaped forward: 28 layers, hidden 1024, 16/8 heads x 128, "
                                   "SwiGLU 3072, vocab 151669; 64 sequences x 512 uniform-random ids; causal; "
                                   "last-token pool + L2; random-init N(0,0.02) bf16 weights",
                       "global_batch": BATCH, "seq_len": SEQ, "parallelism": f"batch-shard x{world}, weights replicated",
                       "l2_policy": "inputs larger than L2 (1.2 GB of weights + activations per step)",
                       "cuda_graph": True, "chunk_seqs": model.chunk_seqs, "gemm_chain": model.chain},
            "step_tflops": round(step_flops / (ms_per_step * 1e-3) / 1e12, 1),
            "seqs_per_s_per_sm_mhz": None if not clocks or not clocks.get("sm_mhz") else round(
                value / clocks["sm_mhz"], 4),
            "e2e": {"value": round(e2e_value, 2), "unit": UNIT, "h2d_bytes_per_step": BATCH * SEQ * 8,
                    "d2h_bytes_per_step": BATCH * H * 4, "ms_per_step": round(e2e_ms / args.steps, 4)},
            "gpu_launches": model.num_launches * args.steps,
            "clocks": clocks, "roofline": roofline, "outputs_finite": finite,
            "step_breakdown_ms": gp["families"],
        }
        if world == 1 and not args.no_kernels:
            weights = model.weights
            del model
            torch.cuda.empty_cache()
            line["serving"] = serving_table(weights)
            del weights
            torch.cuda.empty_cache()
            line["kernels"] = kernel_table(peaks)
            line["loop_records"] = loop_record_table()
        parity_ok = True
        if check:
            # The CPU oracle (eager trunk) on the same weights and the same 64 sequences: it is the timed CPU baseline
            # at one GPU, and at every GPU count its output is what the timed run's embeddings are held against.
            res = cpu_reference_sample(sd_cpu, ocfg, BATCH, repeats=2 if world == 1 else 1)
            ref = res.pop("embeddings")
            cos = torch.nn.functional.cosine_similarity(got_all.double(), ref.double(), dim=-1)
            max_abs = (got_all - ref).abs().max().item()
            parity_ok = bool(cos.min().item() >= 0.999 and max_abs <= 2e-2)
            line["parity"] = {"checked_embeddings": BATCH, "min_cos": round(cos.min().item(), 6),
                              "max_abs": float(f"{max_abs:.3e}"), "tolerance": "cos >= 0.999, max abs <= 2e-2",
                              "against": "eager CPU trunk on the same weights and ids", "ok": parity_ok}
            if world == 1:
                line["cpu_baseline"] = {k: v for k, v in res.items() if k != "seconds"}
        print(json.dumps(line), flush=True)
        if not parity_ok:
            print("bench: embeddings of the timed run are outside the tolerance of the CPU oracle", file=sys.stderr)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0 and not parity_ok:
        raise SystemExit(1)


if __name__ == "__main__":
    main()
