"""Runs ONE of the named kernel configurations a few times on seeded device inputs — the small, self-ending program
the profiler is pointed at (``ncu -k regex:<kernel> ... python -m deplodock_b200.kernel_case <case>``), and a quick
per-kernel timing tool. Cases mirror the benchmark configurations; ``--scale`` shrinks the leading dimension.

The reference's counterpart is ``emmy run -c "<expr>" --bench --profile`` (``emmy/commands/run.py:670-928``), which
re-invokes itself under ``ncu``; here the profiler is started by the caller and this module only launches kernels.
"""

from __future__ import annotations

import argparse

import torch

from deplodock_b200 import ops

CASES = ("rmsnorm", "rmsnorm_big", "softmax", "linear", "linear_model", "linear_w8", "sdpa", "sdpa_model", "qknorm_rope")


def build_case(name: str, scale: float = 1.0):
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(0)

    def rn(*shape):
        return torch.randn(*shape, device=dev, generator=g)

    if name == "rmsnorm":
        x, w = rn(1, 32, 2048), 1 + 0.02 * rn(2048)
        y = torch.empty_like(x)
        return lambda: ops.rmsnorm(x, w, 1e-6, out=y)
    if name == "rmsnorm_big":
        x = rn(int(32768 * scale), 1024).bfloat16()
        w = torch.ones(1024, device=dev, dtype=torch.bfloat16)
        y = torch.empty_like(x)
        return lambda: ops.rmsnorm(x, w, 1e-6, out=y)
    if name == "softmax":
        x = 3 * rn(int(28 * 2048 * scale), 2048)
        m = torch.rand(x.shape, device=dev, generator=g) < 0.01
        m[:, 0] = False
        x[m] = float("-inf")
        y = torch.empty_like(x)
        return lambda: ops.softmax_lastdim(x, out=y)
    if name in ("linear", "linear_w8", "linear_model"):
        M, K, N = (int(4096 * scale), 2048, 6144) if name != "linear_model" else (int(32768 * scale), 1024, 4096)
        x = rn(M, K).bfloat16()
        w32 = 0.02 * rn(N, K)
        y = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        if name == "linear_w8":
            s = (w32.abs().amax(1) / 448.0).contiguous()
            wq = (w32 / s[:, None]).to(torch.float8_e4m3fn)
            return lambda: ops.linear_w8(x, wq, s, out=y)
        w = w32.bfloat16()
        return lambda: ops.linear(x, w, out=y)
    if name == "sdpa":
        B = max(1, int(4 * scale))
        q, k, v = rn(B, 16, 2048, 128).bfloat16(), rn(B, 8, 2048, 128).bfloat16(), rn(B, 8, 2048, 128).bfloat16()
        o = torch.empty_like(q)
        return lambda: ops.sdpa_causal_gqa(q, k, v, out=o)
    if name == "sdpa_model":   # the attention launch of the model plan: token-major fused QKV buffer, 64 x 512 tokens
        B = max(1, int(64 * scale))
        qkv = rn(B * 512, 4096).bfloat16()
        o = torch.empty(B * 512, 2048, device=dev, dtype=torch.bfloat16)
        return lambda: ops.sdpa_causal_gqa_tok(qkv, B, 512, 16, 8, o)
    if name == "qknorm_rope":
        T, S = int(32768 * scale), 512
        qkv = rn(T, 4096).bfloat16()
        qw = torch.ones(128, device=dev, dtype=torch.bfloat16)
        from deplodock_b200.model import rope_tables

        cos, sin = rope_tables(S, 128, 1e6, dev)
        return lambda: ops.qknorm_rope_(qkv, qw, qw, cos, sin, S, 16, 8, 1e-6)
    raise SystemExit(f"unknown case {name!r}; choose from {CASES}")


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("case", choices=CASES)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--scale", type=float, default=1.0)
    args = ap.parse_args()
    fn = build_case(args.case, args.scale)
    fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(args.iters):
        fn()
    e.record()
    ops.device_status()
    print(f"{args.case}: {s.elapsed_time(e) / args.iters * 1e3:.2f} us per launch over {args.iters} launches (eager)")


if __name__ == "__main__":
    main()
