"""The bounds-check build of the library (``libemk_check.so``, ``-DEMK_BOUNDS_CHECK``).

Stands in for a memory checker: indices that come from data are checked where they are used, the access is made safe
(clamped or dropped) in BOTH builds, and the checked build reports the violation through ``emk_device_status``. Nothing
here faults: every bad index is caught before it reaches memory."""

from __future__ import annotations

import subprocess
import sys
import textwrap
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def test_both_builds_export_the_flag(libemk):
    import ctypes

    from deplodock_b200 import build

    assert ctypes.CDLL(str(libemk)).emk_bounds_check_enabled() == 0
    path = build.build(bounds_check=True)
    assert path.name == "libemk_check.so" and ctypes.CDLL(str(path)).emk_bounds_check_enabled() == 1


SCRIPT = textwrap.dedent('''
    import sys
    sys.path.insert(0, %r)
    import numpy as np, torch
    from deplodock_b200 import cabi, ops
    from deplodock_b200.model import rope_tables
    from oracle import cpu_ref, inputs, metrics
    checked = bool(cabi.load_library().emk_bounds_check_enabled())
    assert checked == cabi.BOUNDS_CHECK

    def expect(kind, fn):
        fn()
        if checked:
            try:
                ops.device_status()
            except IndexError as e:
                assert kind in str(e), str(e)
            else:
                raise AssertionError(kind + ": violation not reported")
        else:
            ops.device_status()          # the normal build clamps silently
        ops.device_status()              # the word is cleared, the context is fine

    # in-range work passes in both builds
    x, w = inputs.linear_inputs(300, 256, 520)
    metrics.assert_bf16_tensor_path(ops.linear(x.cuda(), w.cuda()).cpu(), cpu_ref.linear(x, w), what="linear")
    table = torch.randn(50, 1024).bfloat16().cuda()
    ids = inputs.token_ids(2, 9, 50).cuda()
    good = ops.embed_gather(table, ids)
    ops.device_status()
    # 1. token id outside the vocabulary: clamped to the last row, reported by the checked build
    bad = ids.clone(); bad[0, 3] = 10 ** 9; bad[1, 1] = -5
    got = None
    def gather():
        global got
        got = ops.embed_gather(table, bad)
    expect("token id", gather)
    assert torch.equal(got[3], table[49]) and torch.equal(got[10], table[0]) and torch.equal(got[0], good[0])
    # 2. rotary position outside the table
    Hq, Hkv, S = 4, 2, 64
    T = 256
    h = torch.randn(T, 256).bfloat16().cuda()
    wq = (0.05 * torch.randn((Hq + 2 * Hkv) * 128, 256)).bfloat16().cuda()
    qn = torch.ones(128, dtype=torch.bfloat16, device="cuda")
    cos, sin = rope_tables(S, 128, 1e6, "cuda")
    cm = ops.rope_chunk_major(cos, sin)
    qkv = torch.empty(T, (Hq + 2 * Hkv) * 128, dtype=torch.bfloat16, device="cuda")
    pos = (torch.arange(T, dtype=torch.int32) %% S).cuda()
    ops.gemm_fused(h, wq, qkv, epilogue="qknorm_rope", q_weight=qn, k_weight=qn, rope_cm=cm, S=S, Hq=Hq, Hkv=Hkv,
                   positions=pos)
    ops.device_status()
    ref = qkv.clone()
    pos_bad = pos.clone(); pos_bad[17] = S + 5
    expect("rotary position", lambda: ops.gemm_fused(h, wq, qkv, epilogue="qknorm_rope", q_weight=qn, k_weight=qn,
                                                      rope_cm=cm, S=S, Hq=Hq, Hkv=Hkv, positions=pos_bad))
    keep = torch.ones(T, dtype=torch.bool); keep[17] = False
    assert torch.equal(qkv[keep.cuda()], ref[keep.cuda()]) and torch.isfinite(qkv.float()).all()
    # 3. cu_seqlens pointing past the token rows / longer than max_seqlen: cut to what exists, nothing written outside
    lens = [100, 60]
    qkv2 = torch.randn(160 + 8, (Hq + 2 * Hkv) * 128).bfloat16().cuda()
    out = torch.full((168, Hq * 128), 7.0, dtype=torch.bfloat16, device="cuda")
    cu = torch.tensor([0, 100, 160], dtype=torch.int32).cuda()
    ops.sdpa_causal_gqa_varlen(qkv2, cu, 128, Hq, Hkv, out)
    ops.device_status()
    good_out = out.clone()
    out.fill_(7.0)
    expect("cu_seqlens", lambda: ops.sdpa_causal_gqa_varlen(qkv2, torch.tensor([0, 100, 5000], dtype=torch.int32).cuda(),
                                                            128, Hq, Hkv, out))
    assert torch.equal(out[:100], good_out[:100]) and torch.isfinite(out.float()).all()
    print("BOUNDS_OK", checked)
''') % str(ROOT)


@pytest.mark.gpu
@pytest.mark.parametrize("checked", [True, False])
def test_bad_indices_are_made_safe_and_reported_by_the_checked_build(libemk, checked):
    import os

    from deplodock_b200 import build

    if checked:
        build.build(bounds_check=True)
    env = dict(os.environ, EMK_BOUNDS_CHECK="1" if checked else "0")
    res = subprocess.run([sys.executable, "-c", SCRIPT], capture_output=True, text=True, env=env, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-3000:]
    assert f"BOUNDS_OK {checked}" in res.stdout
