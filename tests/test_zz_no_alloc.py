"""The allocation-free entry point (``emk_linear_residual_rmsnorm_bf16_noalloc``) against the ordinary entry points.

Some users of the library cannot allocate device memory at call time — a plugin inside a serving process that handed
the whole device heap to its own pool at start-up, code that runs while a CUDA stream is being captured, a control loop
that cannot afford the device-wide synchronisation cudaMalloc/cudaFree imply. For them the library keeps the scratch
between the projection+residual GEMM and the RMSNorm that follows it in a fixed array of its own. This file checks,
through the C ABI, that the call gives what ``emk_linear_bf16`` (residual epilogue) followed by ``emk_rmsnorm`` gives,
twice in a row (the array keeps the previous call's contents, which must not leak into the next result), that the
caller's buffers are the only memory written, and that sizes beyond the built-in array are refused with a clear error.
It sorts last on purpose so a run that stops at the first failure has already run everything else."""

from __future__ import annotations

import ctypes

import pytest
import torch

from oracle import cpu_ref, inputs, metrics

pytestmark = pytest.mark.gpu


def _call(lib, h, x, w, res, nw, hid, nrm, M, N, K, eps):
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    return lib.emk_linear_residual_rmsnorm_bf16_noalloc(
        h.ptr, ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(w.data_ptr()), ctypes.c_void_p(res.data_ptr()),
        ctypes.c_void_p(nw.data_ptr()), ctypes.c_void_p(hid.data_ptr()), ctypes.c_void_p(nrm.data_ptr()), M, N, K,
        ctypes.c_float(eps), stream)


def test_no_alloc_entry_matches_existing_entries_twice(libemk):
    from deplodock_b200 import cabi, ops

    lib = cabi.load_library()
    h = ops.handle()
    eps = 1e-6
    # the third case has M <= 128: the GEMM behind the call is then the single-CTA kernel, not the CTA-pair one
    for call_no, (M, K, N, seed) in enumerate([(520, 256, 1024, 3), (300, 512, 640, 4), (96, 256, 384, 5)]):
        x, w = inputs.linear_inputs(M, K, N, seed=seed)
        g = torch.Generator().manual_seed(100 + seed)
        res = torch.randn(M, N, generator=g).bfloat16()
        nw = (1 + 0.1 * torch.randn(N, generator=g)).bfloat16()
        xd, wd, rd, nd = x.cuda(), w.cuda(), res.cuda(), nw.cuda()
        hid = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        nrm = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        rc = _call(lib, h, xd, wd, rd, nd, hid, nrm, M, N, K, eps)
        assert rc == cabi.EMK_OK, h.last_error()
        ops.device_status()
        assert torch.cuda.memory_allocated() == before  # nothing came out of torch's allocator either
        # ... nor out of the driver's: a cudaMalloc inside the library is invisible to torch's counters, but not to
        # the device's free-memory figure. The call above was the warm-up of this shape class (module load, symbol
        # look-up, kernel attributes); a second call must leave the free memory where it was.
        free_before = torch.cuda.mem_get_info()[0]
        rc = _call(lib, h, xd, wd, rd, nd, hid, nrm, M, N, K, eps)
        assert rc == cabi.EMK_OK, h.last_error()
        ops.device_status()
        assert torch.cuda.mem_get_info()[0] == free_before
        # existing entry points, same inputs
        want_hid = ops.linear(xd, wd, residual=rd)
        want_nrm = ops.rmsnorm(want_hid, nd, eps)
        ops.device_status()
        assert torch.equal(hid, want_hid), f"call {call_no}: hidden differs from emk_linear_bf16"
        metrics.assert_bf16_tensor_path(nrm.cpu(), want_nrm.cpu(), what=f"call {call_no}: norm vs emk_rmsnorm")
        assert (nrm != want_nrm).float().mean().item() < 0.02  # same rounding steps; only the fp32 sum order differs
        ref_h = cpu_ref.linear(x, w) + res
        metrics.assert_bf16_tensor_path(nrm.cpu(), cpu_ref.rmsnorm_hf(ref_h, nw, eps), abs_tol=6e-2,
                                        what=f"call {call_no}: norm vs eager CPU")


def test_no_alloc_entry_rejects_sizes_beyond_its_array(libemk):
    from deplodock_b200 import cabi, ops

    lib = cabi.load_library()
    h = ops.handle()
    t = torch.zeros(8, dtype=torch.bfloat16, device="cuda")  # never dereferenced: the size check comes first
    M, N, K = 1 << 18, 1024, 64  # 2^18 rows x 8 slots = 2^21 > 2^20
    rc = _call(lib, h, t, t, t, t, t, t, M, N, K, 1e-6)
    assert rc == cabi.EMK_ERR_LIMIT
    assert "exceeds the built-in scratch" in h.last_error()
    with pytest.raises(ValueError):
        h.check(rc, "emk_linear_residual_rmsnorm_bf16_noalloc")
