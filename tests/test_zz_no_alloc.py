"""The batched-GEMM entry point that allocates nothing (dlf_b200_gemm_batched_noalloc).

It exists for callers that cannot provide device scratch and may not allocate any when they call:
inside dlf that is a routine running while the context's LIFO temporary-buffer pool is already
held further up the call stack; outside dlf it is any process that gave all of its device memory
to some other owner at start-up. The entry point keeps the per-batch tables in a fixed array that
is part of the library's device image, so every call reuses the same memory: this test makes two
calls in a row with different problems and checks each against the ordinary entry point (which
takes its scratch from the caller), through the C-ABI in both cases.

This file sorts last on purpose: a run that stops at the first failure has then already executed
every other test."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

HALF_TOL = 2e-2   # fp16 max relative error, as in test_gpu_parity.py
FP32_TOL = 1e-5   # fp32 relative Frobenius error


def _call(L, noalloc, dtype, m, n, k, alphas, A, a_offs, lda, B, b_offs, ldb, betas, C, c_offs, ldc, sync=True):
    batch = len(a_offs)
    prec = 32 if dtype == torch.float32 else 16
    arr = ctypes.c_size_t * batch
    ao, bo, co = arr(*a_offs), arr(*b_offs), arr(*c_offs)
    al = torch.tensor(alphas, dtype=torch.float64).to(dtype).contiguous()
    be = torch.tensor(betas, dtype=torch.float64).to(dtype).contiguous()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    common = [prec, 101, 111, 112, m, n, k, ctypes.c_void_p(al.data_ptr()),
              ctypes.c_void_p(A.data_ptr()), ao, lda, ctypes.c_void_p(B.data_ptr()), bo, ldb,
              ctypes.c_void_p(be.data_ptr()), ctypes.c_void_p(C.data_ptr()), co, ldc, batch]
    if noalloc:
        rc = L.dlf_b200_gemm_batched_noalloc(*common, stream)
    else:
        need = L.dlf_b200_gemm_batched_workspace_bytes(batch)
        ws = torch.empty(need, dtype=torch.uint8, device="cuda")
        rc = L.dlf_b200_gemm_batched(*common, ctypes.c_void_p(ws.data_ptr()), need, stream)
    if sync:
        torch.cuda.synchronize()
    return rc


def _problem(seed, dtype, m, n, k, batch):
    g = torch.Generator().manual_seed(seed)
    a_offs = [3 + i * (m * k + 5) for i in range(batch)]
    b_offs = [(batch - 1 - i) * (n * k + 2) for i in range(batch)]
    c_offs = [1 + i * (m * n + 7) for i in range(batch)]
    A = (torch.rand(a_offs[-1] + m * k, generator=g) * 2 - 1).to(dtype).cuda()
    B = (torch.rand(b_offs[0] + n * k, generator=g) * 2 - 1).to(dtype).cuda()
    C = torch.randn(c_offs[-1] + m * n, generator=g).to(dtype)
    alphas = [0.5 + 0.125 * i for i in range(batch)]
    betas = [0.0 if i % 2 else 0.5 for i in range(batch)]
    return A, a_offs, B, b_offs, C, c_offs, alphas, betas


def test_noalloc_entry_matches_workspace_entry_on_two_calls_in_a_row():
    import dlf_b200
    L = dlf_b200.lib()
    # second problem is smaller than the first: stale table entries of call 1 must not matter
    for seed, dtype, (m, n, k, batch) in ((1, torch.float16, (96, 72, 136, 9)),
                                          (2, torch.float32, (40, 56, 24, 4))):
        A, a_offs, B, b_offs, C, c_offs, alphas, betas = _problem(seed, dtype, m, n, k, batch)
        c_ref, c_new = C.clone().cuda(), C.clone().cuda()
        # row-major, A not transposed (ld = k), B transposed (stored n x k, ld = k)
        assert _call(L, False, dtype, m, n, k, alphas, A, a_offs, k, B, b_offs, k, betas, c_ref, c_offs, n) == 0
        assert _call(L, True, dtype, m, n, k, alphas, A, a_offs, k, B, b_offs, k, betas, c_new, c_offs, n) == 0
        ref, got = c_ref.float().cpu().numpy().astype(np.float64), c_new.float().cpu().numpy().astype(np.float64)
        assert np.isfinite(got).all()
        if dtype == torch.float32:
            assert np.linalg.norm(got - ref) <= FP32_TOL * np.linalg.norm(ref)
        else:
            den = np.maximum(np.abs(ref), 1e-2 * np.abs(ref).max())
            assert (np.abs(got - ref) / den).max() <= HALF_TOL
        # and the ordinary entry point itself is right: one batch entry against float64
        i = batch - 1
        a = A[a_offs[i]:a_offs[i] + m * k].double().cpu().reshape(m, k)
        b = B[b_offs[i]:b_offs[i] + n * k].double().cpu().reshape(n, k)
        c0 = C[c_offs[i]:c_offs[i] + m * n].double().reshape(m, n)
        al = float(torch.tensor(alphas[i]).to(dtype))
        be = float(torch.tensor(betas[i]).to(dtype))
        want = al * (a @ b.t()) + be * c0
        have = c_new[c_offs[i]:c_offs[i] + m * n].double().cpu().reshape(m, n)
        assert float((have - want).norm() / want.norm()) <= (1e-5 if dtype == torch.float32 else 2e-3)
    assert dlf_b200.device_status() == 0


def test_noalloc_calls_queued_back_to_back_share_the_table_in_stream_order():
    """Two calls of different size on one stream with no host wait between them: the second call's
    tables overwrite the first call's only after the first kernel has run. The second problem uses
    every entry the fixed array has (4096 batches). Device memory in use must not change."""
    import dlf_b200
    L = dlf_b200.lib()
    dtype = torch.float16
    p1 = _problem(3, dtype, 64, 48, 72, 11)
    p2 = _problem(4, dtype, 8, 16, 8, 4096)
    outs = []
    for (A, a_offs, B, b_offs, C, c_offs, alphas, betas), (m, n, k) in ((p1, (64, 48, 72)), (p2, (8, 16, 8))):
        c_ref = C.clone().cuda()
        assert _call(L, False, dtype, m, n, k, alphas, A, a_offs, k, B, b_offs, k, betas, c_ref, c_offs, n) == 0
        outs.append((c_ref, C.clone().cuda()))
    # one warmed-up call first, so that the per-device set-up is not what is measured below
    A, a_offs, B, b_offs, C, c_offs, alphas, betas = p1
    scratch = C.clone().cuda()
    assert _call(L, True, dtype, 64, 48, 72, alphas, A, a_offs, 72, B, b_offs, 72, betas, scratch, c_offs, 48) == 0
    free0, _ = torch.cuda.mem_get_info()
    for (A, a_offs, B, b_offs, C, c_offs, alphas, betas), (m, n, k), (_, c_new) in (
            (p1, (64, 48, 72), outs[0]), (p2, (8, 16, 8), outs[1])):
        assert _call(L, True, dtype, m, n, k, alphas, A, a_offs, k, B, b_offs, k, betas, c_new, c_offs, n,
                     sync=False) == 0
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 >= free0  # nothing was taken from the device's free memory
    for c_ref, c_new in outs:
        assert torch.equal(c_ref, c_new)
    assert dlf_b200.device_status() == 0


def test_noalloc_entry_rejects_more_batches_than_its_static_scratch_holds():
    import dlf_b200
    L = dlf_b200.lib()
    batch = 4097  # DLF_B200_NOALLOC_MAX_BATCH + 1
    offs = (ctypes.c_size_t * batch)()
    sc = (ctypes.c_float * batch)()
    buf = torch.zeros(64, device="cuda")
    p = ctypes.c_void_p(buf.data_ptr())
    rc = L.dlf_b200_gemm_batched_noalloc(32, 101, 111, 111, 4, 4, 4, sc, p, offs, 4, p, offs, 4, sc, p,
                                         offs, 4, batch, None)
    assert rc == -2050
    assert dlf_b200.status_string(rc) == "kInsufficientMemoryTemp"
