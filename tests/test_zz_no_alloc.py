"""The allocation-free PQ matvec entry point (ibcu_pq_matmul_fp32_noalloc).

It exists for callers that may not allocate device memory when they call in - a serving loop that
cannot afford cudaMalloc's device-wide synchronisation, a plugin inside a fixed memory budget, a
process whose allocator belongs to another runtime - and keeps its scratch (the fixed-point row
accumulators and arrival counters of the PQ kernel) in an array built into the library. It runs the
same kernel as ibcu_pq_matmul_fp32, so the two must agree to the bit; the test calls it twice in a
row because the array is shared between calls and keeps old contents.
This file sorts last so that a run stopping at the first failure has already run everything else.
"""
import ctypes as C

import numpy as np
import pytest

from tests import _cpu

pytestmark = pytest.mark.gpu


def test_noalloc_matches_allocating_entry_point_twice(backend):
    be = backend
    rng = np.random.default_rng(2024)
    M, N, G, K, B = 1000, 2048, 16, 256, 2
    cb_l, cb_r, il, ir, rs, x = _cpu.make_pq_case(rng, M, N, G, K, B)
    t = be.make_pq(M, N, G, K, cb_l, cb_r, il, ir, rs)
    want = be.pq_matmul(t, x)                                    # existing entry point
    dx, do = be.upload(x), be.alloc(B * M * 4)
    for call in range(2):
        xs = x if call == 0 else (x[::-1].copy() * 0.5)           # second call: other inputs over stale scratch
        ref = want if call == 0 else be.pq_matmul(t, xs)
        be.write(dx, xs)
        be._check(be.lib.ibcu_memset(be.ctx, do.ptr, 0xFF, B * M * 4))
        be._check(be.lib.ibcu_pq_matmul_fp32_noalloc(be.ctx, C.byref(t), dx.ptr, do.ptr, B))
        be.sync()
        got = be.download(do, np.float32, B * M).reshape(B, M)
        assert _cpu.close(got, ref, 1e-3, 1e-4), call
        assert np.array_equal(got, ref), call                     # same kernels, same order of additions


def test_noalloc_refuses_what_does_not_fit(backend):
    be = backend
    cap = be.lib.ibcu_pq_noalloc_max_floats()
    assert cap == 1 << 20
    rng = np.random.default_rng(7)
    M, N, G, K, B = 40000, 256, 16, 256, 16                        # 16 activations x 40000 rows x 8 bytes = 1.28 Mi floats > 1 Mi
    cb_l, cb_r, il, ir, rs, x = _cpu.make_pq_case(rng, M, N, G, K, B)
    t = be.make_pq(M, N, G, K, cb_l, cb_r, il, ir, rs)
    dx, do = be.upload(x), be.alloc(B * M * 4)
    assert be.lib.ibcu_pq_matmul_fp32_noalloc(be.ctx, C.byref(t), dx.ptr, do.ptr, B) == -1
    msg = be.lib.ibcu_last_error(be.ctx)
    assert b"floats of scratch" in msg and str(cap).encode() in msg
    be.lib.ibcu_clear_error(be.ctx)
    # the allocating entry point still serves it, and a smaller batch fits the built-in array
    want = np.empty((B, M), np.float32)
    for b in range(B):
        _cpu.load().oracle.ibo_pq_matmul_fp32(M, N, G, K, cb_l, cb_r, 0, il, ir, rs, x[b], want[b], 1, None)
    assert _cpu.close(be.pq_matmul(t, x), want)
    assert be.lib.ibcu_pq_matmul_fp32_noalloc(be.ctx, C.byref(t), dx.ptr, do.ptr, 2) == 0
    be.sync()
    assert _cpu.close(be.download(do, np.float32, 2 * M).reshape(2, M), want[:2])
