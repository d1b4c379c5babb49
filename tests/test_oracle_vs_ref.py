"""Pins the CPU restatement (oracle/ib_oracle.c) to the unmodified reference library compiled from
the reference checkout (oracle/_ref/libinferbit_ref.so). Skipped where that build is absent."""
import ctypes as C

import numpy as np
import pytest

from tests import _cpu
from tests._cpu import p


@pytest.fixture(scope="module")
def libs(cpu_libs):
    if cpu_libs.ref is None:
        pytest.skip("oracle/_ref/libinferbit_ref.so not built (needs the reference checkout)")
    return cpu_libs


def test_fp16_both_ways_exhaustive(libs):
    o, r = libs.oracle, libs.ref
    for h in range(65536):
        a, b = o.ibo_fp16_to_fp32(h), r.ib_fp16_to_fp32(h)
        assert (a == b) or (a != a and b != b), h
    rng = np.random.default_rng(0)
    vals = np.concatenate([rng.standard_normal(20000) * 10.0 ** rng.integers(-9, 6, 20000),
                           np.array([0.0, -0.0, 65504.0, 65520.0, 65519.9, 1e6, 6e-8, 5.96e-8, 2.98e-8, 1e-9, np.inf, -np.inf])]).astype(np.float32)
    for v in vals:
        assert o.ibo_fp32_to_fp16(float(v)) == r.ib_fp32_to_fp16(float(v)), v
    # every fp16 value round-trips, and the midpoints between neighbours round to even
    for h in range(0, 0x7C00):
        f = np.float32(o.ibo_fp16_to_fp32(h))
        assert o.ibo_fp32_to_fp16(float(f)) == h
        g = np.float32(o.ibo_fp16_to_fp32(h + 1)) if h + 1 < 0x7C00 else None
        if g is not None:
            mid = float(np.float32((np.float64(f) + np.float64(g)) / 2))
            assert o.ibo_fp32_to_fp16(mid) == r.ib_fp32_to_fp16(mid)


@pytest.mark.parametrize("M,N", [(1, 2), (7, 30), (64, 256), (33, 1026), (128, 2048)])
def test_int4_int8_bit_identical_to_scalar_table(libs, M, N):
    rng = np.random.default_rng(M * 1000 + N)
    kern = libs.ref_scalar()
    w4, s16, x = _cpu.make_int4_case(rng, M, N, 3)
    w8, _, _ = _cpu.make_int8_case(rng, M, N, 3)
    s = np.empty(M, np.float32); libs.oracle.ibo_fp16_array_to_fp32(s16, s, M)
    for b in range(3):
        a = np.empty(M, np.float32); r = np.empty(M, np.float32)
        libs.oracle.ibo_matmul_int4(a, w4, s, x[b], M, N); kern.matmul_int4(p(r), p(w4), p(s), p(x[b]), M, N)
        assert np.array_equal(a, r)
        libs.oracle.ibo_matmul_int8(a, w8, s, x[b], M, N); kern.matmul_int8(p(r), p(w8), p(s), p(x[b]), M, N)
        assert np.array_equal(a, r)
    a = np.empty((3, M + 5), np.float32); r = np.empty((3, M + 5), np.float32); a[:] = -1; r[:] = -1
    libs.oracle.ibo_matmul_int8_batch(a, w8, s, x, M, N, 3, M + 5)
    kern.matmul_int8_batch(p(r), p(w8), p(s), p(x), M, N, 3, M + 5)
    assert np.array_equal(a, r)


def test_int4_odd_column_count(libs):
    # the reference guards the last nibble when N is odd (src/kernels/scalar.c:21)
    rng = np.random.default_rng(5)
    M, N = 9, 31
    w = rng.integers(0, 256, size=(M * (N // 2) + 1,), dtype=np.uint8)
    s = rng.uniform(0.002, 0.02, M).astype(np.float32); x = rng.standard_normal(N).astype(np.float32)
    a = np.empty(M, np.float32); r = np.empty(M, np.float32)
    libs.oracle.ibo_matmul_int4(a, w, s, x, M, N); libs.ref_scalar().matmul_int4(p(r), p(w), p(s), p(x), M, N)
    assert np.array_equal(a, r)


@pytest.mark.parametrize("N", [128, 4096, 200, 1])
def test_w4a8_bit_identical(libs, N):
    rng = np.random.default_rng(N)
    B, M = 2, 24
    x = rng.standard_normal((B, N)).astype(np.float32)
    x[0, : min(N, 128)] = 0.0                                  # an all-zero group
    groups = (N + 127) // 128
    qa = np.empty((B, N), np.int8); sa = np.empty((B, groups), np.float32)
    qr = np.empty((B, N), np.int8); sr = np.empty((B, groups), np.float32)
    for b in range(B):
        assert libs.oracle.ibo_quantize_input_int8_g128(x[b], qa[b], sa[b], N) == groups
        assert libs.ref.ib_quantize_input_int8_g128(x[b], qr[b], sr[b], N) == groups
    assert np.array_equal(qa, qr) and np.array_equal(sa, sr)
    if N % 2:
        return
    w = rng.integers(0, 256, size=(M, N // 2), dtype=np.uint8)
    sw = rng.uniform(0.002, 0.02, M).astype(np.float32)
    a = np.empty((B, M), np.float32); r = np.empty((B, M), np.float32)
    libs.oracle.ibo_matmul_w4a8_batch(a, w, sw, qa, sa, M, N, B, M)
    libs.ref_scalar().matmul_w4a8_batch(p(r), p(w), p(sw), p(qr), p(sr), M, N, B, M)
    assert np.array_equal(a, r)
    libs.ref_scalar().matmul_w4a8(p(r[0]), p(w), p(sw), p(qr[0]), p(sr[0]), M, N)
    assert np.array_equal(a[0], r[0])


@pytest.mark.parametrize("M,N,G,K", [(40, 256, 16, 256), (17, 96, 8, 64), (8, 64, 4, 16), (64, 1024, 16, 256)])
def test_pq_matmul_and_reconstruct(libs, M, N, G, K):
    rng = np.random.default_rng(M + N)
    cb_l, cb_r, il, ir, rs, x = _cpu.make_pq_case(rng, M, N, G, K, 2)
    t = libs.ref_pq_tensor(M, N, G, K, cb_l, cb_r, il, ir, rs)
    for b in range(2):
        xb = x[b].copy()
        if b == 1:
            xb[G:3 * G] *= 1e-4                               # two chunks fall under the 1 % rule
        r = np.empty(M, np.float32); a = np.empty(M, np.float32); st = np.empty(M, np.float32)
        assert libs.ref.ib_pq_matmul_fp32(C.byref(t), xb, r) == 0
        skipped = C.c_int(-1)
        assert libs.oracle.ibo_pq_matmul_fp32(M, N, G, K, cb_l, cb_r, 0, il, ir, rs, xb, a, 1, C.byref(skipped)) == 0
        assert skipped.value == (2 if b == 1 else 0)
        # the reference binary's LUT loops are auto-vectorised, so only float-close is promised
        assert _cpu.close(a, r, rtol=1e-5, atol=1e-6)
        assert libs.ref.ib_pq_matmul_fp32_streaming(C.byref(t), xb, st) == 0
        if b == 0:
            assert _cpu.close(st, r, rtol=1e-4, atol=1e-5)
    Wa = np.empty((M, N), np.float32); Wr = np.empty((M, N), np.float32)
    assert libs.oracle.ibo_pq_reconstruct_fp32(M, N, G, K, cb_l, cb_r, il, ir, rs, Wa) == 0
    assert libs.ref.ib_pq_reconstruct_fp32(C.byref(t), Wr) == 0
    assert np.array_equal(Wa, Wr)
    # dense product of the reconstructed weights agrees with the fused path to fp16 rounding of W
    dense = Wr.astype(np.float64) @ x[0].astype(np.float64)
    fused = np.empty(M, np.float32); libs.ref.ib_pq_matmul_fp32(C.byref(t), x[0], fused)
    assert np.max(np.abs(dense - fused)) < 2e-3 * np.max(np.abs(dense))


@pytest.mark.parametrize("M,N,G,K,K_l2,n_out", [(40, 256, 16, 256, 256, 0), (33, 256, 16, 256, 16, 0), (24, 272, 16, 64, 0, 16),
                                               (40, 528, 16, 256, 16, 16), (16, 104, 8, 32, 64, 8)])
def test_pq_second_level_and_outliers(libs, M, N, G, K, K_l2, n_out):
    """Second residual level (byte and 4-bit packed indices) and the outlier sidecar (fewer than 32 columns: the
    reference then takes its scalar form, src/pq_decode.c:1411-1421) against the compiled reference."""
    rng = np.random.default_rng(M + N + K_l2 + n_out)
    d = _cpu.make_pq_case_ex(rng, M, N, G, K, K_l2, n_out, 2)
    t = _cpu.ref_pq_tensor_ex(d)
    for b in range(2):
        xb = d["x"][b].copy()
        if b == 1:
            xb[:2 * G] *= 1e-4                                # chunks under the 1 % rule (some of these columns may be outliers)
        r = np.empty(M, np.float32)
        assert libs.ref.ib_pq_matmul_fp32(C.byref(t), xb, r) == 0
        a = _cpu.oracle_pq_ex(libs.oracle, d, xb)
        assert _cpu.close(a, r, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("M,N,G,K,K_l2,n_out,k_top", [(500, 256, 16, 256, 256, 0, 17), (300, 256, 16, 256, 16, 0, 1), (257, 272, 16, 64, 0, 16, 64),
                                                     (400, 528, 16, 256, 16, 16, 400), (90, 104, 8, 32, 64, 8, 5)])
def test_pq_lm_head_topk(libs, M, N, G, K, K_l2, n_out, k_top):
    """Top-K LM head (src/pq_decode.c:2259-2341): the same token ids in the same order as the compiled reference, logits
    to rounding (the reference's build decides where products and sums contract)."""
    rng = np.random.default_rng(M + N + K_l2 + n_out + k_top)
    d = _cpu.make_pq_case_ex(rng, M, N, G, K, K_l2, n_out, 1)
    t = _cpu.ref_pq_tensor_ex(d)
    xb = d["x"][0].copy()
    xb[:2 * G] *= 1e-4                                        # would fall under the 1 % rule, which this path does not apply
    rl = np.empty(k_top, np.float32); ri = np.empty(k_top, np.int32)
    assert libs.ref.ib_pq_lm_head_topk(C.byref(t), xb, k_top, rl, ri) == 0
    al, ai = _cpu.oracle_pq_topk(libs.oracle, d, xb, k_top)
    assert np.array_equal(ai, ri)
    assert _cpu.close(al, rl, rtol=1e-5, atol=1e-6)
    assert np.all(np.diff(al) <= 0)
    # bad arguments as the reference: K_top outside 1..M
    assert libs.ref.ib_pq_lm_head_topk(C.byref(t), xb, 0, rl, ri) == -1
    assert libs.oracle.ibo_pq_lm_head_topk(M, N, G, K, K_l2, None, None, None, None, None, None, None, None, None, 0, None, None, None,
                                           xb.ctypes.data, M + 1, al.ctypes.data, ai.ctypes.data, None, 1) == -1


def _near_tie_points(rng, D, N):
    Cn = (rng.standard_normal((2, D)) * 0.02).astype(np.float32)
    mid = (Cn[0].astype(np.float64) + Cn[1]) / 2
    d = Cn[1].astype(np.float64) - Cn[0]; d /= np.linalg.norm(d)
    noise = rng.standard_normal((N, D)) * 0.02
    noise -= (noise @ d)[:, None] * d
    return (mid + noise).astype(np.float32), Cn


@pytest.mark.parametrize("D", [1, 2, 3, 4, 5, 7, 8, 9, 12, 16, 17, 32])
def test_kmeans_rounding_mode(libs, D):
    """Points on the bisector of two centroids flip with the last bit of the distance: mode 2 of the
    restatement must reproduce the compiled reference exactly, for every D."""
    rng = np.random.default_rng(100 + D)
    X, Cn = _near_tie_points(rng, D, 1 << 16)
    r = np.empty(len(X), np.int32); a = np.empty(len(X), np.int32)
    assert libs.ref.ib_kmeans_assign(X, len(X), D, Cn, 2, r, None) == 0
    libs.oracle.ibo_kmeans_assign(X, len(X), D, Cn, 2, a, None, 2)
    assert np.array_equal(a, r)


def test_kmeans_assign_config_shape(libs):
    rng = np.random.default_rng(7)
    X = (rng.standard_normal((200000, 8)) * 0.02).astype(np.float32)
    Cn = X[:256].copy()
    X[1000] = X[5]; X[1001] = np.nan                           # an exact tie with centroid 5, and a NaN row
    r = np.empty(len(X), np.int32); a = np.empty(len(X), np.int32)
    libs.ref.ib_kmeans_assign(X, len(X), 8, Cn, 256, r, None)
    libs.oracle.ibo_kmeans_assign(X, len(X), 8, Cn, 256, a, None, 2)
    assert np.array_equal(a, r) and a[1000] == 5 and a[1001] == 0


def test_glue_kernels_bit_identical(libs):
    rng = np.random.default_rng(3)
    kern = libs.ref_scalar()
    N = 1000
    x = rng.standard_normal(N).astype(np.float32); w = rng.uniform(0.9, 1.1, N).astype(np.float32)
    a = np.empty(N, np.float32); r = np.empty(N, np.float32)
    libs.oracle.ibo_rmsnorm(a, x, w, 1e-5, N); kern.rmsnorm(p(r), p(x), p(w), 1e-5, N)
    assert np.array_equal(a, r)
    g = rng.standard_normal(N).astype(np.float32) * 3; u = rng.standard_normal(N).astype(np.float32)
    libs.oracle.ibo_silu_mul(a, g, u, N); kern.silu_mul(p(r), p(g), p(u), N)
    assert np.array_equal(a, r)
    a = x.copy(); r = x.copy()
    libs.oracle.ibo_softmax(a, N); kern.softmax(p(r), N)
    assert np.array_equal(a, r)
    for pos in (0, 1, 512, 4000):
        q1 = rng.standard_normal(128).astype(np.float32); k1 = rng.standard_normal(128).astype(np.float32)
        q2, k2 = q1.copy(), k1.copy()
        libs.oracle.ibo_rope(q1, p(k1), 128, pos, 10000.0); kern.rope(p(q2), p(k2), 128, pos, 10000.0)
        assert np.array_equal(q1, q2) and np.array_equal(k1, k2)
