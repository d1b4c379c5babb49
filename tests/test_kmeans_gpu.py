"""GPU parity of the k-means assign / accumulate / update kernels against the CPU restatement of
src/pq_kmeans.c, through the C ABI. Codes must be bit-identical."""
import ctypes as C

import os

import numpy as np
import pytest

from tests import _cpu

pytestmark = pytest.mark.gpu


def oracle_assign(libs, X, Cn):
    idx = np.empty(len(X), np.int32); dist = np.empty(len(X), np.float32)
    libs.oracle.ibo_kmeans_assign(X, len(X), X.shape[1], Cn, len(Cn), idx, dist.ctypes.data, 2)
    return idx, dist


@pytest.mark.parametrize("N,D,K", [(100000, 8, 256), (5000, 2, 16), (3333, 5, 100), (4097, 16, 64), (1000, 32, 7),
                                   (700, 3, 1000), (64, 8, 1), (1, 8, 256)])
def test_assign_codes_bit_exact(backend, cpu_libs, N, D, K):
    rng = np.random.default_rng(N + D + K)
    X = (rng.standard_normal((N, D)) * 0.02).astype(np.float32)
    Cn = (rng.standard_normal((K, D)) * 0.02).astype(np.float32)
    m = min(N, K); Cn[:m] = X[:m]
    got, gd = backend.kmeans_assign(X, Cn, want_dist=True)
    want, wd = oracle_assign(cpu_libs, X, Cn)
    assert np.array_equal(got, want)
    assert np.array_equal(gd, wd)                               # same roundings, same distance bits


@pytest.mark.parametrize("D", [2, 4, 5, 8, 12])
def test_assign_near_ties_and_exact_ties(backend, cpu_libs, D):
    """Points on the bisector of two centroids decide on the last bit; duplicated centroids are exact
    ties that the lowest index must win; NaN rows fall to centroid 0."""
    rng = np.random.default_rng(40 + D)
    K = 8
    Cn = (rng.standard_normal((K, D)) * 0.02).astype(np.float32)
    Cn[5] = Cn[2]                                               # exact duplicate
    mid = (Cn[0].astype(np.float64) + Cn[1]) / 2
    d = Cn[1].astype(np.float64) - Cn[0]; d /= np.linalg.norm(d)
    noise = rng.standard_normal((50000, D)) * 0.002
    noise -= (noise @ d)[:, None] * d
    X = (mid + noise).astype(np.float32)
    X[10] = Cn[2]; X[11] = np.nan
    got = backend.kmeans_assign(X, Cn)
    want, _ = oracle_assign(cpu_libs, X, Cn)
    assert np.array_equal(got, want)
    assert got[10] == 2 and got[11] == 0
    assert 0 < int((got == 0).sum()) < len(X)


def _lloyd_gpu(be, X, C0, iters, teacher=None):
    N, D = X.shape; K = len(C0)
    dX = be.upload(X); dC = be.upload(C0)
    di, dd = be.alloc(N * 4), be.alloc(N * 4)
    ds, dc, dn = be.alloc(K * D * 4), be.alloc(K * 4), be.alloc(8)
    hist = []
    for it in range(iters):
        if teacher is not None:
            be.write(dC, teacher[it])
        be._check(be.lib.ibcu_kmeans_lloyd_iter(be.ctx, dX.ptr, N, D, dC.ptr, K, di.ptr, dd.ptr, ds.ptr, dc.ptr, dn.ptr))
        be.sync()
        hist.append(dict(idx=be.download(di, np.int32, N), sums=be.download(ds, np.float32, K * D).reshape(K, D),
                         counts=be.download(dc, np.int32, K), inertia=float(be.download(dn, np.float64, 1)[0]),
                         C=be.download(dC, np.float32, K * D).reshape(K, D)))
    return hist


def _lloyd_cpu(libs, X, C0, iters):
    N, D = X.shape; K = len(C0)
    Cn = C0.copy(); hist = []
    for it in range(iters):
        before = Cn.copy()
        idx = np.empty(N, np.int32); sums = np.empty((K, D), np.float32); counts = np.empty(K, np.int32)
        inertia = C.c_double()
        libs.oracle.ibo_kmeans_lloyd_iter(X, N, D, Cn, K, idx, sums, counts, C.byref(inertia), 2)
        hist.append(dict(idx=idx, sums=sums, counts=counts, inertia=inertia.value, C=Cn.copy(), C_in=before))
    return hist


def test_lloyd_teacher_forced_and_free_running(backend, cpu_libs):
    """10 Lloyd iterations from C0 = X[:K]. Teacher-forced (the CPU's centroids fed in each iteration):
    codes and counts bit-exact, sums / centroids / inertia within float tolerance. Free-running: the
    trajectory may drift by summation order; the mismatch count is reported and bounded loosely."""
    rng = np.random.default_rng(77)
    N, D, K, iters = 200000, 8, 256, 10
    X = (rng.standard_normal((N, D)) * 0.02).astype(np.float32)
    C0 = X[:K].copy()
    cpu = _lloyd_cpu(cpu_libs, X, C0, iters)
    forced = _lloyd_gpu(backend, X, C0, iters, teacher=[h["C_in"] for h in cpu])
    for it, (g, c) in enumerate(zip(forced, cpu)):
        assert np.array_equal(g["idx"], c["idx"]), it
        assert np.array_equal(g["counts"], c["counts"]), it
        assert np.allclose(g["sums"], c["sums"], rtol=1e-4, atol=1e-5), it
        assert np.allclose(g["C"], c["C"], rtol=1e-4, atol=1e-6), it
        assert abs(g["inertia"] - c["inertia"]) <= 1e-6 * c["inertia"], it
    free = _lloyd_gpu(backend, X, C0, iters)
    mism = int((free[-1]["idx"] != cpu[-1]["idx"]).sum())
    print(f"free-running: {mism} of {N} codes differ after {iters} iterations; "
          f"max centroid diff {np.max(np.abs(free[-1]['C'] - cpu[-1]['C'])):.3e}")
    assert mism <= N // 100
    assert abs(free[-1]["inertia"] - cpu[-1]["inertia"]) <= 1e-4 * cpu[-1]["inertia"]
    # determinism: the same run again gives the same bits
    again = _lloyd_gpu(backend, X, C0, iters)
    assert np.array_equal(again[-1]["C"], free[-1]["C"]) and np.array_equal(again[-1]["idx"], free[-1]["idx"])


def test_empty_cluster_keeps_its_centroid(backend, cpu_libs):
    rng = np.random.default_rng(5)
    X = (rng.standard_normal((5000, 4)) * 0.02).astype(np.float32)
    C0 = X[:16].copy(); C0[7] = 100.0                            # nobody is near centroid 7
    g = _lloyd_gpu(backend, X, C0, 1)[0]
    c = _lloyd_cpu(cpu_libs, X, C0, 1)[0]
    assert g["counts"][7] == 0 and np.array_equal(g["C"][7], C0[7])
    assert np.array_equal(g["idx"], c["idx"]) and np.array_equal(g["counts"], c["counts"])
    assert np.allclose(g["C"], c["C"], rtol=1e-4, atol=1e-6)


def test_update_rounding_matches(backend, cpu_libs):
    """Given the same sums and counts the centroid move is bit-identical (reciprocal then multiply)."""
    rng = np.random.default_rng(6)
    K, D = 256, 8
    sums = rng.standard_normal((K, D)).astype(np.float32); counts = rng.integers(0, 50, K).astype(np.int32)
    C0 = rng.standard_normal((K, D)).astype(np.float32)
    want = C0.copy(); shift = cpu_libs.oracle.ibo_kmeans_update(want, K, D, sums, counts)
    be = backend
    dC, ds, dc, dsh = be.upload(C0), be.upload(sums), be.upload(counts), be.alloc(4)
    be._check(be.lib.ibcu_kmeans_update(be.ctx, dC.ptr, K, D, ds.ptr, dc.ptr, dsh.ptr)); be.sync()
    assert np.array_equal(be.download(dC, np.float32, K * D).reshape(K, D), want)
    assert abs(float(be.download(dsh, np.float32, 1)[0]) - shift) <= 1e-4 * shift


def test_full_size_properties(backend):
    """Benchmark-size properties (4 Mi points): every code is a valid index, assigning twice is idempotent,
    counts sum to N, and a point equal to a centroid gets that centroid (or an equal-valued earlier one)."""
    rng = np.random.default_rng(1234)
    N, D, K = 1 << 22, 8, 256
    X = (rng.standard_normal((N, D)) * 0.02).astype(np.float32)
    C0 = X[:K].copy()
    h = _lloyd_gpu(backend, X, C0, 1)[0]
    assert h["idx"].min() >= 0 and h["idx"].max() < K
    assert int(h["counts"].sum()) == N and np.array_equal(np.bincount(h["idx"], minlength=K), h["counts"])
    assert np.array_equal(h["idx"][:K], np.arange(K))
    # sums against a float64 bincount
    for d in range(0, D, 3):
        ref = np.bincount(h["idx"], weights=X[:, d].astype(np.float64), minlength=K)
        assert np.allclose(h["sums"][:, d], ref, rtol=1e-4, atol=1e-5)


def test_full_size_codes_against_the_reference(backend, cpu_libs):
    """The benchmark configuration itself: 4 Mi points x 8, K = 256, centroids = the first 256 points, then
    one more assignment with the centroids of one CPU update (teacher-forced): codes bit-equal to the
    unmodified reference's ib_kmeans_assign run on its own thread pool (src/pq_kmeans.c:399-413), or to
    the restatement where the reference library did not travel."""
    rng = np.random.default_rng(1234)
    N, D, K = 1 << 22, 8, 256
    X = (rng.standard_normal((N, D)) * 0.02).astype(np.float32)
    Cn = X[:K].copy()
    want = np.empty(N, np.int32)
    pool = None
    if cpu_libs.ref is not None:
        pool = cpu_libs.ref.ib_pool_create(min(32, os.cpu_count() or 1))
    for step in range(2):
        if cpu_libs.ref is not None:
            assert cpu_libs.ref.ib_kmeans_assign(X, N, D, Cn, K, want, pool) == 0
        else:
            cpu_libs.oracle.ibo_kmeans_assign(X, N, D, Cn, K, want, None, 2)
        got = backend.kmeans_assign(X, Cn)
        bad = np.flatnonzero(got != want)
        assert bad.size == 0, (step, bad[:10], got[bad[:10]], want[bad[:10]])
        # centroids of the next iteration from the reference's own codes (float64 means rounded to FP32: any
        # centroid set will do for a teacher-forced check)
        cnt = np.bincount(want, minlength=K)
        for d in range(D):
            s = np.bincount(want, weights=X[:, d].astype(np.float64), minlength=K)
            Cn[:, d] = np.where(cnt > 0, s / np.maximum(cnt, 1), Cn[:, d]).astype(np.float32)
    if pool:
        cpu_libs.ref.ib_pool_destroy(pool)
