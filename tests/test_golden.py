"""Recorded outputs of the unmodified reference (tests/golden/ref_vectors.npz, made by
tests/golden/make_golden.py) against the CPU restatement (always) and the CUDA kernels (gpu)."""
import os

import numpy as np
import pytest

from tests import _cpu

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "ref_vectors.npz"))


def test_restatement_reproduces_reference_vectors(cpu_libs):
    o = cpu_libs.oracle
    w4, s4, w8, s8, x = G["lin_w4"], G["lin_s4"], G["lin_w8"], G["lin_s8"], G["lin_x"]
    B, N = x.shape; M = w8.shape[0]
    f4 = np.empty(M, np.float32); f8 = np.empty(M, np.float32)
    o.ibo_fp16_array_to_fp32(s4, f4, M); o.ibo_fp16_array_to_fp32(s8, f8, M)
    y = np.empty((B, M), np.float32)
    o.ibo_matmul_int4_batch(y, w4, f4, x, M, N, B, M); assert np.array_equal(y, G["lin_y4"])
    o.ibo_matmul_int8_batch(y, w8, f8, x, M, N, B, M); assert np.array_equal(y, G["lin_y8"]) and np.array_equal(y, G["lin_y8b"])
    q = np.empty((B, N), np.int8); sa = np.empty((B, N // 128), np.float32)
    for b in range(B):
        o.ibo_quantize_input_int8_g128(x[b], q[b], sa[b], N)
    assert np.array_equal(q, G["w4a8_q"]) and np.array_equal(sa, G["w4a8_sa"])
    o.ibo_matmul_w4a8_batch(y, w4, f4, q, sa, M, N, B, M); assert np.array_equal(y, G["w4a8_y"])
    Mp, Np, Gg, K = (int(v) for v in G["pq_shape"])
    yp = np.empty(Mp, np.float32)
    for b in range(2):
        o.ibo_pq_matmul_fp32(Mp, Np, Gg, K, G["pq_cb_l"], G["pq_cb_r"], 0, G["pq_il"], G["pq_ir"], G["pq_rs"], G["pq_x"][b], yp, 1, None)
        assert _cpu.close(yp, G["pq_y"][b], 1e-5, 1e-6)
    for D in (8, 2, 5):
        X, Cn = G[f"km{D}_X"], G[f"km{D}_C"]
        idx = np.empty(len(X), np.int32)
        o.ibo_kmeans_assign(X, len(X), D, Cn, len(Cn), idx, None, 2)
        assert np.array_equal(idx, G[f"km{D}_idx"])


@pytest.mark.gpu
def test_cuda_kernels_reproduce_reference_vectors(backend):
    be = backend
    x = G["lin_x"]
    assert _cpu.close(be.linear(G["lin_w4"], G["lin_s4"], x, 4), G["lin_y4"], 1e-3, 1e-4)
    assert _cpu.close(be.linear(G["lin_w8"], G["lin_s8"], x, 8), G["lin_y8"], 1e-3, 1e-4)
    Mp, Np, Gg, K = (int(v) for v in G["pq_shape"])
    t = be.make_pq(Mp, Np, Gg, K, G["pq_cb_l"], G["pq_cb_r"], G["pq_il"], G["pq_ir"], G["pq_rs"])
    assert _cpu.close(be.pq_matmul(t, G["pq_x"]), G["pq_y"], 1e-3, 1e-4)
    for D in (8, 2, 5):
        assert np.array_equal(be.kmeans_assign(G[f"km{D}_X"], G[f"km{D}_C"]), G[f"km{D}_idx"])
