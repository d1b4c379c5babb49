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


# ── the decode step against the reference's own inferbit_load + inferbit_forward ──────────
DG = np.load(os.path.join(os.path.dirname(__file__), "golden", "decode_ref_logits.npz"))


def _mini_model():
    from tests.golden import ibf_model
    return ibf_model.CFG, ibf_model.tensors(int(DG["seed"][0]))


def _close_logits(got, want):
    scale = float(np.abs(want).max())
    return _cpu.close(got, want, 2e-3, 2e-4 * max(1.0, scale))


def test_decode_restatement_reproduces_reference_forward(cpu_libs):
    """ibo_decode_step, one token per call from an empty cache, against the logits the unmodified reference
    produced for the same IBF-v1 model file (tests/golden/ibf_model.py writes it; recorded by make_golden.py).
    This pins the restatement of forward_single_ex that the GPU decode tests compare with."""
    import ctypes as C
    cfg, (layers, head, (emb, es, fn)) = _mini_model()
    kv = cfg["n_kv_heads"] * cfg["head_dim"]
    om = _cpu.IboModel(); ol = (_cpu.IboLayer * cfg["n_layers"])()
    for f in ("hidden", "inter", "n_layers", "n_heads", "n_kv_heads", "head_dim", "vocab", "max_ctx", "eps", "theta"):
        setattr(om, f, cfg[f])
    keep = []
    for l, (lins, norms) in enumerate(layers):
        for i, (w, s, M, N, bits) in enumerate(lins):
            setattr(ol[l], ("q", "k", "v", "o", "gate", "up", "down")[i], _cpu.IboLinear(w.ctypes.data, s.ctypes.data, M, N, bits))
        kc = np.zeros((cfg["max_ctx"], kv), np.float32); vc = np.zeros((cfg["max_ctx"], kv), np.float32)
        keep.append((kc, vc))
        ol[l].input_norm, ol[l].post_attn_norm = norms[0].ctypes.data, norms[1].ctypes.data
        ol[l].k_cache, ol[l].v_cache = kc.ctypes.data, vc.ctypes.data
    om.embed, om.embed_scale, om.final_norm = emb.ctypes.data, es.ctypes.data, fn.ctypes.data
    om.head = _cpu.IboLinear(head[0].ctypes.data, head[1].ctypes.data, cfg["vocab"], cfg["hidden"], 8)
    om.layers = ol
    toks, want = DG["tokens"], DG["logits"]
    got = np.empty(cfg["vocab"], np.float32)
    for i in range(len(toks)):
        assert cpu_libs.oracle.ibo_decode_step(C.byref(om), toks[i:i + 1].copy(), i, 1, _cpu.p(got), None) == 0
        assert _close_logits(got, want[i]), (i, float(np.max(np.abs(got - want[i]))))


@pytest.mark.gpu
def test_gpu_decode_reproduces_reference_forward():
    """The device decode step (ib_b200_model_*: graph of linears, fused attention, SiLU) on the same model:
    eight single-token steps from an empty cache, then the last three positions again as one batch of 3."""
    import ctypes as C
    from libinferbit_b200 import _ffi
    host = _ffi.load_host()
    assert host.ib_b200_init(0) == 0, host.ib_b200_last_error()
    try:
        cfg, (layers, head, (emb, es, fn)) = _mini_model()
        mc = _ffi.ModelCfg(cfg["hidden"], cfg["inter"], cfg["n_layers"], cfg["n_heads"], cfg["n_kv_heads"], cfg["head_dim"], cfg["vocab"],
                           cfg["max_ctx"], cfg["eps"], cfg["theta"], cfg["attn_bits"], cfg["mlp_bits"], cfg["head_bits"])
        m = host.ib_b200_model_create(host.ib_b200_ctx(), C.byref(mc))
        assert m
        p = _cpu.p
        for l, (lins, norms) in enumerate(layers):
            for i, (w, s, M, N, bits) in enumerate(lins):
                assert host.ib_b200_model_set_linear(m, l, i, p(w), p(s)) == 0
            assert host.ib_b200_model_set_norms(m, l, p(norms[0]), p(norms[1])) == 0
        assert host.ib_b200_model_set_linear(m, 0, 7, p(head[0]), p(head[1])) == 0
        assert host.ib_b200_model_set_embedding(m, p(emb), p(es), p(fn)) == 0
        toks, want = DG["tokens"], DG["logits"]
        got = np.empty(cfg["vocab"], np.float32)
        for i in range(len(toks)):
            assert host.ib_b200_forward_step(m, p(toks[i:i + 1].copy()), i, 1, p(got)) == 0, host.ib_b200_last_error()
            assert _close_logits(got, want[i]), (i, float(np.max(np.abs(got - want[i]))))
        n = len(toks)
        gb = np.empty((3, cfg["vocab"]), np.float32)
        assert host.ib_b200_forward_step(m, p(toks[n - 3:].copy()), n - 3, 3, p(gb)) == 0, host.ib_b200_last_error()
        assert _close_logits(gb, want[n - 3:]), float(np.max(np.abs(gb - want[n - 3:])))
        host.ib_b200_model_free(m)
    finally:
        host.ib_b200_shutdown()
