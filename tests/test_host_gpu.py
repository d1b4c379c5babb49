"""The C host layer (libib_b200.so) through its reference-shaped entry points, host buffers in and
out, checked against the CPU restatement of the reference."""
import ctypes as C

import numpy as np
import pytest

from libinferbit_b200 import _ffi
from tests import _cpu
from tests._cpu import p

pytestmark = pytest.mark.gpu
RTOL, ATOL = 1e-3, 1e-4


@pytest.fixture(scope="module")
def host():
    lib = _ffi.load_host()
    assert lib.ib_b200_init(0) == 0, lib.ib_b200_last_error()
    yield lib
    lib.ib_b200_shutdown()


def test_dispatch_table_matmuls(host, cpu_libs):
    """Install the table into a struct laid out like the reference's ib_kern and call through it."""
    rng = np.random.default_rng(1)
    table = _ffi.HostKernels()
    host.ib_b200_install_kernels(C.byref(table))
    assert not table.matmul_int2                                   # left alone
    M, N, B = 300, 1024, 4
    blob = np.empty(M * N + M * (N // 2), np.uint8)                # one "model mapping": int8 tensor then int4 tensor
    w8, s16, x = _cpu.make_int8_case(rng, M, N, B)
    w4, s16b, _ = _cpu.make_int4_case(rng, M, N, B)
    blob[:M * N] = w8.view(np.uint8).reshape(-1); blob[M * N:] = w4.reshape(-1)
    assert host.ib_b200_register(blob.ctypes.data, blob.nbytes) == 0
    s8 = np.empty(M, np.float32); cpu_libs.oracle.ibo_fp16_array_to_fp32(s16, s8, M)
    s4 = np.empty(M, np.float32); cpu_libs.oracle.ibo_fp16_array_to_fp32(s16b, s4, M)
    want = np.empty(M, np.float32); got = np.empty(M, np.float32)
    cpu_libs.oracle.ibo_matmul_int8(want, w8, s8, x[0], M, N)
    table.matmul_int8(p(got), blob.ctypes.data, p(s8), p(x[0]), M, N)
    assert host.ib_b200_status() == 0, host.ib_b200_last_error()
    assert _cpu.close(got, want, RTOL, ATOL)
    cpu_libs.oracle.ibo_matmul_int4(want, w4, s4, x[1], M, N)
    table.matmul_int4(p(got), blob.ctypes.data + M * N, p(s4), p(x[1]), M, N)
    assert _cpu.close(got, want, RTOL, ATOL)
    # a pool worker's row slice: rows [64, 164), pre-offset pointers, global M as stride (src/threading.c:373-380)
    r0, rows = 64, 100
    wantb = np.empty((B, M), np.float32); cpu_libs.oracle.ibo_matmul_int8_batch(wantb, w8, s8, x, M, N, B, M)
    gotb = np.full((B, M), -5.0, np.float32)
    table.matmul_int8_batch(gotb.ctypes.data + 4 * r0, blob.ctypes.data + r0 * N, s8.ctypes.data + 4 * r0, p(x), rows, N, B, M)
    assert _cpu.close(gotb[:, r0:r0 + rows], wantb[:, r0:r0 + rows], RTOL, ATOL)
    assert np.all(gotb[:, :r0] == -5.0) and np.all(gotb[:, r0 + rows:] == -5.0)
    # W4A8 route, bit exact
    groups = N // 128
    q = np.empty((B, N), np.int8); sa = np.empty((B, groups), np.float32); qg = np.empty(N, np.int8); sg = np.empty(groups, np.float32)
    for b in range(B):
        cpu_libs.oracle.ibo_quantize_input_int8_g128(x[b], q[b], sa[b], N)
    assert host.ib_b200_quantize_input_int8_g128(p(x[2]), p(qg), p(sg), N) == groups
    assert np.array_equal(qg, q[2]) and np.array_equal(sg, sa[2])
    cpu_libs.oracle.ibo_matmul_w4a8_batch(wantb, w4, s4, q, sa, M, N, B, M)
    table.matmul_w4a8_batch(p(gotb), blob.ctypes.data + M * N, p(s4), p(q), p(sa), M, N, B, M)
    assert np.array_equal(gotb, wantb)
    # row scales are cached on the device per tensor and re-sent only when the host vector changes
    h0, d0 = C.c_ulonglong(), C.c_ulonglong(); h1, d1 = C.c_ulonglong(), C.c_ulonglong()
    cpu_libs.oracle.ibo_matmul_int8(want, w8, s8, x[3], M, N)
    host.ib_b200_copy_stats(C.byref(h0), C.byref(d0))
    table.matmul_int8(p(got), blob.ctypes.data, p(s8), p(x[3]), M, N)
    host.ib_b200_copy_stats(C.byref(h1), C.byref(d1))
    assert _cpu.close(got, want, RTOL, ATOL)
    assert h1.value - h0.value == 4 * N and d1.value - d0.value == 4 * M      # activations only; result only
    s8b = (s8 * np.float32(0.5)).astype(np.float32)
    cpu_libs.oracle.ibo_matmul_int8(want, w8, s8b, x[3], M, N)
    table.matmul_int8(p(got), blob.ctypes.data, p(s8b), p(x[3]), M, N)
    host.ib_b200_copy_stats(C.byref(h0), C.byref(d0))
    assert _cpu.close(got, want, RTOL, ATOL)
    assert h0.value - h1.value == 4 * N + 4 * M                                  # changed scales travel again
    # weights outside every registered range: an error, outputs untouched, no CPU path
    other = w8.copy(); got[:] = 9.0
    table.matmul_int8(p(got), p(other), p(s8), p(x[0]), M, N)
    assert host.ib_b200_status() != 0 and np.all(got == 9.0)
    assert b"not inside a registered range" in host.ib_b200_last_error()
    assert host.ib_b200_unregister(blob.ctypes.data) == 0


def test_dispatch_table_elementwise(host, cpu_libs):
    rng = np.random.default_rng(2)
    table = _ffi.HostKernels(); host.ib_b200_install_kernels(C.byref(table))
    N = 4096
    x = rng.standard_normal(N).astype(np.float32); w = rng.uniform(0.9, 1.1, N).astype(np.float32)
    got = np.empty(N, np.float32); want = np.empty(N, np.float32)
    table.rmsnorm(p(got), p(x), p(w), 1e-5, N); cpu_libs.oracle.ibo_rmsnorm(want, x, w, 1e-5, N)
    assert _cpu.close(got, want, RTOL, ATOL)
    g = rng.standard_normal(N).astype(np.float32) * 3
    table.silu_mul(p(got), p(g), p(x), N); cpu_libs.oracle.ibo_silu_mul(want, g, x, N)
    assert _cpu.close(got, want, RTOL, ATOL)
    a = g.copy(); b = g.copy()
    table.softmax(p(a), N); cpu_libs.oracle.ibo_softmax(b, N)
    assert _cpu.close(a, b, RTOL, 1e-7)
    q1 = rng.standard_normal(128).astype(np.float32); k1 = rng.standard_normal(128).astype(np.float32)
    q2, k2 = q1.copy(), k1.copy()
    table.rope(p(q1), p(k1), 128, 517, 10000.0); cpu_libs.oracle.ibo_rope(q2, p(k2), 128, 517, 10000.0)
    assert _cpu.close(q1, q2, RTOL, ATOL) and _cpu.close(k1, k2, RTOL, ATOL)
    assert host.ib_b200_status() == 0, host.ib_b200_last_error()


def test_pq_entry_points(host, cpu_libs):
    rng = np.random.default_rng(3)
    M, N, G, K, B = 512, 2048, 16, 256, 3
    cb_l, cb_r, il, ir, rs, x = _cpu.make_pq_case(rng, M, N, G, K, B)
    t = _ffi.HostPqTensor()
    t.M, t.N, t.G, t.K, t.n_levels, t.C, t.l2_idx_bytes = M, N, G, K, 1, N // G, 1
    t.codebook_l1_l, t.codebook_l1_r = cb_l.ctypes.data, cb_r.ctypes.data
    t.indices_l1_l, t.indices_l1_r, t.row_scale = il.ctypes.data, ir.ctypes.data, rs.ctypes.data
    want = np.empty((B, M), np.float32)
    for b in range(B):
        cpu_libs.oracle.ibo_pq_matmul_fp32(M, N, G, K, cb_l, cb_r, 0, il, ir, rs, x[b], want[b], 1, None)
    got = np.empty(M, np.float32)
    for fn in (host.ib_b200_pq_matmul_fp32, host.ib_b200_pq_matmul_fp32_streaming):
        assert fn(C.byref(t), p(x[0]), p(got)) == 0, host.ib_b200_last_error()
        assert _cpu.close(got, want[0], RTOL, ATOL)
    assert host.ib_b200_pq_matmul_fp32_threaded(C.byref(t), p(x[1]), p(got), None) == 0
    assert _cpu.close(got, want[1], RTOL, ATOL)
    gb = np.empty((B, M), np.float32)
    assert host.ib_b200_pq_matmul_fp32_batch(C.byref(t), p(x), p(gb), B) == 0
    assert _cpu.close(gb, want, RTOL, ATOL)
    # the reference's own argument checks
    assert host.ib_b200_pq_matmul_fp32(None, p(x[0]), p(got)) == -1
    t2 = _ffi.HostPqTensor.from_buffer_copy(t); t2.n_levels = 2
    assert host.ib_b200_pq_matmul_fp32(C.byref(t2), p(x[0]), p(got)) == -1
    assert b"supported subset" in host.ib_b200_last_error()
    host.ib_b200_pq_release(C.byref(t))


def test_kmeans_entry_points(host, cpu_libs):
    rng = np.random.default_rng(4)
    N, D, K = 60000, 8, 256
    X = (rng.standard_normal((N, D)) * 0.02).astype(np.float32)
    C0 = X[:K].copy()
    got = np.empty(N, np.int32); want = np.empty(N, np.int32)
    assert host.ib_b200_kmeans_assign(p(X), N, D, p(C0), K, p(got), None) == 0, host.ib_b200_last_error()
    cpu_libs.oracle.ibo_kmeans_assign(X, N, D, C0, K, want, None, 2)
    assert np.array_equal(got, want)
    assert host.ib_b200_kmeans_assign(None, N, D, p(C0), K, p(got), None) == -1
    # three Lloyd iterations from C0 = X[:K]; the CPU loop is fed the same way
    Cg = C0.copy(); idx = np.empty(N, np.int32); inertia = C.c_double()
    assert host.ib_b200_kmeans_lloyd(p(X), N, D, K, 3, -1.0, p(Cg), p(idx), C.byref(inertia)) == 3
    Cc = C0.copy(); ic = np.empty(N, np.int32); sums = np.empty((K, D), np.float32); cnt = np.empty(K, np.int32); ine = C.c_double()
    for _ in range(3):
        cpu_libs.oracle.ibo_kmeans_lloyd_iter(X, N, D, Cc, K, ic, sums, cnt, C.byref(ine), 2)
    assert np.allclose(Cg, Cc, rtol=1e-3, atol=1e-6)
    assert int((idx != ic).sum()) <= N // 500
    assert abs(inertia.value - ine.value) <= 1e-4 * ine.value
    # with a tolerance the loop stops early like the reference's (src/pq_kmeans.c:285-288)
    Cg2 = C0.copy()
    n = host.ib_b200_kmeans_lloyd(p(X), N, D, K, 50, 1e-4, p(Cg2), None, None)
    assert 1 <= n < 50


def _tiny_model(rng, cfg):
    H, I, kv, V = cfg.hidden, cfg.inter, cfg.n_kv_heads * cfg.head_dim, cfg.vocab
    shapes = [(H, H), (kv, H), (kv, H), (H, H), (I, H), (I, H), (H, I)]
    layers = []
    for _ in range(cfg.n_layers):
        lin = []
        for i, (M, N) in enumerate(shapes):
            bits = cfg.attn_bits if i <= 3 else cfg.mlp_bits
            w, s, _ = (_cpu.make_int8_case if bits == 8 else _cpu.make_int4_case)(rng, M, N, 1)
            s = _cpu.fp16_bits(rng.uniform(0.2, 1.0, M) / (np.sqrt(N) * (73.0 if bits == 8 else 4.6)))
            lin.append((w, s, M, N, bits))
        norms = (_cpu.fp16_bits(rng.uniform(0.9, 1.1, H)), _cpu.fp16_bits(rng.uniform(0.9, 1.1, H)))
        layers.append((lin, norms))
    hw, hs, _ = _cpu.make_int8_case(rng, V, H, 1)
    hs = _cpu.fp16_bits(rng.uniform(0.2, 1.0, V) / (np.sqrt(H) * 73.0))
    emb = rng.integers(-127, 128, (V, H), dtype=np.int8); es = _cpu.fp16_bits(rng.uniform(0.005, 0.02, V))
    fn = _cpu.fp16_bits(rng.uniform(0.9, 1.1, H))
    return layers, (hw, hs), emb, es, fn


@pytest.mark.parametrize("B,pos0", [(1, 0), (1, 37), (4, 37), (8, 5)])
def test_decode_step_matches_forward_restatement(host, cpu_libs, B, pos0):
    """A 3-layer model with the benchmark's structure (GQA, INT8 attention, INT4 MLP, INT8 head, FP32 KV)
    against the restatement of forward_single_ex / forward_batch; twice, so the graph replay is covered."""
    rng = np.random.default_rng(100 + B + pos0)
    cfg = _ffi.ModelCfg(256, 512, 3, 8, 2, 32, 320, 64, 1e-5, 10000.0, 8, 4, 8)
    layers, (hw, hs), emb, es, fn = _tiny_model(rng, cfg)
    kv = cfg.n_kv_heads * cfg.head_dim
    m = host.ib_b200_model_create(host.ib_b200_ctx(), C.byref(cfg))
    assert m
    om = _cpu.IboModel(); olayers = (_cpu.IboLayer * cfg.n_layers)()
    for f in ("hidden", "inter", "n_layers", "n_heads", "n_kv_heads", "head_dim", "vocab", "max_ctx", "eps", "theta"):
        setattr(om, f, getattr(cfg, f))
    caches = []
    for l, (lin, norms) in enumerate(layers):
        for i, (w, s, M, N, bits) in enumerate(lin):
            assert host.ib_b200_model_set_linear(m, l, i, p(w), p(s)) == 0
            setattr(olayers[l], ("q", "k", "v", "o", "gate", "up", "down")[i], _cpu.IboLinear(w.ctypes.data, s.ctypes.data, M, N, bits))
        assert host.ib_b200_model_set_norms(m, l, p(norms[0]), p(norms[1])) == 0
        kc = np.zeros((cfg.max_ctx, kv), np.float32); vc = np.zeros((cfg.max_ctx, kv), np.float32)
        kc[:pos0] = rng.standard_normal((pos0, kv)); vc[:pos0] = rng.standard_normal((pos0, kv))
        assert host.ib_b200_model_set_kv(m, l, p(kc), p(vc), cfg.max_ctx) == 0
        caches.append((kc, vc))
        olayers[l].input_norm, olayers[l].post_attn_norm = norms[0].ctypes.data, norms[1].ctypes.data
        olayers[l].k_cache, olayers[l].v_cache = kc.ctypes.data, vc.ctypes.data
    assert host.ib_b200_model_set_linear(m, 0, 7, p(hw), p(hs)) == 0
    assert host.ib_b200_model_set_embedding(m, p(emb), p(es), p(fn)) == 0
    om.embed, om.embed_scale, om.final_norm = emb.ctypes.data, es.ctypes.data, fn.ctypes.data
    om.head = _cpu.IboLinear(hw.ctypes.data, hs.ctypes.data, cfg.vocab, cfg.hidden, 8)
    om.layers = olayers
    toks = rng.integers(0, cfg.vocab, B).astype(np.int32)
    want = np.empty((B, cfg.vocab), np.float32)
    assert cpu_libs.oracle.ibo_decode_step(C.byref(om), toks, pos0, B, p(want), None) == 0
    assert np.isfinite(want).all() and float(np.abs(want).max()) > 1e-3
    for rep in range(2):
        for l, (kc, vc) in enumerate(caches):                          # rewind the cache rows the step wrote
            kk = kc.copy(); vv = vc.copy(); kk[pos0:] = 0; vv[pos0:] = 0
            host.ib_b200_model_set_kv(m, l, p(kk), p(vv), cfg.max_ctx)
        got = np.empty((B, cfg.vocab), np.float32)
        assert host.ib_b200_forward_step(m, p(toks), pos0, B, p(got)) == 0
        scale = float(np.abs(want).max())
        assert _cpu.close(got, want, 2e-3, 2e-4 * max(1.0, scale)), (rep, float(np.max(np.abs(got - want))))
    gk = np.empty((cfg.max_ctx, kv), np.float32); gv = np.empty((cfg.max_ctx, kv), np.float32)
    assert host.ib_b200_model_get_kv(m, cfg.n_layers - 1, p(gk), p(gv), cfg.max_ctx) == 0
    assert _cpu.close(gk[:pos0 + B], caches[-1][0][:pos0 + B], 2e-3, 2e-4)   # the oracle wrote the same rows into kc
    # the context limit is an error (src/forward.c:857-862)
    assert host.ib_b200_forward_step(m, p(toks), cfg.max_ctx - B + 1, B, None) != 0
    host.ib_b200_model_free(m)


def _build(host, cpu_libs, rng, cfg, kv_fill):
    """a model with the benchmark's structure on the device and its twin for the CPU restatement"""
    layers, (hw, hs), emb, es, fn = _tiny_model(rng, cfg)
    kv = cfg.n_kv_heads * cfg.head_dim
    m = host.ib_b200_model_create(host.ib_b200_ctx(), C.byref(cfg))
    assert m
    om = _cpu.IboModel(); olayers = (_cpu.IboLayer * cfg.n_layers)()
    for f in ("hidden", "inter", "n_layers", "n_heads", "n_kv_heads", "head_dim", "vocab", "max_ctx", "eps", "theta"):
        setattr(om, f, getattr(cfg, f))
    caches = []
    for l, (lin, norms) in enumerate(layers):
        for i, (w, s, M, N, bits) in enumerate(lin):
            assert host.ib_b200_model_set_linear(m, l, i, p(w), p(s)) == 0
            setattr(olayers[l], ("q", "k", "v", "o", "gate", "up", "down")[i], _cpu.IboLinear(w.ctypes.data, s.ctypes.data, M, N, bits))
        assert host.ib_b200_model_set_norms(m, l, p(norms[0]), p(norms[1])) == 0
        kc = np.zeros((cfg.max_ctx, kv), np.float32); vc = np.zeros((cfg.max_ctx, kv), np.float32)
        kc[:kv_fill] = rng.standard_normal((kv_fill, kv)); vc[:kv_fill] = rng.standard_normal((kv_fill, kv))
        assert host.ib_b200_model_set_kv(m, l, p(kc), p(vc), cfg.max_ctx) == 0
        caches.append((kc, vc))
        olayers[l].input_norm, olayers[l].post_attn_norm = norms[0].ctypes.data, norms[1].ctypes.data
        olayers[l].k_cache, olayers[l].v_cache = kc.ctypes.data, vc.ctypes.data
    assert host.ib_b200_model_set_linear(m, 0, 7, p(hw), p(hs)) == 0
    assert host.ib_b200_model_set_embedding(m, p(emb), p(es), p(fn)) == 0
    om.embed, om.embed_scale, om.final_norm = emb.ctypes.data, es.ctypes.data, fn.ctypes.data
    om.head = _cpu.IboLinear(hw.ctypes.data, hs.ctypes.data, cfg.vocab, cfg.hidden, 8)
    om.layers = olayers
    om._keep = (layers, hw, hs, emb, es, fn, caches, olayers)
    return m, om


def test_one_graph_serves_every_position_and_survives_scratch_growth(host, cpu_libs):
    """Autoregressive decoding replays one captured graph per batch size (the position lives on the device),
    and a graph captured early stays valid after later calls made the context's scratch grow: single
    tokens at positions 3..5, then a batch of 8 (needs more scratch), then single tokens again, every step
    against the restatement, which runs the same sequence on its own cache."""
    rng = np.random.default_rng(77)
    cfg = _ffi.ModelCfg(256, 512, 2, 8, 2, 32, 320, 96, 1e-5, 10000.0, 8, 4, 8)
    m, om = _build(host, cpu_libs, rng, cfg, 3)
    lib = _ffi.load_ibcu()
    pos = 3
    plan = [1, 1, 1, 8, 1, 1, 16, 1]
    launches = []
    for B in plan:
        toks = rng.integers(0, cfg.vocab, B).astype(np.int32)
        want = np.empty((B, cfg.vocab), np.float32); got = np.empty((B, cfg.vocab), np.float32)
        assert cpu_libs.oracle.ibo_decode_step(C.byref(om), toks, pos, B, p(want), None) == 0
        before = lib.ibcu_launch_count(host.ib_b200_ctx())
        assert host.ib_b200_forward_step(m, p(toks), pos, B, p(got)) == 0, host.ib_b200_last_error()
        launches.append(int(lib.ibcu_launch_count(host.ib_b200_ctx()) - before))
        scale = float(np.abs(want).max())
        assert _cpu.close(got, want, 2e-3, 2e-4 * max(1.0, scale)), (B, pos, float(np.max(np.abs(got - want))))
        pos += B
    # the first call of a batch size issues the step twice (eagerly, then into the capture); a replay issues
    # only the kernel that stores the position
    assert launches[0] > 20 and launches[1] == 1 and launches[2] == 1 and launches[4] == 1 and launches[7] == 1, launches
    host.ib_b200_model_free(m)


@pytest.mark.parametrize("B", [1, 8])
def test_decode_step_at_7b_layer_shapes(host, cpu_libs, B):
    """One layer and the LM head at the Mistral-7B shapes of the decode configuration (hidden 4096, MLP 14336,
    GQA 32/8 x 128, vocabulary 32000, INT8 attention, INT4 MLP, INT8 head) at context position 512."""
    rng = np.random.default_rng(7000 + B)
    cfg = _ffi.ModelCfg(4096, 14336, 1, 32, 8, 128, 32000, 544, 1e-5, 10000.0, 8, 4, 8)
    m, om = _build(host, cpu_libs, rng, cfg, 512)
    toks = rng.integers(0, cfg.vocab, B).astype(np.int32)
    want = np.empty((B, cfg.vocab), np.float32); got = np.empty((B, cfg.vocab), np.float32)
    assert cpu_libs.oracle.ibo_decode_step(C.byref(om), toks, 512, B, p(want), None) == 0
    assert np.isfinite(want).all() and float(np.abs(want).max()) > 1e-3
    for rep in range(2):                                               # eager + capture, then a replay over the same cache rows
        assert host.ib_b200_forward_step(m, p(toks), 512, B, p(got)) == 0, host.ib_b200_last_error()
        scale = float(np.abs(want).max())
        assert _cpu.close(got, want, 2e-3, 2e-4 * max(1.0, scale)), (rep, float(np.max(np.abs(got - want))))
    host.ib_b200_model_free(m)
