"""GPU parity of the decode-step element-wise kernels against the restated scalar kernels
(src/kernels/scalar.c:126-181) and helpers of src/forward.c. libm-based, so float tolerance."""
import ctypes as C

import numpy as np
import pytest

from tests import _cpu

pytestmark = pytest.mark.gpu
RTOL, ATOL = 1e-3, 1e-4


def test_rmsnorm_silu_softmax_add_embed(backend, cpu_libs):
    rng = np.random.default_rng(2)
    be, o = backend, cpu_libs.oracle
    B, N = 3, 4096
    x = rng.standard_normal((B, N)).astype(np.float32) * 3
    w16 = _cpu.fp16_bits(rng.uniform(0.9, 1.1, N)); w = np.empty(N, np.float32); o.ibo_fp16_array_to_fp32(w16, w, N)
    dx, dw, do = be.upload(x), be.upload(w16), be.alloc(B * N * 4)
    be._check(be.lib.ibcu_rmsnorm_fp16w(be.ctx, do.ptr, dx.ptr, dw.ptr, 1e-5, N, B)); be.sync()
    got = be.download(do, np.float32, B * N).reshape(B, N)
    want = np.empty_like(x)
    for b in range(B):
        o.ibo_rmsnorm(want[b], x[b], w, 1e-5, N)
    assert _cpu.close(got, want, RTOL, ATOL)

    g = rng.standard_normal(B * N).astype(np.float32) * 4; u = rng.standard_normal(B * N).astype(np.float32)
    dg, du = be.upload(g), be.upload(u)
    be._check(be.lib.ibcu_silu_mul(be.ctx, dg.ptr, dg.ptr, du.ptr, B * N)); be.sync()
    want = np.empty_like(g); o.ibo_silu_mul(want, g, u, B * N)
    assert _cpu.close(be.download(dg, np.float32, B * N), want, RTOL, ATOL)

    be._check(be.lib.ibcu_add_inplace(be.ctx, du.ptr, dx.ptr, B * N)); be.sync()
    assert np.array_equal(be.download(du, np.float32, B * N), u + x.reshape(-1))

    s = rng.standard_normal((5, 513)).astype(np.float32) * 5
    ds = be.upload(s)
    be._check(be.lib.ibcu_softmax(be.ctx, ds.ptr, 513, 5)); be.sync()
    want = s.copy()
    for r in range(5):
        o.ibo_softmax(want[r], 513)
    assert _cpu.close(be.download(ds, np.float32, 5 * 513).reshape(5, 513), want, RTOL, 1e-6)

    V, H = 50, 256
    emb = rng.integers(-127, 128, (V, H), dtype=np.int8); es = _cpu.fp16_bits(rng.uniform(0.001, 0.01, V))
    toks = np.array([3, 49, 0], np.int32)
    de, dsx, dt, dxo = be.upload(emb), be.upload(es), be.upload(toks), be.alloc(3 * H * 4)
    be._check(be.lib.ibcu_embed_int8(be.ctx, de.ptr, dsx.ptr, dt.ptr, dxo.ptr, H, 3)); be.sync()
    esf = np.empty(V, np.float32); o.ibo_fp16_array_to_fp32(es, esf, V)
    assert np.array_equal(be.download(dxo, np.float32, 3 * H).reshape(3, H), emb[toks].astype(np.float32) * esf[toks][:, None])


@pytest.mark.parametrize("fused", [False, True])
@pytest.mark.parametrize("n_heads,n_kv,hd,pos0,B", [(32, 8, 128, 512, 1), (32, 8, 128, 512, 8), (4, 4, 64, 0, 3), (8, 2, 32, 5, 2),
                                                     (32, 8, 128, 0, 1), (32, 8, 128, 127, 3), (16, 1, 64, 300, 2), (12, 12, 20, 40, 2)])
def test_rope_kv_write_and_attention(backend, cpu_libs, n_heads, n_kv, hd, pos0, B, fused):
    """fused=False: ibcu_rope_kv_write then ibcu_attention; fused=True: ibcu_attention_decode, which must
    give the same output and cache rows and leave q and k as they were."""
    rng = np.random.default_rng(n_heads + hd + pos0 + B)
    be, o = backend, cpu_libs.oracle
    kv_dim, H, ctx_len = n_kv * hd, n_heads * hd, pos0 + B
    q = rng.standard_normal((B, H)).astype(np.float32); k = rng.standard_normal((B, kv_dim)).astype(np.float32)
    v = rng.standard_normal((B, kv_dim)).astype(np.float32)
    kc = rng.standard_normal((ctx_len, kv_dim)).astype(np.float32); vc = rng.standard_normal((ctx_len, kv_dim)).astype(np.float32)
    dq, dk, dv, dkc, dvc = be.upload(q), be.upload(k), be.upload(v), be.upload(kc), be.upload(vc)
    dout = be.alloc(B * H * 4)
    if fused:
        be._check(be.lib.ibcu_attention_decode(be.ctx, dq.ptr, dk.ptr, dv.ptr, dkc.ptr, dvc.ptr, dout.ptr, n_heads, n_kv, hd, pos0, B, 10000.0))
    else:
        be._check(be.lib.ibcu_rope_kv_write(be.ctx, dq.ptr, dk.ptr, dv.ptr, dkc.ptr, dvc.ptr, n_heads, n_kv, hd, pos0, B, 10000.0))
        be._check(be.lib.ibcu_attention(be.ctx, dq.ptr, dkc.ptr, dvc.ptr, dout.ptr, n_heads, n_kv, hd, pos0, B))
    be.sync()
    # CPU: same sequence as src/forward.c:745-784
    group = n_heads // n_kv
    qr, kr = q.copy(), k.copy(); kcr, vcr = kc.copy(), vc.copy()
    want = np.empty((B, H), np.float32)
    for b in range(B):
        pos = pos0 + b
        for h in range(n_heads):
            qh = qr[b, h * hd:(h + 1) * hd]
            if h % group == 0:
                o.ibo_rope(qh, kr[b, (h // group) * hd:(h // group + 1) * hd].ctypes.data, hd, pos, 10000.0)
            else:
                o.ibo_rope(qh, None, hd, pos, 10000.0)
        kcr[pos] = kr[b]; vcr[pos] = v[b]
        for h in range(n_heads):
            kvh = h // group
            sc = (kcr[:pos + 1, kvh * hd:(kvh + 1) * hd] @ qr[b, h * hd:(h + 1) * hd]).astype(np.float32) * np.float32(1.0 / np.sqrt(np.float32(hd)))
            sc = np.ascontiguousarray(sc, np.float32); o.ibo_softmax(sc, pos + 1)
            want[b, h * hd:(h + 1) * hd] = sc @ vcr[:pos + 1, kvh * hd:(kvh + 1) * hd]
    if fused and n_heads // n_kv <= 8 and hd % 4 == 0:
        assert np.array_equal(be.download(dq, np.float32, B * H).reshape(B, H), q)
        assert np.array_equal(be.download(dk, np.float32, B * kv_dim).reshape(B, kv_dim), k)
    else:
        assert _cpu.close(be.download(dq, np.float32, B * H).reshape(B, H), qr, RTOL, ATOL)
        assert _cpu.close(be.download(dk, np.float32, B * kv_dim).reshape(B, kv_dim), kr, RTOL, ATOL)
    assert _cpu.close(be.download(dkc, np.float32, ctx_len * kv_dim).reshape(ctx_len, kv_dim), kcr, RTOL, ATOL)
    assert np.array_equal(be.download(dvc, np.float32, ctx_len * kv_dim).reshape(ctx_len, kv_dim), vcr)
    assert _cpu.close(be.download(dout, np.float32, B * H).reshape(B, H), want, RTOL, ATOL)


def test_peer_window_single_rank():
    """The peer-window calls on a one-rank context: create, bump allocation with equal alignment, window
    memory survives ibcu_free, the gather of one rank is a no-op, and a second window is refused. (The
    push over NVLink itself needs two GPUs; the multi-rank bench checks it against the NCCL gather.)"""
    from libinferbit_b200 import Backend
    be = Backend(0)
    try:
        lib = be.lib
        p = C.c_void_p()
        assert lib.ibcu_window_alloc(be.ctx, 1024, C.byref(p)) != 0 and lib.ibcu_status(be.ctx) == 0     # no window yet: plain refusal
        h = (C.c_ubyte * 64)()
        be._check(lib.ibcu_window_create(be.ctx, 1 << 20, h))
        assert any(h)
        a, b = C.c_void_p(), C.c_void_p()
        be._check(lib.ibcu_window_alloc(be.ctx, 1000, C.byref(a)))
        be._check(lib.ibcu_window_alloc(be.ctx, 4096, C.byref(b)))
        assert b.value - a.value == 1024 and a.value % 256 == 0
        x = np.arange(1024, dtype=np.float32)
        be._check(lib.ibcu_memcpy_h2d(be.ctx, b, x.ctypes.data, x.nbytes))
        be._check(lib.ibcu_free(be.ctx, b))                          # not returned to the driver: still usable
        bufs = (C.c_void_p * 1)(b.value); Ms = (C.c_int * 1)(1024)
        be._check(lib.ibcu_allgather_rows_n(be.ctx, bufs, Ms, Ms, 1, 1, 32))
        y = np.empty_like(x)
        be._check(lib.ibcu_memcpy_d2h(be.ctx, y.ctypes.data, b, x.nbytes)); be.sync()
        assert np.array_equal(x, y)
        big = C.c_void_p()
        assert lib.ibcu_window_alloc(be.ctx, 2 << 20, C.byref(big)) != 0
        assert lib.ibcu_window_create(be.ctx, 1 << 20, h) != 0
    finally:
        be.close()


def test_bounded_wait_runs_out_and_reports(backend, cpu_libs):
    """A rank whose peer never publishes: the waiting kernel gives up at its limit, the next sync reports a communication
    error, and after clearing it the context works as before (nothing hangs, nothing is lost)."""
    import time
    be = backend
    assert be.lib.ibcu_gather_wait_probe(be.ctx) == 0
    t0 = time.time()
    rc = be.lib.ibcu_sync(be.ctx)
    dt = time.time() - t0
    assert rc == -4, rc                                              # IBCU_ERR_COMM
    assert b"did not arrive within the wait limit" in be.lib.ibcu_last_error(be.ctx)
    assert dt < 30.0
    be.lib.ibcu_clear_error(be.ctx)
    rng = np.random.default_rng(0)
    w, s16, x = _cpu.make_int8_case(rng, 64, 256, 1)
    s = np.empty(64, np.float32); cpu_libs.oracle.ibo_fp16_array_to_fp32(s16, s, 64)
    want = np.empty((1, 64), np.float32); cpu_libs.oracle.ibo_matmul_int8_batch(want, w, s, x, 64, 256, 1, 64)
    assert _cpu.close(be.linear(w, s16, x, 8), want)
