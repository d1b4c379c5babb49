"""Writes tests/golden/ref_vectors.npz: outputs of the UNMODIFIED reference library
(oracle/_ref/libinferbit_ref.so, built from the reference checkout by oracle/Makefile) on small
seeded inputs shaped like the benchmark configurations. The reference's own tests hold no golden
vectors for this path, so these recorded outputs are what pins the CPU restatement and the GPU
kernels on machines that do not have the reference checkout.

    python tests/golden/make_golden.py        (needs oracle/_ref; run `make -C oracle ref` first)
"""
import ctypes as C
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from tests import _cpu                      # noqa: E402
from tests._cpu import p                    # noqa: E402


def main():
    libs = _cpu.load()
    assert libs.ref is not None, "oracle/_ref/libinferbit_ref.so missing: make -C oracle ref"
    kern = libs.ref_scalar()
    rng = np.random.default_rng(20240607)
    out = {}
    # INT4 / INT8 matvec, scalar table (the reference of record)
    M, N, B = 96, 512, 3
    w4, s4, x = _cpu.make_int4_case(rng, M, N, B)
    w8, s8, _ = _cpu.make_int8_case(rng, M, N, B)
    f4 = np.array([libs.ref.ib_fp16_to_fp32(int(v)) for v in s4], np.float32)
    f8 = np.array([libs.ref.ib_fp16_to_fp32(int(v)) for v in s8], np.float32)
    y4 = np.empty((B, M), np.float32); y8 = np.empty((B, M), np.float32)
    for b in range(B):
        kern.matmul_int4(p(y4[b]), p(w4), p(f4), p(x[b]), M, N)
        kern.matmul_int8(p(y8[b]), p(w8), p(f8), p(x[b]), M, N)
    y8b = np.empty((B, M), np.float32)
    kern.matmul_int8_batch(p(y8b), p(w8), p(f8), p(x), M, N, B, M)
    out.update(lin_w4=w4, lin_s4=s4, lin_w8=w8, lin_s8=s8, lin_x=x, lin_y4=y4, lin_y8=y8, lin_y8b=y8b)
    # W4A8
    g = N // 128
    q = np.empty((B, N), np.int8); sa = np.empty((B, g), np.float32)
    for b in range(B):
        libs.ref.ib_quantize_input_int8_g128(x[b], q[b], sa[b], N)
    yw = np.empty((B, M), np.float32)
    kern.matmul_w4a8_batch(p(yw), p(w4), p(f4), p(q), p(sa), M, N, B, M)
    out.update(w4a8_q=q, w4a8_sa=sa, w4a8_y=yw)
    # PQ
    Mp, Np, G, K = 80, 512, 16, 256
    cb_l, cb_r, il, ir, rs, xp = _cpu.make_pq_case(rng, Mp, Np, G, K, 2)
    xp[1, 2 * G:4 * G] *= 1e-4                                   # two chunks under the 1 % rule
    t = libs.ref_pq_tensor(Mp, Np, G, K, cb_l, cb_r, il, ir, rs)
    yp = np.empty((2, Mp), np.float32)
    for b in range(2):
        assert libs.ref.ib_pq_matmul_fp32(C.byref(t), xp[b], yp[b]) == 0
    out.update(pq_cb_l=cb_l, pq_cb_r=cb_r, pq_il=il, pq_ir=ir, pq_rs=rs, pq_x=xp, pq_y=yp, pq_shape=np.array([Mp, Np, G, K]))
    # k-means assignment, including near ties
    for D, Kc in ((8, 256), (2, 16), (5, 32)):
        X = (rng.standard_normal((20000, D)) * 0.02).astype(np.float32)
        Cn = X[:Kc].copy()
        mid = ((Cn[0].astype(np.float64) + Cn[1]) / 2)
        X[1000:3000] = (mid + rng.standard_normal((2000, D)) * 1e-4).astype(np.float32)
        idx = np.empty(len(X), np.int32)
        assert libs.ref.ib_kmeans_assign(X, len(X), D, Cn, Kc, idx, None) == 0
        out[f"km{D}_X"] = X; out[f"km{D}_C"] = Cn; out[f"km{D}_idx"] = idx
    np.savez_compressed(os.path.join(ROOT, "tests", "golden", "ref_vectors.npz"), **out)
    print("wrote", len(out), "arrays")
    decode_golden(libs)


def decode_golden(libs):
    """tests/golden/decode_ref_logits.npz: logits of the reference's own inferbit_load + inferbit_forward on
    the seeded mini model of ibf_model.py, fed one token per call from an empty KV cache (one thread,
    the machine's SIMD table as ibf_load installs it, IB_W4A8=0 so that INT4 layers take the FP32-activation
    kernel this build's decode step uses)."""
    import tempfile
    from tests.golden import ibf_model
    os.environ["IB_W4A8"] = "0"
    r = libs.ref
    r.inferbit_config_create.restype = C.c_void_p
    r.inferbit_config_set_threads.argtypes = [C.c_void_p, C.c_int]
    r.inferbit_config_free.argtypes = [C.c_void_p]
    r.inferbit_load.restype = C.c_void_p; r.inferbit_load.argtypes = [C.c_char_p, C.c_void_p]
    r.inferbit_free.argtypes = [C.c_void_p]
    r.inferbit_forward.restype = C.c_int
    r.inferbit_forward.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int]
    r.inferbit_last_error.restype = C.c_char_p
    r.inferbit_kv_length.restype = C.c_int; r.inferbit_kv_length.argtypes = [C.c_void_p]
    V = ibf_model.CFG["vocab"]
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "mini.ibf")
        ibf_model.write_ibf(path)
        cfg = r.inferbit_config_create()
        r.inferbit_config_set_threads(cfg, 1)
        m = r.inferbit_load(path.encode(), cfg)
        assert m, r.inferbit_last_error()
        toks = np.random.default_rng(5).integers(0, V, 8).astype(np.int32)
        logits = np.empty((len(toks), V), np.float32)
        for i in range(len(toks)):
            rc = r.inferbit_forward(m, p(toks[i:i + 1]), 1, p(logits[i]), V)
            assert rc == 0, r.inferbit_last_error()
        assert r.inferbit_kv_length(m) == len(toks)
        r.inferbit_free(m)
        r.inferbit_config_free(cfg)
    assert np.isfinite(logits).all() and float(np.abs(logits).max()) > 1e-2
    np.savez_compressed(os.path.join(ROOT, "tests", "golden", "decode_ref_logits.npz"), tokens=toks, logits=logits,
                        seed=np.array([ibf_model.SEED]))
    print("wrote decode golden: logits", logits.shape, "max |logit|", float(np.abs(logits).max()))


if __name__ == "__main__":
    main()
