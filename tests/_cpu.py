"""Loads the CPU checkers for the tests: oracle/libib_oracle.so (this repo's restatement, built on
demand with gcc) and oracle/_ref/libinferbit_ref.so (the unmodified reference, present only where
oracle/Makefile could build it from a reference checkout)."""
import ctypes as C
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
ORACLE_SO = os.path.join(ORACLE_DIR, "libib_oracle.so")
REF_SO = os.path.join(ORACLE_DIR, "_ref", "libinferbit_ref.so")

f32 = np.ctypeslib.ndpointer(np.float32, flags="C")
i32 = np.ctypeslib.ndpointer(np.int32, flags="C")
u8 = np.ctypeslib.ndpointer(np.uint8, flags="C")
i8 = np.ctypeslib.ndpointer(np.int8, flags="C")
u16 = np.ctypeslib.ndpointer(np.uint16, flags="C")


class IboLinear(C.Structure):
    _fields_ = [("w", C.c_void_p), ("scale", C.c_void_p), ("M", C.c_int), ("N", C.c_int), ("bits", C.c_int)]


class IboLayer(C.Structure):
    _fields_ = [(n, IboLinear) for n in ("q", "k", "v", "o", "gate", "up", "down")] + [
        ("input_norm", C.c_void_p), ("post_attn_norm", C.c_void_p), ("k_cache", C.c_void_p), ("v_cache", C.c_void_p)]


class IboModel(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("hidden", "inter", "n_layers", "n_heads", "n_kv_heads", "head_dim", "vocab", "max_ctx")] + [
        ("eps", C.c_float), ("theta", C.c_float), ("embed", C.c_void_p), ("embed_scale", C.c_void_p),
        ("final_norm", C.c_void_p), ("head", IboLinear), ("layers", C.POINTER(IboLayer))]


class RefKernels(C.Structure):
    """ib_kernels (src/inferbit_internal.h:199-277), field order as declared there."""
    _mm = C.CFUNCTYPE(None, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int)
    _fields_ = [
        ("matmul_int4", _mm), ("matmul_int8", _mm), ("matmul_int2", _mm),
        ("rmsnorm", C.CFUNCTYPE(None, C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_int)),
        ("rope", C.CFUNCTYPE(None, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_float)),
        ("softmax", C.CFUNCTYPE(None, C.c_void_p, C.c_int)),
        ("silu_mul", C.CFUNCTYPE(None, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int)),
        ("matmul_w4a8", C.CFUNCTYPE(None, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int)),
        ("matmul_w4a8_batch", C.CFUNCTYPE(None, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int)),
        ("matmul_int8_batch", C.CFUNCTYPE(None, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int)),
    ]


class RefPqTensor(C.Structure):
    """ib_pq_tensor (src/pq_decode.h:39-87)."""
    _fields_ = [("M", C.c_int), ("N", C.c_int), ("G", C.c_int), ("K", C.c_int), ("K_l2", C.c_int),
                ("n_levels", C.c_int), ("rotate", C.c_int), ("n_outlier", C.c_int), ("format", C.c_int),
                ("codebook_l1_l", C.c_void_p), ("codebook_l1_r", C.c_void_p),
                ("codebook_l2_l", C.c_void_p), ("codebook_l2_r", C.c_void_p),
                ("indices_l1_l", C.c_void_p), ("indices_l1_r", C.c_void_p),
                ("indices_l2_l", C.c_void_p), ("indices_l2_r", C.c_void_p),
                ("C", C.c_int), ("l2_idx_bytes", C.c_int), ("l2_packed_bits", C.c_int),
                ("row_scale", C.c_void_p), ("outlier_cols", C.c_void_p), ("outlier_sidecar", C.c_void_p),
                ("outlier_scale", C.c_void_p), ("_arena", C.c_void_p), ("_arena_size", C.c_size_t),
                ("_mmap_base", C.c_void_p), ("_mmap_size", C.c_size_t), ("_owns_mmap", C.c_int)]


class RefPqRaw(C.Structure):
    """ib_pq_raw_tensor (src/pq_decode.h:108-116)"""
    _fields_ = [("name", C.c_char_p), ("data", C.c_void_p), ("dtype", C.c_int), ("ndim", C.c_int), ("shape", C.c_int * 4),
                ("size_bytes", C.c_size_t), ("_owns_data", C.c_int)]


class RefPqMulti(C.Structure):
    """ib_pq_multi (src/pq_decode.h:120-131)"""
    _fields_ = [("n", C.c_int), ("names", C.POINTER(C.c_char_p)), ("tensors", C.POINTER(RefPqTensor)), ("_mmap_base", C.c_void_p),
                ("_mmap_size", C.c_size_t), ("n_raw", C.c_int), ("raw_tensors", C.POINTER(RefPqRaw)), ("config_json", C.c_char_p)]


def pq_file_tensor(d, fmt):
    """the writer's description of the tensor that make_pq_case_ex made"""
    blocks = {"codebook_l1_l": d["cb1_l"], "codebook_l1_r": d["cb1_r"], "indices_l1_l": d["idx1_l"], "indices_l1_r": d["idx1_r"], "row_scale": d["rs"]}
    if d["K_l2"]:
        blocks.update({"codebook_l2_l": d["cb2_l"], "codebook_l2_r": d["cb2_r"], "indices_l2_l": d["idx2_l"], "indices_l2_r": d["idx2_r"]})
    if d["n_outlier"]:
        blocks.update({"outlier_cols": d["ocols"], "outlier_sidecar": d["oside"], "outlier_scale": d["oscale"]})
    return dict(format=fmt, M=d["M"], N=d["N"], G=d["G"], K=d["K"], n_levels=2 if d["K_l2"] else 1, K_l2=d["K_l2"],
                n_outlier=d["n_outlier"], blocks=blocks)


def pq_tensor_arrays(t):
    """every array of a loaded ib_pq_tensor (either library's), as numpy copies keyed like the file's blocks"""
    half, Cn = t.G // 2, t.C
    K2 = t.K_l2 if t.K_l2 > 0 else t.K

    def arr(ptr, dtype, n):
        return np.ctypeslib.as_array(C.cast(ptr, C.POINTER(C.c_uint8)), shape=(n * np.dtype(dtype).itemsize,)).view(dtype).copy() if ptr and n else None
    out = {"codebook_l1_l": arr(t.codebook_l1_l, np.uint16, t.K * half), "codebook_l1_r": arr(t.codebook_l1_r, np.uint16, t.K * half),
           "indices_l1_l": arr(t.indices_l1_l, np.uint8, t.M * Cn), "indices_l1_r": arr(t.indices_l1_r, np.uint8, t.M * Cn),
           "row_scale": arr(t.row_scale, np.uint16, t.M)}
    if t.n_levels == 2:
        row = (Cn + 1) // 2 if K2 == 16 else Cn * (2 if t.l2_packed_bits > 0 else t.l2_idx_bytes)
        out.update({"codebook_l2_l": arr(t.codebook_l2_l, np.uint16, K2 * half), "codebook_l2_r": arr(t.codebook_l2_r, np.uint16, K2 * half),
                    "indices_l2_l": arr(t.indices_l2_l, np.uint8, t.M * row), "indices_l2_r": arr(t.indices_l2_r, np.uint8, t.M * row)})
    if t.n_outlier > 0:
        out.update({"outlier_cols": arr(t.outlier_cols, np.int32, t.n_outlier), "outlier_sidecar": arr(t.outlier_sidecar, np.int8, t.M * t.n_outlier),
                    "outlier_scale": arr(t.outlier_scale, np.uint16, t.n_outlier)})
    return out


def build_oracle():
    subprocess.run(["make", "-s", "-C", ORACLE_DIR, "oracle"], check=True)


class Libs:
    def __init__(self):
        if not os.path.exists(ORACLE_SO) or os.path.getmtime(ORACLE_SO) < os.path.getmtime(os.path.join(ORACLE_DIR, "ib_oracle.c")):
            build_oracle()
        o = C.CDLL(ORACLE_SO)
        o.ibo_fp16_to_fp32.restype = C.c_float; o.ibo_fp16_to_fp32.argtypes = [C.c_uint16]
        o.ibo_fp32_to_fp16.restype = C.c_uint16; o.ibo_fp32_to_fp16.argtypes = [C.c_float]
        o.ibo_fp16_array_to_fp32.argtypes = [u16, f32, C.c_int]
        o.ibo_matmul_int4.argtypes = [f32, u8, f32, f32, C.c_int, C.c_int]
        o.ibo_matmul_int8.argtypes = [f32, i8, f32, f32, C.c_int, C.c_int]
        o.ibo_matmul_int8_batch.argtypes = [f32, i8, f32, f32, C.c_int, C.c_int, C.c_int, C.c_int]
        o.ibo_matmul_int4_batch.argtypes = [f32, u8, f32, f32, C.c_int, C.c_int, C.c_int, C.c_int]
        o.ibo_quantize_input_int8_g128.restype = C.c_int
        o.ibo_quantize_input_int8_g128.argtypes = [f32, i8, f32, C.c_int]
        o.ibo_matmul_w4a8_batch.argtypes = [f32, u8, f32, i8, f32, C.c_int, C.c_int, C.c_int, C.c_int]
        o.ibo_pq_matmul_fp32.restype = C.c_int
        o.ibo_pq_matmul_fp32.argtypes = [C.c_int] * 4 + [u16, u16, C.c_long, u8, u8, u16, f32, f32, C.c_int, C.POINTER(C.c_int)]
        o.ibo_pq_matmul_fp32_ex.restype = C.c_int
        o.ibo_pq_matmul_fp32_ex.argtypes = [C.c_int] * 5 + [C.c_void_p] * 9 + [C.c_int] + [C.c_void_p] * 5 + [C.c_int]
        o.ibo_int4g_matmul_fp32.restype = C.c_int
        o.ibo_int4g_matmul_fp32.argtypes = [C.c_int] * 3 + [C.c_void_p] * 2 + [C.c_int] + [C.c_void_p] * 4 + [C.c_float, C.c_int]
        o.ibo_pq_lm_head_topk.restype = C.c_int
        o.ibo_pq_lm_head_topk.argtypes = [C.c_int] * 5 + [C.c_void_p] * 9 + [C.c_int] + [C.c_void_p] * 4 + [C.c_int] + [C.c_void_p] * 3 + [C.c_int]
        o.ibo_pq_reconstruct_fp32.restype = C.c_int
        o.ibo_pq_reconstruct_fp32.argtypes = [C.c_int] * 4 + [u16, u16, u8, u8, u16, f32]
        o.ibo_kmeans_assign.argtypes = [f32, C.c_long, C.c_int, f32, C.c_int, i32, C.c_void_p, C.c_int]
        o.ibo_kmeans_lloyd_iter.restype = C.c_float
        o.ibo_kmeans_lloyd_iter.argtypes = [f32, C.c_long, C.c_int, f32, C.c_int, i32, f32, i32, C.POINTER(C.c_double), C.c_int]
        o.ibo_kmeans_update.restype = C.c_float
        o.ibo_kmeans_update.argtypes = [f32, C.c_int, C.c_int, f32, i32]
        o.ibo_rmsnorm.argtypes = [f32, f32, f32, C.c_float, C.c_int]
        o.ibo_rope.argtypes = [f32, C.c_void_p, C.c_int, C.c_int, C.c_float]
        o.ibo_softmax.argtypes = [f32, C.c_int]
        o.ibo_silu_mul.argtypes = [f32, f32, f32, C.c_int]
        o.ibo_decode_step.restype = C.c_int
        o.ibo_decode_step.argtypes = [C.POINTER(IboModel), i32, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        self.oracle = o
        self.ref = None
        self.ref_kern = None
        if os.path.exists(REF_SO):
            r = C.CDLL(REF_SO)
            r.ib_init_kernels.argtypes = [C.c_int]
            r.ib_detect_simd.restype = C.c_int
            r.ib_fp16_to_fp32.restype = C.c_float; r.ib_fp16_to_fp32.argtypes = [C.c_uint16]
            r.ib_fp32_to_fp16.restype = C.c_uint16; r.ib_fp32_to_fp16.argtypes = [C.c_float]
            r.ib_kmeans_assign.restype = C.c_int
            r.ib_kmeans_assign.argtypes = [f32, C.c_int, C.c_int, f32, C.c_int, i32, C.c_void_p]
            r.ib_pq_matmul_fp32.restype = C.c_int
            r.ib_pq_matmul_fp32.argtypes = [C.POINTER(RefPqTensor), f32, f32]
            r.ib_pq_load_single.restype = C.c_int; r.ib_pq_load_single.argtypes = [C.c_char_p, C.POINTER(RefPqTensor)]
            r.ib_pq_load_multi.restype = C.c_int; r.ib_pq_load_multi.argtypes = [C.c_char_p, C.POINTER(RefPqMulti)]
            r.ib_pq_free.argtypes = [C.POINTER(RefPqTensor)]; r.ib_pq_multi_free.argtypes = [C.POINTER(RefPqMulti)]
            r.ib_pq_lm_head_topk.restype = C.c_int
            r.ib_pq_lm_head_topk.argtypes = [C.POINTER(RefPqTensor), f32, C.c_int, f32, i32]
            r.ib_pq_matmul_fp32_threaded.restype = C.c_int
            r.ib_pq_matmul_fp32_threaded.argtypes = [C.POINTER(RefPqTensor), f32, f32, C.c_void_p]
            r.ib_pq_matmul_fp32_streaming.restype = C.c_int
            r.ib_pq_matmul_fp32_streaming.argtypes = [C.POINTER(RefPqTensor), f32, f32]
            r.ib_pq_reconstruct_fp32.restype = C.c_int
            r.ib_pq_reconstruct_fp32.argtypes = [C.POINTER(RefPqTensor), f32]
            r.ib_quantize_input_int8_g128.restype = C.c_int
            r.ib_quantize_input_int8_g128.argtypes = [f32, i8, f32, C.c_int]
            r.ib_pool_create.restype = C.c_void_p; r.ib_pool_create.argtypes = [C.c_int]
            r.ib_pool_destroy.argtypes = [C.c_void_p]
            r.ib_parallel_matmul.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int]
            r.ib_parallel_matmul_int8_batch.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int]
            self.ref = r
            self.ref_kern = RefKernels.in_dll(r, "ib_kern")

    def ref_scalar(self):
        """Install the reference's scalar table (IB_SIMD_NONE = 0): the reference of record."""
        self.ref.ib_init_kernels(0)
        return self.ref_kern

    def ref_simd(self):
        self.ref.ib_init_kernels(self.ref.ib_detect_simd())
        return self.ref_kern

    def ref_pq_tensor(self, M, N, G, K, cb_l, cb_r, idx_l, idx_r, row_scale):
        t = RefPqTensor()
        t.M, t.N, t.G, t.K, t.K_l2, t.n_levels, t.rotate, t.n_outlier, t.format = M, N, G, K, 0, 1, 0, 0, 0
        t.codebook_l1_l = cb_l.ctypes.data; t.codebook_l1_r = cb_r.ctypes.data
        t.indices_l1_l = idx_l.ctypes.data; t.indices_l1_r = idx_r.ctypes.data
        t.C = N // G; t.l2_idx_bytes = 1; t.row_scale = row_scale.ctypes.data
        t._keep = (cb_l, cb_r, idx_l, idx_r, row_scale)
        return t


def make_pq_case_ex(rng, M, N, G, K, K_l2, n_outlier, B):
    """A PQ tensor with the production extras: K_l2 > 0 adds a second residual level (4-bit packed indices when
    K_l2 == 16, else one byte), n_outlier > 0 an int8 sidecar over that many columns. N - n_outlier = C * G."""
    half = G // 2
    Cn = (N - n_outlier) // G
    assert Cn * G == N - n_outlier
    d = {"M": M, "N": N, "G": G, "K": K, "K_l2": K_l2, "n_outlier": n_outlier, "C": Cn}
    d["cb1_l"] = fp16_bits(rng.standard_normal((K, half)) * 0.02); d["cb1_r"] = fp16_bits(rng.standard_normal((K, half)) * 0.02)
    d["idx1_l"] = rng.integers(0, K, size=(M, Cn), dtype=np.uint8); d["idx1_r"] = rng.integers(0, K, size=(M, Cn), dtype=np.uint8)
    if K_l2:
        d["cb2_l"] = fp16_bits(rng.standard_normal((K_l2, half)) * 0.004); d["cb2_r"] = fp16_bits(rng.standard_normal((K_l2, half)) * 0.004)
        if K_l2 == 16:
            nb = (Cn + 1) // 2
            d["idx2_l"] = rng.integers(0, 256, size=(M, nb), dtype=np.uint8); d["idx2_r"] = rng.integers(0, 256, size=(M, nb), dtype=np.uint8)
        else:
            d["idx2_l"] = rng.integers(0, K_l2, size=(M, Cn), dtype=np.uint8); d["idx2_r"] = rng.integers(0, K_l2, size=(M, Cn), dtype=np.uint8)
    if n_outlier:
        d["ocols"] = np.sort(rng.choice(N, n_outlier, replace=False)).astype(np.int32)
        d["oside"] = rng.integers(-127, 128, size=(M, n_outlier), dtype=np.int8)
        d["oscale"] = fp16_bits(rng.uniform(0.001, 0.01, n_outlier))
    d["rs"] = fp16_bits(rng.uniform(0.5, 2.0, M))
    d["x"] = rng.standard_normal((B, N)).astype(np.float32)
    return d


def _ptr(d, k):
    return d[k].ctypes.data if k in d else None


def oracle_pq_ex(o, d, xb, fused=1):
    out = np.empty(d["M"], np.float32)
    rc = o.ibo_pq_matmul_fp32_ex(d["M"], d["N"], d["G"], d["K"], d["K_l2"], _ptr(d, "cb1_l"), _ptr(d, "cb1_r"), _ptr(d, "cb2_l"), _ptr(d, "cb2_r"),
                                 _ptr(d, "idx1_l"), _ptr(d, "idx1_r"), _ptr(d, "idx2_l"), _ptr(d, "idx2_r"), _ptr(d, "rs"),
                                 d["n_outlier"], _ptr(d, "ocols"), _ptr(d, "oside"), _ptr(d, "oscale"), xb.ctypes.data, out.ctypes.data, fused)
    assert rc == 0
    return out


def make_int4g_case(rng, M, N, G, K_out=0):
    """group-scaled INT4 rows: nibbles uniform, fp16 group scales, one activation, optional per-row outlier columns"""
    q = rng.integers(0, 256, size=(M, N // 2), dtype=np.uint8)
    s = fp16_bits(rng.uniform(0.002, 0.02, (M, N // G)))
    x = rng.standard_normal(N).astype(np.float32)
    oi = ov = None
    if K_out:
        oi = np.stack([rng.choice(N, K_out, replace=False) for _ in range(M)]).astype(np.uint16)
        ov = fp16_bits(rng.standard_normal((M, K_out)) * 0.05)
    return q, s, x, oi, ov


def oracle_int4g(o, q, s, G, x, oi=None, ov=None, eps=0.0, fused=1):
    M, N = q.shape[0], q.shape[1] * 2
    out = np.empty(M, np.float32)
    rc = o.ibo_int4g_matmul_fp32(M, N, G, q.ctypes.data, s.ctypes.data, 0 if oi is None else oi.shape[1],
                                 None if oi is None else oi.ctypes.data, None if ov is None else ov.ctypes.data,
                                 x.ctypes.data, out.ctypes.data, eps, fused)
    assert rc == 0
    return out


def oracle_pq_topk(o, d, xb, k_top, fused=1, want_coarse=False):
    """(logits, ids[, coarse]) of the restated ib_pq_lm_head_topk over the arrays of make_pq_case_ex"""
    logits = np.empty(k_top, np.float32); ids = np.empty(k_top, np.int32); coarse = np.empty(d["M"], np.float32)
    rc = o.ibo_pq_lm_head_topk(d["M"], d["N"], d["G"], d["K"], d["K_l2"], _ptr(d, "cb1_l"), _ptr(d, "cb1_r"), _ptr(d, "cb2_l"), _ptr(d, "cb2_r"),
                               _ptr(d, "idx1_l"), _ptr(d, "idx1_r"), _ptr(d, "idx2_l"), _ptr(d, "idx2_r"), _ptr(d, "rs"),
                               d["n_outlier"], _ptr(d, "ocols"), _ptr(d, "oside"), _ptr(d, "oscale"), xb.ctypes.data, k_top,
                               logits.ctypes.data, ids.ctypes.data, coarse.ctypes.data, fused)
    assert rc == 0
    return (logits, ids, coarse) if want_coarse else (logits, ids)


def ref_pq_tensor_ex(d):
    """the reference's ib_pq_tensor over the arrays of make_pq_case_ex"""
    t = RefPqTensor()
    t.M, t.N, t.G, t.K, t.K_l2 = d["M"], d["N"], d["G"], d["K"], d["K_l2"]
    t.n_levels, t.rotate, t.n_outlier, t.format = (2 if d["K_l2"] else 1), 0, d["n_outlier"], 0
    t.codebook_l1_l, t.codebook_l1_r = _ptr(d, "cb1_l"), _ptr(d, "cb1_r")
    t.codebook_l2_l, t.codebook_l2_r = _ptr(d, "cb2_l"), _ptr(d, "cb2_r")
    t.indices_l1_l, t.indices_l1_r = _ptr(d, "idx1_l"), _ptr(d, "idx1_r")
    t.indices_l2_l, t.indices_l2_r = _ptr(d, "idx2_l"), _ptr(d, "idx2_r")
    t.C, t.l2_idx_bytes, t.l2_packed_bits = d["C"], 1, 0
    t.row_scale = _ptr(d, "rs")
    t.outlier_cols, t.outlier_sidecar, t.outlier_scale = _ptr(d, "ocols"), _ptr(d, "oside"), _ptr(d, "oscale")
    t._keep = d
    return t


_libs = None


def load():
    global _libs
    if _libs is None:
        _libs = Libs()
    return _libs


def p(a):
    return a.ctypes.data_as(C.c_void_p)


# ── seeded synthetic inputs shaped like the benchmark configurations ──
def fp16_bits(x):
    return np.asarray(x, np.float32).astype(np.float16).view(np.uint16)


def make_int8_case(rng, M, N, B):
    w = rng.integers(-127, 128, size=(M, N), dtype=np.int8)
    s16 = fp16_bits(rng.uniform(0.001, 0.01, M))
    x = rng.standard_normal((B, N)).astype(np.float32)
    return w, s16, x


def make_int4_case(rng, M, N, B):
    w = rng.integers(0, 256, size=(M, N // 2), dtype=np.uint8)      # nibbles uniform in [-8, 7]
    s16 = fp16_bits(rng.uniform(0.002, 0.02, M))
    x = rng.standard_normal((B, N)).astype(np.float32)
    return w, s16, x


def make_pq_case(rng, M, N, G, K, B, scale_one=False):
    half, Cn = G // 2, N // G
    cb_l = fp16_bits(rng.standard_normal((K, half)) * 0.02)
    cb_r = fp16_bits(rng.standard_normal((K, half)) * 0.02)
    idx_l = rng.integers(0, K, size=(M, Cn), dtype=np.uint8)
    idx_r = rng.integers(0, K, size=(M, Cn), dtype=np.uint8)
    rs = fp16_bits(np.ones(M) if scale_one else rng.uniform(0.5, 2.0, M))
    x = rng.standard_normal((B, N)).astype(np.float32)
    return cb_l, cb_r, idx_l, idx_r, rs, x


def close(a, b, rtol=1e-3, atol=1e-4):
    """The float parity bar: |a - b| <= atol + rtol * |b| element-wise."""
    a = np.asarray(a, np.float64); b = np.asarray(b, np.float64)
    return bool(np.all(np.abs(a - b) <= atol + rtol * np.abs(b)))
