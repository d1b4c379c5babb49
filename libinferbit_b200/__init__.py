"""libinferbit_b200 — B200 (sm_100a) implementation of libinferbit's quantized-weight product hot path.

The product is two shared libraries built in this directory:

  libibcu.so     CUDA backend, C ABI in include/ibcu.h
  libib_b200.so  C host layer that mirrors the reference's own interfaces for this path
                 (ib_kernels-shaped dispatch table, ib_pq_matmul_fp32, ib_kmeans_assign,
                 a forward step), C ABI in include/ib_b200.h

This Python package is only a thin ctypes convenience layer over those ABIs for tests and
benchmarks: numpy arrays in, numpy arrays out, device buffers as integers. It contains no compute
and no fallback; without the built libraries (or without a GPU) every call raises.
"""
import ctypes as C

import numpy as np

from . import _ffi
from ._ffi import LinearT, PqT

__all__ = ["Backend", "IbcuError", "LinearT", "PqT"]


class IbcuError(RuntimeError):
    pass


class DeviceBuffer:
    """A cudaMalloc'd range owned by a Backend."""

    def __init__(self, be, nbytes):
        self.be = be
        self.nbytes = int(nbytes)
        p = C.c_void_p()
        be._check(be.lib.ibcu_malloc(be.ctx, self.nbytes, C.byref(p)))
        self.ptr = p.value

    def free(self):
        if self.ptr:
            self.be.lib.ibcu_free(self.be.ctx, self.ptr)
            self.ptr = None

    def at(self, byte_offset):
        return self.ptr + int(byte_offset)


class Backend:
    """One GPU context (ibcu_ctx)."""

    def __init__(self, device=0):
        self.lib = _ffi.load_ibcu()
        ctx = C.c_void_p()
        rc = self.lib.ibcu_ctx_create(int(device), C.byref(ctx))
        if rc != 0:
            raise IbcuError(f"ibcu_ctx_create(device={device}) failed with {rc}: no usable sm_100 GPU; "
                            "this library has no CPU fallback")
        self.ctx = ctx
        self.device = device
        self._bufs = []

    # ── plumbing ──
    def _check(self, rc):
        if rc != 0:
            msg = self.lib.ibcu_last_error(self.ctx).decode()
            self.lib.ibcu_clear_error(self.ctx)
            raise IbcuError(f"ibcu error {rc}: {msg}")

    def close(self):
        if self.ctx:
            for b in self._bufs:
                b.free()
            self._bufs = []
            self.lib.ibcu_ctx_destroy(self.ctx)
            self.ctx = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def alloc(self, nbytes):
        b = DeviceBuffer(self, max(int(nbytes), 16))
        self._bufs.append(b)
        return b

    def upload(self, arr):
        arr = np.ascontiguousarray(arr)
        b = self.alloc(arr.nbytes)
        if arr.nbytes:
            self._check(self.lib.ibcu_memcpy_h2d(self.ctx, b.ptr, arr.ctypes.data, arr.nbytes))
            self.sync()
        return b

    def write(self, buf, arr, byte_offset=0):
        arr = np.ascontiguousarray(arr)
        self._check(self.lib.ibcu_memcpy_h2d(self.ctx, buf.at(byte_offset), arr.ctypes.data, arr.nbytes))
        self.sync()

    def download(self, buf, dtype, count, byte_offset=0):
        out = np.empty(int(count), dtype=dtype)
        if out.nbytes:
            self._check(self.lib.ibcu_memcpy_d2h(self.ctx, out.ctypes.data, buf.at(byte_offset) if isinstance(buf, DeviceBuffer) else buf + byte_offset, out.nbytes))
            self.sync()
        return out

    def sync(self):
        self._check(self.lib.ibcu_sync(self.ctx))

    def launches(self):
        return int(self.lib.ibcu_launch_count(self.ctx))

    # ── hot path, numpy convenience (device round trip per call; for tests) ──
    def linear(self, w, scales, x, bits, epilogue=0, out_init=None, force_generic=False):
        """w: int8 [M,N] or uint8 [M,N/2]; scales: uint16 fp16 bits [M] or float32 [M]; x: float32 [B,N]."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        if x.ndim == 1:
            x = x[None, :]
        B, N = x.shape
        M = w.shape[0]
        dw, ds, dx = self.upload(w), self.upload(scales), self.upload(x)
        init = np.zeros((B, M), np.float32) if out_init is None else np.ascontiguousarray(out_init, np.float32)
        do = self.upload(init)
        t = LinearT(dw.ptr, ds.ptr, do.ptr, M, M, 1 if scales.dtype == np.float32 else 0, epilogue)
        self.lib.ibcu_linear_force_generic(self.ctx, 1 if force_generic else 0)
        try:
            self._check(self.lib.ibcu_linear(self.ctx, C.byref(t), 1, dx.ptr, N, B, bits))
            self.sync()
        finally:
            self.lib.ibcu_linear_force_generic(self.ctx, 0)
        out = self.download(do, np.float32, B * M).reshape(B, M)
        for b in (dw, ds, dx, do):
            b.free(); self._bufs.remove(b)
        return out

    def make_pq(self, M, N, G, K, cb_l, cb_r, idx_l, idx_r, row_scale, cb_chunk_stride=0):
        """Upload a PQ tensor (arrays in the reference's layout) and build the subspace-major code plane."""
        t = PqT()
        t.M, t.N, t.G, t.K = M, N, G, K
        bufs = [self.upload(a) for a in (cb_l, cb_r, idx_l, idx_r, row_scale)]
        t.codebook_l, t.codebook_r, t.idx_l, t.idx_r, t.row_scale = [b.ptr for b in bufs]
        t.cb_chunk_stride = cb_chunk_stride
        nb = self.lib.ibcu_pq_idx_t_bytes(M, N, G)
        dt = self.alloc(nb)
        self._check(self.lib.ibcu_pq_prepare(self.ctx, C.byref(t), dt.ptr))
        self.sync()
        t._keep = bufs + [dt]
        return t

    def make_pq_ex(self, d):
        """Upload a PQ tensor given as a dict of arrays in the reference's layout: cb1_l/r, idx1_l/r, rs, and optionally the
        second level (cb2_l/r, idx2_l/r, K_l2; 4-bit packed indices when K_l2 == 16) and the outlier sidecar (ocols, oside,
        oscale, n_outlier)."""
        t = PqT()
        t.M, t.N, t.G, t.K = d["M"], d["N"], d["G"], d["K"]
        keep = []
        def up(name):
            if name not in d:
                return None
            b = self.upload(d[name]); keep.append(b)
            return b.ptr
        t.codebook_l, t.codebook_r, t.idx_l, t.idx_r, t.row_scale = up("cb1_l"), up("cb1_r"), up("idx1_l"), up("idx1_r"), up("rs")
        t.cb_chunk_stride = 0
        t.K_l2 = d.get("K_l2", 0)
        t.codebook2_l, t.codebook2_r, t.idx2_l, t.idx2_r = up("cb2_l"), up("cb2_r"), up("idx2_l"), up("idx2_r")
        t.n_outlier = d.get("n_outlier", 0)
        t.outlier_cols, t.outlier_sidecar, t.outlier_scale = up("ocols"), up("oside"), up("oscale")
        dt = self.alloc(self.lib.ibcu_pq_prepared_bytes(C.byref(t)))
        self._check(self.lib.ibcu_pq_prepare(self.ctx, C.byref(t), dt.ptr))
        self.sync()
        t._keep = keep + [dt]
        return t

    def pq_matmul(self, t, x):
        x = np.ascontiguousarray(x, dtype=np.float32)
        if x.ndim == 1:
            x = x[None, :]
        B = x.shape[0]
        dx = self.upload(x)
        do = self.alloc(B * t.M * 4)
        self._check(self.lib.ibcu_pq_matmul_fp32(self.ctx, C.byref(t), dx.ptr, do.ptr, B))
        self.sync()
        return self.download(do, np.float32, B * t.M).reshape(B, t.M)

    def int4g_matmul(self, q, s, G, x, outl_idx=None, outl_val=None, eps=0.0):
        """group-scaled INT4 rows (ibcu_int4g_matmul_fp32): q [M, N/2] uint8, s [M, N/G] fp16 bits, one activation"""
        from ._ffi import Int4gT
        q = np.ascontiguousarray(q, np.uint8); s = np.ascontiguousarray(s, np.uint16)
        x = np.ascontiguousarray(x, np.float32).reshape(-1)
        t = Int4gT()
        t.M, t.N, t.G = q.shape[0], q.shape[1] * 2, G
        keep = [self.upload(q), self.upload(s), self.upload(x)]
        t.q, t.s = keep[0].ptr, keep[1].ptr
        t.K_out = 0
        if outl_idx is not None:
            oi = np.ascontiguousarray(outl_idx, np.uint16); ov = np.ascontiguousarray(outl_val, np.uint16)
            t.K_out = oi.shape[1]
            keep += [self.upload(oi), self.upload(ov)]
            t.outl_idx, t.outl_val = keep[3].ptr, keep[4].ptr
        do = self.alloc(t.M * 4)
        self._check(self.lib.ibcu_int4g_matmul_fp32(self.ctx, C.byref(t), keep[2].ptr, do.ptr, float(eps)))
        self.sync()
        return self.download(do, np.float32, t.M)

    def pq_lm_head_topk(self, t, x, k_top):
        """(logits[k_top], ids[k_top]) of ib_pq_lm_head_topk (src/pq_decode.c:2259-2341) for one activation"""
        x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
        dx = self.upload(x)
        dl = self.alloc(k_top * 4); di = self.alloc(k_top * 4)
        self._check(self.lib.ibcu_pq_lm_head_topk(self.ctx, C.byref(t), dx.ptr, k_top, dl.ptr, di.ptr))
        self.sync()
        return self.download(dl, np.float32, k_top), self.download(di, np.int32, k_top)

    def kmeans_assign(self, X, Cn, want_dist=False, path=0):
        """path: IBCU_KMEANS_AUTO (0), _EXACT (1) or _MMA_SYNC (2)"""
        X = np.ascontiguousarray(X, np.float32); Cn = np.ascontiguousarray(Cn, np.float32)
        N, D = X.shape; K = Cn.shape[0]
        dX, dC = self.upload(X), self.upload(Cn)
        di = self.alloc(N * 4); dd = self.alloc(N * 4)
        self.lib.ibcu_kmeans_set_path(self.ctx, path)
        try:
            self._check(self.lib.ibcu_kmeans_assign(self.ctx, dX.ptr, N, D, dC.ptr, K, di.ptr, dd.ptr))
            self.sync()
        finally:
            self.lib.ibcu_kmeans_set_path(self.ctx, 0)
        idx = self.download(di, np.int32, N)
        dist = self.download(dd, np.float32, N) if want_dist else None
        for b in (dX, dC, di, dd):
            b.free(); self._bufs.remove(b)
        return (idx, dist) if want_dist else idx
