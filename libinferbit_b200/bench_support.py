"""Workload builders and timers shared by bench.py (device buffers through the C ABI, timing with
CUDA events on the context's stream). Nothing here computes results on the host."""
import ctypes as C
import json
import os

import numpy as np

from ._ffi import LinearT, ModelCfg, PqT


def check(lib, ctx, rc):
    if rc != 0:
        msg = lib.ibcu_last_error(ctx).decode()
        raise RuntimeError(f"ibcu error {rc}: {msg}")


def load_peaks(root):
    path = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d.get("bf16_tflops", 0)), "source": "of measured (MEASURED_PEAKS.json)"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "of fallback (6.65 TB/s, 1.59 PFLOP/s)"}


class Dev:
    """Small helper around ibcu_malloc / copies."""

    def __init__(self, lib, ctx):
        self.lib, self.ctx, self.bufs = lib, ctx, []

    def alloc(self, nbytes):
        p = C.c_void_p()
        check(self.lib, self.ctx, self.lib.ibcu_malloc(self.ctx, max(int(nbytes), 16), C.byref(p)))
        self.bufs.append(p.value)
        return p.value

    def upload(self, arr):
        arr = np.ascontiguousarray(arr)
        d = self.alloc(arr.nbytes)
        check(self.lib, self.ctx, self.lib.ibcu_memcpy_h2d(self.ctx, d, arr.ctypes.data, arr.nbytes))
        check(self.lib, self.ctx, self.lib.ibcu_sync(self.ctx))
        return d

    def free_all(self):
        for b in self.bufs:
            self.lib.ibcu_free(self.ctx, b)
        self.bufs = []

    def alloc_gathered(self, nbytes):
        """a buffer that will be all-gathered: from the peer window when the context has one"""
        p = C.c_void_p()
        if self.lib.ibcu_window_alloc(self.ctx, nbytes, C.byref(p)) == 0:
            return p.value
        return self.alloc(nbytes)

    def timed(self, fn, reps=1):
        """device milliseconds of fn() (issued `reps` times) between two events on the stream"""
        self.lib.ibcu_event_record(self.ctx, 2)
        for _ in range(reps):
            fn()
        self.lib.ibcu_event_record(self.ctx, 3)
        ms = C.c_float()
        check(self.lib, self.ctx, self.lib.ibcu_event_elapsed_ms(self.ctx, 2, 3, C.byref(ms)))
        return ms.value / reps

    def spin_up(self, fn, seconds=0.3):
        """issue fn() until `seconds` of wall time have passed: a GPU that sat idle runs its first
        milliseconds at idle clocks, and the short cases here would otherwise be timed on those"""
        import time
        t0 = time.perf_counter()
        while time.perf_counter() - t0 < seconds:
            for _ in range(8):
                fn()
            check(self.lib, self.ctx, self.lib.ibcu_sync(self.ctx))

    def graph(self, fn):
        """run fn once eagerly (sizes scratch), then capture it; returns the graph id"""
        fn()
        check(self.lib, self.ctx, self.lib.ibcu_sync(self.ctx))
        check(self.lib, self.ctx, self.lib.ibcu_graph_begin(self.ctx))
        fn()
        gid = C.c_int()
        check(self.lib, self.ctx, self.lib.ibcu_graph_end(self.ctx, C.byref(gid)))
        return gid.value


def shard(lib, M, world, rank, align=32):
    r0, rn = C.c_int(), C.c_int()
    lib.ibcu_shard_rows(M, world, rank, align, C.byref(r0), C.byref(rn))
    return r0.value, rn.value


class AttnProjWorkload:
    """RING sets of (q, k, v, o) INT8 projections in HBM; with world > 1 each rank holds its row slices."""

    def __init__(self, lib, ctx, rank, world, ring, proj, B=1, seed=1234):
        self.lib, self.ctx, self.rank, self.world, self.ring, self.proj, self.B = lib, ctx, rank, world, ring, proj, B
        self.dev = Dev(lib, ctx)
        self.N = proj[0][2]
        rng = np.random.default_rng(seed)
        self.xh = rng.standard_normal((B, self.N)).astype(np.float32)
        self.x2h = rng.standard_normal((B, self.N)).astype(np.float32)
        self.x = self.dev.upload(self.xh)
        self.x2 = self.dev.upload(self.x2h)
        self.out = {name: self.dev.alloc_gathered(B * M * 4) for name, M, _ in proj}
        self.sets = []
        self.seeds = []
        s = seed * 977                                       # a tensor is a function of the seed and its place alone: every rank
        for r in range(ring):                                # fills its rows with the bytes the whole tensor has there
            ent, sd = {}, {}
            for name, M, N in proj:
                r0, rn = shard(lib, M, world, rank)
                w = self.dev.alloc(rn * N)
                sc = self.dev.alloc(rn * 2)
                s += 2; sd[name] = (s - 1, s)
                check(lib, ctx, lib.ibcu_fill_hash_bytes_at(ctx, w, rn * N, s - 1, r0 * N))
                check(lib, ctx, lib.ibcu_fill_hash_fp16_uniform_at(ctx, sc, rn, s, 0.001, 0.01, r0))
                ent[name] = (w, sc, M, r0, rn)
            self.sets.append(ent)
            self.seeds.append(sd)
        self.x_host = None
        check(lib, ctx, lib.ibcu_sync(ctx))

    def _desc(self, ent, name):
        w, sc, M, r0, rn = ent[name]
        return LinearT(w, sc, self.out[name] + 4 * r0, rn, M, 0, 0)

    def step(self, i):
        lib, ctx, ent = self.lib, self.ctx, self.sets[i % self.ring]
        qkv = (LinearT * 3)(self._desc(ent, "q"), self._desc(ent, "k"), self._desc(ent, "v"))
        if self.world > 1:                                   # announce the gather: the launch pushes its rows from its epilogue
            bufs = (C.c_void_p * 3)(*[self.out[n] for n in ("q", "k", "v")])
            Ms = (C.c_int * 3)(*[ent[n][2] for n in ("q", "k", "v")])
            check(lib, ctx, lib.ibcu_allgather_rows_prepare(ctx, bufs, Ms, 3))
        check(lib, ctx, lib.ibcu_linear(ctx, qkv, 3, self.x, self.N, self.B, 8))
        if self.world > 1:
            check(lib, ctx, lib.ibcu_allgather_rows_n(ctx, bufs, Ms, Ms, 3, self.B, 32))
        o = self._desc(ent, "o")
        if self.world > 1:
            bufs = (C.c_void_p * 1)(self.out["o"]); Ms = (C.c_int * 1)(ent["o"][2])
            check(lib, ctx, lib.ibcu_allgather_rows_prepare(ctx, bufs, Ms, 1))
        check(lib, ctx, lib.ibcu_linear(ctx, C.byref(o), 1, self.x2, self.N, self.B, 8))
        if self.world > 1:
            check(lib, ctx, lib.ibcu_allgather_rows_n(ctx, bufs, Ms, Ms, 1, self.B, 32))

    def matches_single_gpu(self):
        """The sharded step against the same step on one GPU: set 0 is run once by all ranks (with its gathers), then rank 0
        builds the unsharded tensors of set 0 from the same seeds on a context of its own without a communicator, runs
        q, k, v, o there and compares all four outputs. Returns a dict on rank 0, None elsewhere."""
        lib = self.lib
        self.step(0)
        check(lib, self.ctx, lib.ibcu_sync(self.ctx))
        if self.rank != 0:
            return None
        got = {}
        for name, M, _ in self.proj:
            a = np.empty((self.B, M), np.float32)
            check(lib, self.ctx, lib.ibcu_memcpy_d2h(self.ctx, a.ctypes.data, self.out[name], a.nbytes))
            got[name] = a
        check(lib, self.ctx, lib.ibcu_sync(self.ctx))
        ctx1 = C.c_void_p()
        dev_id = C.c_int()
        assert lib.ibcu_ctx_create(self._device(), C.byref(ctx1)) == 0
        d1 = Dev(lib, ctx1)
        res = {"max_abs_diff": 0.0, "bit_equal": True, "within_tolerance": True}
        for name, M, N in self.proj:
            w = d1.alloc(M * N); sc = d1.alloc(M * 2); o = d1.alloc(self.B * M * 4)
            sw, ss = self.seeds[0][name]
            check(lib, ctx1, lib.ibcu_fill_hash_bytes(ctx1, w, M * N, sw))
            check(lib, ctx1, lib.ibcu_fill_hash_fp16_uniform(ctx1, sc, M, ss, 0.001, 0.01))
            x = d1.upload(self.xh if name != "o" else self.x2h)
            t = LinearT(w, sc, o, M, M, 0, 0)
            check(lib, ctx1, lib.ibcu_linear(ctx1, C.byref(t), 1, x, N, self.B, 8))
            ref = np.empty((self.B, M), np.float32)
            check(lib, ctx1, lib.ibcu_memcpy_d2h(ctx1, ref.ctypes.data, o, ref.nbytes))
            check(lib, ctx1, lib.ibcu_sync(ctx1))
            diff = np.abs(got[name].astype(np.float64) - ref)
            res["max_abs_diff"] = max(res["max_abs_diff"], float(diff.max()))
            res["bit_equal"] = res["bit_equal"] and bool(np.array_equal(got[name], ref))
            res["within_tolerance"] = res["within_tolerance"] and bool(np.all(diff <= 1e-4 + 1e-3 * np.abs(ref)))
        d1.free_all()
        lib.ibcu_ctx_destroy(ctx1)
        return res

    def _device(self):
        return int(os.environ.get("LOCAL_RANK", "0"))

    def capture(self, n):
        self.step(0)
        check(self.lib, self.ctx, self.lib.ibcu_sync(self.ctx))
        before = self.lib.ibcu_launch_count(self.ctx)
        check(self.lib, self.ctx, self.lib.ibcu_graph_begin(self.ctx))
        for i in range(n):
            self.step(i)
        gid = C.c_int()
        check(self.lib, self.ctx, self.lib.ibcu_graph_end(self.ctx, C.byref(gid)))
        self.graph_launches = self.lib.ibcu_launch_count(self.ctx) - before
        return gid.value

    def replay(self, gid):
        check(self.lib, self.ctx, self.lib.ibcu_graph_launch(self.ctx, gid))

    def time_table_calls(self, host, steps, warmup, nsets=4, seed=99):
        """End to end through the ib_kernels-shaped table: host weights registered once (the model
        mapping), then per step four matmul_int8 calls with host activations, host FP32 scales and host
        outputs; every call moves its operands host->device and its result device->host."""
        import time
        rng = np.random.default_rng(seed)
        sets, blobs = [], []
        for _ in range(nsets):
            ent = []
            for name, M, N in self.proj:
                w = rng.integers(-127, 128, (M, N), dtype=np.int8)
                assert host.ib_b200_register(w.ctypes.data, w.nbytes) == 0, host.ib_b200_last_error()
                blobs.append(w)
                ent.append((w, rng.uniform(0.001, 0.01, M).astype(np.float32), np.empty(M, np.float32), M, N))
            sets.append(ent)
        x = rng.standard_normal(self.N).astype(np.float32)
        h2d = d2h = 0
        calls = []
        for ent in sets:
            cs = []
            for w, s, o, M, N in ent:
                r0, rn = shard(self.lib, M, self.world, self.rank)
                cs.append((o.ctypes.data + 4 * r0, w.ctypes.data + r0 * N, s.ctypes.data + 4 * r0, x.ctypes.data, rn, N))
            calls.append(cs)
        def step(i):
            for a in calls[i % nsets]:
                host.ib_b200_matmul_int8(*a)
        for i in range(max(warmup, nsets)):           # every set seen once: row scales are uploaded at a tensor's first call
            step(i)
        a0, b0 = C.c_ulonglong(), C.c_ulonglong()
        host.ib_b200_copy_stats(C.byref(a0), C.byref(b0))
        t0 = time.perf_counter()
        for i in range(steps):
            step(i)
        dt = (time.perf_counter() - t0) / steps
        a1, b1 = C.c_ulonglong(), C.c_ulonglong()
        host.ib_b200_copy_stats(C.byref(a1), C.byref(b1))
        h2d, d2h = (a1.value - a0.value) // steps, (b1.value - b0.value) // steps      # bytes the calls actually moved
        assert host.ib_b200_status() == 0, host.ib_b200_last_error()
        for w in blobs:
            host.ib_b200_unregister(w.ctypes.data)
        return {"t_step": dt, "h2d": h2d, "d2h": d2h}

    def close(self):
        self.dev.free_all()


# ── secondary configurations ────────────────────────────────────────────────────────────
def _linear_ring(lib, ctx, bits, M, N, B, reps_target_bytes=700e6, tcgen05=0):    # tcgen05: 0 library default, 1 / 2 forced on, -1 off
    """us per call and weight GB/s of one linear over a ring of distinct weight buffers (graph replay)."""
    dev = Dev(lib, ctx)
    lib.ibcu_linear_use_tcgen05(ctx, tcgen05)
    rowbytes = N if bits == 8 else N // 2
    wbytes = M * rowbytes
    R = max(2, int(reps_target_bytes // wbytes))
    dW = dev.alloc(R * wbytes); check(lib, ctx, lib.ibcu_fill_hash_bytes(ctx, dW, R * wbytes, 7))
    dS = dev.alloc(M * 2); check(lib, ctx, lib.ibcu_fill_hash_fp16_uniform(ctx, dS, M, 8, 0.002, 0.02))
    dx = dev.upload(np.random.default_rng(0).standard_normal((B, N)).astype(np.float32))
    do = dev.alloc(B * M * 4)
    descs = [LinearT(dW + r * wbytes, dS, do, M, M, 0, 0) for r in range(R)]

    def run():
        for d in descs:
            check(lib, ctx, lib.ibcu_linear(ctx, C.byref(d), 1, dx, N, B, bits))
    gid = dev.graph(run)
    dev.spin_up(lambda: lib.ibcu_graph_launch(ctx, gid))
    ms = min(dev.timed(lambda: lib.ibcu_graph_launch(ctx, gid), reps=5) for _ in range(3)) / R
    lib.ibcu_graph_destroy(ctx, gid)
    dev.free_all()
    lib.ibcu_linear_use_tcgen05(ctx, 0)
    algo = wbytes + 2 * M + 4 * B * N + 4 * B * M
    return {"us": ms * 1e3, "GBps": algo / ms / 1e6, "algorithmic_bytes": algo, "bound": "hbm",
            "shape": {"bits": bits, "M": M, "N": N, "B": B}}


def _w4a8_ring(lib, ctx, M, N, B, reps_target_bytes=300e6):
    """The reference's default route for an INT4 linear (src/forward.c:175-246 with IB_W4A8 on): quantise the activation per
    128-column group, then the INT4 x INT8 matvec; both steps are inside the timed call."""
    dev = Dev(lib, ctx)
    wbytes = M * N // 2
    R = max(2, int(reps_target_bytes // wbytes))
    groups = (N + 127) // 128
    dW = dev.alloc(R * wbytes); check(lib, ctx, lib.ibcu_fill_hash_bytes(ctx, dW, R * wbytes, 17))
    dS = dev.alloc(M * 2); check(lib, ctx, lib.ibcu_fill_hash_fp16_uniform(ctx, dS, M, 18, 0.002, 0.02))
    dx = dev.upload(np.random.default_rng(0).standard_normal((B, N)).astype(np.float32))
    dq, dsa, do = dev.alloc(B * N), dev.alloc(B * groups * 4), dev.alloc(B * M * 4)
    descs = [LinearT(dW + r * wbytes, dS, do, M, M, 0, 0) for r in range(R)]

    def run():
        for d in descs:
            check(lib, ctx, lib.ibcu_linear_w4a8_fp32(ctx, C.byref(d), dx, N, B))
    gid = dev.graph(run)
    dev.spin_up(lambda: lib.ibcu_graph_launch(ctx, gid))
    ms = min(dev.timed(lambda: lib.ibcu_graph_launch(ctx, gid), reps=5) for _ in range(3)) / R
    lib.ibcu_graph_destroy(ctx, gid)
    dev.free_all()
    algo = wbytes + 2 * M + 4 * B * N + 4 * B * M
    return {"us": ms * 1e3, "GBps": algo / ms / 1e6, "algorithmic_bytes": algo, "bound": "hbm",
            "shape": {"bits": 4, "activation_bits": 8, "M": M, "N": N, "B": B}, "route": "quantize_input_int8_g128 + matmul_w4a8 (ibcu_linear_w4a8_fp32)"}


def _pq(lib, ctx, M, N, G, K, B):
    dev = Dev(lib, ctx)
    rng = np.random.default_rng(3)
    half, Cn = G // 2, N // G
    R = 24                                                 # 24 x 7.3 MB of codes > L2
    cb = [dev.upload((rng.standard_normal((K, half)) * 0.02).astype(np.float16)) for _ in range(2)]
    rs = dev.upload(np.ones(M, np.float16))
    x = dev.upload(rng.standard_normal((B, N)).astype(np.float32))
    out = dev.alloc(B * M * 4)
    ts = []
    for r in range(R):
        t = PqT()
        t.M, t.N, t.G, t.K = M, N, G, K
        t.codebook_l, t.codebook_r, t.row_scale, t.cb_chunk_stride = cb[0], cb[1], rs, 0
        il = dev.alloc(M * Cn); ir = dev.alloc(M * Cn)
        check(lib, ctx, lib.ibcu_fill_hash_bytes(ctx, il, M * Cn, 100 + 2 * r))
        check(lib, ctx, lib.ibcu_fill_hash_bytes(ctx, ir, M * Cn, 101 + 2 * r))
        t.idx_l, t.idx_r = il, ir
        it = dev.alloc(lib.ibcu_pq_idx_t_bytes(M, N, G))
        check(lib, ctx, lib.ibcu_pq_prepare(ctx, C.byref(t), it))
        ts.append(t)

    def run():
        for t in ts:
            check(lib, ctx, lib.ibcu_pq_matmul_fp32(ctx, C.byref(t), x, out, B))
    gid = dev.graph(run)
    dev.spin_up(lambda: lib.ibcu_graph_launch(ctx, gid))
    ms = min(dev.timed(lambda: lib.ibcu_graph_launch(ctx, gid), reps=10) for _ in range(3)) / R
    lib.ibcu_graph_destroy(ctx, gid)
    dev.free_all()
    algo = 2 * M * Cn + 2 * K * half * 2 + 2 * M + 4 * B * N + 4 * B * M
    return {"us": ms * 1e3, "GBps": algo / ms / 1e6, "algorithmic_bytes": algo, "bound": "hbm",
            "shape": {"M": M, "N": N, "G": G, "K": K, "B": B}}


def _int4g(lib, ctx, M, N, G):
    """group-scaled INT4 rows, one activation; a ring of tensors larger than L2"""
    from ._ffi import Int4gT
    dev = Dev(lib, ctx)
    rng = np.random.default_rng(9)
    wbytes, sbytes = M * N // 2, 2 * M * (N // G)
    R = max(2, int(300e6 // (wbytes + sbytes)) + 1)
    x = dev.upload(rng.standard_normal(N).astype(np.float32))
    out = dev.alloc(M * 4)
    ts = []
    for r in range(R):
        t = Int4gT()
        t.M, t.N, t.G, t.K_out = M, N, G, 0
        q = dev.alloc(wbytes); sc = dev.alloc(sbytes)
        check(lib, ctx, lib.ibcu_fill_hash_bytes(ctx, q, wbytes, 500 + r))
        check(lib, ctx, lib.ibcu_fill_hash_fp16_uniform(ctx, sc, M * (N // G), 600 + r, 0.002, 0.02))
        t.q, t.s = q, sc
        ts.append(t)

    def run():
        for t in ts:
            check(lib, ctx, lib.ibcu_int4g_matmul_fp32(ctx, C.byref(t), x, out, 0.0))
    gid = dev.graph(run)
    dev.spin_up(lambda: lib.ibcu_graph_launch(ctx, gid))
    ms = min(dev.timed(lambda: lib.ibcu_graph_launch(ctx, gid), reps=10) for _ in range(3)) / R
    lib.ibcu_graph_destroy(ctx, gid)
    dev.free_all()
    algo = wbytes + sbytes + 4 * N + 4 * M
    return {"us": ms * 1e3, "GBps": algo / ms / 1e6, "algorithmic_bytes": algo, "bound": "hbm",
            "shape": {"bits": 4, "group": G, "M": M, "N": N, "B": 1}}


def _pq_topk(lib, ctx, M, N, G, K, K_l2, k_top):
    """ib_pq_lm_head_topk on a two-level LM head: first-level matvec over all rows, choice of k_top rows, every level of
    those rows, order. Eight tensors' code planes (more than L2 together with their regrouped copies) are walked in a ring."""
    dev = Dev(lib, ctx)
    rng = np.random.default_rng(5)
    half, Cn = G // 2, N // G
    R = 8
    cb = [dev.upload((rng.standard_normal((K, half)) * 0.02).astype(np.float16)) for _ in range(2)]
    cb2 = [dev.upload((rng.standard_normal((K_l2, half)) * 0.004).astype(np.float16)) for _ in range(2)]
    rs = dev.upload(np.ones(M, np.float16))
    x = dev.upload(rng.standard_normal(N).astype(np.float32))
    ol = dev.alloc(k_top * 4); oi = dev.alloc(k_top * 4)
    stride2 = (Cn + 1) // 2 if K_l2 == 16 else Cn
    ts = []
    for r in range(R):
        t = PqT()
        t.M, t.N, t.G, t.K, t.K_l2 = M, N, G, K, K_l2
        t.codebook_l, t.codebook_r, t.row_scale, t.cb_chunk_stride = cb[0], cb[1], rs, 0
        t.codebook2_l, t.codebook2_r = cb2[0], cb2[1]
        bufs = [dev.alloc(M * Cn), dev.alloc(M * Cn), dev.alloc(M * stride2), dev.alloc(M * stride2)]
        for j, b in enumerate(bufs):
            check(lib, ctx, lib.ibcu_fill_hash_bytes(ctx, b, M * (Cn if j < 2 else stride2), 300 + 4 * r + j))
        t.idx_l, t.idx_r, t.idx2_l, t.idx2_r = bufs
        it = dev.alloc(lib.ibcu_pq_prepared_bytes(C.byref(t)))
        check(lib, ctx, lib.ibcu_pq_prepare(ctx, C.byref(t), it))
        ts.append(t)

    def run():
        for t in ts:
            check(lib, ctx, lib.ibcu_pq_lm_head_topk(ctx, C.byref(t), x, k_top, ol, oi))
    gid = dev.graph(run)
    dev.spin_up(lambda: lib.ibcu_graph_launch(ctx, gid))
    ms = min(dev.timed(lambda: lib.ibcu_graph_launch(ctx, gid), reps=10) for _ in range(3)) / R
    lib.ibcu_graph_destroy(ctx, gid)
    dev.free_all()
    algo = 2 * M * Cn + 2 * K * half * 2 + 2 * M + 4 * N + k_top * (2 * Cn + 2 * stride2) + 8 * k_top
    return {"us": ms * 1e3, "GBps": algo / ms / 1e6, "algorithmic_bytes": algo, "bound": "hbm",
            "shape": {"M": M, "N": N, "G": G, "K": K, "K_l2": K_l2, "K_top": k_top}}


def _pq_sharded(lib, ctx, rank, world, max_over_ranks, barrier, M, N, G, K, B):
    """The PQ matvec with the rows of every tensor split over the ranks (the reference's threaded form splits rows over
    workers the same way): a rank computes its rows in place into the full-width result, a gather completes it. The
    codes are a function of the seed and the global row, so the sharded tensors are the single-GPU ones."""
    dev = Dev(lib, ctx)
    rng = np.random.default_rng(3)
    half, Cn = G // 2, N // G
    R = 24
    cbh = [(rng.standard_normal((K, half)) * 0.02).astype(np.float16) for _ in range(2)]
    cb = [dev.upload(c) for c in cbh]
    xh = rng.standard_normal((B, N)).astype(np.float32)
    x = dev.upload(xh)
    r0, rn = shard(lib, M, world, rank)
    rs = dev.upload(np.ones(rn, np.float16))
    outs = [dev.alloc_gathered(B * M * 4) for _ in range(2)]      # two result buffers in turn (a buffer is not gathered twice in a row)
    ts = []
    def make(dv, rows, row0, r):
        t = PqT()
        t.M, t.N, t.G, t.K = rows, N, G, K
        t.codebook_l, t.codebook_r, t.cb_chunk_stride = cb[0] if dv is dev else dv.upload(cbh[0]), cb[1] if dv is dev else dv.upload(cbh[1]), 0
        t.row_scale = rs if dv is dev else dv.upload(np.ones(rows, np.float16))
        il = dv.alloc(rows * Cn); ir = dv.alloc(rows * Cn)
        check(dv.lib, dv.ctx, dv.lib.ibcu_fill_hash_bytes_at(dv.ctx, il, rows * Cn, 100 + 2 * r, row0 * Cn))
        check(dv.lib, dv.ctx, dv.lib.ibcu_fill_hash_bytes_at(dv.ctx, ir, rows * Cn, 101 + 2 * r, row0 * Cn))
        t.idx_l, t.idx_r = il, ir
        it = dv.alloc(dv.lib.ibcu_pq_idx_t_bytes(rows, N, G))
        check(dv.lib, dv.ctx, dv.lib.ibcu_pq_prepare(dv.ctx, C.byref(t), it))
        return t
    for r in range(R):
        ts.append(make(dev, rn, r0, r))
    k = [0]
    def one():
        o = outs[k[0] & 1]
        check(lib, ctx, lib.ibcu_pq_matmul_fp32_strided(ctx, C.byref(ts[k[0] % R]), x, o + 4 * r0, M, B))
        bufs = (C.c_void_p * 1)(o); Ms = (C.c_int * 1)(M)
        check(lib, ctx, lib.ibcu_allgather_rows_n(ctx, bufs, Ms, Ms, 1, B, 32))
        k[0] += 1
    for _ in range(200):
        one()
    barrier()
    reps = 240
    ms = max_over_ranks(dev.timed(one, reps=reps))
    algo = 2 * M * Cn + 2 * K * half * 2 + 2 * M + 4 * B * N + 4 * B * M
    out = {"us": ms * 1e3, "GBps": algo / ms / 1e6, "algorithmic_bytes": algo, "bound": "hbm", "rows_per_rank": rn,
           "shape": {"M": M, "N": N, "G": G, "K": K, "B": B}}
    # tensor 0 once more, against the unsharded tensor on one GPU (rank 0, own context)
    k[0] = 0
    one()
    got = np.empty((B, M), np.float32)
    check(lib, ctx, lib.ibcu_memcpy_d2h(ctx, got.ctypes.data, outs[0], got.nbytes))
    check(lib, ctx, lib.ibcu_sync(ctx))
    barrier()
    if rank == 0:
        ctx1 = C.c_void_p()
        assert lib.ibcu_ctx_create(int(os.environ.get("LOCAL_RANK", "0")), C.byref(ctx1)) == 0
        d1 = Dev(lib, ctx1)
        t1 = make(d1, M, 0, 0)
        x1 = d1.upload(xh); o1 = d1.alloc(B * M * 4)
        check(lib, ctx1, lib.ibcu_pq_matmul_fp32(ctx1, C.byref(t1), x1, o1, B))
        ref = np.empty((B, M), np.float32)
        check(lib, ctx1, lib.ibcu_memcpy_d2h(ctx1, ref.ctypes.data, o1, ref.nbytes))
        check(lib, ctx1, lib.ibcu_sync(ctx1))
        d1.free_all(); lib.ibcu_ctx_destroy(ctx1)
        diff = np.abs(got.astype(np.float64) - ref)
        out["matches_single_gpu"] = {"max_abs_diff": float(diff.max()), "bit_equal": bool(np.array_equal(got, ref)),
                                     "within_tolerance": bool(np.all(diff <= 1e-4 + 1e-3 * np.abs(ref)))}
    barrier()
    dev.free_all()
    return out


def _kmeans_shard(r, world, N_total, D, K, C0):
    n0 = N_total * r // world; n1 = N_total * (r + 1) // world
    X = (np.random.default_rng(5000 + r).standard_normal((n1 - n0, D)) * 0.02).astype(np.float32)
    if r == 0:
        X[:K] = C0
    return X


def _kmeans(lib, ctx, rank, world, max_over_ranks, barrier, N_total=1 << 22, D=8, K=256, iters=10):
    dev = Dev(lib, ctx)
    rng = np.random.default_rng(1234)
    C0 = (rng.standard_normal((K, D)) * 0.02).astype(np.float32)        # stands for X[:K]; same on every rank
    X = _kmeans_shard(rank, world, N_total, D, K, C0)
    dX = dev.upload(X); dC = dev.upload(C0)
    n = len(X)
    di, dd = dev.alloc(n * 4), dev.alloc(n * 4)
    ds, dc, dn = dev.alloc(K * D * 4), dev.alloc(K * 4), dev.alloc(16)

    def it():
        check(lib, ctx, lib.ibcu_kmeans_lloyd_iter(ctx, dX, n, D, dC, K, di, dd, ds, dc, dn))
    for _ in range(200):                                   # a fixed count (ranks must issue the same collectives): clocks up
        it()
    barrier()
    check(lib, ctx, lib.ibcu_memcpy_h2d(ctx, dC, C0.ctypes.data, C0.nbytes))
    barrier()
    ms = dev.timed(lambda: [it() for _ in range(iters)])
    ms = max_over_ranks(ms)
    out = {"ms_per_iter": ms / iters, "Mpoints_per_s": N_total / (ms / iters) / 1e3, "points": N_total, "K": K, "D": D, "iters": iters,
           "algorithmic_bytes": N_total * D * 4 + N_total * 4 + K * D * 4, "flops": 2 * N_total * K * D, "bound": "tensor"}
    if world > 1:
        # one iteration from C0, sharded, against the same iteration of all points on one GPU (rank 0, own context)
        check(lib, ctx, lib.ibcu_memcpy_h2d(ctx, dC, C0.ctypes.data, C0.nbytes))
        it()
        cnt = np.empty(K, np.int32); Cs = np.empty((K, D), np.float32)
        check(lib, ctx, lib.ibcu_memcpy_d2h(ctx, cnt.ctypes.data, dc, cnt.nbytes))
        check(lib, ctx, lib.ibcu_memcpy_d2h(ctx, Cs.ctypes.data, dC, Cs.nbytes))
        barrier()
        if rank == 0:
            ctx1 = C.c_void_p()
            assert lib.ibcu_ctx_create(int(os.environ.get("LOCAL_RANK", "0")), C.byref(ctx1)) == 0
            d1 = Dev(lib, ctx1)
            Xall = np.concatenate([_kmeans_shard(r, world, N_total, D, K, C0) for r in range(world)])
            aX, aC = d1.upload(Xall), d1.upload(C0)
            ai, ad = d1.alloc(N_total * 4), d1.alloc(N_total * 4)
            a_s, a_c, a_n = d1.alloc(K * D * 4), d1.alloc(K * 4), d1.alloc(16)
            check(lib, ctx1, lib.ibcu_kmeans_lloyd_iter(ctx1, aX, N_total, D, aC, K, ai, ad, a_s, a_c, a_n))
            rc = np.empty(K, np.int32); rC = np.empty((K, D), np.float32)
            check(lib, ctx1, lib.ibcu_memcpy_d2h(ctx1, rc.ctypes.data, a_c, rc.nbytes))
            check(lib, ctx1, lib.ibcu_memcpy_d2h(ctx1, rC.ctypes.data, aC, rC.nbytes))
            check(lib, ctx1, lib.ibcu_sync(ctx1))
            out["matches_single_gpu"] = {"counts_equal": bool(np.array_equal(cnt, rc)), "max_centroid_diff": float(np.abs(Cs - rC).max()),
                                         "within_tolerance": bool(np.array_equal(cnt, rc) and np.allclose(Cs, rC, rtol=1e-5, atol=1e-7))}
            d1.free_all()
            lib.ibcu_ctx_destroy(ctx1)
        barrier()
    dev.free_all()
    return out


DECODE_CFG = (4096, 14336, 32, 32, 8, 128, 32000, 1024, 1e-5, 10000.0, 8, 4, 8)
DECODE_NOTE = ("random weights as the configuration says except that the per-row scales are drawn twenty times below its ranges "
               "(32 random layers otherwise overflow FP32); KV cache rows 0..511 bell-shaped with unit variance; every step is one "
               "replay of the same CUDA graph (the position is read on the device) at positions 512, 512 + B, ..., 512 + 7 B in turn")


def _decode(lib, host, ctx, B, rank, world, max_over_ranks, barrier, steps=20, warm=60, check_single=True, graph=True):
    cfg = ModelCfg(*DECODE_CFG)
    m = host.ib_b200_model_create(ctx, C.byref(cfg))
    if not m:
        return {"error": "model allocation failed"}
    assert host.ib_b200_model_fill_random(m, 4321, 512) == 0
    if not graph:
        host.ib_b200_model_use_graph(m, 0)                 # launches issued one by one (a profiler then sees kernels)
    toks = np.arange(B, dtype=np.int32) * 7 + 11
    check(lib, ctx, lib.ibcu_memcpy_h2d(ctx, host.ib_b200_model_tokens(m), toks.ctypes.data, toks.nbytes))
    V = cfg.vocab
    out = {}
    if world > 1 and check_single:
        # the sharded model is the one-GPU model: same seed, same step at position 512, logits compared on rank 0
        check(lib, ctx, host.ib_b200_forward_step_device(m, 512, B))
        got = np.empty((B, V), np.float32)
        check(lib, ctx, lib.ibcu_memcpy_d2h(ctx, got.ctypes.data, host.ib_b200_model_logits(m), got.nbytes))
        check(lib, ctx, lib.ibcu_sync(ctx))
        barrier()
        if rank == 0:
            ctx1 = C.c_void_p()
            assert lib.ibcu_ctx_create(int(os.environ.get("LOCAL_RANK", "0")), C.byref(ctx1)) == 0
            m1 = host.ib_b200_model_create(ctx1, C.byref(cfg))
            assert m1 and host.ib_b200_model_fill_random(m1, 4321, 512) == 0
            check(lib, ctx1, lib.ibcu_memcpy_h2d(ctx1, host.ib_b200_model_tokens(m1), toks.ctypes.data, toks.nbytes))
            check(lib, ctx1, host.ib_b200_forward_step_device(m1, 512, B))
            ref = np.empty((B, V), np.float32)
            check(lib, ctx1, lib.ibcu_memcpy_d2h(ctx1, ref.ctypes.data, host.ib_b200_model_logits(m1), ref.nbytes))
            check(lib, ctx1, lib.ibcu_sync(ctx1))
            host.ib_b200_model_free(m1)
            lib.ibcu_ctx_destroy(ctx1)
            diff = np.abs(got.astype(np.float64) - ref)
            out["matches_single_gpu"] = {"max_abs_diff": float(diff.max()), "bit_equal": bool(np.array_equal(got, ref)),
                                         "within_tolerance": bool(np.all(diff <= 1e-4 + 1e-3 * np.abs(ref)))}
        barrier()
    span = 8                                               # positions 512, 512 + B, ... 512 + 7 B, then again
    pos = lambda i: 512 + (i % span) * B
    for i in range(warm):                                  # a fixed count, the same on every rank: clocks up
        check(lib, ctx, host.ib_b200_forward_step_device(m, pos(i), B))
    barrier()
    dev = Dev(lib, ctx)
    k = [0]

    def one():
        check(lib, ctx, host.ib_b200_forward_step_device(m, pos(k[0]), B)); k[0] += 1
    ms = dev.timed(one, reps=steps)
    ms = max_over_ranks(ms)
    logits = np.empty(8, np.float32)
    check(lib, ctx, lib.ibcu_memcpy_d2h(ctx, logits.ctypes.data, host.ib_b200_model_logits(m), 32))
    check(lib, ctx, lib.ibcu_sync(ctx))
    wb = host.ib_b200_model_weight_bytes(m)
    host.ib_b200_model_free(m)
    kv_bytes = 32 * 2 * (512 + B) * 1024 * 4
    out.update({"ms_per_step": ms, "tok_per_s": B / ms * 1e3, "batch": B, "pos": "512 + B * (step % 8)", "weight_GBps_per_gpu": wb / ms / 1e6,
                "algorithmic_bytes": int(wb * world + kv_bytes), "bound": "hbm", "logits_finite": bool(np.isfinite(logits).all()),
                "logits_head": [float(v) for v in logits], "note": DECODE_NOTE})
    return out


def with_roofline(entry, peaks, world=1):
    """adds achieved / peak / frac to an entry that carries its time and algorithmic bytes (or flops)"""
    if "algorithmic_bytes" not in entry:
        return entry
    t = entry["us"] * 1e-6 if "us" in entry else (entry.get("ms_per_iter", entry.get("ms_per_step", 0.0)) * 1e-3)
    if t <= 0:
        return entry
    gbs = entry["algorithmic_bytes"] / t / 1e9 / world           # per GPU
    r = {"bound": entry.get("bound", "hbm"), "hbm_achieved_GBps": gbs, "hbm_peak_GBps": peaks["hbm_gbs"], "hbm_frac": gbs / peaks["hbm_gbs"], "peak_source": peaks["source"]}
    if "flops" in entry:
        tf = entry["flops"] / t / 1e12 / world
        # TF32 is not among the measured peaks; half of the measured dense bf16 rate is the nominal ratio
        r.update({"tensor_achieved_TFLOPs": tf, "tensor_peak_TFLOPs": peaks["bf16_tflops"] / 2, "tensor_frac": tf / (peaks["bf16_tflops"] / 2) if peaks["bf16_tflops"] else None,
                  "tensor_peak_note": "half of the measured dense bf16 GEMM rate (TF32 nominal ratio)"})
    entry["roofline"] = r
    return entry


def other_configs(lib, host, ctx, rank, world, dist, max_over_ranks, barrier, peaks):
    out = {}
    if world == 1:
        out["int4_tinyllama_up_5632x2048_b1"] = _linear_ring(lib, ctx, 4, 5632, 2048, 1)
        out["int4_gate_14336x4096_b1"] = _linear_ring(lib, ctx, 4, 14336, 4096, 1)
        out["int4_down_4096x14336_b1"] = _linear_ring(lib, ctx, 4, 4096, 14336, 1)
        out["w4a8_gate_14336x4096_b1"] = _w4a8_ring(lib, ctx, 14336, 4096, 1)
        out["w4a8_down_4096x14336_b1"] = _w4a8_ring(lib, ctx, 4096, 14336, 1)
        out["int8_q_4096x4096_b1"] = _linear_ring(lib, ctx, 8, 4096, 4096, 1)
        out["int8_q_4096x4096_b4"] = _linear_ring(lib, ctx, 8, 4096, 4096, 4)
        out["int8_q_4096x4096_b16"] = _linear_ring(lib, ctx, 8, 4096, 4096, 16)
        out["int8_head_32000x4096_b1"] = _linear_ring(lib, ctx, 8, 32000, 4096, 1)
        out["pq_down_4096x14336_b1"] = _pq(lib, ctx, 4096, 14336, 16, 256, 1)
        out["pq_down_4096x14336_b8"] = _pq(lib, ctx, 4096, 14336, 16, 256, 8)
        out["pq_topk_head_32000x4096_k64"] = _pq_topk(lib, ctx, 32000, 4096, 16, 256, 16, 64)
        out["int4_group128_4096x4096_b1"] = _int4g(lib, ctx, 4096, 4096, 128)
        out["int4_group128_14336x4096_b1"] = _int4g(lib, ctx, 14336, 4096, 128)
    if world > 1:
        out["pq_down_4096x14336_b1_row_sharded"] = _pq_sharded(lib, ctx, rank, world, max_over_ranks, barrier, 4096, 14336, 16, 256, 1)
    out["kmeans_4Mx8_k256"] = _kmeans(lib, ctx, rank, world, max_over_ranks, barrier)
    out["decode_7b_b1"] = _decode(lib, host, ctx, 1, rank, world, max_over_ranks, barrier)
    out["decode_7b_b8"] = _decode(lib, host, ctx, 8, rank, world, max_over_ranks, barrier)
    if world > 1:
        # the same step with every gather through NCCL: the logits must be the same bits, only the transport differs
        lib.ibcu_window_enable(ctx, 0)
        out["decode_7b_b1_nccl_gathers"] = _decode(lib, host, ctx, 1, rank, world, max_over_ranks, barrier, check_single=False)
        lib.ibcu_window_enable(ctx, 1)
        out["push_gather_matches_nccl"] = out["decode_7b_b1"]["logits_head"] == out["decode_7b_b1_nccl_gathers"]["logits_head"]
    for k, v in out.items():
        if isinstance(v, dict):
            with_roofline(v, peaks, world)
    return out
