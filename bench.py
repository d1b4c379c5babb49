#!/usr/bin/env python
"""Benchmark of the quantized-weight product hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...

Headline workload ("int8_attn_proj_b1"): the INT8 attention projections of a Mistral-7B layer,
q and o 4096x4096, k and v 1024x4096, per-row FP16 scales, one FP32 activation (batch 1). One step =
one pass over one layer's four projections (q, k, v in one launch sharing the activation, then o);
consecutive steps walk a ring of distinct weight sets larger than L2, so every byte comes from HBM.
metric = weight GB/s = algorithmic bytes of a step / device time of a step.
With N > 1 the output rows of every projection are split over the ranks and gathered through the peer
window (tagged stores from the producing kernel's epilogue into every peer's memory, received in the next
kernel's prologue; NCCL is the plumbing and the comparison line) — total work fixed: strong scaling.

The JSON line also carries, under "other", quick measurements of the other configurations (INT4,
PQ, k-means, 7B-shape decode step); they are context, not the headline.
"""
import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

HID, KV = 4096, 1024
PROJ = [("q", HID, HID), ("k", KV, HID), ("v", KV, HID), ("o", HID, HID)]
RING = 16                                # weight sets in the ring: 16 x 42 MB = 671 MB >> 126 MB of L2


def algo_bytes_int8(M, N, B):
    """weights + fp16 scales + FP32 activations in + FP32 outputs"""
    return M * N + 2 * M + 4 * B * N + 4 * B * M


STEP_BYTES = sum(algo_bytes_int8(M, N, 1) for _, M, N in PROJ)


# ── clocks ──────────────────────────────────────────────────────────────────────────────
class ClockSampler:
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.stop, self.th = index, [], False, None

    def _run(self):
        while not self.stop:
            try:
                out = subprocess.run(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits"],
                                     capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.rows.append([c.strip() for c in out.split(",")])
            except Exception:
                pass
            time.sleep(0.1)

    def __enter__(self):
        self.th = threading.Thread(target=self._run, daemon=True)
        self.th.start()
        return self

    def __exit__(self, *a):
        self.stop = True
        self.th.join(timeout=6)

    def summary(self):
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        mhz = sorted(float(r[0]) for r in self.rows if r[0].replace(".", "").isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in self.rows if len(r) >= 6)]
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": float(self.rows[0][1]), "reasons": reasons,
                "samples": len(self.rows)}


# ── CPU baseline: the reference's own kernels when its library was built, else this repo's port ──
def _time_calls(fn, budget_s=2.0, min_reps=2, max_reps=50):
    """best of repeated calls (the reference's own benches report the minimum, tests/bench_pq_decode.c:74-108)"""
    fn()
    best, reps, t_all = 1e30, 0, time.perf_counter()
    while reps < min_reps or (reps < max_reps and time.perf_counter() - t_all < budget_s):
        t0 = time.perf_counter(); fn(); best = min(best, time.perf_counter() - t0); reps += 1
    return best, reps


class CpuBaseline:
    def __init__(self):
        ref = os.path.join(ROOT, "oracle", "_ref", "libinferbit_ref.so")
        self.threads = os.cpu_count() or 1
        if os.path.exists(ref):
            self.kind, self.lib = "reference", C.CDLL(ref)
            L = self.lib
            L.ib_detect_simd.restype = C.c_int
            L.ib_init_kernels(L.ib_detect_simd())          # AVX2 table on x86-64
            L.ib_pool_create.restype = C.c_void_p
            L.ib_pool_create.argtypes = [C.c_int]
            self.pool = L.ib_pool_create(self.threads)
            L.ib_parallel_matmul.argtypes = [C.c_void_p] * 5 + [C.c_int] * 3
            L.ib_parallel_matmul_int8_batch.argtypes = [C.c_void_p] * 5 + [C.c_int] * 3
            L.ib_kmeans_assign.restype = C.c_int
            L.ib_kmeans_assign.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]
            L.ib_pq_matmul_fp32_threaded.restype = C.c_int
            L.ib_pq_matmul_fp32_threaded.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        else:
            port = os.path.join(ROOT, "oracle", "libib_oracle.so")
            if not os.path.exists(port):
                subprocess.run(["make", "-s", "-C", os.path.join(ROOT, "oracle"), "oracle"], check=True)
            self.kind, self.lib, self.threads = "port", C.CDLL(port), 1

    def _base(self, value, unit, sample, cores=None):
        return {"value": value, "unit": unit, "cores": self.threads if cores is None else cores, "kind": self.kind, "sample": sample}

    def matvec_int8(self, out, w, s32, x, M, N):
        if self.kind == "reference":
            self.lib.ib_parallel_matmul(self.pool, out.ctypes.data, w.ctypes.data, s32.ctypes.data, x.ctypes.data, M, N, 8)
        else:
            self.lib.ibo_matmul_int8(out.ctypes.data, w.ctypes.data, s32.ctypes.data, x.ctypes.data, M, N)

    def time_steps(self, steps, warmup, seed=1234):
        """One step = q, k, v, o of one layer on host memory; a ring of 4 sets (168 MB) keeps the weights out of cache."""
        rng = np.random.default_rng(seed)
        sets = []
        for _ in range(4):
            sets.append([(rng.integers(-127, 128, (M, N), dtype=np.int8), rng.uniform(0.001, 0.01, M).astype(np.float32),
                          np.empty(M, np.float32), M, N) for _, M, N in PROJ])
        x = rng.standard_normal(HID).astype(np.float32)
        def step(i):
            for w, s, o, M, N in sets[i % len(sets)]:
                self.matvec_int8(o, w, s, x, M, N)
        for i in range(warmup):
            step(i)
        t0 = time.perf_counter()
        for i in range(steps):
            step(i)
        dt = (time.perf_counter() - t0) / steps
        return dt, STEP_BYTES / dt / 1e9

    # the secondary configurations: the reference's own entry point for each, on its pool with every host thread
    def linear(self, bits, M, N, B, algo_bytes):
        rng = np.random.default_rng(1)
        w = rng.integers(0, 256, (M, N if bits == 8 else N // 2), dtype=np.uint8)
        s = rng.uniform(0.002, 0.02, M).astype(np.float32)
        x = rng.standard_normal((B, N)).astype(np.float32)
        out = np.empty((B, M), np.float32)
        L, p = self.lib, lambda a: a.ctypes.data
        if self.kind != "reference":
            fn = (lambda: L.ibo_matmul_int8(p(out), p(w), p(s), p(x), M, N)) if bits == 8 else (lambda: L.ibo_matmul_int4(p(out), p(w), p(s), p(x), M, N))
            t, reps = _time_calls(fn, 1.0)
            return self._base(algo_bytes / (t * B) / 1e9, "GB/s", f"best of {reps} single-activation calls of the scalar port, scaled to batch {B}")
        single = lambda: [L.ib_parallel_matmul(self.pool, p(out) + 4 * b * M, p(w), p(s), p(x) + 4 * b * N, M, N, bits) for b in range(B)]
        t, reps = _time_calls(single, 1.5)
        r = self._base(algo_bytes / t / 1e9, "GB/s", f"best of {reps}: ib_parallel_matmul x {B} (bits {bits}; the AVX2 table has no batched kernel, so this is what forward.c runs per position)")
        if bits == 8 and B > 1:
            t2, reps2 = _time_calls(lambda: L.ib_parallel_matmul_int8_batch(self.pool, p(out), p(w), p(s), p(x), M, N, B), 1.5)
            r["int8_batch_entry_GBps"] = algo_bytes / t2 / 1e9
            r["sample"] += f"; ib_parallel_matmul_int8_batch (scalar on x86-64): best of {reps2}"
        return r

    def w4a8(self, M, N, B, algo_bytes):
        """the reference's default route for an INT4 linear: ib_quantize_input_int8_g128 per activation, then
        ib_parallel_matmul_w4a8 on the pool (src/forward.c:175-246)"""
        if self.kind != "reference":
            return None
        rng = np.random.default_rng(1)
        w = rng.integers(0, 256, (M, N // 2), dtype=np.uint8)
        s = rng.uniform(0.002, 0.02, M).astype(np.float32)
        x = rng.standard_normal((B, N)).astype(np.float32)
        q = np.empty((B, N), np.int8); sa = np.empty((B, (N + 127) // 128), np.float32)
        out = np.empty((B, M), np.float32)
        L, p = self.lib, lambda a: a.ctypes.data
        L.ib_parallel_matmul_w4a8.argtypes = [C.c_void_p] * 6 + [C.c_int] * 2
        L.ib_quantize_input_int8_g128.argtypes = [C.c_void_p] * 3 + [C.c_int]
        def fn():
            for b in range(B):
                L.ib_quantize_input_int8_g128(p(x) + 4 * b * N, p(q) + b * N, p(sa) + 4 * b * sa.shape[1], N)
                L.ib_parallel_matmul_w4a8(self.pool, p(out) + 4 * b * M, p(w), p(s), p(q) + b * N, p(sa) + 4 * b * sa.shape[1], M, N)
        t, reps = _time_calls(fn, 1.5)
        return self._base(algo_bytes / t / 1e9, "GB/s", f"best of {reps}: ib_quantize_input_int8_g128 + ib_parallel_matmul_w4a8 x {B}")

    def pq(self, M, N, G, K, B, algo_bytes):
        if self.kind != "reference":
            return None
        sys.path.insert(0, ROOT)
        from tests import _cpu
        rng = np.random.default_rng(3)
        cb_l, cb_r, il, ir, rs, x = _cpu.make_pq_case(rng, M, N, G, K, B, scale_one=True)
        t = _cpu.RefPqTensor()
        t.M, t.N, t.G, t.K, t.K_l2, t.n_levels, t.rotate, t.n_outlier, t.format = M, N, G, K, 0, 1, 0, 0, 0
        t.codebook_l1_l, t.codebook_l1_r = cb_l.ctypes.data, cb_r.ctypes.data
        t.indices_l1_l, t.indices_l1_r = il.ctypes.data, ir.ctypes.data
        t.C, t.l2_idx_bytes, t.row_scale = N // G, 1, rs.ctypes.data
        out = np.empty((B, M), np.float32)
        fn = lambda: [self.lib.ib_pq_matmul_fp32_threaded(C.byref(t), x.ctypes.data + 4 * b * N, out.ctypes.data + 4 * b * M, self.pool) for b in range(B)]
        tt, reps = _time_calls(fn, 1.5)
        return self._base(algo_bytes / tt / 1e9, "GB/s", f"best of {reps}: ib_pq_matmul_fp32_threaded x {B}")

    def pq_topk(self, M, N, G, K, K_l2, k_top, algo_bytes):
        if self.kind != "reference":
            return None
        sys.path.insert(0, ROOT)
        from tests import _cpu
        rng = np.random.default_rng(5)
        d = _cpu.make_pq_case_ex(rng, M, N, G, K, K_l2, 0, 1)
        t = _cpu.ref_pq_tensor_ex(d)
        logits = np.empty(k_top, np.float32); ids = np.empty(k_top, np.int32)
        self.lib.ib_pq_lm_head_topk.restype = C.c_int
        self.lib.ib_pq_lm_head_topk.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]
        x = d["x"][0]
        fn = lambda: self.lib.ib_pq_lm_head_topk(C.byref(t), x.ctypes.data, k_top, logits.ctypes.data, ids.ctypes.data)
        assert fn() == 0
        tt, reps = _time_calls(fn, 1.5)
        return self._base(algo_bytes / tt / 1e9, "GB/s", f"best of {reps}: ib_pq_lm_head_topk (one thread: the reference's top-K head has no pooled form)", cores=1)

    def kmeans_assign(self, N, D, K):
        if self.kind != "reference":
            return None
        rng = np.random.default_rng(1234)
        X = (rng.standard_normal((N, D)) * 0.02).astype(np.float32)
        Cn = X[:K].copy()
        idx = np.empty(N, np.int32)
        tt, reps = _time_calls(lambda: self.lib.ib_kmeans_assign(X.ctypes.data, N, D, Cn.ctypes.data, K, idx.ctypes.data, self.pool), 2.0, 2, 5)
        return self._base(N / tt / 1e6, "Mpoints/s", f"best of {reps}: ib_kmeans_assign on {N} points with the pool (the assignment is all but the whole of an iteration; "
                          "the reference's update loop sits inside ib_kmeans_fit, which cannot take initial centroids)")

    def decode(self, B):
        """tokens/s of the reference's own inferbit_forward (B == 1) / ib_forward_positions (B > 1) on 7B-shape IBF-v1 files
        of one and of two layers, extrapolated to 32 layers: t32 = t1 + 31 (t2 - t1). IB_W4A8=0 is set at process start."""
        if self.kind != "reference":
            return None
        import tempfile
        sys.path.insert(0, ROOT)
        from oracle import ibf_writer
        L = self.lib
        L.inferbit_config_create.restype = C.c_void_p
        L.inferbit_config_set_threads.argtypes = [C.c_void_p, C.c_int]
        L.inferbit_load.restype = C.c_void_p; L.inferbit_load.argtypes = [C.c_char_p, C.c_void_p]
        L.inferbit_free.argtypes = [C.c_void_p]
        L.inferbit_forward.restype = C.c_int; L.inferbit_forward.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int]
        L.ib_forward_positions.restype = C.c_int; L.ib_forward_positions.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
        L.inferbit_kv_clear.argtypes = [C.c_void_p]
        H, I, V, kv = 4096, 14336, 32000, 1024
        rng = np.random.default_rng(7)
        f16 = lambda a: np.asarray(a, np.float32).astype(np.float16).view(np.uint16)

        def lin(M, N, bits):
            w = rng.integers(0, 256, (M, N if bits == 8 else N // 2), dtype=np.uint8)
            lo = 0.001 if bits == 8 else 0.002
            return (w.view(np.int8) if bits == 8 else w), f16(rng.uniform(lo * 0.05, lo * 0.5, M)), M, N, bits
        shapes = [(H, H, 8), (kv, H, 8), (kv, H, 8), (H, H, 8), (I, H, 4), (I, H, 4), (H, I, 4)]
        layers = [([lin(*sh) for sh in shapes], (f16(rng.uniform(0.9, 1.1, H)), f16(rng.uniform(0.9, 1.1, H)))) for _ in range(2)]
        head = lin(V, H, 8)
        emb = (rng.integers(-127, 128, (V, H), dtype=np.int8), f16(rng.uniform(0.001, 0.01, V)), f16(rng.uniform(0.9, 1.1, H)))
        times = []
        with tempfile.TemporaryDirectory() as d:
            for nl in (1, 2):
                cfg = dict(hidden=H, inter=I, n_layers=nl, n_heads=32, n_kv_heads=8, head_dim=128, vocab=V, max_ctx=64, eps=1e-5, theta=10000.0, attn_bits=8, mlp_bits=4)
                path = os.path.join(d, f"l{nl}.ibf")
                ibf_writer.write_ibf(path, cfg, layers[:nl], head, emb, name="bench-7b-shape")
                c = L.inferbit_config_create()
                L.inferbit_config_set_threads(c, self.threads)
                m = L.inferbit_load(path.encode(), c)
                assert m, "reference inferbit_load failed"
                toks = (np.arange(B, dtype=np.int32) * 7 + 11)
                logits = np.empty((B, V), np.float32)

                def step():
                    L.inferbit_kv_clear(m)
                    if B == 1:
                        assert L.inferbit_forward(m, toks.ctypes.data, 1, logits.ctypes.data, V) == 0
                    else:
                        assert L.ib_forward_positions(m, toks.ctypes.data, B, logits.ctypes.data) == 0
                tt, reps = _time_calls(step, 1.5, 2, 10)
                times.append(tt)
                L.inferbit_free(m)
        t32 = times[0] + 31 * (times[1] - times[0])
        return self._base(B / t32, "tok/s", f"inferbit_forward / ib_forward_positions of the unmodified reference on 1- and 2-layer 7B-shape files at positions 0..{B - 1} "
                          f"({times[0] * 1e3:.1f} / {times[1] * 1e3:.1f} ms per step), extrapolated to 32 layers; attention over 512 cached positions would add under 2 %")


def bench_config(n_gpus):
    """the same dictionary in both arms: what is measured, not how"""
    return {"workload": "int8_attn_proj_b1", "shapes": "q,o 4096x4096; k,v 1024x4096", "batch": 1, "bytes_per_step": STEP_BYTES,
            "l2": "inputs larger than the cache: consecutive steps walk a ring of distinct weight sets",
            "parallelism": "1 GPU" if n_gpus == 1 else f"rows/{n_gpus} + all-gather"}


def run_reference(args, rank):
    if rank != 0:
        return
    cpu = CpuBaseline()
    steps = max(1, min(args.steps, 200))
    dt, gbs = cpu.time_steps(steps, max(3, min(args.warmup, 10)))
    line = {"impl": "reference", "metric": "int8_matvec_weight_GBps", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
            "steps": steps, "warmup": max(3, min(args.warmup, 10)), "ms_per_step": dt * 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "int8 weights x f32 activations, f32 accumulate",
            "data": "synthetic", "config": bench_config(args.gpus),
            "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cpu.threads, "kind": cpu.kind,
                             "sample": f"{steps} steps of q,k,v,o over a ring of 4 host-resident weight sets (168 MB)"},
            "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ── GPU arm ─────────────────────────────────────────────────────────────────────────────
def dist_setup(n):
    rank = int(os.environ.get("RANK", "0")); world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("gloo", rank=rank, world_size=world)
        return rank, world, local, dist
    return rank, world, local, None


# dram__bytes_read.sum + dram__bytes_write.sum of one captured INT8 4096x4096 launch over its weight bytes
# (the ncu summary of this kernel kept under profiles/); traffic grows with the rows streamed, so a step scales by bytes
NCU_TRAFFIC_PER_ALGORITHMIC_BYTE = 16.873472e6 / 16.777216e6


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=50)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-other", action="store_true", help="skip the secondary configurations")
    ap.add_argument("--case", default=None, help="run one small secondary case alone (for profiler captures): "
                    "int8_4096x4096_b1, int8_4096x4096_b16, int8_32000x4096_b1, int4_14336x4096_b1, int4_5632x2048_b1, pq_4096x14336_b1, pq_4096x14336_b8, pq_topk_32000x4096_k64, int4g_4096x4096_g128_b1, int4g_14336x4096_g128_b1, "
                    "kmeans_4Mx8_k256, decode_7b_b1, decode_7b_b1_eager (launches issued one by one, for per-kernel profiles)")
    args = ap.parse_args()
    rank, world, local, dist = dist_setup(args.gpus)
    os.environ.setdefault("IB_W4A8", "0")                    # the reference reads it once: INT4 layers on FP32 activations, as configured
    if args.impl == "reference":
        run_reference(args, rank)
        return
    from libinferbit_b200 import _ffi, LinearT
    from libinferbit_b200 import bench_support as bs
    lib = _ffi.load_ibcu()
    host = _ffi.load_host()
    if lib.ibcu_device_count() < 1:
        raise SystemExit("bench.py needs a B200: no CUDA device is visible and there is no CPU path")
    assert host.ib_b200_init(local) == 0, host.ib_b200_last_error()
    ctx = host.ib_b200_ctx()
    if world > 1:
        import torch
        idbuf = torch.zeros(128, dtype=torch.uint8)
        if rank == 0:
            raw = (C.c_ubyte * 128)(); assert lib.ibcu_comm_get_id(raw) == 0
            idbuf = torch.tensor(list(raw), dtype=torch.uint8)
        dist.broadcast(idbuf, 0)
        raw = (C.c_ubyte * 128)(*idbuf.tolist())
        assert lib.ibcu_comm_init(ctx, raw, rank, world) == 0, lib.ibcu_last_error(ctx)
        if not os.environ.get("IB_BENCH_NCCL_ONLY"):
            # peer window: every rank maps the others' slab, gathers become pushes over NVLink. If any rank
            # cannot create or map a window, every rank stays on NCCL.
            mine = (C.c_ubyte * 64)()
            ok = lib.ibcu_window_create(ctx, 96 << 20, mine) == 0
            allh = [torch.zeros(64, dtype=torch.uint8) for _ in range(world)]
            dist.all_gather(allh, torch.tensor(list(mine), dtype=torch.uint8))
            for r in range(world):
                if ok and r != rank:
                    ok = lib.ibcu_window_open(ctx, r, (C.c_ubyte * 64)(*allh[r].tolist())) == 0
            flag = torch.tensor([1 if ok else 0], dtype=torch.int32)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            if int(flag.item()) == 0:
                lib.ibcu_clear_error(ctx)
                lib.ibcu_window_enable(ctx, 0)
                os.environ["IB_BENCH_NCCL_ONLY"] = "window unavailable"
            dist.barrier()
    if args.case:
        sync = lambda: bs.check(lib, ctx, lib.ibcu_sync(ctx))
        cases = {
            "int8_4096x4096_b1": lambda: bs._linear_ring(lib, ctx, 8, 4096, 4096, 1, reps_target_bytes=300e6),
            "int8_32000x4096_b1": lambda: bs._linear_ring(lib, ctx, 8, 32000, 4096, 1, reps_target_bytes=400e6),
            "int4_14336x4096_b1": lambda: bs._linear_ring(lib, ctx, 4, 14336, 4096, 1, reps_target_bytes=300e6),
            "w4a8_14336x4096_b1": lambda: bs._w4a8_ring(lib, ctx, 14336, 4096, 1),
            "w4a8_4096x14336_b1": lambda: bs._w4a8_ring(lib, ctx, 4096, 14336, 1),
            "w4a8_14336x4096_b8": lambda: bs._w4a8_ring(lib, ctx, 14336, 4096, 8),
            "int4_28672x4096_b8": lambda: bs._linear_ring(lib, ctx, 4, 28672, 4096, 8, reps_target_bytes=400e6, tcgen05=-1),
            "int4_28672x4096_b8_tcgen05": lambda: bs._linear_ring(lib, ctx, 4, 28672, 4096, 8, reps_target_bytes=400e6, tcgen05=1),
            "int8_32000x4096_b8": lambda: bs._linear_ring(lib, ctx, 8, 32000, 4096, 8, reps_target_bytes=400e6, tcgen05=-1),
            "int8_32000x4096_b8_tcgen05": lambda: bs._linear_ring(lib, ctx, 8, 32000, 4096, 8, reps_target_bytes=400e6, tcgen05=2),
            "int8_4096x4096_b16_tcgen05": lambda: bs._linear_ring(lib, ctx, 8, 4096, 4096, 16, reps_target_bytes=300e6, tcgen05=2),
            "int8_4096x4096_b16": lambda: bs._linear_ring(lib, ctx, 8, 4096, 4096, 16, reps_target_bytes=300e6),
            "int4_5632x2048_b1": lambda: bs._linear_ring(lib, ctx, 4, 5632, 2048, 1, reps_target_bytes=300e6),
            "pq_4096x14336_b1": lambda: bs._pq(lib, ctx, 4096, 14336, 16, 256, 1),
            "pq_4096x14336_b8": lambda: bs._pq(lib, ctx, 4096, 14336, 16, 256, 8),
            "int4g_4096x4096_g128_b1": lambda: bs._int4g(lib, ctx, 4096, 4096, 128),
            "int4g_14336x4096_g128_b1": lambda: bs._int4g(lib, ctx, 14336, 4096, 128),
            "pq_topk_32000x4096_k64": lambda: bs._pq_topk(lib, ctx, 32000, 4096, 16, 256, 16, 64),
            "kmeans_4Mx8_k256": lambda: bs._kmeans(lib, ctx, 0, 1, lambda v: v, sync, iters=2),
            "decode_7b_b1": lambda: bs._decode(lib, host, ctx, 1, 0, 1, lambda v: v, sync, steps=3),
            "decode_7b_b8": lambda: bs._decode(lib, host, ctx, 8, 0, 1, lambda v: v, sync, steps=3),
            "decode_7b_b8_eager": lambda: bs._decode(lib, host, ctx, 8, 0, 1, lambda v: v, sync, steps=3, warm=4, graph=False),
            "decode_7b_b1_eager": lambda: bs._decode(lib, host, ctx, 1, 0, 1, lambda v: v, sync, steps=3, warm=4, graph=False),
        }
        print(json.dumps({"case": args.case, **cases[args.case]()}), flush=True)
        host.ib_b200_shutdown()
        return
    W = max(3, args.warmup)
    K = max(1, args.steps)

    def barrier():
        bs.check(lib, ctx, lib.ibcu_sync(ctx))
        if dist is not None:
            dist.barrier()

    def max_over_ranks(v):
        if dist is None:
            return v
        import torch
        t = torch.tensor([v], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    wl = bs.AttnProjWorkload(lib, ctx, rank, world, RING, PROJ, B=1)
    # device-resident timing: graphs of 100 steps each, replayed
    per_graph = 100 if K >= 100 else K
    n_replay = (K + per_graph - 1) // per_graph
    K = per_graph * n_replay
    gid = wl.capture(per_graph)
    launches_per_graph = wl.graph_launches               # kernels of this library recorded into the graph
    for _ in range((W + per_graph - 1) // per_graph):
        wl.replay(gid)
    barrier()
    with ClockSampler(local) as clk:
        lib.ibcu_event_record(ctx, 0)
        for _ in range(n_replay):
            wl.replay(gid)
        lib.ibcu_event_record(ctx, 1)
        ms = C.c_float()
        bs.check(lib, ctx, lib.ibcu_event_elapsed_ms(ctx, 0, 1, C.byref(ms)))
        barrier()
        # keep the GPU under the same load a little longer so that the clock sampler gets a few
        # readings on short runs; the number of extra replays is agreed between the ranks (a time-based
        # loop would issue different numbers of collectives per rank and deadlock)
        t_graph = max_over_ranks(ms.value / n_replay)
        extra = 0 if ms.value >= 400 else min(20000, int(500.0 / max(t_graph, 1e-3)))
        for _ in range(extra):
            wl.replay(gid)
        barrier()
    t_step = max_over_ranks(ms.value / K) * 1e-3
    value = STEP_BYTES / t_step / 1e9
    mma_launches_per_step = 2
    # the same region five more times: how much one event pair scatters (value above is the first, timed as the contract says)
    repeats = []
    for _ in range(5):
        lib.ibcu_event_record(ctx, 4)
        for _ in range(n_replay):
            wl.replay(gid)
        lib.ibcu_event_record(ctx, 5)
        r_ms = C.c_float()
        bs.check(lib, ctx, lib.ibcu_event_elapsed_ms(ctx, 4, 5, C.byref(r_ms)))
        repeats.append(max_over_ranks(r_ms.value / K))
        barrier()
    single = wl.matches_single_gpu() if world > 1 else None
    # end to end through the reference-shaped table: host buffers, copies inside the timed region
    e2e = wl.time_table_calls(host, min(K, 300), W)
    e2e_t = max_over_ranks(e2e["t_step"])
    peaks = bs.load_peaks(ROOT)
    line = {
        "metric": "int8_matvec_weight_GBps", "value": value, "unit": "GB/s", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": t_step * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "int8 weights x int8 limbs of 32-bit fixed-point activations, s32 accumulate (exact); f32 in/out",
        "data": "synthetic",
        "config": bench_config(world),
        "timing": {"ring": f"{RING} distinct weight sets ({RING * STEP_BYTES >> 20} MiB) > L2", "steps_per_graph": per_graph,
                   "transport": ("NCCL all-gather" if os.environ.get("IB_BENCH_NCCL_ONLY") else "push all-gather over peer memory (NVLink)") if world > 1 else None,
                   "repeat_ms_per_step": repeats, "median_ms_per_step": sorted(repeats)[len(repeats) // 2], "min_ms_per_step": min(repeats)},
        "clocks": clk.summary(),
        "gpu_launches": int(launches_per_graph * n_replay),
        "e2e": {"value": STEP_BYTES / e2e_t / 1e9, "unit": "GB/s", "h2d_bytes_per_step": e2e["h2d"], "d2h_bytes_per_step": e2e["d2h"],
                "ms_per_step": e2e_t * 1e3, "api": "ib_kernels table: matmul_int8 x4 with host buffers"},
        "roofline": {"bound": "hbm", "achieved": value / world, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": value / world / peaks["hbm_gbs"], "traffic": NCU_TRAFFIC_PER_ALGORITHMIC_BYTE * STEP_BYTES / world,
                     "peak_source": peaks["source"],
                     "kernel": "linear_mma_kernel<8,...>", "launches_per_step": mma_launches_per_step,
                     "note": "achieved = algorithmic bytes of a step / device time of a step, both launches of the step together; "
                             "traffic = DRAM bytes of a step, scaled from the ncu capture of one 4096x4096 launch "
                             "(16.873 MB read + 0 written for 16.777 MB of weights; the 32000x4096 launch gives the same ratio)"},
    }
    if single is not None:
        line["matches_single_gpu"] = single
    cpu = None
    if rank == 0 and world == 1:
        cpu = CpuBaseline()
        dt, gbs = cpu.time_steps(60, 5)
        line["cpu_baseline"] = {"value": gbs, "unit": "GB/s", "cores": cpu.threads, "kind": cpu.kind,
                                "sample": "60 steps of q,k,v,o over a ring of 4 host-resident weight sets"}
    if not args.no_other:
        other = bs.other_configs(lib, host, ctx, rank, world, dist, max_over_ranks, barrier, peaks)
        if cpu is not None:
            # the reference's own entry point for each configuration, timed here on the host cores (a reported baseline)
            for name, e in other.items():
                if not isinstance(e, dict):
                    continue
                try:
                    if name.startswith("int4_group"):
                        e["cpu_baseline"] = None              # the reference has this matvec only as static functions of its session engine
                    elif name.startswith("pq_topk_"):
                        sh = e["shape"]; e["cpu_baseline"] = cpu.pq_topk(sh["M"], sh["N"], sh["G"], sh["K"], sh["K_l2"], sh["K_top"], e["algorithmic_bytes"])
                    elif name.startswith("w4a8_"):
                        sh = e["shape"]; e["cpu_baseline"] = cpu.w4a8(sh["M"], sh["N"], sh["B"], e["algorithmic_bytes"])
                    elif name.startswith(("int4_", "int8_")):
                        sh = e["shape"]; e["cpu_baseline"] = cpu.linear(sh["bits"], sh["M"], sh["N"], sh["B"], e["algorithmic_bytes"])
                    elif name.startswith("pq_"):
                        sh = e["shape"]; e["cpu_baseline"] = cpu.pq(sh["M"], sh["N"], sh["G"], sh["K"], sh["B"], e["algorithmic_bytes"])
                    elif name.startswith("kmeans_"):
                        e["cpu_baseline"] = cpu.kmeans_assign(e["points"], e["D"], e["K"])
                    elif name.startswith("decode_7b_b") and "nccl" not in name:
                        e["cpu_baseline"] = cpu.decode(e["batch"])
                except Exception as ex:                        # a baseline that cannot be taken must not cost the GPU numbers
                    e["cpu_baseline"] = {"error": repr(ex)[:200]}
        line["other"] = other
    wl.close()
    if rank == 0:
        print(json.dumps(line), flush=True)
    host.ib_b200_shutdown()
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
