"""World-size-2 runs of the multi-GPU host logic on CPU (gloo): the row-shard plan the CUDA library
uses (ibcu_shard_rows) with an all-gather of row-sharded linear outputs, and the k-means exchange
(all-reduce of per-rank sums and counts, redundant centroid update). The arithmetic on each rank is
the CPU restatement; what is under test is the partitioning and the exchange pattern."""
import ctypes as C
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    from libinferbit_b200 import _ffi
    from tests import _cpu
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    lib = _ffi.load_ibcu(); o = _cpu.load().oracle
    ok = True
    # ── row-sharded INT8 linear + all-gather (shards of unequal size: 100 rows, 32-row units) ──
    rng = np.random.default_rng(5)                                  # same data on every rank
    for M, N, B in ((100, 256, 2), (1024, 512, 1)):
        w, s16, x = _cpu.make_int8_case(rng, M, N, B)
        s = np.empty(M, np.float32); o.ibo_fp16_array_to_fp32(s16, s, M)
        full = np.empty((B, M), np.float32); o.ibo_matmul_int8_batch(full, w, s, x, M, N, B, M)
        r0, rn = C.c_int(), C.c_int()
        lib.ibcu_shard_rows(M, world, rank, 32, C.byref(r0), C.byref(rn))
        r0, rn = r0.value, rn.value
        buf = np.zeros((B, M), np.float32)
        if rn:
            part = np.empty((B, rn), np.float32)
            o.ibo_matmul_int8_batch(part, np.ascontiguousarray(w[r0:r0 + rn]), np.ascontiguousarray(s[r0:r0 + rn]), x, rn, N, B, rn)
            buf[:, r0:r0 + rn] = part
        # the exchange: every rank broadcasts its slice of every activation row (ragged all-gather)
        for r in range(world):
            q0, qn = C.c_int(), C.c_int()
            lib.ibcu_shard_rows(M, world, r, 32, C.byref(q0), C.byref(qn))
            if qn.value:
                t = torch.from_numpy(np.ascontiguousarray(buf[:, q0.value:q0.value + qn.value]))
                dist.broadcast(t, r)
                buf[:, q0.value:q0.value + qn.value] = t.numpy()
        ok &= bool(np.array_equal(buf, full))
    # ── k-means: points sharded, sums / counts all-reduced, update on every rank ──
    N, D, K = 20000, 8, 64
    X = (rng.standard_normal((N, D)) * 0.02).astype(np.float32); C0 = X[:K].copy()
    ref_C = C0.copy(); idx = np.empty(N, np.int32); sums = np.empty((K, D), np.float32); cnt = np.empty(K, np.int32); ine = C.c_double()
    o.ibo_kmeans_lloyd_iter(X, N, D, ref_C, K, idx, sums, cnt, C.byref(ine), 2)
    n0, n1 = N * rank // world, N * (rank + 1) // world
    Xs = np.ascontiguousarray(X[n0:n1]); Cs = C0.copy()
    li = np.empty(n1 - n0, np.int32); ls = np.empty((K, D), np.float32); lc = np.empty(K, np.int32); lin = C.c_double()
    tmpC = C0.copy()
    o.ibo_kmeans_lloyd_iter(Xs, n1 - n0, D, tmpC, K, li, ls, lc, C.byref(lin), 2)    # local assign + accumulate
    ts, tc, ti = torch.from_numpy(ls), torch.from_numpy(lc), torch.tensor([lin.value], dtype=torch.float64)
    dist.all_reduce(ts); dist.all_reduce(tc); dist.all_reduce(ti)
    o.ibo_kmeans_update(Cs, K, D, ls, lc)
    ok &= bool(np.array_equal(li, idx[n0:n1])) and bool(np.array_equal(lc, cnt))
    ok &= bool(np.allclose(Cs, ref_C, rtol=1e-5, atol=1e-7)) and abs(float(ti[0]) - ine.value) <= 1e-9 * ine.value
    # every rank ends with the same centroids
    tC = torch.from_numpy(Cs.copy()); dist.broadcast(tC, 0)
    ok &= bool(np.array_equal(tC.numpy(), Cs))
    q.put((rank, ok))
    dist.destroy_process_group()


def test_two_ranks_gloo():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p_ in procs:
        p_.start()
    res = sorted(q.get(timeout=120) for _ in procs)
    for p_ in procs:
        p_.join(timeout=60)
    assert res == [(0, True), (1, True)]
