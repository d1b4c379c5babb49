"""Child process of tests/test_multirank_gpu.py: rank `rank` of `world` on GPU `rank`. The ranks find each other
through files in a shared directory (communicator id, window handles), load the seeded mini model through
ib_b200_model_set_linear (every rank keeps its row slices), run the decode steps of the golden recording - every
linear row-sharded, the slices gathered over the peer window, or over NCCL when argv says so - and print one JSON
line with the largest deviation from the reference's recorded logits.

argv: <rank> <world> <dir> <transport: push|nccl>"""
import ctypes as C
import json
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def _put(path, data):
    with open(path + ".tmp", "wb") as f:
        f.write(bytes(data))
    os.rename(path + ".tmp", path)


def _get(path, timeout=120):
    t0 = time.time()
    while not os.path.exists(path):
        if time.time() - t0 > timeout:
            raise TimeoutError(path)
        time.sleep(0.01)
    return open(path, "rb").read()


def main():
    rank, world, d, transport = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], sys.argv[4]
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    from libinferbit_b200 import _ffi
    from tests import _cpu
    from tests.test_golden import DG, _mini_model, _close_logits
    lib, host = _ffi.load_ibcu(), _ffi.load_host()
    assert host.ib_b200_init(rank) == 0, host.ib_b200_last_error()
    ctx = host.ib_b200_ctx()
    if rank == 0:
        raw = (C.c_ubyte * 128)(); assert lib.ibcu_comm_get_id(raw) == 0
        _put(os.path.join(d, "id"), raw)
    raw = (C.c_ubyte * 128)(*_get(os.path.join(d, "id")))
    assert lib.ibcu_comm_init(ctx, raw, rank, world) == 0, lib.ibcu_last_error(ctx)
    if transport == "push":
        mine = (C.c_ubyte * 64)()
        assert lib.ibcu_window_create(ctx, 8 << 20, mine) == 0, lib.ibcu_last_error(ctx)
        _put(os.path.join(d, f"win{rank}"), mine)
        for r in range(world):
            if r != rank:
                h = (C.c_ubyte * 64)(*_get(os.path.join(d, f"win{r}")))
                assert lib.ibcu_window_open(ctx, r, h) == 0, lib.ibcu_last_error(ctx)
    cfg, (layers, head, (emb, es, fn)) = _mini_model()
    mc = _ffi.ModelCfg(cfg["hidden"], cfg["inter"], cfg["n_layers"], cfg["n_heads"], cfg["n_kv_heads"], cfg["head_dim"], cfg["vocab"],
                       cfg["max_ctx"], cfg["eps"], cfg["theta"], cfg["attn_bits"], cfg["mlp_bits"], cfg["head_bits"])
    m = host.ib_b200_model_create(ctx, C.byref(mc))
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
    worst, ok = 0.0, True
    before = lib.ibcu_launch_count(ctx)
    for i in range(len(toks)):
        assert host.ib_b200_forward_step(m, p(toks[i:i + 1].copy()), i, 1, p(got)) == 0, lib.ibcu_last_error(ctx)
        worst = max(worst, float(np.max(np.abs(got - want[i]))))
        ok = ok and _close_logits(got, want[i])
    n = len(toks)
    gb = np.empty((3, cfg["vocab"]), np.float32)
    assert host.ib_b200_forward_step(m, p(toks[n - 3:].copy()), n - 3, 3, p(gb)) == 0, lib.ibcu_last_error(ctx)
    ok = ok and _close_logits(gb, want[n - 3:])
    launches = int(lib.ibcu_launch_count(ctx) - before)
    host.ib_b200_model_free(m)
    _put(os.path.join(d, f"done{rank}"), b"1")              # nobody tears its window down while a peer may still push
    for r in range(world):
        _get(os.path.join(d, f"done{r}"))
    host.ib_b200_shutdown()
    print(json.dumps({"rank": rank, "ok": bool(ok), "max_abs_diff": worst, "launches": launches, "transport": transport}), flush=True)


if __name__ == "__main__":
    main()
