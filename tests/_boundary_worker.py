"""Child process of tests/test_boundary_gpu.py: the UNMODIFIED reference (oracle/_ref/libinferbit_ref.so)
loads the seeded mini model with its own inferbit_load, runs its own inferbit_forward on its CPU table,
then the GPU table is installed into the reference's exported global ib_kern (after the load, because
ibf_load re-initialises it, src/ibf_loader.c:538-540), the model's weight mapping is registered, and the
same inferbit_forward calls run again: every linear layer, RMSNorm, RoPE, softmax and SiLU of the
reference's forward pass now goes through ib_b200_* on the GPU. Prints one JSON line.

argv: <threads> <IB_W4A8 value>"""
import ctypes as C
import json
import os
import sys
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    threads, w4a8 = int(sys.argv[1]), sys.argv[2]
    os.environ["IB_W4A8"] = w4a8                      # read once by the reference (src/forward.c:14-21)
    from libinferbit_b200 import _ffi
    from tests import _cpu
    from tests.golden import ibf_model
    libs = _cpu.load()
    r = libs.ref
    assert r is not None, "oracle/_ref/libinferbit_ref.so missing"
    host = _ffi.load_host()
    r.inferbit_config_create.restype = C.c_void_p
    r.inferbit_config_set_threads.argtypes = [C.c_void_p, C.c_int]
    r.inferbit_load.restype = C.c_void_p; r.inferbit_load.argtypes = [C.c_char_p, C.c_void_p]
    r.inferbit_free.argtypes = [C.c_void_p]
    r.inferbit_forward.restype = C.c_int; r.inferbit_forward.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int]
    r.inferbit_kv_clear.argtypes = [C.c_void_p]
    r.inferbit_last_error.restype = C.c_char_p
    V = ibf_model.CFG["vocab"]
    toks = np.random.default_rng(5).integers(0, V, 6).astype(np.int32)
    out = {"threads": threads, "w4a8": w4a8}
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "mini.ibf")
        ibf_model.write_ibf(path)
        cfg = r.inferbit_config_create()
        r.inferbit_config_set_threads(cfg, threads)
        m = r.inferbit_load(path.encode(), cfg)
        assert m, r.inferbit_last_error()

        def run():
            r.inferbit_kv_clear(m)
            lg = np.empty((len(toks) + 1, V), np.float32)
            for i in range(len(toks)):
                assert r.inferbit_forward(m, _cpu.p(toks[i:i + 1]), 1, _cpu.p(lg[i]), V) == 0, r.inferbit_last_error()
            r.inferbit_kv_clear(m)                    # and the prompt in one call (last logits only)
            assert r.inferbit_forward(m, _cpu.p(toks), len(toks), _cpu.p(lg[-1]), V) == 0, r.inferbit_last_error()
            return lg
        cpu = run()
        # the model's weight mapping: the whole file is mapped (src/ibf_loader.c:471), found here through
        # /proc/self/maps; a C integration passes model->weight_data and model->weight_data_size instead
        base = size = None
        for line in open("/proc/self/maps"):
            if line.rstrip().endswith(path):
                a, b = (int(v, 16) for v in line.split()[0].split("-"))
                base = a if base is None else min(base, a)
                size = b - base
        assert base, "weight mapping not found"
        size = min(size, os.path.getsize(path))
        assert host.ib_b200_init(0) == 0, host.ib_b200_last_error()
        assert host.ib_b200_register(base, size) == 0, host.ib_b200_last_error()
        before = _ffi.load_ibcu().ibcu_launch_count(host.ib_b200_ctx())
        host.ib_b200_install_kernels(C.addressof(libs.ref_kern))      # the reference's own global table
        gpu = run()
        out["launches"] = int(_ffi.load_ibcu().ibcu_launch_count(host.ib_b200_ctx()) - before)
        out["status"] = host.ib_b200_status()
        if out["status"]:
            out["error"] = host.ib_b200_last_error().decode()
        scale = float(np.abs(cpu).max())
        out["max_abs_diff"] = float(np.max(np.abs(gpu - cpu)))
        out["scale"] = scale
        out["close"] = bool(np.all(np.abs(gpu.astype(np.float64) - cpu) <= 2e-4 * max(1.0, scale) + 2e-3 * np.abs(cpu)))
        out["finite"] = bool(np.isfinite(gpu).all())
        r.ib_init_kernels(r.ib_detect_simd())         # hand the table back before the model goes
        r.inferbit_free(m)
        host.ib_b200_unregister(base)
        host.ib_b200_shutdown()
    print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
