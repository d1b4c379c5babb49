"""The C ABI loads without a GPU and exports every symbol its header declares."""
import ctypes as C
import os
import re

from libinferbit_b200 import _ffi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared(header):
    txt = open(os.path.join(ROOT, "include", header)).read()
    txt = re.sub(r"/\*.*?\*/", "", txt, flags=re.S)
    return sorted(set(re.findall(r"\b((?:ibcu|ib_b200)_[a-z0-9_]+)\s*\(", txt)))


def test_libibcu_exports_every_declared_symbol():
    lib = _ffi.load_ibcu()
    names = declared("ibcu.h")
    assert len(names) > 40
    for n in names:
        assert hasattr(lib, n), n
    assert sorted(_ffi.IBCU_SYMBOLS) == names          # the Python prototypes cover the header exactly


def test_libib_b200_exports_every_declared_symbol():
    lib = _ffi.load_host()
    names = [n for n in declared("ib_b200.h") if n.startswith("ib_b200_")]
    assert len(names) > 30
    for n in names:
        assert hasattr(lib, n), n
    assert sorted(_ffi.HOST_SYMBOLS) == names


def test_libinferbit_front_exports_every_declared_symbol():
    lib = _ffi.load_front()
    txt = open(os.path.join(ROOT, "include", "inferbit_gpu.h")).read()
    txt = re.sub(r"/\*.*?\*/", "", txt, flags=re.S)
    names = sorted(set(re.findall(r"\b((?:inferbit|ib_pq)_[a-z0-9_]+)\s*\(", txt)))
    assert len(names) >= 30 and "ib_pq_load_multi" in names
    for n in names:
        assert hasattr(lib, n), n
    assert sorted(_ffi.FRONT_SYMBOLS) == names


def test_host_layer_without_gpu_reports_errors():
    import numpy as np
    lib = _ffi.load_host()
    if _ffi.load_ibcu().ibcu_device_count() > 0:
        return
    assert lib.ib_b200_init(0) != 0
    assert b"no usable" in lib.ib_b200_last_error()
    out = np.full(4, 7.0, np.float32); w = np.zeros(64, np.int8); s = np.ones(4, np.float32); x = np.ones(16, np.float32)
    lib.ib_b200_matmul_int8(out.ctypes.data, w.ctypes.data, s.ctypes.data, x.ctypes.data, 4, 16)
    assert lib.ib_b200_status() != 0 and np.all(out == 7.0)          # error recorded, output untouched
    assert b"before ib_b200_init" in lib.ib_b200_last_error()
    assert lib.ib_b200_status() == 0                                  # read-once


def test_no_gpu_means_an_error_not_a_fallback():
    lib = _ffi.load_ibcu()
    if lib.ibcu_device_count() > 0:
        return
    ctx = C.c_void_p()
    assert lib.ibcu_ctx_create(0, C.byref(ctx)) != 0 and not ctx.value


def test_shard_rows_partitions_exactly():
    lib = _ffi.load_ibcu()
    for M in (0, 1, 100, 1024, 4096, 14336, 32000, 32001):
        for world in (1, 2, 3, 4, 8):
            for align in (1, 16, 32):
                nxt = 0
                for r in range(world):
                    r0, rn = C.c_int(), C.c_int()
                    lib.ibcu_shard_rows(M, world, r, align, C.byref(r0), C.byref(rn))
                    assert r0.value == nxt and rn.value >= 0
                    if rn.value and r0.value + rn.value < M:
                        assert rn.value % align == 0
                    nxt += rn.value
                assert nxt == M


def test_hash_fill_host_side_is_position_addressable():
    import numpy as np
    lib = _ffi.load_ibcu()
    a = np.empty(1000, np.uint8); lib.ibcu_hash_bytes_host(a.ctypes.data, 1000, 42, 0)
    b = np.empty(100, np.uint8); lib.ibcu_hash_bytes_host(b.ctypes.data, 100, 42, 333)
    assert np.array_equal(a[333:433], b) and len(set(a.tolist())) > 200
