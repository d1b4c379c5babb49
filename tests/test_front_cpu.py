"""The reference-named front (libinferbit.so, include/inferbit_gpu.h) on the CPU: configuration, the
error paths of inferbit_load that the reference's own loader tests walk (tests/test_ibf_loader.c:169-304:
wrong extension, file too small, bad magic) plus malformed headers, and - where the unmodified
reference was built - that it refuses the same files. With a valid file and no GPU the load fails with an
error: there is no CPU path."""
import ctypes as C
import json
import os
import struct

import pytest

from libinferbit_b200 import _ffi
from tests.golden import ibf_model


@pytest.fixture(scope="module")
def front():
    return _ffi.load_front()


def _err(front):
    e = front.inferbit_last_error()
    return e.decode() if e else None


def _write(path, header_bytes, version=1, magic=b"INFERBIT", declared=None, tail=b""):
    with open(path, "wb") as f:
        f.write(magic + struct.pack("<III", version, len(header_bytes) if declared is None else declared, 0) + bytes(12))
        f.write(header_bytes)
        f.write(tail)


def test_config_and_null_safety(front):
    cfg = front.inferbit_config_create()
    assert cfg
    front.inferbit_config_set_threads(cfg, 16)
    front.inferbit_config_set_context_length(cfg, 32)
    front.inferbit_config_set_kv_cache_dynamic(cfg, 1)
    front.inferbit_config_set_native_bits(cfg, 8)
    front.inferbit_config_free(cfg)
    assert _err(front) is None                                         # nothing pending
    assert front.inferbit_kv_length(None) == 0
    front.inferbit_kv_clear(None); front.inferbit_kv_truncate(None, 3); front.inferbit_free(None)
    assert front.inferbit_model_architecture(None) == b"unknown"
    assert front.inferbit_model_num_layers(None) == 0 and front.inferbit_model_total_memory(None) == 0
    assert front.inferbit_forward(None, None, 1, None, 10) == -5       # INFERBIT_ERROR_PARAM
    assert "NULL argument" in _err(front)
    assert _err(front) is None                                         # read-once
    assert front.inferbit_load(None, None) is None and "NULL" in _err(front)


def test_load_refuses_what_the_reference_refuses(front, tmp_path, cpu_libs):
    cases = {}
    p = str(tmp_path / "model.safetensors"); cases["ext"] = (p, ".ibf")
    p = str(tmp_path / "small.ibf"); open(p, "wb").write(b"INF"); cases["small"] = (p, "too small")
    p = str(tmp_path / "magic.ibf"); open(p, "wb").write(b"NOTVALID" + bytes(56)); cases["magic"] = (p, "magic")
    p = str(tmp_path / "version.ibf"); _write(p, b"{}", version=9); cases["version"] = (p, "version")
    p = str(tmp_path / "hsize.ibf"); _write(p, b"{}", declared=10_000); cases["hsize"] = (p, "header size")
    p = str(tmp_path / "json.ibf"); _write(p, b'{"architecture": {"num_layers": 2,, }'); cases["json"] = (p, "JSON")
    p = str(tmp_path / "fields.ibf"); _write(p, json.dumps({"architecture": {"num_layers": 0, "num_heads": 4}}).encode()); cases["fields"] = (p, "required")
    p = str(tmp_path / "missing.ibf"); cases["missing"] = (p, "failed to open")
    ref = cpu_libs.ref
    if ref is not None:
        ref.inferbit_load.restype = C.c_void_p; ref.inferbit_load.argtypes = [C.c_char_p, C.c_void_p]
        ref.inferbit_last_error.restype = C.c_char_p
    for name, (path, needle) in cases.items():
        assert front.inferbit_load(path.encode(), None) is None, name
        msg = _err(front)
        assert msg and needle in msg, (name, msg)
        if ref is not None:
            assert ref.inferbit_load(path.encode(), None) is None, name
            rmsg = ref.inferbit_last_error()
            assert rmsg and needle in rmsg.decode(), (name, rmsg)
    cfg = front.inferbit_config_create()
    front.inferbit_config_set_native_parse(cfg, 1)
    assert front.inferbit_load(b"x.ibf", cfg) is None and "native parse" in _err(front)
    front.inferbit_config_free(cfg)


def _mini_with(tmp_path, name, edit):
    """the seeded mini model's file with its JSON header edited"""
    src = str(tmp_path / "mini_src.ibf")
    ibf_model.write_ibf(src)
    raw = open(src, "rb").read()
    hs = struct.unpack("<I", raw[12:16])[0]
    hdr = json.loads(raw[32:32 + hs])
    data_off = (32 + hs + 63) & ~63
    edit(hdr)
    js = json.dumps(hdr).encode()
    out = str(tmp_path / name)
    with open(out, "wb") as f:
        f.write(b"INFERBIT" + struct.pack("<III", 1, len(js), 0) + bytes(12) + js)
        f.write(bytes((-(32 + len(js))) % 64))
        f.write(raw[data_off:])
    return out


def test_load_refuses_formats_outside_the_path(front, tmp_path):
    def kv8(h): h["kv_cache"]["bits"] = 8
    def tern(h): h["layers"][1]["weights"]["up_proj"]["bits"] = 2
    def gelu(h): h["architecture"]["activation"] = "gelu"
    def oob(h): h["layers"][0]["weights"]["q_proj"]["offset"] = 10 ** 9
    def few(h): h["layers"] = h["layers"][:1]
    for name, edit, needle in (("kv8.ibf", kv8, "kv_bits=8"), ("tern.ibf", tern, "2 bits"), ("gelu.ibf", gelu, "gelu"), ("few.ibf", few, "layers")):
        assert front.inferbit_load(_mini_with(tmp_path, name, edit).encode(), None) is None
        assert needle in _err(front), name
    if _ffi.load_ibcu().ibcu_device_count() > 0:
        assert front.inferbit_load(_mini_with(tmp_path, "oob.ibf", oob).encode(), None) is None
        assert "outside the weight data" in _err(front)


def test_valid_file_without_a_gpu_is_an_error_not_a_fallback(front, tmp_path):
    if _ffi.load_ibcu().ibcu_device_count() > 0:
        pytest.skip("a GPU is visible: covered by the gpu tests")
    path = str(tmp_path / "mini.ibf")
    ibf_model.write_ibf(path)
    assert front.inferbit_load(path.encode(), None) is None
    assert "no usable B200" in _err(front)
