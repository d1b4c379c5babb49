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


# ── product-quantised model files ("IBF v5"): ib_pq_load_single / ib_pq_load_multi ──
def _v5_cases(tmp_path):
    import numpy as np
    from oracle import ibf_writer
    from tests import _cpu
    rng = np.random.default_rng(77)
    ds = {"layers.0.down": _cpu.make_pq_case_ex(rng, 40, 256, 16, 256, 0, 0, 1),
          "layers.0.gate": _cpu.make_pq_case_ex(rng, 33, 272, 16, 256, 16, 16, 1),      # 4-bit packed second level + outlier columns
          "head": _cpu.make_pq_case_ex(rng, 24, 104, 8, 32, 64, 8, 1)}
    fmts = {"layers.0.down": "pq2d_v1_l1", "layers.0.gate": "pq2d_v1_l1_l2", "head": "pq2d_v1_l1_l2"}
    raws = {"tok_embeddings": rng.standard_normal((7, 5)).astype(np.float16), "norm": rng.standard_normal(11).astype(np.float32),
            "ids": np.arange(6, dtype=np.int32)}
    cfg = {"arch": "llama", "hidden": 256, "rope": {"theta": 10000.5, "scaled": False}, "names": ["a", "b\"c"], "none": None}
    path = os.path.join(str(tmp_path), "m.ibf")
    ibf_writer.write_ibf_v5(path, {k: _cpu.pq_file_tensor(d, fmts[k]) for k, d in ds.items()}, raws, cfg)
    return path, ds, raws, cfg


def _multi_as_dict(m):
    import numpy as np
    from tests import _cpu
    out = {"tensors": {}, "raw": {}, "config": json.loads(m.config_json.decode()) if m.config_json else None}
    for i in range(m.n):
        t = m.tensors[i]
        scal = {f: getattr(t, f) for f in ("M", "N", "G", "K", "K_l2", "n_levels", "rotate", "n_outlier", "format", "C", "l2_idx_bytes", "l2_packed_bits")}
        out["tensors"][m.names[i].decode()] = (scal, _cpu.pq_tensor_arrays(t))
    for i in range(m.n_raw):
        r = m.raw_tensors[i]
        data = np.ctypeslib.as_array(C.cast(r.data, C.POINTER(C.c_uint8)), shape=(r.size_bytes,)).copy()
        out["raw"][r.name.decode()] = (r.dtype, r.ndim, list(r.shape)[:r.ndim], data)
    return out


def _same(a, b):
    import numpy as np
    assert a["config"] == b["config"] and a["tensors"].keys() == b["tensors"].keys() and list(a["tensors"]) == list(b["tensors"])
    for k in a["tensors"]:
        assert a["tensors"][k][0] == b["tensors"][k][0], k
        for key, arr in a["tensors"][k][1].items():
            assert np.array_equal(arr, b["tensors"][k][1][key]), (k, key)
    assert list(a["raw"]) == list(b["raw"])
    for k in a["raw"]:
        assert a["raw"][k][:3] == b["raw"][k][:3] and np.array_equal(a["raw"][k][3], b["raw"][k][3])


def test_pq_file_reader_matches_the_reference(front, tmp_path):
    """ib_pq_load_multi / ib_pq_load_single of this library fill the reference's structs with what the compiled reference's
    own readers produce from the same file (every scalar field, every array, names in file order, raw tensors, config), and
    refuse the files the reference refuses."""
    import numpy as np
    from tests import _cpu
    path, ds, raws, cfg = _v5_cases(tmp_path)
    mine = _cpu.RefPqMulti()
    assert front.ib_pq_load_multi(path.encode(), C.byref(mine)) == 0
    got = _multi_as_dict(mine)
    assert got["config"] == cfg and list(got["tensors"]) == list(ds)
    for name, d in ds.items():                                # against what was written
        scal, arrs = got["tensors"][name]
        assert (scal["M"], scal["N"], scal["G"], scal["K"], scal["K_l2"], scal["n_outlier"], scal["C"]) == (d["M"], d["N"], d["G"], d["K"], d["K_l2"], d["n_outlier"], d["C"])
        assert np.array_equal(arrs["indices_l1_l"], d["idx1_l"].reshape(-1)) and np.array_equal(arrs["row_scale"], d["rs"].reshape(-1))
    for name, a in raws.items():
        assert np.array_equal(got["raw"][name][3], np.frombuffer(a.tobytes(), np.uint8)) and got["raw"][name][2] == list(a.shape)
    ref = _cpu.load().ref
    if ref is not None:
        theirs = _cpu.RefPqMulti()
        assert ref.ib_pq_load_multi(path.encode(), C.byref(theirs)) == 0
        _same(got, _multi_as_dict(theirs))
        ref.ib_pq_multi_free(C.byref(theirs))
    # the single-tensor reader takes the first tensor of the file
    one = _cpu.RefPqTensor()
    assert front.ib_pq_load_single(path.encode(), C.byref(one)) == 0
    first = next(iter(ds))
    assert np.array_equal(_cpu.pq_tensor_arrays(one)["indices_l1_r"], ds[first]["idx1_r"].reshape(-1)) and one.format == 1
    found = front.ib_pq_multi_find(C.byref(mine), b"head")
    assert found and C.cast(found, C.POINTER(_cpu.RefPqTensor)).contents.M == ds["head"]["M"]
    assert not front.ib_pq_multi_find(C.byref(mine), b"nope")
    front.ib_pq_free(C.byref(one))
    assert one.M == 0 and not one._arena
    front.ib_pq_multi_free(C.byref(mine))
    assert mine.n == 0 and not mine.tensors
    # files both refuse: truncated blocks, wrong version, a block of the wrong size, a second level outside {16, 64, K}
    raw = open(path, "rb").read()
    bad = {}
    bad["truncated"] = raw[:len(raw) - 100]
    bad["version"] = raw[:8] + struct.pack("<I", 4) + raw[12:]
    hl = struct.unpack("<I", raw[12:16])[0]
    hdr = json.loads(raw[32:32 + hl].decode())
    h2 = json.loads(json.dumps(hdr)); h2["tensors"]["layers.0.down"]["row_scale"]["size"] += 2
    h3 = json.loads(json.dumps(hdr)); h3["tensors"]["head"]["K_l2"] = 48
    for key, h in (("size", h2), ("k_l2", h3)):
        text = json.dumps(h).encode()
        assert len(text) <= hl
        bad[key] = raw[:32] + text + b" " * (hl - len(text)) + raw[32 + hl:]
    for key, blob in bad.items():
        p = os.path.join(str(tmp_path), key + ".ibf")
        open(p, "wb").write(blob)
        m = _cpu.RefPqMulti()
        assert front.ib_pq_load_multi(p.encode(), C.byref(m)) == -1 and m.n == 0, key
        if ref is not None:
            t = _cpu.RefPqMulti()
            assert ref.ib_pq_load_multi(p.encode(), C.byref(t)) == -1, key
    assert front.ib_pq_load_single(b"/nonexistent/file.ibf", C.byref(one)) == -1 and front.ib_pq_load_single(None, C.byref(one)) == -1
