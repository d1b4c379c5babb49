"""The reference-named front (libinferbit.so) on the GPU: the seeded mini model written as an IBF-v1
file loads through inferbit_load, and inferbit_forward reproduces the logits the unmodified reference
recorded for the same file (tests/golden/decode_ref_logits.npz); prompt batches, KV truncation, the error
codes of src/forward.c:850-871 and a file whose o_proj is stored at the default width."""
import ctypes as C
import os

import numpy as np
import pytest

from libinferbit_b200 import _ffi
from tests import _cpu
from tests.golden import ibf_model
from tests.test_golden import DG, _close_logits

pytestmark = pytest.mark.gpu
p = _cpu.p


@pytest.fixture(scope="module")
def front():
    return _ffi.load_front()


def _err(front):
    e = front.inferbit_last_error()
    return e.decode() if e else None


def test_front_reproduces_reference_forward(front, tmp_path):
    cfg = ibf_model.CFG
    path = str(tmp_path / "mini.ibf")
    ibf_model.write_ibf(path, seed=int(DG["seed"][0]))
    m = front.inferbit_load(path.encode(), None)
    assert m, _err(front)
    assert front.inferbit_model_architecture(m) == b"llama"
    assert front.inferbit_model_num_layers(m) == cfg["n_layers"] and front.inferbit_model_hidden_size(m) == cfg["hidden"]
    assert front.inferbit_model_vocab_size(m) == cfg["vocab"] and front.inferbit_model_max_context(m) == cfg["max_ctx"]
    assert front.inferbit_model_default_bits(m) == cfg["mlp_bits"]
    assert front.inferbit_model_weight_memory(m) > 0
    kvm = cfg["n_layers"] * cfg["max_ctx"] * cfg["n_kv_heads"] * cfg["head_dim"] * 2 * 2
    assert front.inferbit_model_kv_memory(m) == kvm
    assert front.inferbit_model_total_memory(m) == kvm + front.inferbit_model_weight_memory(m)
    assert front.inferbit_kv_length(m) == 0
    toks, want = DG["tokens"], DG["logits"]
    V = cfg["vocab"]
    got = np.empty(V, np.float32)
    for i in range(len(toks)):                                        # one token per call, as the recording was made
        assert front.inferbit_forward(m, p(toks[i:i + 1].copy()), 1, p(got), V) == 0, _err(front)
        assert _close_logits(got, want[i]), (i, float(np.max(np.abs(got - want[i]))))
    assert front.inferbit_kv_length(m) == len(toks)
    # the whole prompt in one call: only the last position's logits come back (src/forward.c:872-901)
    front.inferbit_kv_clear(m)
    assert front.inferbit_kv_length(m) == 0
    assert front.inferbit_forward(m, p(toks.copy()), len(toks), p(got), V) == 0, _err(front)
    assert _close_logits(got, want[-1])
    # truncate to five positions and feed the last three again
    front.inferbit_kv_truncate(m, 5)
    assert front.inferbit_kv_length(m) == 5
    assert front.inferbit_forward(m, p(toks[5:].copy()), 3, p(got), V) == 0
    assert _close_logits(got, want[-1]) and front.inferbit_kv_length(m) == 8
    # errors (src/generate.c:232-239, src/forward.c:851-871)
    assert front.inferbit_forward(m, p(toks), 1, p(got), V + 1) == -5 and "vocab_size mismatch" in _err(front)
    bad = np.array([V], np.int32)
    assert front.inferbit_forward(m, p(bad), 1, p(got), V) == -5 and "out of range" in _err(front)
    assert front.inferbit_forward(m, p(toks), 0, p(got), V) == -5
    _err(front)
    long = np.zeros(cfg["max_ctx"], np.int32)
    assert front.inferbit_forward(m, p(long), len(long), p(got), V) == -4 and "context length exceeded" in _err(front)
    assert front.inferbit_kv_length(m) == 8                           # a refused call leaves the cache as it was
    # more than 32 positions in one call go through in groups; the cache ends full
    front.inferbit_kv_clear(m)
    rng = np.random.default_rng(9)
    prompt = rng.integers(0, V, cfg["max_ctx"]).astype(np.int32)
    assert front.inferbit_forward(m, p(prompt), len(prompt), p(got), V) == 0, _err(front)
    assert front.inferbit_kv_length(m) == cfg["max_ctx"] and np.isfinite(got).all()
    assert front.inferbit_forward(m, p(toks), 1, p(got), V) == -4
    _err(front)
    front.inferbit_free(m)


def test_front_context_length_config(front, tmp_path):
    path = str(tmp_path / "mini.ibf")
    ibf_model.write_ibf(path)
    cfg = front.inferbit_config_create()
    front.inferbit_config_set_context_length(cfg, 16)
    front.inferbit_config_set_threads(cfg, 4)
    m = front.inferbit_load(path.encode(), cfg)
    assert m, _err(front)
    V = ibf_model.CFG["vocab"]
    got = np.empty(V, np.float32)
    toks = np.arange(16, dtype=np.int32)
    assert front.inferbit_forward(m, p(toks), 16, p(got), V) == 0
    assert front.inferbit_forward(m, p(toks), 1, p(got), V) == -4
    front.inferbit_free(m)
    front.inferbit_config_free(cfg)


def test_front_per_tensor_bit_widths(front, tmp_path, cpu_libs):
    """o_proj stored as INT4 while q, k, v are INT8 (what the reference's converter writes with its
    defaults): the file's per-tensor widths are honoured. Checked against the restatement of forward_single_ex."""
    cfg = dict(ibf_model.CFG, o_bits=4)
    path = str(tmp_path / "mixed.ibf")
    ibf_model.write_ibf(path, cfg=cfg, seed=4242)
    layers, head, (emb, es, fn) = ibf_model.tensors(4242, cfg)
    assert layers[0][0][3][4] == 4 and layers[0][0][0][4] == 8
    kv = cfg["n_kv_heads"] * cfg["head_dim"]
    om = _cpu.IboModel(); ol = (_cpu.IboLayer * cfg["n_layers"])()
    for f in ("hidden", "inter", "n_layers", "n_heads", "n_kv_heads", "head_dim", "vocab", "max_ctx", "eps", "theta"):
        setattr(om, f, cfg[f])
    keep = []
    for l, (lins, norms) in enumerate(layers):
        for i, (w, s, M, N, bits) in enumerate(lins):
            setattr(ol[l], ("q", "k", "v", "o", "gate", "up", "down")[i], _cpu.IboLinear(w.ctypes.data, s.ctypes.data, M, N, bits))
        kc = np.zeros((cfg["max_ctx"], kv), np.float32); vc = np.zeros((cfg["max_ctx"], kv), np.float32)
        keep.append((kc, vc))
        ol[l].input_norm, ol[l].post_attn_norm = norms[0].ctypes.data, norms[1].ctypes.data
        ol[l].k_cache, ol[l].v_cache = kc.ctypes.data, vc.ctypes.data
    om.embed, om.embed_scale, om.final_norm = emb.ctypes.data, es.ctypes.data, fn.ctypes.data
    om.head = _cpu.IboLinear(head[0].ctypes.data, head[1].ctypes.data, cfg["vocab"], cfg["hidden"], 8)
    om.layers = ol
    m = front.inferbit_load(path.encode(), None)
    assert m, _err(front)
    V = cfg["vocab"]
    toks = np.random.default_rng(1).integers(0, V, 6).astype(np.int32)
    got = np.empty(V, np.float32); want = np.empty(V, np.float32)
    for i in range(len(toks)):
        assert cpu_libs.oracle.ibo_decode_step(C.byref(om), toks[i:i + 1].copy(), i, 1, p(want), None) == 0
        assert front.inferbit_forward(m, p(toks[i:i + 1].copy()), 1, p(got), V) == 0, _err(front)
        assert _close_logits(got, want), (i, float(np.max(np.abs(got - want))))
    front.inferbit_free(m)


def test_pq_tensors_from_a_file_run_on_the_gpu(front, cpu_libs, tmp_path):
    """A product-quantised model file read by ib_pq_load_multi (the reference's name and struct) feeds ib_pq_matmul_fp32 and
    ib_pq_lm_head_topk of the same library: a loaded tensor carries the file's format tag (1..3), which the host layer
    takes; results against the restatement."""
    from libinferbit_b200 import _ffi as ffi
    from oracle import ibf_writer
    host = ffi.load_host()
    assert host.ib_b200_init(0) == 0, host.ib_b200_last_error()
    try:
        rng = np.random.default_rng(31)
        ds = {"down": _cpu.make_pq_case_ex(rng, 512, 1024, 16, 256, 0, 0, 1),
              "head": _cpu.make_pq_case_ex(rng, 3000, 512 + 16, 16, 256, 16, 16, 1)}
        fmts = {"down": "pq2d_v1_l1", "head": "pq2d_v1_l1_l2"}
        path = str(tmp_path / "pq.ibf")
        ibf_writer.write_ibf_v5(path, {k: _cpu.pq_file_tensor(d, fmts[k]) for k, d in ds.items()})
        m = _cpu.RefPqMulti()
        assert front.ib_pq_load_multi(path.encode(), C.byref(m)) == 0
        for name, d in ds.items():
            t = front.ib_pq_multi_find(C.byref(m), name.encode())
            assert t
            x = d["x"][0]
            out = np.empty(d["M"], np.float32)
            assert front.ib_pq_matmul_fp32(t, x.ctypes.data, out.ctypes.data) == 0, host.ib_b200_last_error()
            assert _cpu.close(out, _cpu.oracle_pq_ex(cpu_libs.oracle, d, x), 1e-3, 1e-4)
        d = ds["head"]
        gl = np.empty(20, np.float32); gi = np.empty(20, np.int32)
        assert front.ib_pq_lm_head_topk(front.ib_pq_multi_find(C.byref(m), b"head"), d["x"][0].ctypes.data, 20, gl.ctypes.data, gi.ctypes.data) == 0
        wl, wi = _cpu.oracle_pq_topk(cpu_libs.oracle, d, d["x"][0], 20)
        assert set(gi.tolist()) == set(wi.tolist()) and np.all(np.diff(gl) <= 0)
        front.ib_pq_multi_free(C.byref(m))                    # also drops the copies in HBM
        assert m.n == 0
    finally:
        host.ib_b200_shutdown()
