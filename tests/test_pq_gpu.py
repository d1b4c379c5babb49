"""GPU parity of the PQ LUT + gather matvec against the CPU restatement of matmul_impl
(src/pq_decode.c:1504-1682), through the C ABI (ibcu_pq_prepare / ibcu_pq_matmul_fp32)."""
import ctypes as C

import numpy as np
import pytest

from tests import _cpu

pytestmark = pytest.mark.gpu
RTOL, ATOL = 1e-3, 1e-4


def oracle_pq(libs, M, N, G, K, cb_l, cb_r, il, ir, rs, x, stride=0):
    out = np.empty((x.shape[0], M), np.float32)
    for b in range(x.shape[0]):
        assert libs.oracle.ibo_pq_matmul_fp32(M, N, G, K, cb_l, cb_r, stride, il, ir, rs, x[b], out[b], 1, None) == 0
    return out


@pytest.mark.parametrize("M,N,G,K,B", [
    (4096, 14336, 16, 256, 1),      # Mistral-7B down_proj: 1792 subspaces of length 8
    (4096, 14336, 16, 256, 8),
    (1000, 2048, 16, 256, 3),       # rows not a multiple of 16
    (300, 1200, 16, 100, 5),        # several activations: 150 subspaces, the second unit of 128 is mostly padding; 100 codebook entries
    (48, 640, 16, 256, 32),         # 32 activations, fewer pieces of work than SMs
    (16, 40960, 16, 256, 32),       # 1280 units of one group each: a block walks nine of them and reports its arrivals in two batches
    (512, 1024, 16, 256, 2),        # two activations: one pass of the slab kernel with entries two floats wide
    (64, 256, 8, 64, 2), (33, 96, 4, 16, 1), (2048, 512, 32, 256, 1), (5, 16, 16, 256, 1),
])
def test_pq_matches_reference_restatement(backend, cpu_libs, M, N, G, K, B):
    rng = np.random.default_rng(M + N + G + K + B)
    cb_l, cb_r, il, ir, rs, x = _cpu.make_pq_case(rng, M, N, G, K, B)
    t = backend.make_pq(M, N, G, K, cb_l, cb_r, il, ir, rs)
    got = backend.pq_matmul(t, x)
    want = oracle_pq(cpu_libs, M, N, G, K, cb_l, cb_r, il, ir, rs, x)
    assert _cpu.close(got, want, RTOL, ATOL), float(np.max(np.abs(got - want)))


@pytest.mark.parametrize("M,N,G,K,K_l2,n_out,B", [
    (4096, 14336, 16, 256, 256, 0, 1),    # down_proj shape with a full second level
    (4096, 14336, 16, 256, 16, 0, 2),     # 6-bit-per-weight variant: 16-entry second level, two 4-bit indices per byte
    (1000, 2048 + 48, 16, 256, 0, 48, 3), # outlier sidecar only; rows not a multiple of 16
    (4096, 4096 + 64, 16, 256, 16, 64, 1),
    (77, 8 * 13 + 5, 8, 32, 64, 5, 2), (33, 96, 4, 16, 16, 0, 1),
])
def test_pq_second_level_and_outliers(backend, cpu_libs, M, N, G, K, K_l2, n_out, B):
    """The production forms of the tensor (src/pq_decode.c:1441-1496 second residual level, :1058-1075 index forms, :1394-1409
    outlier sidecar, :1538-1546 inner columns) against the CPU restatement, which is pinned to the compiled reference."""
    rng = np.random.default_rng(M + N + K_l2 + n_out + B)
    d = _cpu.make_pq_case_ex(rng, M, N, G, K, K_l2, n_out, B)
    d["x"][B - 1, :3 * G] *= 1e-4                            # some chunks fall under the 1 % rule
    t = backend.make_pq_ex(d)
    got = backend.pq_matmul(t, d["x"])
    want = np.stack([_cpu.oracle_pq_ex(cpu_libs.oracle, d, d["x"][b]) for b in range(B)])
    assert _cpu.close(got, want, RTOL, ATOL), float(np.max(np.abs(got - want)))
    got2 = backend.pq_matmul(t, d["x"])                      # accumulators and counters were left clean
    assert np.array_equal(got, got2)


@pytest.mark.parametrize("M,N,G,K,K_l2,n_out,k_top", [
    (32000, 4096, 16, 256, 16, 0, 64),     # LM head of the 7B shape, 16-entry second level
    (32000, 4096 + 32, 16, 256, 256, 32, 256),
    (5000, 1024, 16, 256, 0, 0, 1024),     # single level: the full logits are the first-level ones
    (300, 8 * 13 + 5, 8, 32, 64, 5, 1), (40, 96, 4, 16, 16, 0, 40),
    (40000, 256, 16, 256, 16, 0, 100),     # more rows than four keys per thread of the cluster: its 32-key instance
    (270000, 32, 16, 256, 0, 0, 50),       # more rows than the cluster keeps in registers: the one-block selection
])
def test_pq_lm_head_topk(backend, cpu_libs, M, N, G, K, K_l2, n_out, k_top):
    """ib_pq_lm_head_topk (src/pq_decode.c:2259-2341) against its restatement, which is pinned to the compiled reference: the
    same rows in the same order wherever neighbouring logits differ by more than rounding, logits within tolerance."""
    rng = np.random.default_rng(M + N + K_l2 + n_out + k_top)
    d = _cpu.make_pq_case_ex(rng, M, N, G, K, K_l2, n_out, 1)
    x = d["x"][0].copy()
    x[:3 * G] *= 1e-4                                         # would fall under the 1 % rule, which this path does not apply
    t = backend.make_pq_ex(d)
    gl, gi = backend.pq_lm_head_topk(t, x, k_top)
    wl, wi, coarse = _cpu.oracle_pq_topk(cpu_libs.oracle, d, x, k_top, want_coarse=True)
    assert np.all(np.diff(gl) <= 0) and len(set(gi.tolist())) == k_top
    # the chosen set: equal, except for rows whose first-level logit sits within rounding of the boundary
    kth = np.sort(coarse)[-k_top]
    margin = 1e-4 * max(1.0, float(np.max(np.abs(coarse))))
    sure = set(np.flatnonzero(coarse > kth + margin).tolist())
    maybe = set(np.flatnonzero(coarse >= kth - margin).tolist())
    assert sure <= set(gi.tolist()) <= maybe and sure <= set(wi.tolist())
    # full logits of the rows both chose, and their order
    full = dict(zip(wi.tolist(), wl.tolist()))
    both = [(i, v) for i, v in zip(gi.tolist(), gl.tolist()) if i in full]
    assert len(both) >= len(sure)
    assert _cpu.close(np.array([v for _, v in both], np.float32), np.array([full[i] for i, _ in both], np.float32), RTOL, ATOL)
    if set(gi.tolist()) == set(wi.tolist()):                 # a row whose logit is clear of both neighbours sits at the same place
        tol = 2 * (ATOL + RTOL * np.abs(wl))
        clear = np.ones(k_top, bool)
        clear[1:] &= np.abs(np.diff(wl)) > tol[1:]
        clear[:-1] &= np.abs(np.diff(wl)) > tol[:-1]
        assert np.array_equal(gi[clear], wi[clear])
    gl2, gi2 = backend.pq_lm_head_topk(t, x, k_top)          # scratch left clean, same bits again
    assert np.array_equal(gl, gl2) and np.array_equal(gi, gi2)
    full_mv = backend.pq_matmul(t, d["x"][0])                 # the matvec still works after the first-level-only launch
    assert _cpu.close(full_mv[0], _cpu.oracle_pq_ex(cpu_libs.oracle, d, d["x"][0]), RTOL, ATOL)
    assert backend.lib.ibcu_pq_lm_head_topk(backend.ctx, C.byref(t), backend.upload(x).ptr, 0, 1, 1) == -1
    backend.lib.ibcu_clear_error(backend.ctx)


def test_pq_lm_head_topk_equal_logits(backend, cpu_libs):
    """Rows with equal logits: the lowest rows are kept at the boundary and equal full logits come out in ascending row order,
    which is also what the reference's heap and stable insertion sort give when every row is equal."""
    rng = np.random.default_rng(5)
    d = _cpu.make_pq_case_ex(rng, 3000, 256, 16, 256, 16, 0, 1)
    for key in ("idx1_l", "idx1_r", "idx2_l", "idx2_r"):
        d[key][:] = d[key][0]                                 # every row is row 0
    d["rs"][:] = d["rs"][0]
    t = backend.make_pq_ex(d)
    gl, gi = backend.pq_lm_head_topk(t, d["x"][0], 7)
    wl, wi = _cpu.oracle_pq_topk(cpu_libs.oracle, d, d["x"][0], 7)
    assert np.array_equal(gi, np.arange(7)) and np.array_equal(wi, np.arange(7)) and np.all(gl == gl[0])
    # two values: rows 100.. carry a larger scale, the boundary falls inside the smaller value's rows
    half = d["rs"].copy(); half[:] = _cpu.fp16_bits(np.float32(0.5)); half[100:110] = _cpu.fp16_bits(np.float32(1.0))
    d["rs"][:] = half
    t2 = backend.make_pq_ex(d)
    gl, gi = backend.pq_lm_head_topk(t2, d["x"][0], 14)
    big = set(range(100, 110))
    if _cpu.oracle_pq_topk(cpu_libs.oracle, d, d["x"][0], 1)[0][0] > 0:      # positive logits: the scaled rows lead, then the lowest of the rest
        assert set(gi[:10].tolist()) == big and gi[10:].tolist() == [0, 1, 2, 3]
    else:                                                     # negative logits: the scaled rows are the smallest and are not chosen
        assert gi.tolist() == list(range(14))


def test_pq_lm_head_topk_through_the_host_layer(cpu_libs):
    """ib_b200_pq_lm_head_topk takes the reference's own struct and host pointers."""
    from libinferbit_b200 import _ffi
    host = _ffi.load_host()
    assert host.ib_b200_init(0) == 0, host.ib_b200_last_error()
    try:
        rng = np.random.default_rng(21)
        d = _cpu.make_pq_case_ex(rng, 2000, 1024 + 16, 16, 256, 16, 16, 1)
        t = _cpu.ref_pq_tensor_ex(d)
        k_top = 32
        gl = np.empty(k_top, np.float32); gi = np.empty(k_top, np.int32)
        x = d["x"][0]
        host.ib_b200_pq_lm_head_topk.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]   # the reference's struct as it is
        assert host.ib_b200_pq_lm_head_topk(C.byref(t), x.ctypes.data, k_top, gl.ctypes.data, gi.ctypes.data) == 0, host.ib_b200_last_error()
        wl, wi = _cpu.oracle_pq_topk(cpu_libs.oracle, d, x, k_top)
        assert set(gi.tolist()) == set(wi.tolist()) and np.all(np.diff(gl) <= 0)
        order = {i: v for i, v in zip(wi.tolist(), wl.tolist())}
        assert _cpu.close(gl, np.array([order[i] for i in gi.tolist()], np.float32), RTOL, ATOL)
        assert host.ib_b200_pq_lm_head_topk(C.byref(t), x.ctypes.data, 0, gl.ctypes.data, gi.ctypes.data) == -1
        assert host.ib_b200_pq_lm_head_topk(C.byref(t), x.ctypes.data, 2001, gl.ctypes.data, gi.ctypes.data) == -1
    finally:
        host.ib_b200_shutdown()


def test_pq_extras_through_the_host_layer(cpu_libs):
    """ib_b200_pq_matmul_fp32 takes the reference's own struct with two levels and outliers (host pointers)."""
    from libinferbit_b200 import _ffi
    host = _ffi.load_host()
    assert host.ib_b200_init(0) == 0, host.ib_b200_last_error()
    try:
        rng = np.random.default_rng(11)
        d = _cpu.make_pq_case_ex(rng, 300, 1024 + 32, 16, 256, 16, 32, 1)
        t = _cpu.ref_pq_tensor_ex(d)
        out = np.empty(300, np.float32)
        host.ib_b200_pq_matmul_fp32.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        assert host.ib_b200_pq_matmul_fp32(C.byref(t), d["x"][0].ctypes.data, out.ctypes.data) == 0, host.ib_b200_last_error()
        want = _cpu.oracle_pq_ex(cpu_libs.oracle, d, d["x"][0])
        assert _cpu.close(out, want, RTOL, ATOL)
        t.l2_idx_bytes = 2; t.K_l2 = 4096                    # uint16 second-level indices: refused, never computed on the CPU
        host.ib_b200_pq_release.argtypes = [C.c_void_p]
        host.ib_b200_pq_release(C.byref(t))
        assert host.ib_b200_pq_matmul_fp32(C.byref(t), d["x"][0].ctypes.data, out.ctypes.data) == -1
    finally:
        host.ib_b200_shutdown()


def test_row_slices_written_in_place(backend, cpu_libs):
    """Two tensors that hold the upper and the lower rows of one tensor write their rows straight into the full-width
    result (ibcu_pq_matmul_fp32_strided): the same bits as the whole tensor in one call."""
    rng = np.random.default_rng(17)
    M, N, G, K, B = 200, 512, 16, 256, 3
    cb_l, cb_r, il, ir, rs, x = _cpu.make_pq_case(rng, M, N, G, K, B)
    whole = backend.pq_matmul(backend.make_pq(M, N, G, K, cb_l, cb_r, il, ir, rs), x)
    cut = 96
    top = backend.make_pq(cut, N, G, K, cb_l, cb_r, il[:cut].copy(), ir[:cut].copy(), rs[:cut].copy())
    bot = backend.make_pq(M - cut, N, G, K, cb_l, cb_r, il[cut:].copy(), ir[cut:].copy(), rs[cut:].copy())
    dx = backend.upload(x)
    do = backend.upload(np.full((B, M + 8), -3.0, np.float32))
    backend._check(backend.lib.ibcu_pq_matmul_fp32_strided(backend.ctx, C.byref(top), dx.ptr, do.ptr, M + 8, B))
    backend._check(backend.lib.ibcu_pq_matmul_fp32_strided(backend.ctx, C.byref(bot), dx.ptr, do.ptr + 4 * cut, M + 8, B))
    backend.sync()
    got = backend.download(do, np.float32, B * (M + 8)).reshape(B, M + 8)
    assert np.array_equal(got[:, :M], whole) and np.all(got[:, M:] == -3.0)
    assert backend.lib.ibcu_pq_matmul_fp32_strided(backend.ctx, C.byref(top), dx.ptr, do.ptr, cut - 1, B) == -1      # stride below the rows
    backend.lib.ibcu_clear_error(backend.ctx)


@pytest.mark.parametrize("dim,G,K1,n_vec", [(1024, 16, 256, 3), (128, 8, 16, 2), (1024, 16, 100, 1)])
def test_pq_kv_encode(backend, cpu_libs, dim, G, K1, n_vec):
    """PQ KV-cache encode (src/pq_decode.c:5008-5066): per-vector scale and nearest codeword per half chunk, against the CPU
    restatement (which has no entry point of the reference to be pinned to). Codes and scales must be the same bits;
    a zero vector and duplicated codebook entries (the first of equals wins) are among the cases."""
    rng = np.random.default_rng(dim + K1)
    half, Cn = G // 2, dim // G
    cb_l = _cpu.fp16_bits(rng.standard_normal((K1, half)) * 3.0); cb_r = _cpu.fp16_bits(rng.standard_normal((K1, half)) * 3.0)
    cb_l[K1 // 2] = cb_l[1]                                  # equal entries: the lower index must win
    vec = (rng.standard_normal((n_vec, dim)) * 0.7).astype(np.float32)
    if n_vec > 1:
        vec[1] = 0.0
    o = cpu_libs.oracle
    o.ibo_pqkv_encode.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
    o.ibo_pqkv_encode.restype = None
    want_idx = np.empty((n_vec, 2 * Cn), np.uint8); want_s = np.empty(n_vec, np.float32)
    for v in range(n_vec):
        o.ibo_pqkv_encode(vec[v].ctypes.data, dim, G, K1, cb_l.ctypes.data, cb_r.ctypes.data, want_idx[v].ctypes.data,
                          want_s[v:].ctypes.data, 1)
    be = backend
    dv, dl, dr = be.upload(vec), be.upload(cb_l), be.upload(cb_r)
    di, ds = be.alloc(n_vec * 2 * Cn), be.alloc(n_vec * 4)
    be._check(be.lib.ibcu_pqkv_encode(be.ctx, dv.ptr, dim, n_vec, G, K1, dl.ptr, dr.ptr, di.ptr, ds.ptr)); be.sync()
    assert np.array_equal(be.download(di, np.uint8, n_vec * 2 * Cn).reshape(n_vec, 2 * Cn), want_idx)
    assert np.array_equal(be.download(ds, np.float32, n_vec), want_s)


def test_packed_code_plane_is_a_faithful_copy(backend):
    """ibcu_pq_prepare regroups the codes as [slab of 32 subspaces][group of 16 rows][lane][16 rows]
    (subspace 2 * chunk + side = 32 * slab + lane; byte i of lane l is row i ^ (l >> 1) of the group, the order the
    kernel's lane-to-lane reduction wants); padding rows and padding subspaces hold zeros, and the tail of the array
    holds the largest codebook magnitude."""
    rng = np.random.default_rng(3)
    M, N, G, K = 77, 160, 16, 256
    cb_l, cb_r, il, ir, rs, _ = _cpu.make_pq_case(rng, M, N, G, K, 1)
    t = backend.make_pq(M, N, G, K, cb_l, cb_r, il, ir, rs)
    Cn = N // G
    assert t.M_pad == 80
    nslab = (2 * Cn + 31) // 32
    total = backend.lib.ibcu_pq_idx_t_bytes(M, N, G)
    assert total == nslab * 32 * t.M_pad + 256
    raw = backend.download(t.idx_t, np.uint8, total)
    plane = raw[:nslab * 32 * t.M_pad].reshape(nslab, t.M_pad // 16, 32, 16)          # [slab][group][lane][byte]
    order = np.arange(16)[None, :] ^ (np.arange(32)[:, None] >> 1)                        # [lane][row in group] -> byte
    plane = np.take_along_axis(plane, np.broadcast_to(order, plane.shape), axis=3)        # [slab][group][lane][row in group]
    sub = plane.transpose(0, 2, 1, 3).reshape(nslab * 32, t.M_pad)                        # [subspace][row]
    assert np.array_equal(sub[0:2 * Cn:2, :M], il.T) and np.array_equal(sub[1:2 * Cn:2, :M], ir.T)
    assert np.all(sub[:, M:] == 0) and np.all(sub[2 * Cn:] == 0)
    cbmax = raw[nslab * 32 * t.M_pad:][:4].view(np.float32)[0]
    want = max(float(np.abs(cb_l.view(np.float16).astype(np.float32)).max()), float(np.abs(cb_r.view(np.float16).astype(np.float32)).max()))
    assert cbmax == np.float32(want)


def test_codes_select_the_right_table_entries(backend):
    """Codebook entry k of side L holds k in its first element and zeros elsewhere, side R holds 1000*k,
    and x is one-hot per chunk: the output must be exactly the selected integers."""
    M, N, G, K = 48, 64, 16, 256
    half, Cn = 8, 4
    cb_l = np.zeros((K, half), np.float32); cb_l[:, 0] = np.arange(K)
    cb_r = np.zeros((K, half), np.float32); cb_r[:, 0] = np.arange(K) * 8.0
    rng = np.random.default_rng(1)
    il = rng.integers(0, K, (M, Cn), dtype=np.uint8); ir = rng.integers(0, K, (M, Cn), dtype=np.uint8)
    rs = np.full(M, 0x3C00, np.uint16)
    t = backend.make_pq(M, N, G, K, _cpu.fp16_bits(cb_l), _cpu.fp16_bits(cb_r), il, ir, rs)
    for c in range(Cn):
        x = np.zeros((1, N), np.float32); x[0, c * G] = 1.0; x[0, c * G + half] = 1.0
        got = backend.pq_matmul(t, x)[0]
        assert np.array_equal(got, il[:, c].astype(np.float32) + 8.0 * ir[:, c].astype(np.float32))


def test_chunk_skip_rule(backend, cpu_libs):
    """Chunks whose 16 activations all stay under 1 % of the vector's max contribute nothing
    (src/pq_decode.c:1582-1616); an all-zero activation gives zeros."""
    rng = np.random.default_rng(8)
    M, N, G, K = 256, 1024, 16, 256
    cb_l, cb_r, il, ir, rs, x = _cpu.make_pq_case(rng, M, N, G, K, 3)
    x[0, 5 * G:9 * G] *= 1e-3
    x[1, :] = 0.0
    x[2, ::2] *= 1e-5
    t = backend.make_pq(M, N, G, K, cb_l, cb_r, il, ir, rs)
    got = backend.pq_matmul(t, x)
    want = np.empty((3, M), np.float32); skipped = []
    for b in range(3):
        n = C.c_int()
        cpu_libs.oracle.ibo_pq_matmul_fp32(M, N, G, K, cb_l, cb_r, 0, il, ir, rs, x[b], want[b], 1, C.byref(n))
        skipped.append(n.value)
    assert skipped[0] >= 4 and skipped[1] == 0
    assert _cpu.close(got, want, RTOL, ATOL)
    assert np.all(got[1] == 0.0)
    # dropping is visible: without the rule row 0 would differ
    x0 = x[0].copy(); x0[5 * G:9 * G] = 0.0
    ref0 = np.empty(M, np.float32)
    cpu_libs.oracle.ibo_pq_matmul_fp32(M, N, G, K, cb_l, cb_r, 0, il, ir, rs, x0, ref0, 1, None)
    assert _cpu.close(got[0], ref0, RTOL, ATOL)


def test_per_subspace_codebooks(backend, cpu_libs):
    """A codebook per chunk (stride between chunk tables), same arithmetic."""
    rng = np.random.default_rng(12)
    M, N, G, K = 128, 512, 16, 256
    half, Cn = 8, N // G
    cb_l = _cpu.fp16_bits(rng.standard_normal((Cn, K, half)) * 0.02)
    cb_r = _cpu.fp16_bits(rng.standard_normal((Cn, K, half)) * 0.02)
    _, _, il, ir, rs, x = _cpu.make_pq_case(rng, M, N, G, K, 2)
    t = backend.make_pq(M, N, G, K, cb_l, cb_r, il, ir, rs, cb_chunk_stride=K * half)
    got = backend.pq_matmul(t, x)
    want = oracle_pq(cpu_libs, M, N, G, K, cb_l.reshape(-1), cb_r.reshape(-1), il, ir, rs, x, stride=K * half)
    assert _cpu.close(got, want, RTOL, ATOL)


def test_linearity_at_full_size(backend):
    """Size-independent property at the benchmark shape: with the skip rule inactive the map is linear,
    f(x + y) = f(x) + f(y) and f(2x) = 2 f(x) exactly (the same number of activations in both calls: one activation
    and several take different kernels, whose FP32 partial sums are ordered differently)."""
    rng = np.random.default_rng(4)
    M, N, G, K = 4096, 14336, 16, 256
    cb_l, cb_r, il, ir, rs, x = _cpu.make_pq_case(rng, M, N, G, K, 2)
    t = backend.make_pq(M, N, G, K, cb_l, cb_r, il, ir, rs)
    fx = backend.pq_matmul(t, x)
    f2 = backend.pq_matmul(t, 2.0 * x)
    assert np.array_equal(f2, 2.0 * fx)
    f1 = backend.pq_matmul(t, x[:1])
    assert np.array_equal(backend.pq_matmul(t, 2.0 * x[:1]), 2.0 * f1) and _cpu.close(f1[0], fx[0], 1e-5, 1e-5)
    fs = backend.pq_matmul(t, (x[0] + x[1])[None, :])
    assert _cpu.close(fs[0], fx[0] + fx[1], 1e-3, 1e-4)
