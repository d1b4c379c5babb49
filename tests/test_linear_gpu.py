"""GPU parity of the INT4 / INT8 linear kernels against the CPU restatement of the reference's scalar
kernels (src/kernels/scalar.c:9-41,70-84), through the C ABI (ibcu_linear)."""
import ctypes as C

import numpy as np
import pytest

from libinferbit_b200 import LinearT
from tests import _cpu

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1e-3, 1e-4        # the float bar: |gpu - ref| <= 1e-4 + 1e-3 |ref|


def oracle_linear(libs, w, s16, x, bits):
    M = w.shape[0]; B, N = x.shape
    s = np.empty(M, np.float32); libs.oracle.ibo_fp16_array_to_fp32(s16, s, M)
    out = np.empty((B, M), np.float32)
    if bits == 8:
        libs.oracle.ibo_matmul_int8_batch(out, w, s, x, M, N, B, M)
    else:
        libs.oracle.ibo_matmul_int4_batch(out, w, s, x, M, N, B, M)
    return out


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("M,N,B", [
    (5632, 2048, 1),      # TinyLlama up_proj
    (1024, 4096, 1), (1024, 4096, 4), (1024, 4096, 16),     # k/v proj
    (4096, 4096, 4), (4096, 4096, 16),                      # q/o proj at the batch sizes of the attention configuration
    (512, 4096, 2), (512, 4096, 3), (512, 4096, 8), (256, 4096, 32),
    (4096, 14336, 1),     # down_proj shape
    (100, 320, 5),        # rows not a multiple of the tile, short rows
    (33, 96, 1), (1, 64, 1), (17, 4128, 7),
])
def test_linear_matches_scalar_reference(backend, cpu_libs, bits, M, N, B):
    rng = np.random.default_rng(bits * 7919 + M * 31 + N + B)
    w, s16, x = (_cpu.make_int8_case if bits == 8 else _cpu.make_int4_case)(rng, M, N, B)
    got = backend.linear(w, s16, x, bits)
    want = oracle_linear(cpu_libs, w, s16, x, bits)
    assert _cpu.close(got, want, RTOL, ATOL), float(np.max(np.abs(got - want)))


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("M,N,B", [(4096, 4096, 8), (4096, 4096, 16), (1000, 4096, 11), (130, 256, 8), (4096, 14336, 8), (2048, 14336, 16),
                                   (300, 1152, 9)])
def test_batched_tcgen05_path(backend, cpu_libs, bits, M, N, B):
    """The optional kernel for 8 to 16 activations on the tcgen05 tensor cores (accumulators in tensor memory): against
    the scalar restatement, and against the mma.sync kernel on the same inputs. Both sum exact
    integers; they can differ in the last place only where the columns were split into different numbers of slices."""
    rng = np.random.default_rng(bits * 13 + M + N + B)
    w, s16, x = (_cpu.make_int8_case if bits == 8 else _cpu.make_int4_case)(rng, M, N, B)
    init = rng.standard_normal((B, M)).astype(np.float32)
    want = oracle_linear(cpu_libs, w, s16, x, bits)
    backend.lib.ibcu_linear_use_tcgen05(backend.ctx, 2)
    try:
        before = backend.launches()
        got = backend.linear(w, s16, x, bits)
        assert backend.launches() - before >= (2 if N % 512 == 0 else 1)    # conversion kernel + tcgen05 kernel (+ recombination); other rows take the usual kernel
        assert _cpu.close(got, want, RTOL, ATOL), float(np.max(np.abs(got - want)))
        got_add = backend.linear(w, s16, x, bits, epilogue=1, out_init=init)
        assert np.allclose(got_add, init + got, rtol=1e-6, atol=1e-6 * float(np.abs(got).max()))    # the residual epilogue adds the same product
        backend.lib.ibcu_linear_use_tcgen05(backend.ctx, -1)
        other = backend.linear(w, s16, x, bits)
    finally:
        backend.lib.ibcu_linear_use_tcgen05(backend.ctx, 0)
    assert np.allclose(got, other, rtol=2e-6, atol=1e-6 * float(np.abs(other).max()))
    assert backend.lib.ibcu_sync(backend.ctx) == 0           # no wait inside the kernel ran out


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("M,N,B", [(40, 66, 2), (9, 30, 1), (257, 1000, 3), (64, 4096, 4)])
def test_portable_kernel(backend, cpu_libs, bits, M, N, B):
    """Shapes the tensor-core path does not take (row bytes not a multiple of 16) and the forced
    portable kernel on a shape it does take."""
    rng = np.random.default_rng(M + N)
    w, s16, x = (_cpu.make_int8_case if bits == 8 else _cpu.make_int4_case)(rng, M, N, B)
    got = backend.linear(w, s16, x, bits, force_generic=True)
    want = oracle_linear(cpu_libs, w, s16, x, bits)
    assert _cpu.close(got, want, RTOL, ATOL)
    got2 = backend.linear(w, s16, x, bits)
    assert _cpu.close(got2, want, RTOL, ATOL)


@pytest.mark.parametrize("bits", [8, 4])
def test_unpack_is_exact(backend, bits):
    """One-hot activations read single weights back: out/scale must be the integer itself, for every
    column position modulo 128 and every nibble / byte value."""
    rng = np.random.default_rng(11)
    M, N = 64, 256
    if bits == 8:
        w = rng.integers(-128, 128, size=(M, N), dtype=np.int8)
        w[:, 0] = np.arange(M) - 128; w[:, 1] = np.arange(M) + 64
        vals = w.astype(np.float32)
    else:
        w = rng.integers(0, 256, size=(M, N // 2), dtype=np.uint8)
        w[:16, 0] = np.arange(16) | (np.arange(16)[::-1] << 4)
        vals = np.empty((M, N), np.float32)
        vals[:, 0::2] = (w & 15).astype(np.float32) - 8
        vals[:, 1::2] = (w >> 4).astype(np.float32) - 8
    ones = np.full(M, 0x3C00, np.uint16)                       # fp16 1.0
    for j0 in range(0, N, 32):
        x = np.zeros((32, N), np.float32)
        x[np.arange(32), j0 + np.arange(32)] = 1.0
        got = backend.linear(w, ones, x, bits)                 # [32, M]
        assert np.array_equal(got, vals[:, j0:j0 + 32].T)


@pytest.mark.parametrize("bits", [8, 4])
def test_scales_fp32_and_residual_epilogue(backend, cpu_libs, bits):
    rng = np.random.default_rng(5)
    M, N, B = 200, 512, 4
    w, s16, x = (_cpu.make_int8_case if bits == 8 else _cpu.make_int4_case)(rng, M, N, B)
    want = oracle_linear(cpu_libs, w, s16, x, bits)
    s32 = np.empty(M, np.float32); cpu_libs.oracle.ibo_fp16_array_to_fp32(s16, s32, M)
    assert _cpu.close(backend.linear(w, s32, x, bits), want, RTOL, ATOL)
    base = rng.standard_normal((B, M)).astype(np.float32)
    got = backend.linear(w, s16, x, bits, epilogue=1, out_init=base)
    assert _cpu.close(got, base + want, RTOL, ATOL)


def test_wide_dynamic_range_activations(backend, cpu_libs):
    """Activations spanning six orders of magnitude inside one vector, and huge and tiny vectors: the
    per-slice power-of-two scaling keeps the fixed-point limbs exact enough. The absolute term of the
    bar is scaled by the largest activation, which is what sets the reference's own rounding noise."""
    rng = np.random.default_rng(9)
    M, N = 128, 1024
    w, s16, _ = _cpu.make_int8_case(rng, M, N, 1)
    for scale in (1e-20, 1e-6, 1.0, 3e4, 1e12):
        x = (rng.standard_normal((2, N)) * scale * 10.0 ** rng.integers(-3, 3, (2, N))).astype(np.float32)
        got = backend.linear(w, s16, x, 8)
        want = oracle_linear(cpu_libs, w, s16, x, 8)
        assert _cpu.close(got, want, RTOL, ATOL * float(np.abs(x).max())), scale
    x = np.zeros((1, N), np.float32)
    assert np.array_equal(backend.linear(w, s16, x, 8), np.zeros((1, M), np.float32))


def test_three_tensors_one_launch_with_strided_output(backend, cpu_libs):
    """q, k, v share the activation: one launch, each tensor with its own rows, scales and output
    stride (the reference's M_stride, src/threading.c:373-380)."""
    rng = np.random.default_rng(21)
    N, B = 1024, 4
    Ms = [256, 64, 80]
    be = backend
    x = rng.standard_normal((B, N)).astype(np.float32)
    dx = be.upload(x)
    descs = (LinearT * 3)()
    keep, wants, outs = [], [], []
    for i, M in enumerate(Ms):
        w, s16, _ = _cpu.make_int8_case(rng, M, N, 1)
        wants.append(oracle_linear(cpu_libs, w, s16, x, 8))
        dw, ds = be.upload(w), be.upload(s16)
        stride = M + 8
        do = be.upload(np.full((B, stride), -7.0, np.float32))
        keep += [dw, ds]; outs.append((do, stride))
        descs[i] = LinearT(dw.ptr, ds.ptr, do.ptr, M, stride, 0, 0)
    be._check(be.lib.ibcu_linear(be.ctx, descs, 3, dx.ptr, N, B, 8))
    be.sync()
    for (do, stride), want, M in zip(outs, wants, Ms):
        got = be.download(do, np.float32, B * stride).reshape(B, stride)
        assert _cpu.close(got[:, :M], want, RTOL, ATOL)
        assert np.all(got[:, M:] == -7.0)                      # padding untouched


def test_gate_up_silu(backend, cpu_libs):
    rng = np.random.default_rng(22)
    M, N, B = 300, 512, 2
    be = backend
    x = rng.standard_normal((B, N)).astype(np.float32)
    wg, sg, _ = _cpu.make_int4_case(rng, M, N, 1)
    wu, su, _ = _cpu.make_int4_case(rng, M, N, 1)
    g = oracle_linear(cpu_libs, wg, sg, x, 4); u = oracle_linear(cpu_libs, wu, su, x, 4)
    want = np.empty_like(g)
    for b in range(B):
        cpu_libs.oracle.ibo_silu_mul(want[b], g[b], u[b], M)
    dx = be.upload(x)
    descs = (LinearT * 2)()
    og, ou = be.alloc(B * M * 4), be.alloc(B * M * 4)
    descs[0] = LinearT(be.upload(wg).ptr, be.upload(sg).ptr, og.ptr, M, M, 0, 0)
    descs[1] = LinearT(be.upload(wu).ptr, be.upload(su).ptr, ou.ptr, M, M, 0, 0)
    be._check(be.lib.ibcu_linear_gate_up_silu(be.ctx, descs, dx.ptr, N, B, 4))
    be.sync()
    got = be.download(og, np.float32, B * M).reshape(B, M)
    assert _cpu.close(got, want, 2e-3, 2e-4)


def test_bad_arguments_are_refused(backend):
    be = backend
    d = be.alloc(1024)
    t = LinearT(d.ptr, d.ptr, d.ptr, 4, 4, 0, 0)
    assert be.lib.ibcu_linear(be.ctx, C.byref(t), 1, d.ptr, 64, 1, 3) == -1       # bits
    assert b"bits" in be.lib.ibcu_last_error(be.ctx)
    assert be.lib.ibcu_status(be.ctx) == -1
    be.lib.ibcu_clear_error(be.ctx)
    assert be.lib.ibcu_linear(be.ctx, C.byref(t), 1, d.ptr, 64, 33, 8) == -1      # B > IB_BATCH_MAX
    be.lib.ibcu_clear_error(be.ctx)
    assert be.lib.ibcu_linear(be.ctx, C.byref(t), 1, d.ptr, 63, 1, 4) == -1       # odd N for nibbles
    be.lib.ibcu_clear_error(be.ctx)
    assert be.lib.ibcu_linear(be.ctx, C.byref(t), 0, d.ptr, 64, 1, 8) == -1
    be.lib.ibcu_clear_error(be.ctx)
    assert be.lib.ibcu_status(be.ctx) == 0


@pytest.mark.parametrize("N,B,M", [(128, 3, 70), (4096, 3, 70), (200, 3, 70), (14336, 1, 333), (4096, 8, 512), (2048, 11, 100),
                                   (4096, 1, 4096)])
def test_w4a8_route_bit_exact(backend, cpu_libs, N, B, M):
    """Activation quantiser (src/threading.c:401-432) and INT4 x INT8 kernel (src/kernels/scalar.c:43-124):
    integer work, so the bar is bit-exact, including the FP32 accumulation order. Whole groups of 128 columns
    take the tensor-core kernel (more than 8 activations in chunks of 8), N = 200 the row-per-warp kernel;
    both are also run against each other."""
    rng = np.random.default_rng(N + B)
    be = backend
    x = rng.standard_normal((B, N)).astype(np.float32)
    if B >= 3:
        x[1, :64] = 0; x[2, :] *= 1e-12
    groups = (N + 127) // 128
    q = np.empty((B, N), np.int8); sa = np.empty((B, groups), np.float32)
    for b in range(B):
        cpu_libs.oracle.ibo_quantize_input_int8_g128(x[b], q[b], sa[b], N)
    dx = be.upload(x); dq = be.alloc(B * N); dsa = be.alloc(B * groups * 4)
    be._check(be.lib.ibcu_quantize_input_int8_g128(be.ctx, dx.ptr, dq.ptr, dsa.ptr, N, B)); be.sync()
    assert np.array_equal(be.download(dq, np.int8, B * N).reshape(B, N), q)
    assert np.array_equal(be.download(dsa, np.float32, B * groups).reshape(B, groups), sa)
    w = rng.integers(0, 256, size=(M, N // 2), dtype=np.uint8)
    s16 = _cpu.fp16_bits(rng.uniform(0.002, 0.02, M))
    sw = np.empty(M, np.float32); cpu_libs.oracle.ibo_fp16_array_to_fp32(s16, sw, M)
    want = np.empty((B, M), np.float32)
    cpu_libs.oracle.ibo_matmul_w4a8_batch(want, w, sw, q, sa, M, N, B, M)
    do = be.alloc(B * M * 4)
    t = LinearT(be.upload(w).ptr, be.upload(s16).ptr, do.ptr, M, M, 0, 0)
    be._check(be.lib.ibcu_linear_w4a8(be.ctx, C.byref(t), dq.ptr, dsa.ptr, N, B)); be.sync()
    assert np.array_equal(be.download(do, np.float32, B * M).reshape(B, M), want)
    do3 = be.alloc(B * M * 4)                               # quantiser and matvec in one call from the FP32 activations
    t3 = LinearT(t.w, t.scales, do3.ptr, M, M, 0, 0)
    be._check(be.lib.ibcu_linear_w4a8_fp32(be.ctx, C.byref(t3), dx.ptr, N, B)); be.sync()
    assert np.array_equal(be.download(do3, np.float32, B * M).reshape(B, M), want)
    be.lib.ibcu_linear_force_generic(be.ctx, 1)             # the row-per-warp kernel on the same inputs
    try:
        do2 = be.alloc(B * M * 4)
        t2 = LinearT(t.w, t.scales, do2.ptr, M, M, 0, 0)
        be._check(be.lib.ibcu_linear_w4a8(be.ctx, C.byref(t2), dq.ptr, dsa.ptr, N, B)); be.sync()
        assert np.array_equal(be.download(do2, np.float32, B * M).reshape(B, M), want)
    finally:
        be.lib.ibcu_linear_force_generic(be.ctx, 0)


@pytest.mark.parametrize("bits,N", [(8, 1024), (4, 2048), (8, 200)])
def test_prologues_rmsnorm_and_silu_mul(backend, cpu_libs, bits, N):
    """RMSNorm (fp16 weights) and silu(x)*x2 folded into the call equal the separate scalar kernels
    (src/kernels/scalar.c:126-138,175-181) followed by the matvec; N = 200 takes the portable path."""
    from libinferbit_b200 import _ffi
    rng = np.random.default_rng(bits + N)
    be, o = backend, cpu_libs.oracle
    M, B = 96, 3
    w, s16, x = (_cpu.make_int8_case if bits == 8 else _cpu.make_int4_case)(rng, M, N, B)
    x *= 3.0
    x2 = rng.standard_normal((B, N)).astype(np.float32)
    nw16 = _cpu.fp16_bits(rng.uniform(0.9, 1.1, N)); nw = np.empty(N, np.float32); o.ibo_fp16_array_to_fp32(nw16, nw, N)
    dw, ds, dx, dx2, dn, do = be.upload(w), be.upload(s16), be.upload(x), be.upload(x2), be.upload(nw16), be.alloc(B * M * 4)
    t = LinearT(dw.ptr, ds.ptr, do.ptr, M, M, 0, 0)
    for op in (1, 2):
        xin = np.empty_like(x)
        for b in range(B):
            if op == 1:
                o.ibo_rmsnorm(xin[b], x[b], nw, 1e-5, N)
            else:
                o.ibo_silu_mul(xin[b], x[b], x2[b], N)
        want = oracle_linear(cpu_libs, w, s16, xin, bits)
        pro = _ffi.PrologueT(op, dx2.ptr, dn.ptr, 1e-5)
        be._check(be.lib.ibcu_linear_ex(be.ctx, C.byref(t), 1, dx.ptr, N, B, bits, C.byref(pro)))
        be.sync()
        got = be.download(do, np.float32, B * M).reshape(B, M)
        assert _cpu.close(got, want, 2e-3, 2e-4), op


@pytest.mark.parametrize("bits,M,N,B,parts", [(4, 96, 14336, 1, 28), (8, 80, 4096, 2, 7), (4, 64, 2048, 3, 5), (8, 48, 200, 2, 3), (8, 40, 40960, 1, 16)])
def test_silu_mul_amax_then_known_max_prologue(backend, cpu_libs, bits, M, N, B, parts):
    """ibcu_silu_mul_amax followed by a linear call told max|x| (IBCU_PRO_KNOWN_MAX) gives bit for bit what the
    silu(x)*x2 prologue gives: same activation values, same maximum, hence the same fixed-point operand.
    The pieces written by the element-wise step are checked against numpy."""
    from libinferbit_b200 import _ffi
    rng = np.random.default_rng(bits * 1000 + N + B)
    be, o = backend, cpu_libs.oracle
    w, s16, g = (_cpu.make_int8_case if bits == 8 else _cpu.make_int4_case)(rng, M, N, B)
    g *= 2.0
    u = rng.standard_normal((B, N)).astype(np.float32)
    dw, ds, dg, du = be.upload(w), be.upload(s16), be.upload(g), be.upload(u)
    dh, da, do1, do2 = be.alloc(B * N * 4), be.alloc(B * parts * 4), be.alloc(B * M * 4), be.alloc(B * M * 4)
    t1, t2 = LinearT(dw.ptr, ds.ptr, do1.ptr, M, M, 0, 0), LinearT(dw.ptr, ds.ptr, do2.ptr, M, M, 0, 0)
    p_silu = _ffi.PrologueT(2, du.ptr, None, 0.0, None, 0)
    be._check(be.lib.ibcu_linear_ex(be.ctx, C.byref(t1), 1, dg.ptr, N, B, bits, C.byref(p_silu)))
    be._check(be.lib.ibcu_silu_mul_amax(be.ctx, dh.ptr, dg.ptr, du.ptr, N, B, da.ptr, parts))
    p_known = _ffi.PrologueT(3, None, None, 0.0, da.ptr, parts)
    be._check(be.lib.ibcu_linear_ex(be.ctx, C.byref(t2), 1, dh.ptr, N, B, bits, C.byref(p_known)))
    be.sync()
    h = be.download(dh, np.float32, B * N).reshape(B, N)
    want_h = np.empty_like(h)
    for b in range(B):
        o.ibo_silu_mul(want_h[b], g[b], u[b], N)
    assert _cpu.close(h, want_h, 1e-5, 1e-6)
    am = be.download(da, np.float32, B * parts).reshape(B, parts)
    chunk = (N + parts - 1) // parts
    for b in range(B):
        for p in range(parts):
            seg = np.abs(h[b, p * chunk:(p + 1) * chunk])
            assert am[b, p] == (seg.max() if seg.size else 0.0)
    got1 = be.download(do1, np.float32, B * M).reshape(B, M)
    got2 = be.download(do2, np.float32, B * M).reshape(B, M)
    if N % 16 == 0:                       # the tensor-core path: identical fixed-point operands
        assert np.array_equal(got1, got2)
    assert _cpu.close(got2, oracle_linear(cpu_libs, w, s16, want_h, bits), 2e-3, 2e-4)


@pytest.mark.parametrize("bits,Ms,N,B", [
    (8, [7, 250, 3], 512, 1),            # ragged tensors: runs of rows never cross a tensor, tiles shorter than 16 rows
    (4, [1, 2, 5000, 33], 1024, 2),      # four tensors, one of them larger than the whole grid's worth of 4-row runs
    (8, [4096, 1024, 1024], 4096, 1),    # the q,k,v launch of the headline step
    (4, [14336, 14336], 4096, 1),        # the gate,up launch of the 7B decode step
    (8, [0, 64, 0], 256, 3),             # empty shards (a rank that owns no rows of a tensor)
])
def test_several_tensors_with_ragged_rows(backend, cpu_libs, bits, Ms, N, B):
    rng = np.random.default_rng(bits + sum(Ms) + N)
    be = backend
    x = rng.standard_normal((B, N)).astype(np.float32)
    dx = be.upload(x)
    n = len(Ms)
    descs = (LinearT * n)()
    keep, wants, outs = [], [], []
    for i, M in enumerate(Ms):
        Mr = max(M, 1)
        w, s16, _ = (_cpu.make_int8_case if bits == 8 else _cpu.make_int4_case)(rng, Mr, N, 1)
        wants.append(oracle_linear(cpu_libs, w, s16, x, bits)[:, :M])
        dw, ds = be.upload(w), be.upload(s16)
        do = be.upload(np.full((B, Mr), -3.0, np.float32))
        keep += [dw, ds]; outs.append(do)
        descs[i] = LinearT(dw.ptr, ds.ptr, do.ptr, M, Mr, 0, 0)
    be._check(be.lib.ibcu_linear(be.ctx, descs, n, dx.ptr, N, B, bits))
    be.sync()
    for do, want, M in zip(outs, wants, Ms):
        Mr = max(M, 1)
        got = be.download(do, np.float32, B * Mr).reshape(B, Mr)
        assert _cpu.close(got[:, :M], want, RTOL, ATOL), (M, float(np.max(np.abs(got[:, :M] - want))) if M else 0)
        if M == 0:
            assert np.all(got == -3.0)


@pytest.mark.parametrize("bits,M,N,B", [(8, 32000, 4096, 1), (8, 48, 65536, 2), (4, 40, 131072, 1), (8, 200, 16384, 6)])
def test_full_size_head_and_rows_longer_than_shared_memory(backend, cpu_libs, bits, M, N, B):
    """The LM-head shape against the scalar restatement, and rows whose limbs do not fit one block's shared
    memory (columns split over several blocks, integer partial sums recombined by linear_finalize_kernel)."""
    rng = np.random.default_rng(bits * 13 + M + N + B)
    w, s16, x = (_cpu.make_int8_case if bits == 8 else _cpu.make_int4_case)(rng, M, N, B)
    got = backend.linear(w, s16, x, bits)
    want = oracle_linear(cpu_libs, w, s16, x, bits)
    assert _cpu.close(got, want, RTOL, ATOL * max(1.0, float(np.abs(want).max()))), float(np.max(np.abs(got - want)))


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,G,K_out,eps", [
    (4096, 4096, 128, 0, 0.0),        # attention projection of the 7B shape, groups of 128
    (5632, 2048, 64, 8, 0.0),         # TinyLlama up_proj shape with eight outlier columns per row
    (4099, 14336, 32, 0, 0.0),        # rows not a multiple of the four a warp carries; rows longer than one pass of the lanes
    (1000, 4096, 128, 16, 0.05),      # groups under 5 % of the largest activation are left out
    (33, 96, 32, 3, 0.0), (40, 48, 16, 2, 0.0), (17, 200, 8, 0, 0.2),   # small shapes; the last two take the generic kernel
])
def test_group_scaled_int4_rows(backend, cpu_libs, M, N, G, K_out, eps):
    """Group-scaled INT4 rows of the reference's session engine (src/pq_decode.c:3565-3651; skip rule :3854-3882) against
    their restatement (parity unpinned: static functions in the reference), within the float bar."""
    rng = np.random.default_rng(M + N + G + K_out)
    q, s, x, oi, ov = _cpu.make_int4g_case(rng, M, N, G, K_out)
    if eps:
        x[: N // 4] *= 1e-3                                   # a quarter of the groups fall under the threshold
    got = backend.int4g_matmul(q, s, G, x, oi, ov, eps)
    want = _cpu.oracle_int4g(cpu_libs.oracle, q, s, G, x, oi, ov, eps)
    assert _cpu.close(got, want, RTOL, ATOL), float(np.max(np.abs(got - want)))
    if eps:                                                   # the rule is visible: without it the result differs
        full = _cpu.oracle_int4g(cpu_libs.oracle, q, s, G, x, oi, ov, 0.0)
        assert not np.array_equal(full, want)
    assert np.array_equal(got, backend.int4g_matmul(q, s, G, x, oi, ov, eps))       # same bits again
    # linearity at full size: f(2x) = 2 f(x) exactly (every product and sum scales by a power of two)
    assert np.array_equal(backend.int4g_matmul(q, s, G, 2.0 * x, oi, ov, eps), 2.0 * got)
