// Per-row-scaled INT4 / INT8 linear layers for 1..32 FP32 activations.
//
// Data in HBM: weights keep the reference layout bit for bit (INT8 row-major; INT4 two columns per
// byte, low nibble first, bias 8), scales are FP16 (or FP32) per output row.
//
// Fast path (linear_mma_kernel): HBM-bound streaming of the weights with 128-bit no-allocate loads.
// Every lane unpacks its 16 bytes in registers to exact fp16 pairs with the "1024 + n" bit trick
// (PRMT/LOP3 + one HSUB2/HFMA2 per pair) and feeds them to mma.sync.m16n8k16 (fp16 in, fp32
// accumulate). The eight MMA columns carry the FP32 activations as exact fp16 pieces
// (x * 2^-e = hi + mid [+ lo], written once per call by xprep_kernel), so the product is FP32-grade
// while costing ~1.3 issue slots per weight instead of ~3 for convert + FFMA.
// Because a dot product is invariant under a permutation of k applied to both operands, each lane
// simply owns 16 contiguous bytes of a row; no shared-memory transpose or ldmatrix is needed.
// K is split over the warps of a CTA and, for short/wide tensors, over the CTAs of a thread-block
// cluster; partial sums meet in shared memory / distributed shared memory in a fixed order.
//
// Portable path (linear_generic_kernel): one warp per output row, plain FP32 FMAs; used for shapes
// the fast path does not take (row bytes not a multiple of 16, unaligned pointers) and by tests.
#include "common.cuh"
#include <cooperative_groups.h>
namespace cg = cooperative_groups;

namespace {

struct LinTensor {
    const uint8_t* w;
    const void* scales;
    float* out;
    int M, out_stride, scales_fp32, epilogue;
    int rg_start;                  // first row-group of this tensor in the launch
};

struct LinearParams {
    LinTensor t[4];
    int n_tensors;
    int rowbytes;                  // bytes per weight row
    int nkb;                       // 64-byte k-blocks per row
    int B, P, ncols;               // activations, fp16 pieces per activation, B*P
    const __half* xpack;           // [ncols][xld] fp16 pieces, fragment order
    int xld;
    const float* xscale;           // [B] power-of-two factor removed from x
    int ks;                        // cluster size = CTAs sharing one row-group
};

// ── activation split ────────────────────────────────────────────────────────────────────
// One CTA per activation vector. x is scaled by a power of two so that its largest magnitude
// lands in [2^14, 2^15) (exact, keeps fp16 away from overflow and from its subnormals), then split
// into P fp16 pieces whose sum reproduces x to 2^-22 (P = 2) or better (P = 3) relative.
// perm8 != 0 stores each aligned group of 8 columns as [c0,c4,c1,c5,c2,c6,c3,c7], the order in
// which the INT4 unpack yields its nibbles.
__global__ void __launch_bounds__(1024) xprep_kernel(const float* __restrict__ x, int N, int n_pad, int P, int perm8,
                                                    __half* __restrict__ xpack, float* __restrict__ xscale) {
    __shared__ float red[32];
    __shared__ float s_mul;
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x;
    const float* xb = x + (size_t)b * N;
    float amax = 0.0f;
    for (int j = threadIdx.x; j < N; j += blockDim.x) amax = fmaxf(amax, fabsf(xb[j]));
    amax = warp_max(amax);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.0f;
        v = warp_max(v);
        if (threadIdx.x == 0) {
            int ex = 0;
            float mul = 1.0f, back = 1.0f;
            if (v > 0.0f && v < INFINITY) {
                frexpf(v, &ex);                       // v = m * 2^ex, m in [0.5, 1)
                int sh = 15 - ex;
                sh = sh > 100 ? 100 : (sh < -100 ? -100 : sh);
                mul = ldexpf(1.0f, sh);
                back = ldexpf(1.0f, -sh);
            }
            s_mul = mul;
            xscale[b] = back;
        }
    }
    __syncthreads();
    const float mul = s_mul;
    for (int j = threadIdx.x; j < n_pad; j += blockDim.x) {
        float v = j < N ? xb[j] * mul : 0.0f;
        int jj = perm8 ? ((j & ~7) | (((j & 3) << 1) | ((j >> 2) & 1))) : j;
#pragma unroll 3
        for (int p = 0; p < P; p++) {
            __half h = __float2half_rn(v);
            xpack[(size_t)(b * P + p) * n_pad + jj] = h;
            v -= __half2float(h);
        }
    }
}

// ── register unpack ─────────────────────────────────────────────────────────────────────
__device__ __forceinline__ uint32_t hsub2_u32(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t hfma2_u32(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
// four int8 -> (w0,w1), (w2,w3) as exact fp16 pairs
__device__ __forceinline__ void unpack_int8x4(uint32_t raw, uint32_t& h01, uint32_t& h23) {
    uint32_t u = raw ^ 0x80808080u;                          // w + 128 as unsigned bytes
    h01 = hsub2_u32(__byte_perm(u, 0x64646464u, 0x4140), 0x64806480u);   // (1024 + u) - 1152
    h23 = hsub2_u32(__byte_perm(u, 0x64646464u, 0x4342), 0x64806480u);
}
// eight nibbles n0..n7 -> (n0,n4), (n1,n5), (n2,n6), (n3,n7), each minus 8, as exact fp16 pairs
__device__ __forceinline__ void unpack_int4x8(uint32_t raw, uint32_t& a, uint32_t& b, uint32_t& c, uint32_t& d) {
    uint32_t hi = raw >> 8;
    a = hsub2_u32((raw & 0x000F000Fu) | 0x64006400u, 0x64086408u);                 // (1024 + n) - 1032
    b = hfma2_u32((raw & 0x00F000F0u) | 0x64006400u, 0x2C002C00u, 0xD480D480u);    // (1024 + 16n)/16 - 72
    c = hsub2_u32((hi & 0x000F000Fu) | 0x64006400u, 0x64086408u);
    d = hfma2_u32((hi & 0x00F000F0u) | 0x64006400u, 0x2C002C00u, 0xD480D480u);
}
__device__ __forceinline__ void mma16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t u4_get(const uint4& v, int i) { return i == 0 ? v.x : (i == 1 ? v.y : (i == 2 ? v.z : v.w)); }

// ── fast path ───────────────────────────────────────────────────────────────────────────
// BITS: 4 or 8. NCG: groups of 8 MMA columns (ceil(B*P/8)). RT: 16-row tiles per warp.
// W: warps per CTA (all on the same RT*16 rows, interleaved over 64-byte k-blocks).
// U: k-blocks loaded per batch.
template <int BITS, int NCG, int RT, int W, int U>
__global__ void __launch_bounds__(W * 32) linear_mma_kernel(const LinearParams p) {
    constexpr int ROWS = RT * 16;
    constexpr int COLS = NCG * 8;
    constexpr int XK = BITS == 8 ? 64 : 128;                  // activation columns per k-block
    extern __shared__ __align__(16) float smem[];             // [W][ROWS][COLS] partials, then [ROWS][COLS]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    pdl_launch_dependents();

    const int ks = p.ks;
    const int rg = blockIdx.x / ks;
    const int crank = blockIdx.x - rg * ks;
    int ti = 0;
#pragma unroll
    for (int i = 1; i < 4; i++) if (i < p.n_tensors && rg >= p.t[i].rg_start) ti = i;
    const LinTensor T = p.t[ti];
    const int row0 = (rg - T.rg_start) * ROWS;

    const uint8_t* rowp[RT * 2];
#pragma unroll
    for (int j = 0; j < RT * 2; j++) {
        int r = row0 + (j >> 1) * 16 + (j & 1) * 8 + g;
        r = r < T.M ? r : T.M - 1;
        rowp[j] = T.w + (size_t)r * p.rowbytes + 16 * t;
    }
    const __half* xcol[NCG];
#pragma unroll
    for (int c = 0; c < NCG; c++) {
        int col = c * 8 + g;
        col = col < p.ncols ? col : 0;                        // spare MMA columns reread column 0
        xcol[c] = p.xpack + (size_t)col * p.xld + (XK / 4) * t;
    }
    float acc[RT][NCG][4];
#pragma unroll
    for (int i = 0; i < RT; i++)
#pragma unroll
        for (int c = 0; c < NCG; c++) { acc[i][c][0] = acc[i][c][1] = acc[i][c][2] = acc[i][c][3] = 0.0f; }

    const int S = ks * W;
    const uint32_t fill = BITS == 8 ? 0u : 0x88888888u;      // encodes weight 0
    bool waited = false;
    for (int kb0 = crank * W + warp; kb0 < p.nkb; kb0 += S * U) {
        uint4 wreg[U][RT * 2];
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int kb = kb0 + u * S;
            const bool in = kb < p.nkb && kb * 64 + 16 * t < p.rowbytes;
#pragma unroll
            for (int j = 0; j < RT * 2; j++)
                wreg[u][j] = in ? ld_stream_u4(rowp[j] + (size_t)kb * 64) : make_uint4(fill, fill, fill, fill);
        }
        if (!waited) { pdl_wait(); waited = true; }          // weights are in flight; now x may be read
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int kb = kb0 + u * S;
            if (kb >= p.nkb) break;
            if (BITS == 8) {
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    uint4 xf[NCG];
#pragma unroll
                    for (int c = 0; c < NCG; c++) xf[c] = *reinterpret_cast<const uint4*>(xcol[c] + (size_t)kb * XK + 8 * h);
#pragma unroll
                    for (int s = 0; s < 2; s++) {
                        uint32_t lo[RT * 2], hi[RT * 2];
#pragma unroll
                        for (int j = 0; j < RT * 2; j++) unpack_int8x4(u4_get(wreg[u][j], 2 * h + s), lo[j], hi[j]);
#pragma unroll
                        for (int i = 0; i < RT; i++)
#pragma unroll
                            for (int c = 0; c < NCG; c++)
                                mma16816(acc[i][c], lo[2 * i], lo[2 * i + 1], hi[2 * i], hi[2 * i + 1],
                                         s ? xf[c].z : xf[c].x, s ? xf[c].w : xf[c].y);
                    }
                }
            } else {
#pragma unroll
                for (int wd = 0; wd < 4; wd++) {
                    uint4 xf[NCG];
#pragma unroll
                    for (int c = 0; c < NCG; c++) xf[c] = *reinterpret_cast<const uint4*>(xcol[c] + (size_t)kb * XK + 8 * wd);
                    uint32_t qa[RT * 2], qb[RT * 2], qc[RT * 2], qd[RT * 2];
#pragma unroll
                    for (int j = 0; j < RT * 2; j++) unpack_int4x8(u4_get(wreg[u][j], wd), qa[j], qb[j], qc[j], qd[j]);
#pragma unroll
                    for (int i = 0; i < RT; i++)
#pragma unroll
                        for (int c = 0; c < NCG; c++) {
                            mma16816(acc[i][c], qa[2 * i], qa[2 * i + 1], qb[2 * i], qb[2 * i + 1], xf[c].x, xf[c].y);
                            mma16816(acc[i][c], qc[2 * i], qc[2 * i + 1], qd[2 * i], qd[2 * i + 1], xf[c].z, xf[c].w);
                        }
                }
            }
        }
    }
    if (!waited) pdl_wait();

    // per-warp partials -> shared memory
    float* part = smem + (size_t)warp * ROWS * COLS;
#pragma unroll
    for (int i = 0; i < RT; i++)
#pragma unroll
        for (int c = 0; c < NCG; c++) {
            *reinterpret_cast<float2*>(part + (i * 16 + g) * COLS + c * 8 + 2 * t) = make_float2(acc[i][c][0], acc[i][c][1]);
            *reinterpret_cast<float2*>(part + (i * 16 + g + 8) * COLS + c * 8 + 2 * t) = make_float2(acc[i][c][2], acc[i][c][3]);
        }
    __syncthreads();
    // sum over the warps in warp order; result lands in warp 0's slab
    for (int e = threadIdx.x; e < ROWS * COLS; e += W * 32) {
        float s = smem[e];
#pragma unroll
        for (int w = 1; w < W; w++) s += smem[(size_t)w * ROWS * COLS + e];
        smem[e] = s;
    }
    if (ks > 1) cg::this_cluster().sync(); else __syncthreads();

    if (crank == 0) {
        const int B = p.B, P = p.P;
        for (int e = threadIdx.x; e < ROWS * B; e += W * 32) {
            const int b = e / ROWS, r = e - b * ROWS;
            const int row = row0 + r;
            if (row >= T.M) continue;
            float y = 0.0f;
            for (int k = 0; k < ks; k++) {
                const float* src = k == 0 ? smem : cg::this_cluster().map_shared_rank(smem, k);
                for (int q = 0; q < P; q++) y += src[r * COLS + b * P + q];
            }
            const float sc = T.scales_fp32 ? reinterpret_cast<const float*>(T.scales)[row]
                                           : __half2float(reinterpret_cast<const __half*>(T.scales)[row]);
            y = y * p.xscale[b] * sc;
            float* o = T.out + (size_t)b * T.out_stride + row;
            *o = T.epilogue == IBCU_EPI_ADD ? *o + y : y;
        }
    }
    if (ks > 1) cg::this_cluster().sync();                    // keep remote shared memory alive until read
}

// ── portable path ───────────────────────────────────────────────────────────────────────
// One warp per output row; lanes stride over the columns; FP32 FMAs; activations straight from x.
template <int BITS>
__global__ void __launch_bounds__(256) linear_generic_kernel(LinTensor T, const float* __restrict__ x, int N, int B) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= T.M) return;
    const size_t rowbytes = BITS == 8 ? (size_t)N : (size_t)(N / 2);
    const uint8_t* wr = T.w + (size_t)row * rowbytes;
    const float sc = T.scales_fp32 ? reinterpret_cast<const float*>(T.scales)[row]
                                   : __half2float(reinterpret_cast<const __half*>(T.scales)[row]);
    for (int b = 0; b < B; b++) {
        const float* xb = x + (size_t)b * N;
        float s = 0.0f;
        if (BITS == 8) {
            for (int j = lane; j < N; j += 32) s = fmaf((float)(int8_t)wr[j], xb[j], s);
        } else {
            for (int j = 2 * lane; j < N; j += 64) {
                uint8_t v = wr[j >> 1];
                s = fmaf((float)((int)(v & 15) - 8), xb[j], s);
                if (j + 1 < N) s = fmaf((float)((int)(v >> 4) - 8), xb[j + 1], s);
            }
        }
        s = warp_sum(s);
        if (lane == 0) {
            float y = s * sc;
            float* o = T.out + (size_t)b * T.out_stride + row;
            *o = T.epilogue == IBCU_EPI_ADD ? *o + y : y;
        }
    }
}

template <int BITS, int NCG, int RT, int W, int U>
int launch_mma(ibcu_ctx* ctx, const LinearParams& p, int total_rg) {
    auto kern = linear_mma_kernel<BITS, NCG, RT, W, U>;
    size_t smem = (size_t)W * RT * 16 * NCG * 8 * sizeof(float);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return ibcu_fail(ctx, IBCU_ERR_CUDA, "cudaFuncSetAttribute(smem=%zu): %s", smem, cudaGetErrorString(e));
    }
    return ibcu_launch(ctx, kern, dim3(total_rg * p.ks), dim3(W * 32), smem, p.ks, true, p);
}

template <int BITS, int NCG>
int dispatch_shape(ibcu_ctx* ctx, const LinearParams& p, int total_rg, int rt) {
    if (rt == 2) return launch_mma<BITS, NCG, 2, 8, 2>(ctx, p, total_rg);
    return launch_mma<BITS, NCG, 1, 8, 2>(ctx, p, total_rg);
}

}  // namespace

// Tuning knobs read once from the environment (for sweeps; defaults are the measured best).
static int env_int(const char* name, int dflt) {
    const char* v = getenv(name);
    return v && *v ? atoi(v) : dflt;
}

extern "C" void ibcu_linear_force_generic(ibcu_ctx* ctx, int on) { if (ctx) ctx->force_generic = on; }

extern "C" int ibcu_linear(ibcu_ctx* ctx, const ibcu_linear_t* tensors, int n_tensors,
                           const float* x, int N, int B, int bits) {
    IBCU_CHECK_CTX(ctx);
    IBCU_REQUIRE(ctx, tensors && x, "ibcu_linear: null pointer");
    IBCU_REQUIRE(ctx, n_tensors >= 1 && n_tensors <= 4, "ibcu_linear: n_tensors=%d not in 1..4", n_tensors);
    IBCU_REQUIRE(ctx, bits == 4 || bits == 8, "ibcu_linear: bits=%d (4 or 8 supported)", bits);
    IBCU_REQUIRE(ctx, B >= 1 && B <= 32, "ibcu_linear: B=%d not in 1..32", B);
    IBCU_REQUIRE(ctx, N >= 1 && (bits == 8 || (N & 1) == 0), "ibcu_linear: N=%d invalid for %d-bit rows", N, bits);
    for (int i = 0; i < n_tensors; i++) {
        IBCU_REQUIRE(ctx, tensors[i].w && tensors[i].scales && tensors[i].out, "ibcu_linear: tensor %d has a null pointer", i);
        IBCU_REQUIRE(ctx, tensors[i].M >= 0 && tensors[i].out_stride >= tensors[i].M, "ibcu_linear: tensor %d M=%d stride=%d", i, tensors[i].M, tensors[i].out_stride);
    }
    const int rowbytes = bits == 8 ? N : N / 2;
    bool fast = !ctx->force_generic && (rowbytes % 16 == 0);
    for (int i = 0; i < n_tensors; i++) if (((uintptr_t)tensors[i].w & 15) != 0) fast = false;

    if (!fast) {
        for (int i = 0; i < n_tensors; i++) {
            if (tensors[i].M == 0) continue;
            LinTensor T = { (const uint8_t*)tensors[i].w, tensors[i].scales, tensors[i].out, tensors[i].M,
                            tensors[i].out_stride, tensors[i].scales_fp32, tensors[i].epilogue, 0 };
            dim3 grid((tensors[i].M + 7) / 8);
            int rc = bits == 8 ? ibcu_launch(ctx, linear_generic_kernel<8>, grid, dim3(256), 0, 1, true, T, x, N, B)
                               : ibcu_launch(ctx, linear_generic_kernel<4>, grid, dim3(256), 0, 1, true, T, x, N, B);
            if (rc) return rc;
        }
        return IBCU_OK;
    }

    // fast path: split activations, then stream the weights
    const int P = B <= 2 ? 3 : 2;
    const int ncols = B * P;
    const int ncg = ncols <= 8 ? 1 : (ncols <= 16 ? 2 : (ncols <= 32 ? 4 : 8));
    const int nkb = (rowbytes + 63) / 64;
    const int xk = bits == 8 ? 64 : 128;
    const int xld = nkb * xk;
    size_t xbytes = (size_t)ncols * xld * sizeof(__half);
    xbytes = (xbytes + 255) & ~(size_t)255;
    int rc = ibcu_reserve(ctx, &ctx->xpack, &ctx->xpack_bytes, xbytes + 32 * sizeof(float));
    if (rc) return rc;
    __half* xpack = (__half*)ctx->xpack;
    float* xscale = (float*)((char*)ctx->xpack + xbytes);
    int threads = N >= 4096 ? 1024 : (N >= 1024 ? 512 : 128);
    rc = ibcu_launch(ctx, xprep_kernel, dim3(B), dim3(threads), 0, 1, true, x, N, xld, P, bits == 4 ? 1 : 0, xpack, xscale);
    if (rc) return rc;

    static const int rt_env = env_int("IBCU_LINEAR_RT", 0);
    static const int ks_env = env_int("IBCU_LINEAR_KS", 0);
    long total_rows = 0;
    for (int i = 0; i < n_tensors; i++) total_rows += tensors[i].M;
    int rt = rt_env ? rt_env : ((ncg >= 8 || total_rows < 32L * ctx->sm_count) ? 1 : 2);
    const int rows_per_rg = rt * 16;
    LinearParams p;
    memset(&p, 0, sizeof p);
    int total_rg = 0;
    for (int i = 0; i < n_tensors; i++) {
        p.t[i] = { (const uint8_t*)tensors[i].w, tensors[i].scales, tensors[i].out, tensors[i].M,
                   tensors[i].out_stride, tensors[i].scales_fp32, tensors[i].epilogue, total_rg };
        total_rg += (tensors[i].M + rows_per_rg - 1) / rows_per_rg;
    }
    if (total_rg == 0) return IBCU_OK;
    p.n_tensors = n_tensors; p.rowbytes = rowbytes; p.nkb = nkb; p.B = B; p.P = P; p.ncols = ncols;
    p.xpack = xpack; p.xld = xld; p.xscale = xscale;
    // cluster split of K: enough CTAs to fill the machine a few times over, at least 2 k-blocks per warp
    int ks = 1;
    while (ks < 8 && total_rg * ks < 4 * ctx->sm_count && nkb / (ks * 2 * 8) >= 2) ks *= 2;
    if (ks_env) ks = ks_env;
    p.ks = ks;

#define IBCU_DISPATCH(BITS) \
    switch (ncg) { \
        case 1: rc = dispatch_shape<BITS, 1>(ctx, p, total_rg, rt); break; \
        case 2: rc = dispatch_shape<BITS, 2>(ctx, p, total_rg, rt); break; \
        case 4: rc = dispatch_shape<BITS, 4>(ctx, p, total_rg, rt); break; \
        default: rc = dispatch_shape<BITS, 8>(ctx, p, total_rg, rt); break; \
    }
    if (bits == 8) { IBCU_DISPATCH(8) } else { IBCU_DISPATCH(4) }
#undef IBCU_DISPATCH
    return rc;
}

// v1: the two projections in one launch, then the element-wise kernel over gate.out.
extern "C" int ibcu_linear_gate_up_silu(ibcu_ctx* ctx, const ibcu_linear_t* gate_up, const float* x, int N, int B, int bits) {
    IBCU_CHECK_CTX(ctx);
    IBCU_REQUIRE(ctx, gate_up && gate_up[0].M == gate_up[1].M && gate_up[0].out_stride == gate_up[1].out_stride,
                 "ibcu_linear_gate_up_silu: gate and up must have equal shapes");
    IBCU_REQUIRE(ctx, gate_up[0].epilogue == IBCU_EPI_STORE && gate_up[1].epilogue == IBCU_EPI_STORE, "ibcu_linear_gate_up_silu: store epilogue only");
    int rc = ibcu_linear(ctx, gate_up, 2, x, N, B, bits);
    if (rc) return rc;
    return ibcu_silu_mul(ctx, gate_up[0].out, gate_up[0].out, gate_up[1].out,
                         (size_t)(B - 1) * gate_up[0].out_stride + gate_up[0].M);
}
