// INT4 weights x INT8 activations (the reference's default route for INT4 linears): activations are
// quantised per 128-column group on the device, group dot products are exact int32, and the per-row
// FP32 accumulation over groups runs in group order with separately rounded multiply and add, so the
// results equal the reference's scalar kernel bit for bit.
#include "common.cuh"

namespace {

// one warp per (activation, group of 128)
__global__ void __launch_bounds__(256) quantize_g128_kernel(const float* __restrict__ x, int8_t* __restrict__ q, float* __restrict__ sa,
                                                            int N, int groups, int total) {
    pdl_launch_dependents();
    pdl_wait();
    const int wid = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (wid >= total) return;
    const int b = wid / groups, g = wid - b * groups;
    const int lo = g * 128, hi = min(lo + 128, N);
    const float* xb = x + (size_t)b * N;
    float v[4];
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int j = lo + lane + 32 * i;
        v[i] = j < hi ? xb[j] : 0.0f;
        amax = fmaxf(amax, fabsf(v[i]));
    }
    amax = warp_max(amax);
    float scale, inv = 0.0f;
    const bool dead = amax < 1e-10f;
    if (dead) scale = 1e-10f;
    else { scale = __fdiv_rn(amax, 127.0f); inv = __fdiv_rn(1.0f, scale); }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int j = lo + lane + 32 * i;
        if (j >= hi) continue;
        int qi = 0;
        if (!dead) {
            qi = __float2int_rz(__fadd_rn(__fmul_rn(v[i], inv), v[i] >= 0.0f ? 0.5f : -0.5f));
            qi = max(-127, min(127, qi));
        }
        q[(size_t)b * N + j] = (int8_t)qi;
    }
    if (lane == 0) sa[(size_t)b * groups + g] = scale;
}

// one warp per output row; lanes split each 128-column group (4 columns = 2 weight bytes per lane)
__global__ void __launch_bounds__(256) w4a8_kernel(const uint8_t* __restrict__ w, const void* __restrict__ scales, int scales_fp32,
                                                   float* __restrict__ out, int M, int out_stride, int epilogue,
                                                   const int8_t* __restrict__ xq, const float* __restrict__ sa, int N, int B) {
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= M) return;
    const int groups = (N + 127) / 128;
    const uint8_t* wr = w + (size_t)row * (N / 2);
    const float sw = scales_fp32 ? reinterpret_cast<const float*>(scales)[row]
                                 : __half2float(reinterpret_cast<const __half*>(scales)[row]);
    for (int b = 0; b < B; b++) {
        const int8_t* xb = xq + (size_t)b * N;
        float acc = 0.0f;
        for (int g = 0; g < groups; g++) {
            const int j = g * 128 + 4 * lane;
            int dot = 0;
#pragma unroll
            for (int u = 0; u < 2; u++) {
                const int jj = j + 2 * u;
                if (jj < N) {
                    const uint8_t byte = wr[jj >> 1];
                    dot += ((int)(byte & 15) - 8) * (int)xb[jj];
                    if (jj + 1 < N) dot += ((int)(byte >> 4) - 8) * (int)xb[jj + 1];
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
            acc = __fadd_rn(acc, __fmul_rn((float)dot, sa[(size_t)b * groups + g]));
        }
        if (lane == 0) {
            const float y = __fmul_rn(acc, sw);
            float* o = out + (size_t)b * out_stride + row;
            *o = epilogue == IBCU_EPI_ADD ? *o + y : y;
        }
    }
}


// ── tensor-core path ────────────────────────────────────────────────────────────────────
// The same exact arithmetic on the integer tensor cores. A group of 128 columns is 64 weight bytes, one
// k-block; mma.sync.m16n8k32 (u8 x s8 -> s32) gives the group's dot product for 16 rows and up to 8
// activations from four instructions: raw & 0x0F0F0F0F are the even columns, raw & 0xF0F0F0F0 sixteen
// times the odd ones (separate accumulator, shifted back exactly), and the nibble bias 8 comes off as
// 8 * (sum of the group's activation bytes). The group dot products of a tile of rows are parked in
// shared memory, [group][row][activation]; one thread per (row, activation) then walks the groups in
// order with separately rounded multiply and add, which is the reference's own sequence of roundings.
// Block = 8 warps, a run of rows walked in tiles of 16; weights stream through a cp.async ring of
// (16 rows x 512 bytes) stages, warp w taking k-block w of every stage.
constexpr int WT_W = 8, WT_R = 16, WT_SK = WT_W * 64, WT_LD = WT_SK + 64;

__device__ __forceinline__ void wt_imma_u8(int* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void wt_cp16(uint32_t smem_dst, const void* gsrc, bool valid) {
    const int n = valid ? 16 : 0;                             // 0 source bytes -> 16 zero bytes
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"(smem_dst), "l"(gsrc), "r"(n) : "memory");
}
__device__ __forceinline__ uint32_t wt_word(const uint4& v, int i) { return i == 0 ? v.x : (i == 1 ? v.y : (i == 2 ? v.z : v.w)); }

struct WtParams {
    const uint8_t* w; const void* scales; int scales_fp32;
    float* out; int M, out_stride, epilogue;
    const int8_t* xq; const float* sa;                        // [B][N], [B][groups]
    const float* xf;                                          // not NULL: FP32 activations [B][N], quantised per group by every block for itself (xq, sa unused)
    int N, B, groups, rows_per_block, xs_ld;
    int dld;                                                  // words per row of the parked dot products: B made odd, so that rows fall on different banks
};

template <int STAGES, int RT>
__global__ void __launch_bounds__(WT_W * 32) w4a8_mma_kernel(const WtParams p) {
    constexpr int R = WT_R * RT;                              // rows per tile
    constexpr int STAGE_BYTES = R * WT_LD;
    constexpr int CPR = WT_SK / 16;                           // 16-byte chunks per row per stage
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    pdl_launch_dependents();
    const int row_begin = blockIdx.x * p.rows_per_block, row_end = min(p.M, row_begin + p.rows_per_block);
    const int nk = p.groups, nst = (nk + WT_W - 1) / WT_W;
    const int rowbytes = p.N / 2;
    unsigned char* ring = smem_raw;
    int* gdot = reinterpret_cast<int*>(smem_raw + STAGES * STAGE_BYTES);                      // [groups][R][dld]
    int* qsum = gdot + (((size_t)nk * R * p.dld + 3) & ~(size_t)3);                           // [B][groups] 8 x sums of the groups' activation bytes
    float* s_sa = reinterpret_cast<float*>(qsum + (((size_t)p.B * nk + 3) & ~(size_t)3));     // [B][groups]
    int8_t* xs = reinterpret_cast<int8_t*>(s_sa + (((size_t)p.B * nk + 3) & ~(size_t)3));     // [B][xs_ld], columns of every 8 as c0,c2,c4,c6,c1,c3,c5,c7

    // producer: this thread owns chunk column cc of rows pr + 8 i of every stage
    const int cc = threadIdx.x % CPR, pr = threadIdx.x / CPR;
    const uint32_t ring_u32 = (uint32_t)__cvta_generic_to_shared(ring) + pr * WT_LD + cc * 16;
    int pf_row = row_begin, pf_it = 0, pf_slot = 0;
    auto pf_issue = [&]() {
        if (pf_row < row_end) {
            const int rows = min(R, row_end - pf_row);
            const bool kv = pf_it * WT_SK + cc * 16 < rowbytes;
            const uint32_t d = ring_u32 + pf_slot * STAGE_BYTES;
#pragma unroll
            for (int i = 0; i < 2 * RT; i++) {
                const bool v = kv && pr + 8 * i < rows;
                const uint8_t* src = p.w + (size_t)(pf_row + (v ? pr + 8 * i : 0)) * rowbytes + (v ? (size_t)pf_it * WT_SK + cc * 16 : 0);
                wt_cp16(d + i * 8 * WT_LD, src, v);
            }
            pf_slot = pf_slot + 1 == STAGES ? 0 : pf_slot + 1;
            if (++pf_it == nst) { pf_it = 0; pf_row += rows; }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
#pragma unroll
    for (int s = 0; s < STAGES - 1; s++) pf_issue();          // weights first: they do not depend on the activations
    pdl_wait();

    // activations: bytes of every 8 columns reordered to evens then odds; per group 8 x the sum of its bytes and its scale
    if (p.xf) {
        // the reference's quantiser (src/threading.c:401-432) on the fly: a warp per (activation, group of 128 columns),
        // scale = max|x| / 127 (1e-10 and all zeros for a dead group), round half away from zero, clamp to +-127
        for (int e = warp; e < p.B * nk; e += WT_W) {
            const int b = e / nk, k = e % nk;
            const float4 v = *reinterpret_cast<const float4*>(p.xf + (size_t)b * p.N + (size_t)k * 128 + 4 * lane);
            const float amax = warp_max(fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
            const bool dead = amax < 1e-10f;
            const float scale = dead ? 1e-10f : __fdiv_rn(amax, 127.0f);
            const float inv = dead ? 0.0f : __fdiv_rn(1.0f, scale);
            const float f[4] = { v.x, v.y, v.z, v.w };
            int q[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                int qi = 0;
                if (!dead) {
                    qi = __float2int_rz(__fadd_rn(__fmul_rn(f[i], inv), f[i] >= 0.0f ? 0.5f : -0.5f));
                    qi = max(-127, min(127, qi));
                }
                q[i] = qi;
            }
            // lane holds columns 4 lane .. 4 lane + 3: the even lane of a pair has c0..c3 of its 8 columns, the odd lane c4..c7
            const uint32_t mine = (uint32_t)(q[0] & 255) | ((uint32_t)(q[1] & 255) << 8) | ((uint32_t)(q[2] & 255) << 16) | ((uint32_t)(q[3] & 255) << 24);
            const uint32_t other = __shfl_xor_sync(0xffffffffu, mine, 1);
            const uint32_t lo = (lane & 1) ? other : mine, hi = (lane & 1) ? mine : other;
            if ((lane & 1) == 0)
                *reinterpret_cast<uint2*>(xs + (size_t)b * p.xs_ld + (size_t)k * 128 + 4 * lane) =
                    make_uint2(__byte_perm(lo, hi, 0x6420), __byte_perm(lo, hi, 0x7531));
            int ssum = q[0] + q[1] + q[2] + q[3];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ssum += __shfl_xor_sync(0xffffffffu, ssum, o);
            if (lane == 0) { qsum[e] = 8 * ssum; s_sa[e] = scale; }
        }
    } else {
        for (int e = threadIdx.x; e < p.B * (p.N / 8); e += WT_W * 32) {
            const int b = e / (p.N / 8), c8 = e % (p.N / 8);
            const uint2 v = *reinterpret_cast<const uint2*>(p.xq + (size_t)b * p.N + (size_t)c8 * 8);
            const uint2 o = make_uint2(__byte_perm(v.x, v.y, 0x6420), __byte_perm(v.x, v.y, 0x7531));
            *reinterpret_cast<uint2*>(xs + (size_t)b * p.xs_ld + (size_t)c8 * 8) = o;
        }
        for (int e = threadIdx.x; e < p.B * nk; e += WT_W * 32) {
            const int b = e / nk, k = e % nk;
            const int4* q4 = reinterpret_cast<const int4*>(p.xq + (size_t)b * p.N + (size_t)k * 128);
            int s = 0;
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const int4 v = q4[i];
                s = __dp4a(v.x, 0x01010101, s); s = __dp4a(v.y, 0x01010101, s); s = __dp4a(v.z, 0x01010101, s); s = __dp4a(v.w, 0x01010101, s);
            }
            qsum[e] = 8 * s;
            s_sa[e] = p.sa[e];
        }
    }
    __syncthreads();
    const int col = g < p.B ? g : 0;                          // spare MMA columns reread activation 0
    const int8_t* xcol = xs + (size_t)col * p.xs_ld + 32 * t;

    int slot = 0;
    for (int row0 = row_begin; row0 < row_end; row0 += R) {
        const int tile_rows = min(R, row_end - row0);
        for (int it = 0; it < nst; it++) {
            asm volatile("cp.async.wait_group %0;" :: "n"(STAGES - 2) : "memory");
            __syncthreads();                                  // this stage has landed for everyone; the previous one is free
            pf_issue();
            const int k = it * WT_W + warp;                   // this warp's group
            if (k < nk) {
                const unsigned char* sw = ring + slot * STAGE_BYTES + warp * 64 + 16 * t;
                uint4 xf[2];
#pragma unroll
                for (int h = 0; h < 2; h++) xf[h] = *reinterpret_cast<const uint4*>(xcol + (size_t)k * 128 + 16 * h);
                int* d = gdot + (size_t)k * R * p.dld;
#pragma unroll
                for (int i = 0; i < RT; i++) {
                    const uint4 c0 = *reinterpret_cast<const uint4*>(sw + (i * 16 + g) * WT_LD);
                    const uint4 c1 = *reinterpret_cast<const uint4*>(sw + (i * 16 + g + 8) * WT_LD);
                    int lo[4] = { 0, 0, 0, 0 }, hi[4] = { 0, 0, 0, 0 };
#pragma unroll
                    for (int h = 0; h < 2; h++) {
                        const uint32_t r0a = wt_word(c0, 2 * h), r0b = wt_word(c0, 2 * h + 1);
                        const uint32_t r1a = wt_word(c1, 2 * h), r1b = wt_word(c1, 2 * h + 1);
                        wt_imma_u8(lo, r0a & 0x0F0F0F0Fu, r1a & 0x0F0F0F0Fu, r0b & 0x0F0F0F0Fu, r1b & 0x0F0F0F0Fu, xf[h].x, xf[h].z);
                        wt_imma_u8(hi, r0a & 0xF0F0F0F0u, r1a & 0xF0F0F0F0u, r0b & 0xF0F0F0F0u, r1b & 0xF0F0F0F0u, xf[h].y, xf[h].w);
                    }
                    if (2 * t < p.B) {
                        d[(i * 16 + g) * p.dld + 2 * t] = lo[0] + (hi[0] >> 4);
                        d[(i * 16 + g + 8) * p.dld + 2 * t] = lo[2] + (hi[2] >> 4);
                    }
                    if (2 * t + 1 < p.B) {
                        d[(i * 16 + g) * p.dld + 2 * t + 1] = lo[1] + (hi[1] >> 4);
                        d[(i * 16 + g + 8) * p.dld + 2 * t + 1] = lo[3] + (hi[3] >> 4);
                    }
                }
            }
            slot = slot + 1 == STAGES ? 0 : slot + 1;
        }
        __syncthreads();
        // one thread per (row, activation): groups in order, multiply and add rounded separately
        for (int e = threadIdx.x; e < R * p.B; e += WT_W * 32) {
            const int r = e % R, b = e / R;
            if (r >= tile_rows) continue;
            const int row = row0 + r;
            const float* sab = s_sa + (size_t)b * nk;
            const int* qs = qsum + (size_t)b * nk;
            const int* dr = gdot + (size_t)r * p.dld + b;
            const int gstride = R * p.dld;
            float acc = 0.0f;
#pragma unroll 8
            for (int k = 0; k < nk; k++)
                acc = __fadd_rn(acc, __fmul_rn((float)(dr[(size_t)k * gstride] - qs[k]), sab[k]));
            const float sw = p.scales_fp32 ? reinterpret_cast<const float*>(p.scales)[row]
                                           : __half2float(reinterpret_cast<const __half*>(p.scales)[row]);
            const float y = __fmul_rn(acc, sw);
            float* o = p.out + (size_t)b * p.out_stride + row;
            *o = p.epilogue == IBCU_EPI_ADD ? *o + y : y;
        }
        __syncthreads();                                      // the parked dot products are free for the next tile
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
}

template <int STAGES, int RT>
int w4a8_mma_launch(ibcu_ctx* ctx, const WtParams& p, int grid, size_t smem) {
    auto kern = w4a8_mma_kernel<STAGES, RT>;
    if (smem > 48 * 1024) {
        static size_t allowed[64];
        size_t& have = allowed[ctx->device & 63];
        if (smem > have) {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return ibcu_fail(ctx, IBCU_ERR_CUDA, "cudaFuncSetAttribute(smem=%zu): %s", smem, cudaGetErrorString(e));
            have = smem;
        }
    }
    return ibcu_launch(ctx, kern, dim3(grid), dim3(WT_W * 32), smem, 1, true, p);
}

}  // namespace

extern "C" int ibcu_quantize_input_int8_g128(ibcu_ctx* ctx, const float* x, int8_t* q, float* sa, int N, int B) {
    IBCU_CHECK_CTX(ctx);
    IBCU_REQUIRE(ctx, x && q && sa && N > 0 && B > 0, "ibcu_quantize_input_int8_g128: bad arguments");
    const int groups = (N + 127) / 128, total = groups * B;
    return ibcu_launch(ctx, quantize_g128_kernel, dim3((total + 7) / 8), dim3(256), 0, 1, true, x, q, sa, N, groups, total);
}

static int w4a8_call(ibcu_ctx* ctx, const ibcu_linear_t* t, const int8_t* xq, const float* sa, const float* xf, int N, int B);

extern "C" int ibcu_linear_w4a8(ibcu_ctx* ctx, const ibcu_linear_t* t, const int8_t* xq, const float* sa, int N, int B) {
    IBCU_CHECK_CTX(ctx);
    IBCU_REQUIRE(ctx, t && t->w && t->scales && t->out && xq && sa, "ibcu_linear_w4a8: null pointer");
    return w4a8_call(ctx, t, xq, sa, nullptr, N, B);
}

// FP32 activations in: quantiser and matvec in one launch when the tensor-core kernel takes the shape, else the quantiser
// kernel into the context's activation buffer and then the matvec.
extern "C" int ibcu_linear_w4a8_fp32(ibcu_ctx* ctx, const ibcu_linear_t* t, const float* x, int N, int B) {
    IBCU_CHECK_CTX(ctx);
    IBCU_REQUIRE(ctx, t && t->w && t->scales && t->out && x, "ibcu_linear_w4a8_fp32: null pointer");
    // every block of the matvec would quantise all activations for itself: worth it only while that is a few groups
    // (one 4096-column activation); otherwise the quantiser runs once, as a launch of its own
    if (N % 128 == 0 && ((uintptr_t)x & 15) == 0 && (long)B * (N / 128) <= 32) return w4a8_call(ctx, t, nullptr, nullptr, x, N, B);
    const int groups = (N + 127) / 128;
    const size_t qbytes = ((size_t)B * N + 255) & ~(size_t)255;
    int rc = ibcu_reserve(ctx, &ctx->xpack, &ctx->xpack_bytes, qbytes + (size_t)B * groups * sizeof(float));
    if (rc) return rc;
    int8_t* q = (int8_t*)ctx->xpack;
    float* sa = (float*)((char*)ctx->xpack + qbytes);
    rc = ibcu_quantize_input_int8_g128(ctx, x, q, sa, N, B);
    if (rc) return rc;
    return w4a8_call(ctx, t, q, sa, nullptr, N, B);
}

static int w4a8_call(ibcu_ctx* ctx, const ibcu_linear_t* t, const int8_t* xq, const float* sa, const float* xf, int N, int B) {
    IBCU_REQUIRE(ctx, N > 0 && (N & 1) == 0 && B >= 1 && B <= 32 && t->M >= 0 && t->out_stride >= t->M, "ibcu_linear_w4a8: bad shape");
    if (t->M == 0) return IBCU_OK;
    // tensor-core path: whole groups of 128 columns, aligned operands; up to 8 activations per launch
    if (N % 128 == 0 && !ctx->force_generic && ((uintptr_t)t->w & 15) == 0 && (xf || ((uintptr_t)xq & 7) == 0)) {
        const int groups = N / 128;
        for (int b0 = 0; b0 < B; b0 += 8) {
            const int Bc = B - b0 < 8 ? B - b0 : 8;
            WtParams p;
            memset(&p, 0, sizeof p);
            p.w = (const uint8_t*)t->w; p.scales = t->scales; p.scales_fp32 = t->scales_fp32;
            p.out = t->out + (size_t)b0 * t->out_stride; p.M = t->M; p.out_stride = t->out_stride; p.epilogue = t->epilogue;
            p.xq = xq ? xq + (size_t)b0 * N : nullptr; p.sa = sa ? sa + (size_t)b0 * groups : nullptr; p.xf = xf ? xf + (size_t)b0 * N : nullptr;
            p.N = N; p.B = Bc; p.groups = groups;
            p.xs_ld = N + 16;
            p.dld = Bc | 1;
            // rows per block: one wave of two blocks per SM when shared memory allows; 32-row tiles once a block's run is longer than 16
            auto plan = [&](int rt, int stages, size_t* smem_out) {
                const size_t tail = (((size_t)groups * 16 * rt * p.dld * 4 + 15) & ~(size_t)15) + 2 * ((((size_t)Bc * groups + 3) & ~(size_t)3) * 4) + (size_t)Bc * p.xs_ld;
                *smem_out = (size_t)stages * 16 * rt * WT_LD + tail;
                int fit = (int)((227 * 1024) / (*smem_out + 1024));
                return fit > 2 ? 2 : fit;
            };
            int rt = (t->M + 2 * ctx->sm_count - 1) / (2 * ctx->sm_count) > 16 ? 2 : 1;
            size_t smem = 0;
            int stages = rt == 2 ? 6 : 8;
            int fit = plan(rt, stages, &smem);
            if (fit < 2) { stages = 4; fit = plan(rt, stages, &smem); }
            if (fit < 1 && rt == 2) { rt = 1; fit = plan(rt, stages, &smem); }
            if (fit < 1) break;                               // does not fit: the row-per-warp kernel below takes the call
            const int slots = fit * ctx->sm_count;
            int rpb = (t->M + slots - 1) / slots;
            if (rpb < 4) rpb = 4;
            p.rows_per_block = rpb;
            const int grid = (t->M + rpb - 1) / rpb;
            const int rc = rt == 2 ? (stages == 6 ? w4a8_mma_launch<6, 2>(ctx, p, grid, smem) : w4a8_mma_launch<4, 2>(ctx, p, grid, smem))
                                   : (stages == 8 ? w4a8_mma_launch<8, 1>(ctx, p, grid, smem) : w4a8_mma_launch<4, 1>(ctx, p, grid, smem));
            if (rc) return rc;
            if (b0 + Bc >= B) return IBCU_OK;
        }
    }
    if (!xq) {                                                // FP32 activations and a shape the kernel above did not take: quantise first
        const int groups = (N + 127) / 128;
        const size_t qbytes = ((size_t)B * N + 255) & ~(size_t)255;
        int rc = ibcu_reserve(ctx, &ctx->xpack, &ctx->xpack_bytes, qbytes + (size_t)B * groups * sizeof(float));
        if (rc) return rc;
        int8_t* q = (int8_t*)ctx->xpack;
        float* sq = (float*)((char*)ctx->xpack + qbytes);
        rc = ibcu_quantize_input_int8_g128(ctx, xf, q, sq, N, B);
        if (rc) return rc;
        xq = q; sa = sq;
    }
    return ibcu_launch(ctx, w4a8_kernel, dim3((t->M + 7) / 8), dim3(256), 0, 1, true, (const uint8_t*)t->w, t->scales, t->scales_fp32,
                       t->out, t->M, t->out_stride, t->epilogue, xq, sa, N, B);
}
