// Product-quantised matvec: out[r] = row_scale[r] * sum over subspaces s of LUT_s[code[r][s]],
// LUT_s[k] = codebook_s[k] . x_s (FP32), for 1..32 activations. One launch per call.
//
// Data in HBM: codebooks, row scales and the two row-major code planes exactly as the reference
// holds them, plus one derived array made once per tensor by ibcu_pq_prepare: the codes regrouped into
// slabs of 32 subspaces (subspace s = 2 * chunk + side) so that lane l of a warp owns subspace 32 j + l:
//   idx_t[slab j][group g of 16 rows][lane l][16 rows]   (one byte each)
// A warp instruction that loads 16 bytes per lane reads 512 contiguous bytes: 16 rows x 32 subspaces.
// The last 256 bytes of the array hold the largest magnitude of any codebook entry.
//
// pq_slab_kernel: grid = (blocks of rows) x (slabs). A block builds the lookup table of its slab in shared
// memory in the bank-per-lane layout, word (k * 32 + l): lane l only ever touches bank l, so neither the
// build nor the gather has a bank conflict whatever the codes are. A warp then walks its groups of 16
// rows: one 16-byte code load per lane, 16 table reads, and a butterfly over the lanes that leaves each
// row's sum over the slab's 32 subspaces in one lane. Slab sums of a row meet in a 64-bit fixed-point
// accumulator in global memory through integer atomic adds: integer addition is associative, so the
// result does not depend on the order in which blocks arrive and is identical from run to run. The
// quantum of the fixed point is 2^-62 of a bound on |sum| that every block derives from max|x|, the
// largest codebook magnitude and N. The block that arrives last for its rows (an arrival counter) reads the
// accumulators back, leaves them zero for the next call, applies the row scale and stores.
#include "common.cuh"
#include <mutex>

namespace {

constexpr int PQ_THREADS = 512;
constexpr int PQ_WARPS = PQ_THREADS / 32;
constexpr int PQ_TAIL = 256;                 // bytes after the code array: [0] = max |codebook entry| as float bits

struct PqParams {
    int M, M_pad, N, G, K, C, B, nslab, rows_per_block;
    const __half* cb_l; const __half* cb_r; long cb_stride;
    const uint8_t* idx_t;
    const __half* row_scale;
    const float* x;                            // [B][N]
    float* out;                                // [B][M]
    unsigned long long* acc;                   // [B][M_pad] fixed-point sums, zero between calls
    unsigned int* arrive;                      // [passes][row blocks] arrival counters, zero between calls
};

// codes [M][C] x 2 planes -> slabs of 32 subspaces, 16 rows per lane (see the head of the file)
__global__ void __launch_bounds__(256) pq_pack_kernel(const uint8_t* __restrict__ idx_l, const uint8_t* __restrict__ idx_r,
                                                      int M, int C, int M_pad, int nslab, uint8_t* __restrict__ idx_t) {
    const int G16 = M_pad / 16;
    const long total = (long)nslab * G16 * 32;
    for (long e = (long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long)gridDim.x * blockDim.x) {
        const int l = (int)(e & 31);
        const long jg = e >> 5;
        const int g = (int)(jg % G16), j = (int)(jg / G16);
        const int s = 32 * j + l, c = s >> 1;
        const uint8_t* src = (s & 1) ? idx_r : idx_l;
        uint32_t w[4] = { 0, 0, 0, 0 };
#pragma unroll
        for (int i = 0; i < 16; i++) {
            const int r = 16 * g + i;
            const uint32_t v = (c < C && r < M) ? src[(size_t)r * C + c] : 0u;
            w[i >> 2] |= v << (8 * (i & 3));
        }
        reinterpret_cast<uint4*>(idx_t)[e] = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

__global__ void __launch_bounds__(256) pq_absmax_kernel(const __half* __restrict__ a, const __half* __restrict__ b, size_t n, float* __restrict__ out) {
    float m = 0.0f;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float u = fabsf(__half2float(a[i])), v = fabsf(__half2float(b[i]));
        if (u == u) m = fmaxf(m, u);
        if (v == v) m = fmaxf(m, v);
    }
    m = warp_max(m);
    if ((threadIdx.x & 31) == 0) atomicMax(reinterpret_cast<int*>(out), __float_as_int(m));     // non-negative floats order like ints
}

// one halving step of the butterfly: N values per lane -> N/2, each the sum over the lane pair {l, l ^ o}
template <int N>
__device__ __forceinline__ void fold(float* v, int o, int lane) {
    const bool up = (lane & o) != 0;
#pragma unroll
    for (int i = 0; i < N / 2; i++) {
        const float send = up ? v[i] : v[i + N / 2];
        const float keep = up ? v[i + N / 2] : v[i];
        v[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
    }
}

// BT activations share one pass over the codes: table entries are BT floats wide (1 or 4)
template <int BT>
__global__ void __launch_bounds__(PQ_THREADS, BT == 1 ? 2 : 1) pq_slab_kernel(const PqParams p) {
    extern __shared__ __align__(16) float lut[];            // [256][32][BT]
    __shared__ float xs[BT][32][17];                         // this slab's activation slices, one row per lane (half <= 16)
    __shared__ float red[BT][PQ_WARPS];
    __shared__ int bad_s[PQ_WARPS];
    __shared__ unsigned char live[BT][32];
    __shared__ int last_s;
    pdl_launch_dependents();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int half = p.G >> 1, nsub = 2 * p.C;
    const int row_lo = blockIdx.x * p.rows_per_block;
    const int row_hi = min(p.M_pad, row_lo + p.rows_per_block);
    const int G16 = p.M_pad >> 4;
    const int g_lo = row_lo >> 4, g_hi = row_hi >> 4;
    const float cbmax = __int_as_float(*reinterpret_cast<const int*>(p.idx_t + (size_t)p.nslab * G16 * 512));

    pdl_wait();
    const bool vec_x = (p.N & 3) == 0 && ((uintptr_t)p.x & 15) == 0;
    for (int b0 = 0; b0 < p.B; b0 += BT) {
        const int nb = min(BT, p.B - b0);
        // ── max |x| of each activation (the reference's 1 %-of-max rule and the fixed-point scale need it) ──
        float am[BT]; int bad = 0;
#pragma unroll
        for (int t = 0; t < BT; t++) {
            am[t] = 0.0f;
            if (t >= nb) continue;
            const float* xb = p.x + (size_t)(b0 + t) * p.N;
            if (vec_x) {
                const float4* x4 = reinterpret_cast<const float4*>(xb);
                const int n4 = p.N >> 2;
#pragma unroll 8
                for (int j = tid; j < n4; j += PQ_THREADS) {
                    const float4 v = x4[j];
                    const float m4 = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
                    am[t] = fmaxf(am[t], m4);
                    bad |= !(fabsf(v.x) <= 3.0e38f) | !(fabsf(v.y) <= 3.0e38f) | !(fabsf(v.z) <= 3.0e38f) | !(fabsf(v.w) <= 3.0e38f);
                }
            } else {
#pragma unroll 8
                for (int j = tid; j < p.N; j += PQ_THREADS) { const float v = xb[j]; am[t] = fmaxf(am[t], fabsf(v)); bad |= !(fabsf(v) <= 3.0e38f); }
            }
        }
#pragma unroll
        for (int t = 0; t < BT; t++) am[t] = warp_max(am[t]);
        bad = __any_sync(0xffffffffu, bad);
        __syncthreads();                                     // the previous pass is done with the table and xs
        if (lane == 0) {
#pragma unroll
            for (int t = 0; t < BT; t++) red[t][warp] = am[t];
            bad_s[warp] = bad;
        }
        for (int j = 0; j < (p.nslab - (int)blockIdx.y + (int)gridDim.y - 1) / (int)gridDim.y; j++) {
            const int slab = blockIdx.y + j * gridDim.y;
            const int s0 = slab * 32;
            if (j) __syncthreads();
            // this slab's slices of x: subspace s covers x[s * half, (s + 1) * half)
            for (int e = tid; e < BT * 32 * half; e += PQ_THREADS) {
                const int t = e / (32 * half), r = e - t * 32 * half, l = r / half, i = r - l * half;
                const int s = s0 + l;
                xs[t][l][i] = (t < nb && s < nsub) ? p.x[(size_t)(b0 + t) * p.N + (size_t)s * half + i] : 0.0f;
            }
            __syncthreads();
            float amax[BT];
            int anybad = 0;
#pragma unroll
            for (int w = 0; w < PQ_WARPS; w++) anybad |= bad_s[w];
#pragma unroll
            for (int t = 0; t < BT; t++) {
                amax[t] = red[t][0];
#pragma unroll
                for (int w = 1; w < PQ_WARPS; w++) amax[t] = fmaxf(amax[t], red[t][w]);
            }
            if (tid < 32 * BT) {
                const int t = tid >> 5, l = tid & 31;
                bool keep = t < nb && s0 + l < nsub;
                if (keep && amax[t] > 0.0f) {                // a chunk (both halves) whose largest |x| is under 1 % of the largest overall is dropped
                    const int l0 = l & ~1;
                    float cm = 0.0f;
                    for (int i = 0; i < half; i++) cm = fmaxf(cm, fmaxf(fabsf(xs[t][l0][i]), fabsf(xs[t][l0 + 1][i])));
                    keep = cm >= amax[t] * 0.01f;
                }
                live[t][l] = keep;
            }
            __syncthreads();
            // ── lookup table of the slab: thread (k, lane) for k = warp, warp + 16, ...; word (k * 32 + lane) ──
            {
                const int s = s0 + lane;
                const bool sub_ok = s < nsub;
                const __half* cb = ((s & 1) ? p.cb_r : p.cb_l) + (size_t)(s >> 1) * p.cb_stride;
                const bool vec_cb = half == 8 && (p.cb_stride & 7) == 0 && ((uintptr_t)p.cb_l & 15) == 0 && ((uintptr_t)p.cb_r & 15) == 0;
                bool lv[BT];
#pragma unroll
                for (int t = 0; t < BT; t++) lv[t] = live[t][lane];
                if (vec_cb) {
                    constexpr int U = 4;
                    float xr[BT][8];
#pragma unroll
                    for (int t = 0; t < BT; t++)
#pragma unroll
                        for (int i = 0; i < 8; i++) xr[t][i] = xs[t][lane][i];
                    for (int k0 = warp; k0 < 256; k0 += PQ_WARPS * U) {
                        uint4 raw[U];
#pragma unroll
                        for (int u = 0; u < U; u++) {
                            const int k = k0 + u * PQ_WARPS;
                            raw[u] = (sub_ok && k < p.K) ? *reinterpret_cast<const uint4*>(cb + (size_t)k * 8) : make_uint4(0, 0, 0, 0);
                        }
#pragma unroll
                        for (int u = 0; u < U; u++) {
                            const int k = k0 + u * PQ_WARPS;
                            const __half2* h = reinterpret_cast<const __half2*>(&raw[u]);
                            const float2 f0 = __half22float2(h[0]), f1 = __half22float2(h[1]), f2 = __half22float2(h[2]), f3 = __half22float2(h[3]);
                            float v[BT];
#pragma unroll
                            for (int t = 0; t < BT; t++) {
                                float a = 0.0f;
                                a = fmaf(f0.x, xr[t][0], a); a = fmaf(f0.y, xr[t][1], a); a = fmaf(f1.x, xr[t][2], a); a = fmaf(f1.y, xr[t][3], a);
                                a = fmaf(f2.x, xr[t][4], a); a = fmaf(f2.y, xr[t][5], a); a = fmaf(f3.x, xr[t][6], a); a = fmaf(f3.y, xr[t][7], a);
                                v[t] = lv[t] ? a : 0.0f;
                            }
                            float* dst = lut + ((size_t)k * 32 + lane) * BT;
                            if constexpr (BT == 4) *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
                            else dst[0] = v[0];
                        }
                    }
                } else {
                    for (int k = warp; k < 256; k += PQ_WARPS) {
                        float v[BT];
#pragma unroll
                        for (int t = 0; t < BT; t++) v[t] = 0.0f;
                        if (sub_ok && k < p.K) {
                            for (int i = 0; i < half; i++) {
                                const float c = __half2float(cb[(size_t)k * half + i]);
#pragma unroll
                                for (int t = 0; t < BT; t++) v[t] = fmaf(c, xs[t][lane][i], v[t]);
                            }
#pragma unroll
                            for (int t = 0; t < BT; t++) v[t] = lv[t] ? v[t] : 0.0f;
                        }
                        float* dst = lut + ((size_t)k * 32 + lane) * BT;
#pragma unroll
                        for (int t = 0; t < BT; t++) dst[t] = v[t];
                    }
                }
            }
            __syncthreads();
            // ── fixed-point scale: 2^e >= N * max|codebook| * max|x| bounds every row sum ──
            float inv_q[BT];
#pragma unroll
            for (int t = 0; t < BT; t++) {
                const float bound = (float)p.N * cbmax * amax[t];
                int e = (int)((__float_as_uint(bound) >> 23) & 0xFF) - 126;       // bound < 2^e
                e = max(-60, min(120, e));
                inv_q[t] = __uint_as_float((uint32_t)(127 + 62 - e) << 23);          // 2^(62 - e)
            }
            // ── gather: a warp per group of 16 rows ──
            const uint4* codes = reinterpret_cast<const uint4*>(p.idx_t) + (size_t)slab * G16 * 32 + lane;
            for (int g = g_lo + warp; g < g_hi; g += PQ_WARPS) {
                const uint4 cd = ld_stream_u4(codes + (size_t)g * 32);
                float v[16 * BT];
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    const uint32_t w = i < 4 ? cd.x : (i < 8 ? cd.y : (i < 12 ? cd.z : cd.w));
                    const uint32_t code = (w >> (8 * (i & 3))) & 0xFF;
                    if constexpr (BT == 4) {
                        const float4 q = *reinterpret_cast<const float4*>(lut + ((size_t)code * 32 + lane) * 4);
                        v[i] = q.x; v[16 + i] = q.y; v[32 + i] = q.z; v[48 + i] = q.w;       // index = t * 16 + row
                    } else v[i] = lut[code * 32 + lane];
                }
                if constexpr (BT == 4) { fold<64>(v, 16, lane); fold<32>(v, 8, lane); fold<16>(v, 4, lane); fold<8>(v, 2, lane); fold<4>(v, 1, lane); }
                else { fold<16>(v, 16, lane); fold<8>(v, 8, lane); fold<4>(v, 4, lane); fold<2>(v, 2, lane); v[0] += __shfl_xor_sync(0xffffffffu, v[0], 1); }
                // which (activation, row) a lane ends up with: bit 16 of the lane picked the upper half of the
                // index range in the first step, bit 8 the upper half of that half, and so on
                if constexpr (BT == 4) {
                    const int base = ((lane & 16) ? 32 : 0) + ((lane & 8) ? 16 : 0) + ((lane & 4) ? 8 : 0) + ((lane & 2) ? 4 : 0) + ((lane & 1) ? 2 : 0);
#pragma unroll
                    for (int q = 0; q < 2; q++) {
                        const int idx = base + q, t = idx >> 4, r = 16 * g + (idx & 15);
                        if (t < nb) atomicAdd(p.acc + (size_t)(b0 + t) * p.M_pad + r, (unsigned long long)__float2ll_rn(v[q] * inv_q[t]));
                    }
                } else if ((lane & 1) == 0) {
                    const int r = 16 * g + (lane >> 1);
                    atomicAdd(p.acc + (size_t)b0 * p.M_pad + r, (unsigned long long)__float2ll_rn(v[0] * inv_q[0]));
                }
            }
        }
        // ── the block that arrives last for these rows turns the sums into the result ──
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            unsigned int* cnt = p.arrive + (size_t)(b0 / BT) * gridDim.x + blockIdx.x;     // one counter per pass and block of rows
            const unsigned int n = atomicAdd(cnt, 1u);
            last_s = n == gridDim.y - 1;
            if (last_s) *cnt = 0;
        }
        __syncthreads();
        if (last_s) {
            __threadfence();
            float amax[BT]; int anybad = 0;
#pragma unroll
            for (int w = 0; w < PQ_WARPS; w++) anybad |= bad_s[w];
#pragma unroll
            for (int t = 0; t < BT; t++) {
                amax[t] = red[t][0];
#pragma unroll
                for (int w = 1; w < PQ_WARPS; w++) amax[t] = fmaxf(amax[t], red[t][w]);
            }
            const int rows = min(row_hi, p.M) - row_lo;
            for (int e = tid; e < rows * nb; e += PQ_THREADS) {
                const int t = e / rows, r = row_lo + (e - t * rows);
                const float bound = (float)p.N * cbmax * amax[t];
                int ex = (int)((__float_as_uint(bound) >> 23) & 0xFF) - 126;
                ex = max(-60, min(120, ex));
                const long long s = (long long)atomicExch(p.acc + (size_t)(b0 + t) * p.M_pad + r, 0ull);
                const double q = __longlong_as_double((long long)(1023 + ex - 62) << 52);          // 2^(ex - 62)
                float y = (float)((double)s * q) * __half2float(p.row_scale[r]);
                if (anybad) y = __int_as_float(0x7fc00000);                                         // an activation held NaN or Inf
                p.out[(size_t)(b0 + t) * p.M + r] = y;
            }
            // padded rows of the last group also received sums
            for (int e = tid; e < (row_hi - min(row_hi, p.M)) * nb; e += PQ_THREADS) {
                const int pad = row_hi - min(row_hi, p.M), t = e / pad, r = min(row_hi, p.M) + (e - t * pad);
                p.acc[(size_t)(b0 + t) * p.M_pad + r] = 0ull;
            }
        }
        __syncthreads();
    }
}

struct PqPlan { int C, nslab, row_blocks, rows_per_block, slab_blocks; size_t acc_words; };

PqPlan pq_plan(const ibcu_ctx* ctx, const ibcu_pq_t* t, int B) {
    PqPlan pl;
    pl.C = t->N / t->G;
    pl.nslab = (2 * pl.C + 31) / 32;
    const int per_sm = B >= 2 ? 1 : 2;
    const int slots = ctx->sm_count * per_sm;
    pl.slab_blocks = pl.nslab < slots ? pl.nslab : slots;                    // more slabs than blocks: a block walks several
    int rb = slots / pl.slab_blocks;
    const int groups = t->M_pad / 16;
    if (rb > groups) rb = groups;
    if (rb < 1) rb = 1;
    const int gpb = (groups + rb - 1) / rb;
    pl.rows_per_block = gpb * 16;
    pl.row_blocks = (groups + gpb - 1) / gpb;
    pl.acc_words = (size_t)B * t->M_pad;
    return pl;
}

int pq_launch(ibcu_ctx* ctx, const ibcu_pq_t* t, const float* x, float* out, int B, const PqPlan& pl,
              unsigned long long* acc, unsigned int* arrive) {
    PqParams p;
    p.M = t->M; p.M_pad = t->M_pad; p.N = t->N; p.G = t->G; p.K = t->K; p.C = pl.C; p.B = B; p.nslab = pl.nslab;
    p.rows_per_block = pl.rows_per_block;
    p.cb_l = (const __half*)t->codebook_l; p.cb_r = (const __half*)t->codebook_r; p.cb_stride = t->cb_chunk_stride;
    p.idx_t = t->idx_t; p.row_scale = (const __half*)t->row_scale; p.x = x; p.out = out; p.acc = acc; p.arrive = arrive;
    const dim3 grid(pl.row_blocks, pl.slab_blocks), block(PQ_THREADS);
    if (B >= 2) {
        const size_t smem = (size_t)256 * 32 * 4 * sizeof(float);
        static std::once_flag once[64];
        cudaError_t e = cudaSuccess;
        std::call_once(once[ctx->device & 63], [&] { e = cudaFuncSetAttribute(pq_slab_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); });
        if (e != cudaSuccess) return ibcu_fail(ctx, IBCU_ERR_CUDA, "cudaFuncSetAttribute(pq_slab_kernel): %s", cudaGetErrorString(e));
        return ibcu_launch(ctx, pq_slab_kernel<4>, grid, block, smem, 1, true, p);
    }
    return ibcu_launch(ctx, pq_slab_kernel<1>, grid, block, (size_t)256 * 32 * sizeof(float), 1, true, p);
}

int pq_check(ibcu_ctx* ctx, const ibcu_pq_t* t, const float* x, float* out, int B, const char* who) {
    IBCU_REQUIRE(ctx, t && x && out, "%s: null pointer", who);
    IBCU_REQUIRE(ctx, t->codebook_l && t->codebook_r && t->row_scale, "%s: tensor has a null pointer", who);
    IBCU_REQUIRE(ctx, t->idx_t && t->M_pad >= t->M && (t->M_pad & 15) == 0, "%s: call ibcu_pq_prepare on the tensor first", who);
    IBCU_REQUIRE(ctx, t->M > 0 && t->N > 0 && t->G > 0 && (t->G & 1) == 0 && t->G <= 32 && t->N % t->G == 0 && t->K >= 1 && t->K <= 256,
                 "%s: bad shape M=%d N=%d G=%d K=%d", who, t->M, t->N, t->G, t->K);
    IBCU_REQUIRE(ctx, B >= 1 && B <= 32, "%s: B=%d not in 1..32", who, B);
    return IBCU_OK;
}

}  // namespace

constexpr size_t PQ_COUNTER_BYTES = 16384;                   // 4096 arrival counters ahead of the accumulators

static size_t pq_scratch_bytes(const PqPlan& pl) { return PQ_COUNTER_BYTES + pl.acc_words * sizeof(unsigned long long); }

extern "C" size_t ibcu_pq_idx_t_bytes(int M, int N, int G) {
    if (M <= 0 || N <= 0 || G <= 0 || N % G) return 0;
    const size_t M_pad = ((size_t)M + 15) & ~(size_t)15;
    const size_t nslab = (2 * (size_t)(N / G) + 31) / 32;
    return nslab * 32 * M_pad + PQ_TAIL;
}

extern "C" int ibcu_pq_prepare(ibcu_ctx* ctx, ibcu_pq_t* t, uint8_t* idx_t_out) {
    IBCU_CHECK_CTX(ctx);
    IBCU_REQUIRE(ctx, t && idx_t_out && t->idx_l && t->idx_r && t->codebook_l && t->codebook_r, "ibcu_pq_prepare: null pointer");
    IBCU_REQUIRE(ctx, t->M > 0 && t->N > 0 && t->G > 0 && (t->G & 1) == 0 && t->N % t->G == 0 && t->K >= 1 && t->K <= 256,
                 "ibcu_pq_prepare: bad shape M=%d N=%d G=%d K=%d", t->M, t->N, t->G, t->K);
    IBCU_REQUIRE(ctx, ((uintptr_t)idx_t_out & 15) == 0, "ibcu_pq_prepare: idx_t_out must be 16-byte aligned");
    const int C = t->N / t->G, half = t->G / 2;
    const int M_pad = (t->M + 15) & ~15;
    const int nslab = (2 * C + 31) / 32;
    const size_t body = (size_t)nslab * 32 * M_pad;
    const long vecs = (long)(body / 16);
    int blocks = (int)((vecs + 255) / 256);
    if (blocks > ctx->sm_count * 8) blocks = ctx->sm_count * 8;
    int rc = ibcu_launch(ctx, pq_pack_kernel, dim3(blocks), dim3(256), 0, 1, false, t->idx_l, t->idx_r, t->M, C, M_pad, nslab, idx_t_out);
    if (rc) return rc;
    IBCU_CUDA(ctx, cudaMemsetAsync(idx_t_out + body, 0, PQ_TAIL, ctx->stream));
    // entries of both tables: one pair when the tables are shared, one pair per chunk otherwise
    const size_t n = t->cb_chunk_stride ? (size_t)(C - 1) * t->cb_chunk_stride + (size_t)t->K * half : (size_t)t->K * half;
    int ab = (int)((n + 255) / 256);
    if (ab > ctx->sm_count * 4) ab = ctx->sm_count * 4;
    rc = ibcu_launch(ctx, pq_absmax_kernel, dim3(ab), dim3(256), 0, 1, false, (const __half*)t->codebook_l, (const __half*)t->codebook_r, n,
                     reinterpret_cast<float*>(idx_t_out + body));
    if (rc) return rc;
    t->idx_t = idx_t_out;
    t->M_pad = M_pad;
    return IBCU_OK;
}

extern "C" int ibcu_pq_matmul_fp32(ibcu_ctx* ctx, const ibcu_pq_t* t, const float* x, float* out, int B) {
    IBCU_CHECK_CTX(ctx);
    int rc = pq_check(ctx, t, x, out, B, "ibcu_pq_matmul_fp32");
    if (rc) return rc;
    const PqPlan pl = pq_plan(ctx, t, B);
    const size_t need = pq_scratch_bytes(pl);
    if (ctx->pq_acc_bytes < need) {
        // the accumulators and counters must read zero when a call starts and every call leaves them so:
        // they are cleared once, when the buffer is made
        rc = ibcu_reserve(ctx, &ctx->pq_acc, &ctx->pq_acc_bytes, need);
        if (rc) return rc;
        IBCU_CUDA(ctx, cudaMemsetAsync(ctx->pq_acc, 0, ctx->pq_acc_bytes, ctx->stream));
    }
    return pq_launch(ctx, t, x, out, B, pl, (unsigned long long*)((char*)ctx->pq_acc + PQ_COUNTER_BYTES), (unsigned int*)ctx->pq_acc);
}

// ── PQ matvec without any allocation ────────────────────────────────────────────────────
// Some callers must not (or cannot) allocate device memory at call time: code that runs inside a
// latency-critical serving loop where cudaMalloc's implicit device synchronisation is unacceptable,
// plugins that are handed a fixed memory budget by their host application, and processes whose
// allocator is owned by another runtime. For them the fixed-point row accumulators and the arrival
// counters live in a fixed array that is part of the library image: every GPU that loads the library
// holds PQ_STATIC_FLOATS four-byte words (4 MiB) from load until exit, whether or not this entry point is
// used.
constexpr size_t PQ_STATIC_FLOATS = (size_t)1 << 20;
static __device__ __align__(256) float pq_static_scratch[PQ_STATIC_FLOATS];

// In host code `pq_static_scratch` is only a handle for the runtime, not a device address; the
// address a kernel can use is looked up once per device, with that device current.
static float* pq_static_address(ibcu_ctx* ctx) {
    static float* per_device[64];
    static std::mutex lock;
    if (ctx->device < 0 || ctx->device >= 64) return nullptr;
    std::lock_guard<std::mutex> guard(lock);
    if (!per_device[ctx->device]) {
        int cur = -1;
        cudaGetDevice(&cur);
        if (cudaSetDevice(ctx->device) != cudaSuccess) return nullptr;
        float* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress((void**)&p, pq_static_scratch);
        if (cur >= 0 && cur != ctx->device) cudaSetDevice(cur);            // leave the caller's current device as it was
        if (e != cudaSuccess) { ibcu_fail(ctx, IBCU_ERR_CUDA, "cudaGetSymbolAddress(pq_static_scratch) failed: %s", cudaGetErrorString(e)); return nullptr; }
        per_device[ctx->device] = p;
    }
    return per_device[ctx->device];
}

extern "C" size_t ibcu_pq_noalloc_max_floats(void) { return PQ_STATIC_FLOATS; }

extern "C" int ibcu_pq_matmul_fp32_noalloc(ibcu_ctx* ctx, const ibcu_pq_t* t, const float* x, float* out, int B) {
    IBCU_CHECK_CTX(ctx);
    int rc = pq_check(ctx, t, x, out, B, "ibcu_pq_matmul_fp32_noalloc");
    if (rc) return rc;
    const PqPlan pl = pq_plan(ctx, t, B);
    const size_t need = pq_scratch_bytes(pl);
    if (need > PQ_STATIC_FLOATS * sizeof(float))
        return ibcu_fail(ctx, IBCU_ERR_PARAM, "ibcu_pq_matmul_fp32_noalloc: this call needs %zu floats of scratch (%d activations x %d padded rows x 2, plus %zu for counters), "
                         "the built-in array holds %zu; use ibcu_pq_matmul_fp32", need / sizeof(float), B, t->M_pad, PQ_COUNTER_BYTES / sizeof(float), PQ_STATIC_FLOATS);
    float* base = pq_static_address(ctx);
    if (!base) return ctx->status ? ctx->status : ibcu_fail(ctx, IBCU_ERR_CUDA, "ibcu_pq_matmul_fp32_noalloc: no address for the built-in scratch on device %d", ctx->device);
    // The accumulators and counters must start at zero. A call that ran to its end leaves them so, but the
    // array is shared by every caller on the device and one that was cut short may not have: clear the part
    // this call uses (an asynchronous fill on the stream, no allocation).
    IBCU_CUDA(ctx, cudaMemsetAsync(base, 0, need, ctx->stream));
    return pq_launch(ctx, t, x, out, B, pl, (unsigned long long*)((char*)base + PQ_COUNTER_BYTES), (unsigned int*)base);
}
