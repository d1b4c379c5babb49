// Product-quantised matvec: out[r] = row_scale[r] * sum over subspaces s of LUT_s[code[r][s]],
// LUT_s[k] = codebook_s[k] . x_s (FP32), for 1..32 activations. One launch per call.
//
// Data in HBM: codebooks, row scales and the two row-major code planes exactly as the reference
// holds them, plus one derived array made once per tensor by ibcu_pq_prepare: the codes regrouped into
// slabs of 32 subspaces (subspace s = 2 * chunk + side) so that lane l of a warp owns subspace 32 j + l:
//   idx_t[slab j][group g of 16 rows][lane l][16 rows]   (one byte each; byte i of lane l is row i ^ (l >> 1) of the group)
// A warp instruction that loads 16 bytes per lane reads 512 contiguous bytes: 16 rows x 32 subspaces. The rows of a
// lane are stored in the order in which the lane-to-lane reduction wants them: with value j of lane l standing for
// row j ^ (l >> 1), every halving step keeps the lower half of the registers and sends the upper half, in every lane.
// The last 256 bytes of the array hold the largest magnitude of any codebook entry.
//
// pq_slab_kernel: grid = (blocks of rows) x (slabs) x (passes of one or two activations). A block builds the lookup table of its slab in shared
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
#include <cooperative_groups.h>
#include <mutex>

namespace {

constexpr int PQ_THREADS = 512;
constexpr int PQ_WARPS = PQ_THREADS / 32;
constexpr size_t PQ_COUNTER_BYTES = 16384;   // 4096 four-byte slots ahead of the accumulators: arrival counters, the last 64 for max|x|
constexpr int PQ_TAIL = 256;                 // bytes after the code array: [0] = max |codebook entry| as float bits

struct PqParams {
    int M, M_pad, N, G, K, C, B, nslab, rows_per_block;
    const __half* cb_l; const __half* cb_r; long cb_stride;
    const uint8_t* idx_t;
    const __half* row_scale;
    const float* x;                            // [B][N]
    float* out;                                // [B][out_stride], the first M of every row written
    int out_stride;
    unsigned long long* acc;                   // [B][M_pad] fixed-point sums, zero between calls
    unsigned int* arrive;                      // [passes][row blocks] arrival counters, zero between calls
    const unsigned* amax_bits;                 // [B] bit patterns of max|x[b]| when pq_amax_kernel ran ahead, else NULL
    // production extras (src/pq_decode.c:1441-1496, :1538-1546): slabs [nslab1, nslab) hold the codes of a second
    // residual level over the same activation slices, with shared codebooks of K2 entries; inner != NULL lists the
    // columns of x that the tables are built from (the others are outlier columns), n_inner = C * G of them
    int nslab1, K2;
    const __half* cb2_l; const __half* cb2_r;
    const int* inner; int n_inner;
    int tail_slabs;                            // slabs of the whole code array: the tail with max |codebook entry| follows them
    int no_skip;                               // the 1 % rule is off (the first-level pass of the top-K head, src/pq_decode.c:2085-2143)
};

// codes [M][C] x 2 planes -> slabs of 32 subspaces, 16 rows per lane (see the head of the file)
// packed != 0: two 4-bit codes per byte, low nibble = even chunk, rows of (C + 1) / 2 bytes (second level with 16 entries)
__global__ void __launch_bounds__(256) pq_pack_kernel(const uint8_t* __restrict__ idx_l, const uint8_t* __restrict__ idx_r,
                                                      int M, int C, int M_pad, int nslab, uint8_t* __restrict__ idx_t, int packed) {
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
            const int r = 16 * g + (i ^ (l >> 1));
            uint32_t v = 0u;
            if (c < C && r < M) {
                if (packed) { const uint32_t b = src[(size_t)r * ((C + 1) / 2) + (c >> 1)]; v = (c & 1) ? (b >> 4) & 15u : b & 15u; }
                else v = src[(size_t)r * C + c];
            }
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

// tail[0] += tail[1]: the bound used for the fixed-point scale covers one entry of each level
__global__ void pq_add_tail_kernel(float* tail) { if (threadIdx.x == 0) tail[0] += tail[1]; }

// grid (B): the bit pattern of max|x[b]| (NaN and Inf sort above every finite value)
__global__ void __launch_bounds__(512) pq_amax_kernel(const float* __restrict__ x, int N, unsigned* __restrict__ out,
                                                      const int* __restrict__ inner, int n_inner) {
    __shared__ unsigned red[16];
    pdl_launch_dependents();
    pdl_wait();
    const float* xb = x + (size_t)blockIdx.x * N;
    unsigned m = 0u;
    if (inner) {
        for (int j = threadIdx.x; j < n_inner; j += 512) m = max(m, __float_as_uint(xb[inner[j]]) & 0x7fffffffu);
    } else if ((N & 3) == 0 && ((uintptr_t)x & 15) == 0) {
        const uint4* x4 = reinterpret_cast<const uint4*>(xb);
#pragma unroll 8
        for (int j = threadIdx.x; j < (N >> 2); j += 512) {
            const uint4 v = x4[j];
            m = max(max(m, v.x & 0x7fffffffu), max(max(v.y & 0x7fffffffu, v.z & 0x7fffffffu), v.w & 0x7fffffffu));
        }
    } else {
        for (int j = threadIdx.x; j < N; j += 512) m = max(m, __float_as_uint(xb[j]) & 0x7fffffffu);
    }
    m = __reduce_max_sync(0xffffffffu, m);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 16; w++) m = max(m, red[w]);
        out[blockIdx.x] = m;
    }
}

// one halving step of the butterfly: N values per lane -> N/2, each the sum over the lane pair {l, l ^ o}. Value j of
// lane l stands for index j ^ m(l), where the lane bit o is the bit N/2 of m: the partner's value i is then this lane's
// value i + N/2, so every lane keeps its lower half and sends its upper half, without a select.
template <int N>
__device__ __forceinline__ void fold(float* v, int o) {
#pragma unroll
    for (int i = 0; i < N / 2; i++) v[i] += __shfl_xor_sync(0xffffffffu, v[i + N / 2], o);
}

// BT activations (1 or 2) share a pass over the codes: table entries are BT floats wide. grid = (blocks of rows,
// blocks of slabs, passes); pass z serves activations BT z .. BT z + BT - 1.
// EX: the tensor has a second level or outlier columns; plain tensors take the instance without that code.
template <int BT, bool EX>
__global__ void __launch_bounds__(PQ_THREADS, 2) pq_slab_kernel(const PqParams p) {
    constexpr int PQ_NG = BT == 1 ? 4 : 2;                   // groups of 16 rows whose codes a warp keeps in flight
    extern __shared__ __align__(16) float lut[];            // [256][32][BT]
    __shared__ float xs[BT][32][17];                         // this slab's activation slices, one row per lane (half <= 16)
    __shared__ __align__(16) float4 cbf[256][2][2];          // [k][side][half of the entry]: the two shared codebooks (half == 8) widened to FP32, staged once;
                                                             // even and odd lanes (sides L and R) of a warp read neighbouring 32-byte pieces
    __shared__ unsigned red[BT][PQ_WARPS];
    __shared__ int last_s;
    pdl_launch_dependents();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int half = p.G >> 1, nsub = 2 * p.C;
    const int b0 = blockIdx.z * BT, nb = min(BT, p.B - b0);
    const int row_lo = blockIdx.x * p.rows_per_block;
    const int row_hi = min(p.M_pad, row_lo + p.rows_per_block);
    const int G16 = p.M_pad >> 4;
    const int g_lo = row_lo >> 4, g_hi = row_hi >> 4;
    const int ngw = g_lo + warp < g_hi ? (g_hi - g_lo - warp + PQ_WARPS - 1) / PQ_WARPS : 0;     // this warp's groups: g_lo + warp + 16 i
    const int nj = (p.nslab - (int)blockIdx.y + (int)gridDim.y - 1) / (int)gridDim.y;             // this block's slabs: blockIdx.y + gridDim.y j
    const bool cb1_al = ((uintptr_t)p.cb_l & 15) == 0 && ((uintptr_t)p.cb_r & 15) == 0;
    const bool cb2_al = ((uintptr_t)p.cb2_l & 15) == 0 && ((uintptr_t)p.cb2_r & 15) == 0;
    // per level (0: first, 1: second residual level): may the two shared codebooks be staged in shared memory, may they be read 16 bytes at a time
    auto lvl_smem = [&](int lvl) { return half == 8 && (lvl ? cb2_al : (p.cb_stride == 0 && cb1_al)); };
    auto lvl_vec = [&](int lvl) { return half == 8 && (lvl ? cb2_al : ((p.cb_stride & 7) == 0 && cb1_al)); };
    auto stage_cb = [&](int lvl) {                            // every thread: one entry of one side, widened to FP32
        const int side = tid >> 8, k = tid & 255;
        const __half* src = lvl ? (side ? p.cb2_r : p.cb2_l) : (side ? p.cb_r : p.cb_l);
        const uint4 raw = k < (lvl ? p.K2 : p.K) ? reinterpret_cast<const uint4*>(src)[k] : make_uint4(0, 0, 0, 0);
        const __half2* h = reinterpret_cast<const __half2*>(&raw);
        const float2 f0 = __half22float2(h[0]), f1 = __half22float2(h[1]), f2 = __half22float2(h[2]), f3 = __half22float2(h[3]);
        cbf[k][side][0] = make_float4(f0.x, f0.y, f1.x, f1.y);
        cbf[k][side][1] = make_float4(f2.x, f2.y, f3.x, f3.y);
    };
    int staged = -1;                                          // the level whose codebooks sit in cbf

    // weights first, they do not depend on the previous kernel: the first codes, the shared codebooks, the row scales
    auto load_codes = [&](int slab, int c0, uint4* cd) {
        const uint4* codes = reinterpret_cast<const uint4*>(p.idx_t) + (size_t)slab * G16 * 32 + lane;
#pragma unroll
        for (int i = 0; i < PQ_NG; i++) {
            const int g = g_lo + warp + PQ_WARPS * (c0 + i);
            cd[i] = (c0 + i < ngw) ? ld_stream_u4(codes + (size_t)g * 32) : make_uint4(0, 0, 0, 0);
        }
    };
    uint4 cd[PQ_NG];
    if (nj > 0) {
        load_codes(blockIdx.y, 0, cd);
        const int lvl0 = EX && (int)blockIdx.y >= p.nslab1;
        if (lvl_smem(lvl0)) { stage_cb(lvl0); staged = lvl0; }
    }
    const float cbmax = __int_as_float(*reinterpret_cast<const int*>(p.idx_t + (size_t)p.tail_slabs * G16 * 512));
    // the rows this thread would finish if its block turns out to arrive last (PQ_FIN at a time)
    constexpr int PQ_FIN = 4;
    const int rows = max(0, min(row_hi, p.M) - row_lo);
    float rsc[PQ_FIN];
#pragma unroll
    for (int u = 0; u < PQ_FIN; u++) {
        const int e = tid + u * PQ_THREADS;
        rsc[u] = e < rows * nb ? __half2float(p.row_scale[row_lo + e % rows]) : 0.0f;
    }

    pdl_wait();
    const bool vec_x = (p.N & 3) == 0 && ((uintptr_t)p.x & 15) == 0;
    auto fill_xs = [&](int s0) {                            // this slab's slices of x: subspace s covers x[s * half, (s + 1) * half)
        if (half == 8) {
            for (int e = tid; e < BT * 256; e += PQ_THREADS) {
                const int t = e >> 8, l = (e >> 3) & 31, i = e & 7, s = s0 + l;
                xs[t][l][i] = (t < nb && s < nsub) ? p.x[(size_t)(b0 + t) * p.N + ((EX && p.inner) ? p.inner[s * 8 + i] : s * 8 + i)] : 0.0f;
            }
            return;
        }
        for (int e = tid; e < BT * 32 * half; e += PQ_THREADS) {
            const int t = e / (32 * half), r = e - t * 32 * half, l = r / half, i = r - l * half;
            const int s = s0 + l;
            xs[t][l][i] = (t < nb && s < nsub) ? p.x[(size_t)(b0 + t) * p.N + ((EX && p.inner) ? p.inner[s * half + i] : s * half + i)] : 0.0f;
        }
    };
    // ── max |x| of each activation (the reference's 1 %-of-max rule and the fixed-point scale need it), as the
    //    largest bit pattern of |x|: patterns of non-negative floats order like the floats, and NaN / Inf sort last.
    //    The loads are issued here and first used after the table has been built. ──
    unsigned ab[BT];
#pragma unroll
    for (int t = 0; t < BT; t++) {
        ab[t] = 0u;
        if (t >= nb) continue;
        if (p.amax_bits) { ab[t] = p.amax_bits[b0 + t]; continue; }            // made by pq_amax_kernel ahead of this launch
        const float* xb = p.x + (size_t)(b0 + t) * p.N;
        if (EX && p.inner) {                                 // outlier columns do not count (src/pq_decode.c:1582-1588)
            for (int j = tid; j < p.n_inner; j += PQ_THREADS) ab[t] = max(ab[t], __float_as_uint(xb[p.inner[j]]) & 0x7fffffffu);
        } else if (vec_x) {
            const uint4* x4 = reinterpret_cast<const uint4*>(xb);
            const int n4 = p.N >> 2;
#pragma unroll 8
            for (int j = tid; j < n4; j += PQ_THREADS) {
                const uint4 v = x4[j];
                ab[t] = max(max(ab[t], v.x & 0x7fffffffu), max(max(v.y & 0x7fffffffu, v.z & 0x7fffffffu), v.w & 0x7fffffffu));
            }
        } else {
#pragma unroll 8
            for (int j = tid; j < p.N; j += PQ_THREADS) ab[t] = max(ab[t], __float_as_uint(xb[j]) & 0x7fffffffu);
        }
    }
    float amax[BT], inv_q[BT];
    int anybad = 0;
    for (int j = 0; j < nj; j++) {
        const int slab = blockIdx.y + j * gridDim.y;
        const int lvl = EX && slab >= p.nslab1;              // slabs of the second level follow those of the first, over the same slices of x
        const int s0 = (lvl ? slab - p.nslab1 : slab) * 32;
        const int Kl = lvl ? p.K2 : p.K;
        const bool cb_smem = lvl_smem(lvl), cb_vec = lvl_vec(lvl);
        if (j) {
            __syncthreads();                                 // the gather of the previous slab is done with the table and xs
            load_codes(slab, 0, cd);
            if (EX && cb_smem && staged != lvl) { stage_cb(lvl); staged = lvl; }
        }
        fill_xs(s0);
        __syncthreads();
        // ── lookup table of the slab: thread (k, lane) for k = warp, warp + 16, ...; word (k * 32 + lane). Padding
        //    subspaces have zero slices, hence zero tables; subspaces the 1 % rule drops are dealt with in the gather ──
        {
            const int s = s0 + lane;
            const bool sub_ok = s < nsub;
            const __half* cb = lvl ? ((s & 1) ? p.cb2_r : p.cb2_l) : ((s & 1) ? p.cb_r : p.cb_l) + (size_t)(s >> 1) * p.cb_stride;
            if (cb_vec) {
                float xr[BT][8];
#pragma unroll
                for (int t = 0; t < BT; t++)
#pragma unroll
                    for (int i = 0; i < 8; i++) xr[t][i] = xs[t][lane][i];
                if (cb_smem) {
                    const int side = s & 1;
#pragma unroll 4
                    for (int k = warp; k < 256; k += PQ_WARPS) {
                        const float4 ca = cbf[k][side][0], cc = cbf[k][side][1];
                        float v[BT];
#pragma unroll
                        for (int t = 0; t < BT; t++) {
                            float a = 0.0f;
                            a = fmaf(ca.x, xr[t][0], a); a = fmaf(ca.y, xr[t][1], a); a = fmaf(ca.z, xr[t][2], a); a = fmaf(ca.w, xr[t][3], a);
                            a = fmaf(cc.x, xr[t][4], a); a = fmaf(cc.y, xr[t][5], a); a = fmaf(cc.z, xr[t][6], a); a = fmaf(cc.w, xr[t][7], a);
                            v[t] = a;
                        }
                        float* dst = lut + ((size_t)k * 32 + lane) * BT;
                        if constexpr (BT == 2) *reinterpret_cast<float2*>(dst) = (lane & 1) ? make_float2(v[1], v[0]) : make_float2(v[0], v[1]);
                        else dst[0] = v[0];
                    }
                } else {
                    constexpr int U = 4;
                    for (int k0 = warp; k0 < 256; k0 += PQ_WARPS * U) {
                        uint4 raw[U];
#pragma unroll
                        for (int u = 0; u < U; u++) {
                            const int k = k0 + u * PQ_WARPS;
                            raw[u] = (sub_ok && k < Kl) ? *reinterpret_cast<const uint4*>(cb + (size_t)k * 8) : make_uint4(0, 0, 0, 0);
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
                                v[t] = a;
                            }
                            float* dst = lut + ((size_t)k * 32 + lane) * BT;
                            if constexpr (BT == 2) *reinterpret_cast<float2*>(dst) = (lane & 1) ? make_float2(v[1], v[0]) : make_float2(v[0], v[1]);
                            else dst[0] = v[0];
                        }
                    }
                }
            } else {
                for (int k = warp; k < 256; k += PQ_WARPS) {
                    float v[BT];
#pragma unroll
                    for (int t = 0; t < BT; t++) v[t] = 0.0f;
                    if (sub_ok && k < Kl) {
                        for (int i = 0; i < half; i++) {
                            const float c = __half2float(cb[(size_t)k * half + i]);
#pragma unroll
                            for (int t = 0; t < BT; t++) v[t] = fmaf(c, xs[t][lane][i], v[t]);
                        }
                    }
                    float* dst = lut + ((size_t)k * 32 + lane) * BT;
#pragma unroll
                    for (int t = 0; t < BT; t++) dst[BT == 2 ? t ^ (lane & 1) : t] = v[t];
                }
            }
        }
        if (j == 0) {
            if (!p.amax_bits) {
#pragma unroll
                for (int t = 0; t < BT; t++) ab[t] = __reduce_max_sync(0xffffffffu, ab[t]);
            }
            if (lane == 0) {
#pragma unroll
                for (int t = 0; t < BT; t++) red[t][warp] = ab[t];
            }
        }
        __syncthreads();                                     // the table is complete (and, for the first slab, the maxima are in place)
        if (j == 0) {
#pragma unroll
            for (int t = 0; t < BT; t++) {
                unsigned m = red[t][0];
#pragma unroll
                for (int w = 1; w < PQ_WARPS; w++) m = max(m, red[t][w]);
                anybad |= m > 0x7f7fffffu;                                         // a NaN or an Inf among the activations of this pass
                amax[t] = __uint_as_float(m);
                // fixed-point scale: 2^e >= N * max|codebook| * max|x| bounds every row sum
                const float bound = (float)p.N * cbmax * amax[t];
                int e = (int)((__float_as_uint(bound) >> 23) & 0xFF) - 126;         // bound < 2^e
                e = max(-60, min(120, e));
                inv_q[t] = __uint_as_float((uint32_t)(127 + 62 - e) << 23);            // 2^(62 - e)
            }
        }
        // the reference drops a chunk (both of its subspaces) whose largest |x| is under 1 % of the largest overall:
        // this lane's subspace then contributes nothing
        bool dead[BT];
        unsigned any_dead = 0;
#pragma unroll
        for (int t = 0; t < BT; t++) {
            dead[t] = false;
            if (t < nb && s0 + lane < nsub && amax[t] > 0.0f && !p.no_skip) {
                const int l0 = lane & ~1;
                float cm = 0.0f;
                for (int i = 0; i < half; i++) cm = fmaxf(cm, fmaxf(fabsf(xs[t][l0][i]), fabsf(xs[t][l0 + 1][i])));
                dead[t] = !(cm >= amax[t] * 0.01f);
            }
            any_dead |= __ballot_sync(0xffffffffu, dead[t]);
        }
        // ── gather: a warp per group of 16 rows, the codes of the next PQ_NG groups in flight meanwhile ──
        for (int c0 = 0; c0 < ngw; c0 += PQ_NG) {
            uint4 nx[PQ_NG];
            if (c0 + PQ_NG < ngw) load_codes(slab, c0 + PQ_NG, nx);
#pragma unroll
            for (int q4 = 0; q4 < PQ_NG; q4++) {
                if (c0 + q4 >= ngw) break;
                const int g = g_lo + warp + PQ_WARPS * (c0 + q4);
                const uint4 cw = cd[q4];
                float v[16 * BT];
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    const uint32_t w = i < 4 ? cw.x : (i < 8 ? cw.y : (i < 12 ? cw.z : cw.w));
                    const uint32_t code = __byte_perm(w, 0u, 0x4440u | (i & 3));     // one byte-permute; shift-and-mask became a byte-to-word conversion on the quarter-rate conversion pipe, which then bounded the gather
                    if constexpr (BT == 2) {
                        const float2 q = *reinterpret_cast<const float2*>(lut + ((size_t)code * 32 + lane) * 2);
                        v[2 * i] = q.x; v[2 * i + 1] = q.y;                                 // value 2 i + u: row i ^ (lane >> 1), activation u ^ (lane & 1)
                    } else v[i] = lut[code * 32 + lane];
                }
                if (any_dead) {
#pragma unroll
                    for (int u = 0; u < BT; u++)
#pragma unroll
                        for (int i = 0; i < 16; i++) v[i * BT + u] = dead[BT == 2 ? u ^ (lane & 1) : u] ? 0.0f : v[i * BT + u];
                }
                if constexpr (BT == 2) { fold<32>(v, 16); fold<16>(v, 8); fold<8>(v, 4); fold<4>(v, 2); fold<2>(v, 1); }
                else { fold<16>(v, 16); fold<8>(v, 8); fold<4>(v, 4); fold<2>(v, 2); v[0] += __shfl_xor_sync(0xffffffffu, v[0], 1); }
                // value 0 of lane l is now the sum over the 32 subspaces of row l >> 1 (and, with two activations, of activation l & 1)
                if constexpr (BT == 2) {
                    const int t = lane & 1, r = 16 * g + (lane >> 1);
                    if (t < nb) atomicAdd(p.acc + (size_t)(b0 + t) * p.M_pad + r, (unsigned long long)__float2ll_rn(v[0] * inv_q[t]));
                } else if ((lane & 1) == 0) {
                    const int r = 16 * g + (lane >> 1);
                    atomicAdd(p.acc + (size_t)b0 * p.M_pad + r, (unsigned long long)__float2ll_rn(v[0] * inv_q[0]));
                }
            }
            if (c0 + PQ_NG < ngw) {
#pragma unroll
                for (int i = 0; i < PQ_NG; i++) cd[i] = nx[i];
            }
        }
    }
    // ── the block that arrives last for these rows turns the sums into the result ──
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        unsigned int* cnt = p.arrive + (size_t)blockIdx.z * gridDim.x + blockIdx.x;        // one counter per pass and block of rows
        const unsigned int n = atomicAdd(cnt, 1u);
        last_s = n == gridDim.y - 1;
        if (last_s) *cnt = 0;
    }
    __syncthreads();
    if (!last_s) return;
    __threadfence();
    if (nj == 0) {                                            // a block without slabs saw no maxima; it cannot be last unless it is alone
#pragma unroll
        for (int t = 0; t < BT; t++) { amax[t] = 0.0f; }
    }
    for (int e0 = 0; e0 < rows * nb; e0 += PQ_FIN * PQ_THREADS) {
        long long sum[PQ_FIN];
#pragma unroll
        for (int u = 0; u < PQ_FIN; u++) {
            const int e = e0 + tid + u * PQ_THREADS;
            sum[u] = 0;
            if (e < rows * nb) sum[u] = (long long)atomicExch(p.acc + (size_t)(b0 + e / rows) * p.M_pad + row_lo + e % rows, 0ull);
        }
#pragma unroll
        for (int u = 0; u < PQ_FIN; u++) {
            const int e = e0 + tid + u * PQ_THREADS;
            if (e >= rows * nb) continue;
            const int t = e / rows, r = row_lo + e % rows;
            const float bound = (float)p.N * cbmax * amax[t];
            int ex = (int)((__float_as_uint(bound) >> 23) & 0xFF) - 126;
            ex = max(-60, min(120, ex));
            const double q = __longlong_as_double((long long)(1023 + ex - 62) << 52);              // 2^(ex - 62)
            const float sc = e0 == 0 ? rsc[u] : __half2float(p.row_scale[r]);
            float y = (float)((double)sum[u] * q) * sc;
            if (anybad) y = __int_as_float(0x7fc00000);                                             // an activation held NaN or Inf
            p.out[(size_t)(b0 + t) * p.out_stride + r] = y;
        }
    }
    // padded rows of the last group also received sums
    const int pad = row_hi - min(row_hi, p.M);
    for (int e = tid; e < pad * nb; e += PQ_THREADS) {
        const int t = e / pad, r = min(row_hi, p.M) + (e - t * pad);
        p.acc[(size_t)(b0 + t) * p.M_pad + r] = 0ull;
    }
}

// ── Several activations, plain tensor with shared codebooks of 8-wide entries: pq_wide_kernel ──
// The gather is bound by the shared-memory pipe: a table read and a lane-to-lane shuffle each move 32 values per cycle, and
// the reduction over the lanes costs one shuffle per 32 values looked up. Here a lane owns four subspaces (a unit of work is
// one activation x 128 subspaces, table of 128 KB) and adds their entries in registers before the lanes meet: a quarter of
// the shuffles. Units x groups of 16 rows form one list that the blocks (one per SM) cut into equal contiguous pieces, so
// every SM has the same share whatever the shape; a piece that crosses a unit builds a second table. Sums meet in the same
// fixed-point accumulators; the block whose arrival completes an activation's count of pieces converts that activation.
constexpr int PW_THREADS = 1024;
constexpr int PW_WARPS = PW_THREADS / 32;
constexpr int PW_Q = 4;                                      // subspaces per lane: slabs 4 u .. 4 u + 3 of the code plane
constexpr int PW_MAXSEG = 8;
// Table layout: quarters 2 h and 2 h + 1 share a region of 64 KB that starts at shared-memory address 64 KB * (h + 1); entry k of
// quarter q, lane l sits at byte k * 256 + (q & 1) * 128 + 4 l of its region: bank l as before, and the code is byte 1 of the
// address, so one byte-permute of the code word and the lane's base address yields the address of a table read. The codebooks
// and the slices of x live below the first region.
constexpr size_t PW_SMEM = 3 * 65536;
constexpr size_t PW_LOW_BYTES = 256 * 2 * 2 * sizeof(float4) + PW_Q * 32 * 9 * sizeof(float);

__global__ void __launch_bounds__(PW_THREADS, 1) pq_wide_kernel(const PqParams p, int nunit, int per_block, int* err) {
    extern __shared__ __align__(16) unsigned char pw_smem[];
    const uint32_t dyn = (uint32_t)__cvta_generic_to_shared(pw_smem);                                                           // shared-memory address of the dynamic part
    float4 (*cbf)[2][2] = reinterpret_cast<float4 (*)[2][2]>(pw_smem);                                // [k][side][half of the entry], FP32
    float (*xs)[9] = reinterpret_cast<float (*)[9]>(pw_smem + 256 * 2 * 2 * sizeof(float4));          // [4 * 32 subspaces][8 (+1)]
    unsigned char* lut_b = pw_smem + (65536u - dyn);                                                  // the byte at shared-memory address 64 KB
    if (dyn + PW_LOW_BYTES > 65536u) { if (threadIdx.x == 0) *err = 7001; return; }               // the host reports it at the next sync; cannot happen with this kernel's static data
    __shared__ int seg_tok[PW_MAXSEG], seg_n[PW_MAXSEG], seg_last[PW_MAXSEG];
    __shared__ unsigned char sub_dead[PW_Q * 32];             // per subspace of the unit: its chunk falls under the 1 % rule
    __shared__ unsigned amax_s[32], red_s[2][PW_WARPS];       // bit pattern of max |x| of the activations this block meets
    pdl_launch_dependents();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int G16 = p.M_pad >> 4, nsub = 2 * p.C;
    // positions in the list of (unit, activation, group) fit 32 bits (the host checks): 64-bit divisions would cost more
    // instructions per segment than the table build
    const unsigned total = (unsigned)nunit * (unsigned)p.B * (unsigned)G16;
    const unsigned lo = min(total, blockIdx.x * (unsigned)per_block);
    const unsigned hi = min(total, lo + (unsigned)per_block);
    // weights first, they do not depend on the previous kernel
    if (tid < 512) {
        const int side = tid >> 8, k = tid & 255;
        const uint4 raw = k < p.K ? reinterpret_cast<const uint4*>(side ? p.cb_r : p.cb_l)[k] : make_uint4(0, 0, 0, 0);
        const __half2* h = reinterpret_cast<const __half2*>(&raw);
        const float2 f0 = __half22float2(h[0]), f1 = __half22float2(h[1]), f2 = __half22float2(h[2]), f3 = __half22float2(h[3]);
        cbf[k][side][0] = make_float4(f0.x, f0.y, f1.x, f1.y);
        cbf[k][side][1] = make_float4(f2.x, f2.y, f3.x, f3.y);
    }
    const float cbmax = __int_as_float(*reinterpret_cast<const int*>(p.idx_t + (size_t)p.tail_slabs * G16 * 512));
    const uint4* plane = reinterpret_cast<const uint4*>(p.idx_t) + lane;
    // this thread's activation of a segment: subspace s of a unit covers x[8 s, 8 s + 8)
    auto load_x = [&](unsigned at_) -> float {
        if (at_ >= hi) return 0.0f;
        const unsigned ut_ = at_ / (unsigned)G16;
        const int u_ = (int)(ut_ / (unsigned)p.B), t_ = (int)(ut_ - (unsigned)u_ * (unsigned)p.B);
        const int sb = u_ * (PW_Q * 32) + (tid >> 3);
        return sb < nsub ? p.x[(size_t)t_ * p.N + (size_t)sb * 8 + (tid & 7)] : 0.0f;
    };
    pdl_wait();
    float xnext = load_x(lo);                                // in flight while the maxima are taken
    // max |x| of the activations in this block's piece of the list (consecutive ones, two at a time so that their loads
    // travel together): the 1 % rule and the fixed-point scale need it. As bit patterns: those of non-negative floats
    // order like the floats, and NaN / Inf sort last.
    if (lo < hi) {
        const unsigned ut_lo = lo / (unsigned)G16, ut_hi = (hi - 1) / (unsigned)G16;
        const int ntok = (int)min((unsigned)p.B, ut_hi - ut_lo + 1);
        const bool vec_x = (p.N & 3) == 0 && ((uintptr_t)p.x & 15) == 0;
        for (int j0 = 0; j0 < ntok; j0 += 2) {
            unsigned m[2] = { 0u, 0u };
            int tk[2];
            tk[0] = (int)((ut_lo + (unsigned)j0) % (unsigned)p.B);
            tk[1] = j0 + 1 < ntok ? (int)((ut_lo + (unsigned)j0 + 1u) % (unsigned)p.B) : tk[0];       // alone: the same activation twice
            const float* xb0 = p.x + (size_t)tk[0] * p.N;
            const float* xb1 = p.x + (size_t)tk[1] * p.N;
            if (vec_x) {
                const uint4* xa = reinterpret_cast<const uint4*>(xb0);
                const uint4* xc = reinterpret_cast<const uint4*>(xb1);
#pragma unroll 4
                for (int i = tid; i < (p.N >> 2); i += PW_THREADS) {
                    const uint4 v = xa[i], w = xc[i];
                    m[0] = max(max(m[0], v.x & 0x7fffffffu), max(max(v.y & 0x7fffffffu, v.z & 0x7fffffffu), v.w & 0x7fffffffu));
                    m[1] = max(max(m[1], w.x & 0x7fffffffu), max(max(w.y & 0x7fffffffu, w.z & 0x7fffffffu), w.w & 0x7fffffffu));
                }
            } else {
                for (int i = tid; i < p.N; i += PW_THREADS) {
                    m[0] = max(m[0], __float_as_uint(xb0[i]) & 0x7fffffffu);
                    m[1] = max(m[1], __float_as_uint(xb1[i]) & 0x7fffffffu);
                }
            }
#pragma unroll
            for (int h = 0; h < 2; h++) {
                m[h] = __reduce_max_sync(0xffffffffu, m[h]);
                if (lane == 0) red_s[h][warp] = m[h];
            }
            __syncthreads();
            if (warp < 2 && j0 + warp < ntok) {
                const unsigned r = __reduce_max_sync(0xffffffffu, red_s[warp][lane]);
                if (lane == 0) amax_s[tk[warp]] = r;
            }
            __syncthreads();
        }
    }

    // what the block owes the arrival counters: (activation, pieces) of every segment since the last flush
    int nseg = 0;
    auto flush = [&]() {
        __threadfence();
        __syncthreads();
        if (tid < nseg) {
            const unsigned want = (unsigned)nunit * (unsigned)G16;
            const unsigned old = atomicAdd(p.arrive + seg_tok[tid], (unsigned)seg_n[tid]);
            seg_last[tid] = old + (unsigned)seg_n[tid] == want;
            if (seg_last[tid]) p.arrive[seg_tok[tid]] = 0;
        }
        __syncthreads();
        for (int sgi = 0; sgi < nseg; sgi++) {
            if (!seg_last[sgi]) continue;
            // every piece of this activation has arrived, each behind its block's fence: plain loads past L1 read the sums
            __threadfence();
            const int t = seg_tok[sgi];
            const unsigned ab = amax_s[t];
            const float bound = (float)p.N * cbmax * __uint_as_float(ab);
            int ex = (int)((__float_as_uint(bound) >> 23) & 0xFF) - 126;
            ex = max(-60, min(120, ex));
            const double q = __longlong_as_double((long long)(1023 + ex - 62) << 52);                  // 2^(ex - 62)
            const bool bad = ab > 0x7f7fffffu;                                                            // a NaN or an Inf among the activations
            unsigned long long* acc = p.acc + (size_t)t * p.M_pad;
            for (int r0 = 0; r0 < p.M_pad; r0 += 4 * PW_THREADS) {
                long long sum[4];
                float sc[4];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int r = r0 + tid + i * PW_THREADS;
                    sum[i] = r < p.M_pad ? (long long)__ldcg(acc + r) : 0;
                    sc[i] = r < p.M ? __half2float(p.row_scale[r]) : 0.0f;
                }
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int r = r0 + tid + i * PW_THREADS;
                    if (r < p.M_pad) acc[r] = 0ull;                                                      // zero for the next call, padded rows too
                    if (r < p.M) p.out[(size_t)t * p.out_stride + r] = bad ? __int_as_float(0x7fc00000) : (float)((double)sum[i] * q) * sc[i];
                }
            }
        }
        __syncthreads();
        nseg = 0;
    };

    for (unsigned at = lo; at < hi;) {
        const unsigned ut = at / (unsigned)G16;               // unit * B + activation
        const int g0 = (int)(at - ut * (unsigned)G16);
        const int g1 = (int)min((unsigned)G16, (unsigned)g0 + (hi - at));
        const int u = (int)(ut / (unsigned)p.B), t = (int)(ut - (unsigned)u * (unsigned)p.B);
        at += (unsigned)(g1 - g0);
        // codes of this warp's first group: in flight during the table build
        uint4 cd[PW_Q];
        auto load_codes = [&](int g, int q) {
            return (4 * u + q < p.nslab && g < g1) ? ld_stream_u4(plane + ((size_t)(4 * u + q) * G16 + g) * 32) : make_uint4(0, 0, 0, 0);
        };
#pragma unroll
        for (int q = 0; q < PW_Q; q++) cd[q] = load_codes(g0 + warp, q);
        __syncthreads();                                      // the previous segment's gather is done with the table and the slices (first: cbf is staged)
        if (nseg == PW_MAXSEG) flush();
        if (tid == 0) { seg_tok[nseg] = t; seg_n[nseg] = g1 - g0; }
        nseg++;
        xs[tid >> 3][tid & 7] = xnext;                        // this unit's 1024 activations
        xnext = load_x(at);                                   // the next segment's, in flight during this one
        const float amax = __uint_as_float(amax_s[t]);         // written before the barriers above
        const float bound = (float)p.N * cbmax * amax;
        int e = (int)((__float_as_uint(bound) >> 23) & 0xFF) - 126;                                     // bound < 2^e
        e = max(-60, min(120, e));
        const float inv_q = __uint_as_float((uint32_t)(127 + 62 - e) << 23);                              // 2^(62 - e)
        __syncthreads();
        // the reference drops a chunk (both of its subspaces) whose largest |x| is under 1 % of the largest overall
        if (tid < PW_Q * 16) {                                // one thread per chunk of the unit
            float cm = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; i++) cm = fmaxf(cm, fmaxf(fabsf(xs[2 * tid][i]), fabsf(xs[2 * tid + 1][i])));
            const unsigned char d = amax > 0.0f && !p.no_skip && u * (PW_Q * 32) + 2 * tid < nsub && !(cm >= amax * 0.01f);
            sub_dead[2 * tid] = d; sub_dead[2 * tid + 1] = d;
        }
        __syncthreads();
        // table: warp w builds entries k = w + 32 i, two quarters at a time (a codebook entry is read once for the two);
        // each entry is summed in the same order as in the slab kernel
        const int side = lane & 1;
#pragma unroll 1
        for (int qp = 0; qp < PW_Q; qp += 2) {
            float xr[2][8];
#pragma unroll
            for (int q = 0; q < 2; q++) {
                const bool dead = sub_dead[(qp + q) * 32 + lane];            // a dropped subspace gets a table of zeros: the gather need not know
#pragma unroll
                for (int i = 0; i < 8; i++) xr[q][i] = dead ? 0.0f : xs[(qp + q) * 32 + lane][i];
            }
#pragma unroll 2
            for (int k = warp; k < 256; k += PW_WARPS) {
                const float4 ca = cbf[k][side][0], cc = cbf[k][side][1];
#pragma unroll
                for (int q = 0; q < 2; q++) {
                    float a = 0.0f;
                    a = fmaf(ca.x, xr[q][0], a); a = fmaf(ca.y, xr[q][1], a); a = fmaf(ca.z, xr[q][2], a); a = fmaf(ca.w, xr[q][3], a);
                    a = fmaf(cc.x, xr[q][4], a); a = fmaf(cc.y, xr[q][5], a); a = fmaf(cc.z, xr[q][6], a); a = fmaf(cc.w, xr[q][7], a);
                    *reinterpret_cast<float*>(lut_b + (size_t)(qp >> 1) * 65536 + (size_t)k * 256 + q * 128 + lane * 4) = a;
                }
            }
        }
        __syncthreads();                                      // the table is complete
        for (int g = g0 + warp; g < g1; g += PW_WARPS) {
            float v[16];
#pragma unroll
            for (int q = 0; q < PW_Q; q++) {
                const uint4 cw = cd[q];
                cd[q] = load_codes(g + PW_WARPS, q);          // the next group's codes travel while this one is looked up
                const uint32_t tb = 65536u * (1u + (q >> 1)) + (q & 1) * 128u + lane * 4u;     // entry 0 of this lane's subspace; byte 1 of the address is zero
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    const uint32_t w = i < 4 ? cw.x : (i < 8 ? cw.y : (i < 12 ? cw.z : cw.w));
                    const uint32_t addr = __byte_perm(w, tb, 0x7604u | ((i & 3) << 4));          // bytes (tb3, tb2, code, tb0)
                    float val;
                    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(val) : "r"(addr) : "memory");
                    v[i] = q == 0 ? val : v[i] + val;
                }
            }
            fold<16>(v, 16); fold<8>(v, 8); fold<4>(v, 4); fold<2>(v, 2);
            v[0] += __shfl_xor_sync(0xffffffffu, v[0], 1);
            if ((lane & 1) == 0)                              // value 0 of lane l: row l >> 1 of the group
                atomicAdd(p.acc + (size_t)t * p.M_pad + 16 * g + (lane >> 1), (unsigned long long)__float2ll_rn(v[0] * inv_q));
        }
    }
    if (nseg) flush();
}

// Outlier sidecar (src/pq_decode.c:1394-1409): out[r] += sum over j of (sidecar[r][j] * scale[j]) * x[col[j]], added to the finished
// rows. grid (blocks of 8 rows, activations), a warp per row, lanes over the outlier columns.
__global__ void __launch_bounds__(256) pq_outlier_kernel(const int8_t* __restrict__ side, const int32_t* __restrict__ cols, const __half* __restrict__ scale,
                                                         int no, const float* __restrict__ x, int N, float* __restrict__ out, int M, int out_stride) {
    extern __shared__ float xo[];                            // x[col[j]] of this activation
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int j = threadIdx.x; j < no; j += 256) xo[j] = x[(size_t)b * N + cols[j]];
    __syncthreads();
    const int r = blockIdx.x * 8 + warp;
    if (r >= M) return;
    float acc = 0.0f;
    for (int j = lane; j < no; j += 32) {
        const float w = (float)side[(size_t)r * no + j] * __half2float(scale[j]);
        acc = fmaf(w, xo[j], acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) out[(size_t)b * out_stride + r] += acc;
}

struct PqPlan { int C, nslab1, nslab, bt, passes, row_blocks, rows_per_block, slab_blocks; size_t acc_words; int wide, nunit, per_block, nblocks; };

PqPlan pq_plan(const ibcu_ctx* ctx, const ibcu_pq_t* t, int B, bool l1_only = false) {
    PqPlan pl;
    pl.C = (t->N - t->n_outlier) / t->G;
    pl.nslab1 = (2 * pl.C + 31) / 32;
    pl.nslab = (t->K_l2 > 0 && !l1_only) ? 2 * pl.nslab1 : pl.nslab1;
    pl.bt = B >= 2 ? 2 : 1;
    pl.passes = (B + pl.bt - 1) / pl.bt;
    const int slots = ctx->sm_count * 2;
    const int groups = t->M_pad / 16;
    pl.slab_blocks = pl.nslab < slots ? pl.nslab : slots;                    // more slabs than blocks: a block walks several
    // Blocks of rows: every one of them builds the tables of its slab again, so few are cheap in arithmetic, but the
    // grid should fill whole rounds of the machine. Cost model in warp instructions: a table ~ 3000 * bt, the
    // gather of all rows ~ groups * 125 * bt, per slab and pass.
    const long units = (long)pl.slab_blocks * pl.passes;
    const long slabs_per_block = (pl.nslab + pl.slab_blocks - 1) / pl.slab_blocks;
    int best_rb = 1; double best = 1e30;
    for (int rb = 1; rb <= 16 && rb <= groups; rb++) {
        const long rounds = (units * rb + slots - 1) / slots;
        const double cost = (double)rounds * slabs_per_block * (3000.0 + 125.0 * ((groups + rb - 1) / rb));
        if (cost < best * 0.98) { best = cost; best_rb = rb; }
    }
    const int gpb = (groups + best_rb - 1) / best_rb;
    pl.rows_per_block = gpb * 16;
    pl.row_blocks = (groups + gpb - 1) / gpb;
    pl.acc_words = (size_t)B * t->M_pad;
    // three or more activations of a plain tensor with shared 8-wide codebooks: the kernel with four subspaces per lane
    // (4096 x 14336: 21.8 against 26.5 us at three activations; at two the slab kernel's single pass wins, 17.6 against 20.2 us)
    pl.wide = B >= 3 && !l1_only && t->K_l2 == 0 && t->n_outlier == 0 && t->G == 16 && t->cb_chunk_stride == 0 &&
              (((uintptr_t)t->codebook_l | (uintptr_t)t->codebook_r) & 15) == 0;
    pl.nunit = (pl.nslab + PW_Q - 1) / PW_Q;
    const long total = (long)pl.nunit * B * groups;
    if (total >= (1l << 30)) pl.wide = 0;                    // the kernel counts its pieces in 32 bits
    const long nb = total < ctx->sm_count ? total : ctx->sm_count;
    pl.per_block = (int)((total + nb - 1) / nb);
    pl.nblocks = (int)((total + pl.per_block - 1) / pl.per_block);
    return pl;
}

int pq_launch(ibcu_ctx* ctx, const ibcu_pq_t* t, const float* x, float* out, int out_stride, int B, const PqPlan& pl,
              unsigned long long* acc, unsigned int* arrive, bool l1_only = false) {
    PqParams p;
    p.M = t->M; p.M_pad = t->M_pad; p.N = t->N; p.G = t->G; p.K = t->K; p.C = pl.C; p.B = B; p.nslab = pl.nslab;
    p.rows_per_block = pl.rows_per_block;
    p.cb_l = (const __half*)t->codebook_l; p.cb_r = (const __half*)t->codebook_r; p.cb_stride = t->cb_chunk_stride;
    p.idx_t = t->idx_t; p.row_scale = (const __half*)t->row_scale; p.x = x; p.out = out; p.out_stride = out_stride; p.acc = acc; p.arrive = arrive;
    p.amax_bits = nullptr;
    p.nslab1 = pl.nslab1; p.K2 = t->K_l2; p.cb2_l = (const __half*)t->codebook2_l; p.cb2_r = (const __half*)t->codebook2_r;
    p.inner = t->n_outlier > 0 ? t->inner_cols : nullptr; p.n_inner = t->N - t->n_outlier;
    p.tail_slabs = t->K_l2 > 0 ? 2 * pl.nslab1 : pl.nslab1; p.no_skip = l1_only ? 1 : 0;
    const bool ex = t->K_l2 > 0 || t->n_outlier > 0;
    const dim3 grid(pl.row_blocks, pl.slab_blocks, pl.passes), block(PQ_THREADS);
    // static plus dynamic shared memory passes 48 KB: opt in once per device
    static std::once_flag once[64];
    cudaError_t e = cudaSuccess;
    std::call_once(once[ctx->device & 63], [&] {
        e = cudaFuncSetAttribute(pq_slab_kernel<2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 256 * 32 * 2 * (int)sizeof(float));
        if (e == cudaSuccess) e = cudaFuncSetAttribute(pq_slab_kernel<1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 256 * 32 * (int)sizeof(float));
        if (e == cudaSuccess) e = cudaFuncSetAttribute(pq_slab_kernel<2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 256 * 32 * 2 * (int)sizeof(float));
        if (e == cudaSuccess) e = cudaFuncSetAttribute(pq_slab_kernel<1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 256 * 32 * (int)sizeof(float));
        if (e == cudaSuccess) e = cudaFuncSetAttribute(pq_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PW_SMEM);
    });
    if (e != cudaSuccess) return ibcu_fail(ctx, IBCU_ERR_CUDA, "cudaFuncSetAttribute(pq_slab_kernel): %s", cudaGetErrorString(e));
    if (pl.wide)                               // takes the maxima of the activations it meets itself
        return ibcu_launch(ctx, pq_wide_kernel, dim3(pl.nblocks), dim3(PW_THREADS), PW_SMEM, 1, true, p, pl.nunit, pl.per_block, ctx->kern_err);
    if (pl.bt == 2) {
        // with several activations every block would scan all of them for their maxima: one small launch does it once;
        // its results sit in the last 64 counter slots, which no pass uses
        unsigned* amax_bits = arrive + (PQ_COUNTER_BYTES / sizeof(unsigned) - 64);
        int rc = ibcu_launch(ctx, pq_amax_kernel, dim3(B), dim3(512), 0, 1, true, x, t->N, amax_bits, p.inner, p.n_inner);
        if (rc) return rc;
        p.amax_bits = amax_bits;
        rc = ex ? ibcu_launch(ctx, pq_slab_kernel<2, true>, grid, block, (size_t)256 * 32 * 2 * sizeof(float), 1, true, p)
                : ibcu_launch(ctx, pq_slab_kernel<2, false>, grid, block, (size_t)256 * 32 * 2 * sizeof(float), 1, true, p);
        if (rc) return rc;
    } else {
        const int rc = ex ? ibcu_launch(ctx, pq_slab_kernel<1, true>, grid, block, (size_t)256 * 32 * sizeof(float), 1, true, p)
                          : ibcu_launch(ctx, pq_slab_kernel<1, false>, grid, block, (size_t)256 * 32 * sizeof(float), 1, true, p);
        if (rc) return rc;
    }
    if (t->n_outlier > 0)                                    // the sidecar's share is added to the finished rows (src/pq_decode.c:1676)
        return ibcu_launch(ctx, pq_outlier_kernel, dim3((t->M + 7) / 8, B), dim3(256), (size_t)t->n_outlier * sizeof(float), 1, true,
                           t->outlier_sidecar, t->outlier_cols, (const __half*)t->outlier_scale, t->n_outlier, x, t->N, out, t->M, out_stride);
    return IBCU_OK;
}

int pq_check(ibcu_ctx* ctx, const ibcu_pq_t* t, const float* x, float* out, int B, const char* who) {
    IBCU_REQUIRE(ctx, t && x && out, "%s: null pointer", who);
    IBCU_REQUIRE(ctx, t->codebook_l && t->codebook_r && t->row_scale, "%s: tensor has a null pointer", who);
    IBCU_REQUIRE(ctx, t->idx_t && t->M_pad >= t->M && (t->M_pad & 15) == 0, "%s: call ibcu_pq_prepare on the tensor first", who);
    IBCU_REQUIRE(ctx, t->M > 0 && t->N > 0 && t->G > 0 && (t->G & 1) == 0 && t->G <= 32 && t->n_outlier >= 0 && t->n_outlier < t->N &&
                      (t->N - t->n_outlier) % t->G == 0 && t->K >= 1 && t->K <= 256,
                 "%s: bad shape M=%d N=%d G=%d K=%d outliers=%d", who, t->M, t->N, t->G, t->K, t->n_outlier);
    IBCU_REQUIRE(ctx, t->K_l2 == 0 || (t->K_l2 >= 1 && t->K_l2 <= 256 && t->codebook2_l && t->codebook2_r), "%s: second level with K_l2=%d", who, t->K_l2);
    IBCU_REQUIRE(ctx, t->n_outlier == 0 || (t->outlier_cols && t->outlier_sidecar && t->outlier_scale && t->inner_cols), "%s: outlier arrays missing", who);
    IBCU_REQUIRE(ctx, B >= 1 && B <= 32, "%s: B=%d not in 1..32", who, B);
    return IBCU_OK;
}

}  // namespace

static size_t pq_scratch_bytes(const PqPlan& pl) { return PQ_COUNTER_BYTES + pl.acc_words * sizeof(unsigned long long); }

extern "C" size_t ibcu_pq_idx_t_bytes(int M, int N, int G) {
    if (M <= 0 || N <= 0 || G <= 0 || N % G) return 0;
    const size_t M_pad = ((size_t)M + 15) & ~(size_t)15;
    const size_t nslab = (2 * (size_t)(N / G) + 31) / 32;
    return nslab * 32 * M_pad + PQ_TAIL;
}

extern "C" size_t ibcu_pq_prepared_bytes(const ibcu_pq_t* t) {
    if (!t || t->M <= 0 || t->N <= 0 || t->G <= 0 || t->n_outlier < 0 || t->n_outlier >= t->N || (t->N - t->n_outlier) % t->G) return 0;
    const size_t M_pad = ((size_t)t->M + 15) & ~(size_t)15;
    const size_t nslab1 = (2 * (size_t)((t->N - t->n_outlier) / t->G) + 31) / 32;
    const size_t nslab = t->K_l2 > 0 ? 2 * nslab1 : nslab1;
    return nslab * 32 * M_pad + PQ_TAIL + (t->n_outlier > 0 ? (size_t)(t->N - t->n_outlier) * sizeof(int32_t) : 0);
}

// inner[k] = k-th column that is not an outlier column (ascending), as src/pq_decode.c:1538-1546 builds it
__global__ void __launch_bounds__(256) pq_inner_cols_kernel(const int32_t* __restrict__ ocols, int no, int N, int32_t* __restrict__ inner) {
    for (int j = blockIdx.x * blockDim.x + threadIdx.x; j < N; j += gridDim.x * blockDim.x) {
        // rank of j among the outlier columns (sorted): columns below j that are outliers
        int lo = 0, hi = no;
        while (lo < hi) { const int mid = (lo + hi) >> 1; if (ocols[mid] < j) lo = mid + 1; else hi = mid; }
        if (lo < no && ocols[lo] == j) continue;             // an outlier column itself
        inner[j - lo] = j;
    }
}

extern "C" int ibcu_pq_prepare(ibcu_ctx* ctx, ibcu_pq_t* t, uint8_t* idx_t_out) {
    IBCU_CHECK_CTX(ctx);
    IBCU_REQUIRE(ctx, t && idx_t_out && t->idx_l && t->idx_r && t->codebook_l && t->codebook_r, "ibcu_pq_prepare: null pointer");
    IBCU_REQUIRE(ctx, t->M > 0 && t->N > 0 && t->G > 0 && (t->G & 1) == 0 && t->n_outlier >= 0 && t->n_outlier < t->N &&
                      (t->N - t->n_outlier) % t->G == 0 && t->K >= 1 && t->K <= 256,
                 "ibcu_pq_prepare: bad shape M=%d N=%d G=%d K=%d outliers=%d", t->M, t->N, t->G, t->K, t->n_outlier);
    IBCU_REQUIRE(ctx, t->K_l2 == 0 || (t->K_l2 >= 1 && t->K_l2 <= 256 && t->codebook2_l && t->codebook2_r && t->idx2_l && t->idx2_r),
                 "ibcu_pq_prepare: second level with K_l2=%d (at most 256 entries, one-byte or 4-bit indices)", t->K_l2);
    IBCU_REQUIRE(ctx, t->n_outlier == 0 || (t->outlier_cols && t->outlier_sidecar && t->outlier_scale), "ibcu_pq_prepare: outlier arrays missing");
    IBCU_REQUIRE(ctx, t->K_l2 == 0 || t->cb_chunk_stride == 0, "ibcu_pq_prepare: a second level needs shared codebooks");
    IBCU_REQUIRE(ctx, ((uintptr_t)idx_t_out & 15) == 0, "ibcu_pq_prepare: idx_t_out must be 16-byte aligned");
    const int C = (t->N - t->n_outlier) / t->G, half = t->G / 2;
    const int M_pad = (t->M + 15) & ~15;
    const int nslab1 = (2 * C + 31) / 32, nslab = t->K_l2 > 0 ? 2 * nslab1 : nslab1;
    const size_t plane = (size_t)nslab1 * 32 * M_pad, body = (size_t)nslab * 32 * M_pad;
    const long vecs = (long)(plane / 16);
    int blocks = (int)((vecs + 255) / 256);
    if (blocks > ctx->sm_count * 8) blocks = ctx->sm_count * 8;
    int rc = ibcu_launch(ctx, pq_pack_kernel, dim3(blocks), dim3(256), 0, 1, false, t->idx_l, t->idx_r, t->M, C, M_pad, nslab1, idx_t_out, 0);
    if (rc) return rc;
    if (t->K_l2 > 0) {
        rc = ibcu_launch(ctx, pq_pack_kernel, dim3(blocks), dim3(256), 0, 1, false, t->idx2_l, t->idx2_r, t->M, C, M_pad, nslab1, idx_t_out + plane,
                         t->K_l2 == 16 ? 1 : 0);
        if (rc) return rc;
    }
    IBCU_CUDA(ctx, cudaMemsetAsync(idx_t_out + body, 0, PQ_TAIL, ctx->stream));
    // largest magnitude over the entries of all tables: one pair when the tables are shared, one pair per chunk otherwise; then the second level's
    const size_t n = t->cb_chunk_stride ? (size_t)(C - 1) * t->cb_chunk_stride + (size_t)t->K * half : (size_t)t->K * half;
    int ab = (int)((n + 255) / 256);
    if (ab > ctx->sm_count * 4) ab = ctx->sm_count * 4;
    rc = ibcu_launch(ctx, pq_absmax_kernel, dim3(ab), dim3(256), 0, 1, false, (const __half*)t->codebook_l, (const __half*)t->codebook_r, n,
                     reinterpret_cast<float*>(idx_t_out + body));
    if (rc) return rc;
    if (t->K_l2 > 0) {
        // the fixed-point bound is N * (largest entry) * max|x| per level: with two levels the sum of both levels' largest entries bounds a pair of terms
        rc = ibcu_launch(ctx, pq_absmax_kernel, dim3(1), dim3(256), 0, 1, false, (const __half*)t->codebook2_l, (const __half*)t->codebook2_r,
                         (size_t)t->K_l2 * half, reinterpret_cast<float*>(idx_t_out + body) + 1);
        if (rc) return rc;
        rc = ibcu_launch(ctx, pq_add_tail_kernel, dim3(1), dim3(32), 0, 1, false, reinterpret_cast<float*>(idx_t_out + body));
        if (rc) return rc;
    }
    if (t->n_outlier > 0) {
        int32_t* inner = reinterpret_cast<int32_t*>(idx_t_out + body + PQ_TAIL);
        int ib = (t->N + 255) / 256;
        if (ib > ctx->sm_count * 4) ib = ctx->sm_count * 4;
        rc = ibcu_launch(ctx, pq_inner_cols_kernel, dim3(ib), dim3(256), 0, 1, false, t->outlier_cols, t->n_outlier, t->N, inner);
        if (rc) return rc;
        t->inner_cols = inner;
    }
    t->idx_t = idx_t_out;
    t->M_pad = M_pad;
    return IBCU_OK;
}

extern "C" int ibcu_pq_matmul_fp32(ibcu_ctx* ctx, const ibcu_pq_t* t, const float* x, float* out, int B) {
    return ibcu_pq_matmul_fp32_strided(ctx, t, x, out, t ? t->M : 0, B);
}

extern "C" int ibcu_pq_matmul_fp32_strided(ibcu_ctx* ctx, const ibcu_pq_t* t, const float* x, float* out, int out_stride, int B) {
    IBCU_CHECK_CTX(ctx);
    int rc = pq_check(ctx, t, x, out, B, "ibcu_pq_matmul_fp32");
    if (rc) return rc;
    IBCU_REQUIRE(ctx, out_stride >= t->M, "ibcu_pq_matmul_fp32_strided: out_stride=%d below M=%d", out_stride, t->M);
    const PqPlan pl = pq_plan(ctx, t, B);
    const size_t need = pq_scratch_bytes(pl);
    if (ctx->pq_acc_bytes < need) {
        // the accumulators and counters must read zero when a call starts and every call leaves them so:
        // they are cleared once, when the buffer is made
        rc = ibcu_reserve(ctx, &ctx->pq_acc, &ctx->pq_acc_bytes, need);
        if (rc) return rc;
        IBCU_CUDA(ctx, cudaMemsetAsync(ctx->pq_acc, 0, ctx->pq_acc_bytes, ctx->stream));
    }
    return pq_launch(ctx, t, x, out, out_stride, B, pl, (unsigned long long*)((char*)ctx->pq_acc + PQ_COUNTER_BYTES), (unsigned int*)ctx->pq_acc);
}

// ── top-K LM head (src/pq_decode.c:2259-2341) ───────────────────────────────────────────
// Three launches: the first-level matvec over all rows without the 1 % rule (the kernels above), the choice of the
// K_top rows with the largest first-level logits, and every level of those rows, whose last block orders them by full logit.
namespace {

constexpr int TOPK_MAX = 1024;
constexpr int TOPK_THREADS = 1024;

// What the kernel before wrote (first-level logits, chosen rows, their full logits) is read past L1 (__ldcg): these
// kernels start while their predecessor still runs, and a read-only-path load after the dependency wait returned the
// previous call's values here (the chosen rows came out paired with another call's order).
// keys order like the floats (negative values reversed, positive ones above them)
__device__ __forceinline__ unsigned topk_key(float v) {
    const unsigned u = __float_as_uint(v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// One block (the fallback for more rows than the cluster kernel below keeps in registers). The K_top-th largest key by
// passes of 8-bit digit counts over (key - smallest key), from its highest set bit down: counted from the smallest key
// the first digit already spreads the rows over the table (logits themselves share their leading bits, and adds to a
// few shared counters queue behind one another), and later passes only touch the rows of one digit. Then the rows above
// the threshold in any order and, of the rows equal to it, those with the lowest indices: cand[0 .. K_top). The
// reference keeps the first row it met among equal first-level logits at the boundary too (a later row replaces the
// heap's root only when strictly larger), but which equal rows survive inside its heap depends on the heap's shape;
// equal logits at the boundary are a tie that callers cannot rely on either way.
__global__ void __launch_bounds__(TOPK_THREADS) pq_topk_select_kernel(const float* __restrict__ coarse, int M, int K_top, int32_t* __restrict__ cand) {
    __shared__ unsigned hist[256], red_lo[TOPK_THREADS / 32], red_hi[TOPK_THREADS / 32];
    __shared__ unsigned s_prefix, s_need, s_gt, s_eq_before, warp_tot[TOPK_THREADS / 32];
    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nchunk = (M + TOPK_THREADS - 1) / TOPK_THREADS;
    auto key_at = [&](int j) -> unsigned {                    // key of row tid + 1024 j
        const int i = tid + j * TOPK_THREADS;
        return i < M ? topk_key(__ldcg(coarse + i)) : 0u;
    };
    unsigned lo = 0xffffffffu, hi = 0u;
    for (int j = 0; j < nchunk; j++) if (tid + j * TOPK_THREADS < M) { const unsigned k = key_at(j); lo = min(lo, k); hi = max(hi, k); }
    lo = __reduce_min_sync(0xffffffffu, lo); hi = __reduce_max_sync(0xffffffffu, hi);
    if (lane == 0) { red_lo[warp] = lo; red_hi[warp] = hi; }
    if (tid == 0) { s_prefix = 0u; s_need = (unsigned)K_top; }
    __syncthreads();
    lo = __reduce_min_sync(0xffffffffu, red_lo[lane]); hi = __reduce_max_sync(0xffffffffu, red_hi[lane]);
    int shift = 32 - __clz(hi - lo);                          // bits of (key - lo) in use; 0 when all keys are equal
    while (shift > 0) {
        const int width = shift < 8 ? shift : 8;
        const int top = shift;                                // the bits at and above `top` are settled: they equal s_prefix there
        shift -= width;
        if (tid < 256) hist[tid] = 0u;
        __syncthreads();
        const unsigned prefix = s_prefix, need0 = s_need, mask = top >= 32 ? 0u : 0xffffffffu << top;
        for (int j = 0; j < nchunk; j++) {
            const unsigned k = key_at(j) - lo;
            if (tid + j * TOPK_THREADS < M && (k & mask) == prefix) atomicAdd(&hist[(k >> shift) & ((1u << width) - 1u)], 1u);
        }
        __syncthreads();
        // counts from the top digit down, as running sums over 256 threads: the digit at which the sum reaches what is still needed
        unsigned c = 0, incl = 0;
        if (tid < 256) {
            c = hist[255 - tid];
            incl = c;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) { const unsigned n = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += n; }
            if (lane == 31) warp_tot[warp] = incl;
        }
        __syncthreads();
        if (tid < 256) {
            for (int w = 0; w < warp; w++) incl += warp_tot[w];
            const unsigned excl = incl - c;
            if (excl < need0 && need0 <= incl) {
                s_need = need0 - excl;                        // rows still to take among those whose key starts with (prefix, digit)
                s_prefix = prefix | ((unsigned)(255 - tid) << shift);
            }
        }
        __syncthreads();
    }
    const unsigned T = s_prefix, need_eq = s_need;           // (the K_top-th largest key) - lo; need_eq rows equal to it are taken
    if (tid == 0) { s_gt = 0u; s_eq_before = 0u; }
    __syncthreads();
    const int n_gt = K_top - (int)need_eq;
    for (int j = 0; j < nchunk; j++) {
        const int i = j * TOPK_THREADS + tid;
        const unsigned k = key_at(j) - lo;
        const bool gt = i < M && k > T, eq = i < M && k == T;
        if (gt) { const unsigned slot = atomicAdd(&s_gt, 1u); if ((int)slot < n_gt) cand[slot] = i; }
        if (__syncthreads_or(eq)) {                           // rows equal to the threshold: taken in index order
            const unsigned bal = __ballot_sync(0xffffffffu, eq);
            if (lane == 0) warp_tot[warp] = __popc(bal);
            __syncthreads();
            unsigned before = s_eq_before;
            for (int w = 0; w < warp; w++) before += warp_tot[w];
            const unsigned rank = before + __popc(bal & ((1u << lane) - 1u));
            if (eq && rank < need_eq) cand[n_gt + (int)rank] = i;
            __syncthreads();
            if (tid == 0) { unsigned t = 0; for (int w = 0; w < TOPK_THREADS / 32; w++) t += warp_tot[w]; s_eq_before += t; }
            __syncthreads();
        }
    }
}

// The same selection by a cluster of eight blocks: a block keeps chunks rank, rank + 8, ... of 1024 rows (NREG keys per
// thread), counts its digits in its own table, and every block adds the eight tables through distributed shared memory
// and reaches the same decision. Places in cand: rows above the threshold first, then rows equal to it, both in index
// order (counts per chunk, summed over the chunks ahead), so the list is the same from run to run. One block of 1024
// threads takes about 20 us for 32000 rows, most of it barriers and shared-memory adds that wait for one another.
constexpr int TOPK_CL = 8;
template <int NREG>
__global__ void __launch_bounds__(TOPK_THREADS) pq_topk_select_cluster_kernel(const float* __restrict__ coarse, int M, int K_top, int32_t* __restrict__ cand) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    __shared__ unsigned hist[256], red_lo[TOPK_THREADS / 32], red_hi[TOPK_THREADS / 32], warp_tot[TOPK_THREADS / 32];
    __shared__ unsigned s_lo, s_hi, s_prefix, s_need;
    __shared__ unsigned cnt_gt[NREG], cnt_eq[NREG], all_gt[NREG * TOPK_CL], all_eq[NREG * TOPK_CL];
    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const unsigned rank = cluster.block_rank();
    unsigned keys[NREG];
    unsigned lo = 0xffffffffu, hi = 0u;
#pragma unroll
    for (int j = 0; j < NREG; j++) {
        const int i = (j * TOPK_CL + (int)rank) * TOPK_THREADS + tid;      // chunk j * 8 + rank
        keys[j] = i < M ? topk_key(__ldcg(coarse + i)) : 0u;
        if (i < M) { lo = min(lo, keys[j]); hi = max(hi, keys[j]); }
    }
    lo = __reduce_min_sync(0xffffffffu, lo); hi = __reduce_max_sync(0xffffffffu, hi);
    if (lane == 0) { red_lo[warp] = lo; red_hi[warp] = hi; }
    __syncthreads();
    lo = __reduce_min_sync(0xffffffffu, red_lo[lane]); hi = __reduce_max_sync(0xffffffffu, red_hi[lane]);
    if (tid == 0) { s_lo = lo; s_hi = hi; s_prefix = 0u; s_need = (unsigned)K_top; }
    cluster.sync();
    for (unsigned r = 0; r < (unsigned)TOPK_CL; r++) {        // a block without rows leaves lo = all ones, hi = 0
        lo = min(lo, *cluster.map_shared_rank(&s_lo, r));
        hi = max(hi, *cluster.map_shared_rank(&s_hi, r));
    }
    int shift = hi >= lo ? 32 - __clz(hi - lo) : 0;           // bits of (key - lo) in use; 0 when all keys are equal
    while (shift > 0) {                                       // the same number of rounds in every block: the barriers below are the cluster's
        const int width = shift < 8 ? shift : 8;
        const int top = shift;
        shift -= width;
        if (tid < 256) hist[tid] = 0u;
        __syncthreads();
        const unsigned prefix = s_prefix, need0 = s_need, mask = top >= 32 ? 0u : 0xffffffffu << top;
#pragma unroll
        for (int j = 0; j < NREG; j++) {
            const int i = (j * TOPK_CL + (int)rank) * TOPK_THREADS + tid;
            const unsigned k = keys[j] - lo;
            if (i < M && (k & mask) == prefix) atomicAdd(&hist[(k >> shift) & ((1u << width) - 1u)], 1u);
        }
        cluster.sync();                                       // every block's table is complete
        unsigned c = 0, incl = 0;
        if (tid < 256) {
            for (unsigned r = 0; r < (unsigned)TOPK_CL; r++) c += cluster.map_shared_rank(hist, r)[255 - tid];
            incl = c;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) { const unsigned n = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += n; }
            if (lane == 31) warp_tot[warp] = incl;
        }
        __syncthreads();
        if (tid < 256) {
            for (int w = 0; w < warp; w++) incl += warp_tot[w];
            const unsigned excl = incl - c;
            if (excl < need0 && need0 <= incl) {
                s_need = need0 - excl;
                s_prefix = prefix | ((unsigned)(255 - tid) << shift);
            }
        }
        cluster.sync();                                       // nobody reads a table any more: it may be cleared for the next round
    }
    const unsigned T = s_prefix, need_eq = s_need;
    const int n_gt = K_top - (int)need_eq;
    // rows above the threshold and rows equal to it, per chunk
    bool gt[NREG], eq[NREG];
#pragma unroll
    for (int j = 0; j < NREG; j++) {
        const int i = (j * TOPK_CL + (int)rank) * TOPK_THREADS + tid;
        const unsigned k = keys[j] - lo;
        gt[j] = i < M && k > T; eq[j] = i < M && k == T;
        const int ng = __syncthreads_count(gt[j]), ne = __syncthreads_count(eq[j]);
        if (tid == 0) { cnt_gt[j] = (unsigned)ng; cnt_eq[j] = (unsigned)ne; }
    }
    cluster.sync();
    if (tid < NREG * TOPK_CL) {                               // chunk c = j * 8 + r lives in block r, slot j
        const unsigned r = (unsigned)tid % TOPK_CL, j = (unsigned)tid / TOPK_CL;
        all_gt[tid] = cluster.map_shared_rank(cnt_gt, r)[j];
        all_eq[tid] = cluster.map_shared_rank(cnt_eq, r)[j];
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < NREG; j++) {
        const int cidx = j * TOPK_CL + (int)rank, i = cidx * TOPK_THREADS + tid;
        if (all_gt[cidx] == 0 && all_eq[cidx] == 0) continue;                      // uniform over the block
        unsigned before_gt = 0, before_eq = 0;
        for (int c2 = 0; c2 < cidx; c2++) { before_gt += all_gt[c2]; before_eq += all_eq[c2]; }
        const unsigned bg = __ballot_sync(0xffffffffu, gt[j]), be = __ballot_sync(0xffffffffu, eq[j]);
        __syncthreads();                                      // warp_tot of the previous chunk has been read
        if (lane == 0) warp_tot[warp] = (unsigned)__popc(bg) | ((unsigned)__popc(be) << 16);
        __syncthreads();
        unsigned wg = 0, we = 0;
        for (int w = 0; w < warp; w++) { wg += warp_tot[w] & 0xffffu; we += warp_tot[w] >> 16; }
        const unsigned lower = (1u << lane) - 1u;
        if (gt[j]) { const unsigned slot = before_gt + wg + (unsigned)__popc(bg & lower); if ((int)slot < n_gt) cand[slot] = i; }
        if (eq[j]) { const unsigned rk = before_eq + we + (unsigned)__popc(be & lower); if (rk < need_eq) cand[n_gt + (int)rk] = i; }
    }
    cluster.sync();                                           // no block leaves while another may still read its counts
}

// A block per chosen row: every level of the row, entry times activation (src/pq_decode.c:2145-2248), threads over the
// chunks so that the dependent reads (code, then codebook entry) of all chunks travel together; a fixed butterfly over
// the lanes, the warps' sums added in warp order; row scale, then the outlier sidecar.
constexpr int TOPK_SUB_THREADS = 128;
__global__ void __launch_bounds__(TOPK_SUB_THREADS) pq_topk_subset_kernel(const ibcu_pq_t t, int C, const float* __restrict__ x, const int32_t* cand,
                                                                          int K_top, float* refined, unsigned* done,
                                                                          float* __restrict__ out_logits, int32_t* __restrict__ out_ids) {
    __shared__ float wsum[2][TOPK_SUB_THREADS / 32];
    __shared__ float sv[TOPK_MAX];
    __shared__ int32_t si[TOPK_MAX];
    __shared__ int last_s;
    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int r = __ldcg(cand + blockIdx.x), half = t.G >> 1;
    const bool two = t.K_l2 > 0, packed = t.K_l2 == 16;
    const size_t l2_stride = packed ? (size_t)((C + 1) / 2) : (size_t)C;
    const __half* cb1l = reinterpret_cast<const __half*>(t.codebook_l);
    const __half* cb1r = reinterpret_cast<const __half*>(t.codebook_r);
    const __half* cb2l = reinterpret_cast<const __half*>(t.codebook2_l);
    const __half* cb2r = reinterpret_cast<const __half*>(t.codebook2_r);
    const int32_t* inner = t.n_outlier > 0 ? t.inner_cols : nullptr;
    const uint8_t* jl = two ? t.idx2_l + (size_t)r * l2_stride : nullptr;
    const uint8_t* jr = two ? t.idx2_r + (size_t)r * l2_stride : nullptr;
    // 8-wide entries at 16-byte boundaries and contiguous activations: one 16-byte read per entry, two per slice of x
    const bool vec = half == 8 && !inner && (t.cb_chunk_stride & 7) == 0 && ((uintptr_t)x & 15) == 0 &&
                     ((((uintptr_t)cb1l | (uintptr_t)cb1r) & 15) == 0) && (!two || (((uintptr_t)cb2l | (uintptr_t)cb2r) & 15) == 0);
    float acc = 0.0f;
    for (int c = tid; c < C; c += TOPK_SUB_THREADS) {
        const int base = c * t.G;
        const int a1 = t.idx_l[(size_t)r * C + c], b1 = t.idx_r[(size_t)r * C + c];
        const __half* el = cb1l + (size_t)c * t.cb_chunk_stride + (size_t)a1 * half;
        const __half* er = cb1r + (size_t)c * t.cb_chunk_stride + (size_t)b1 * half;
        const __half *fl = nullptr, *fr = nullptr;
        if (two) {
            const int a2 = packed ? ((c & 1) ? (jl[c >> 1] >> 4) & 15 : jl[c >> 1] & 15) : jl[c];
            const int b2 = packed ? ((c & 1) ? (jr[c >> 1] >> 4) & 15 : jr[c >> 1] & 15) : jr[c];
            fl = cb2l + (size_t)a2 * half; fr = cb2r + (size_t)b2 * half;
        }
        if (vec) {
            const uint4 ql = *reinterpret_cast<const uint4*>(el), qr = *reinterpret_cast<const uint4*>(er);
            uint4 pl = make_uint4(0, 0, 0, 0), pr = make_uint4(0, 0, 0, 0);
            if (two) { pl = *reinterpret_cast<const uint4*>(fl); pr = *reinterpret_cast<const uint4*>(fr); }
            const float4 x0 = *reinterpret_cast<const float4*>(x + base), x1 = *reinterpret_cast<const float4*>(x + base + 4);
            const float4 x2 = *reinterpret_cast<const float4*>(x + base + 8), x3 = *reinterpret_cast<const float4*>(x + base + 12);
            const float xl[8] = { x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w };
            const float xr[8] = { x2.x, x2.y, x2.z, x2.w, x3.x, x3.y, x3.z, x3.w };
            const __half* hl = reinterpret_cast<const __half*>(&ql); const __half* hr = reinterpret_cast<const __half*>(&qr);
            const __half* gl = reinterpret_cast<const __half*>(&pl); const __half* gr = reinterpret_cast<const __half*>(&pr);
#pragma unroll
            for (int j = 0; j < 8; j++) {
                float wl = __half2float(hl[j]), wr = __half2float(hr[j]);
                if (two) { wl += __half2float(gl[j]); wr += __half2float(gr[j]); }      // (e1 + e2) x: both levels share the activation
                acc = fmaf(wl, xl[j], acc);
                acc = fmaf(wr, xr[j], acc);
            }
        } else {
            for (int j = 0; j < half; j++) {
                const float xl = x[inner ? inner[base + j] : base + j], xr = x[inner ? inner[base + half + j] : base + half + j];
                float wl = __half2float(el[j]), wr = __half2float(er[j]);
                if (two) { wl += __half2float(fl[j]); wr += __half2float(fr[j]); }
                acc = fmaf(wl, xl, acc);
                acc = fmaf(wr, xr, acc);
            }
        }
    }
    float oc = 0.0f;
    for (int j = tid; j < t.n_outlier; j += TOPK_SUB_THREADS) {
        const float wgt = (float)t.outlier_sidecar[(size_t)r * t.n_outlier + j] * __half2float(reinterpret_cast<const __half*>(t.outlier_scale)[j]);
        oc = fmaf(wgt, x[t.outlier_cols[j]], oc);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { acc += __shfl_xor_sync(0xffffffffu, acc, o); oc += __shfl_xor_sync(0xffffffffu, oc, o); }
    if (lane == 0) { wsum[0][warp] = acc; wsum[1][warp] = oc; }
    __syncthreads();
    if (tid == 0) {
        float a = wsum[0][0], o = wsum[1][0];
        for (int w = 1; w < TOPK_SUB_THREADS / 32; w++) { a += wsum[0][w]; o += wsum[1][w]; }
        refined[blockIdx.x] = a * __half2float(reinterpret_cast<const __half*>(t.row_scale)[r]) + o;
        // the block that finishes last orders the rows: by full logit, descending; equal logits by ascending row
        __threadfence();
        const unsigned n_done = atomicAdd(done, 1u);
        last_s = n_done == gridDim.x - 1;
        if (last_s) *done = 0u;                               // zero again for the next call
    }
    __syncthreads();
    if (!last_s) return;
    __threadfence();
    int n = 1;
    while (n < K_top) n <<= 1;
    for (int e = tid; e < n; e += TOPK_SUB_THREADS) { sv[e] = e < K_top ? __ldcg(refined + e) : -INFINITY; si[e] = e < K_top ? __ldcg(cand + e) : 0x7fffffff; }
    __syncthreads();
    // a before b: larger logit, then smaller row; NaN logits go last
    auto before = [](float av, int32_t ai, float bv, int32_t bi) {
        const bool an = av != av, bn = bv != bv;
        if (an != bn) return bn;
        if (!an && av != bv) return av > bv;
        return ai < bi;
    };
    for (int k = 2; k <= n; k <<= 1) {                        // bitonic network over the next power of two
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int e = tid; e < n; e += TOPK_SUB_THREADS) {
                const int p = e ^ j;
                if (p > e) {
                    const bool up = (e & k) == 0;             // this pair sorts towards "before first"
                    const float av = sv[e], bv = sv[p];
                    const int32_t ai = si[e], bi = si[p];
                    const bool swap = up ? before(bv, bi, av, ai) : before(av, ai, bv, bi);
                    if (swap) { sv[e] = bv; sv[p] = av; si[e] = bi; si[p] = ai; }
                }
            }
            __syncthreads();
        }
    }
    for (int e = tid; e < K_top; e += TOPK_SUB_THREADS) { out_logits[e] = sv[e]; out_ids[e] = si[e]; }
}

}  // namespace

extern "C" int ibcu_pq_lm_head_topk(ibcu_ctx* ctx, const ibcu_pq_t* t, const float* x, int K_top, float* out_logits, int32_t* out_ids) {
    IBCU_CHECK_CTX(ctx);
    IBCU_REQUIRE(ctx, out_logits && out_ids, "ibcu_pq_lm_head_topk: null output");
    int rc = pq_check(ctx, t, x, out_logits, 1, "ibcu_pq_lm_head_topk");
    if (rc) return rc;
    IBCU_REQUIRE(ctx, K_top >= 1 && K_top <= t->M && K_top <= TOPK_MAX, "ibcu_pq_lm_head_topk: K_top=%d not in 1..min(M, %d)", K_top, TOPK_MAX);
    IBCU_REQUIRE(ctx, t->idx_l && t->idx_r && (t->K_l2 == 0 || (t->idx2_l && t->idx2_r)), "ibcu_pq_lm_head_topk: the row-major code planes must stay resident");
    const PqPlan pl = pq_plan(ctx, t, 1, true);
    const size_t need = pq_scratch_bytes(pl);
    if (ctx->pq_acc_bytes < need) {
        rc = ibcu_reserve(ctx, &ctx->pq_acc, &ctx->pq_acc_bytes, need);
        if (rc) return rc;
        IBCU_CUDA(ctx, cudaMemsetAsync(ctx->pq_acc, 0, ctx->pq_acc_bytes, ctx->stream));
    }
    const size_t coarse_bytes = ((size_t)t->M * sizeof(float) + 255) & ~(size_t)255;
    rc = ibcu_reserve(ctx, &ctx->scratch, &ctx->scratch_bytes, coarse_bytes + 2 * TOPK_MAX * sizeof(float));
    if (rc) return rc;
    float* coarse = (float*)ctx->scratch;
    int32_t* cand = (int32_t*)((char*)ctx->scratch + coarse_bytes);
    float* refined = (float*)(cand + TOPK_MAX);
    rc = pq_launch(ctx, t, x, coarse, t->M, 1, pl, (unsigned long long*)((char*)ctx->pq_acc + PQ_COUNTER_BYTES), (unsigned int*)ctx->pq_acc, true);
    if (rc) return rc;
    if (t->M <= 4 * TOPK_CL * TOPK_THREADS)
        rc = ibcu_launch(ctx, pq_topk_select_cluster_kernel<4>, dim3(TOPK_CL), dim3(TOPK_THREADS), 0, TOPK_CL, true, (const float*)coarse, t->M, K_top, cand);
    else if (t->M <= 32 * TOPK_CL * TOPK_THREADS)
        rc = ibcu_launch(ctx, pq_topk_select_cluster_kernel<32>, dim3(TOPK_CL), dim3(TOPK_THREADS), 0, TOPK_CL, true, (const float*)coarse, t->M, K_top, cand);
    else
        rc = ibcu_launch(ctx, pq_topk_select_kernel, dim3(1), dim3(TOPK_THREADS), 0, 1, true, (const float*)coarse, t->M, K_top, cand);
    if (rc) return rc;
    // arrival counter of the row kernel: a slot of the counter area that no matvec launch uses (zero between calls)
    unsigned* done = (unsigned int*)ctx->pq_acc + (PQ_COUNTER_BYTES / sizeof(unsigned) - 128);
    return ibcu_launch(ctx, pq_topk_subset_kernel, dim3(K_top), dim3(TOPK_SUB_THREADS), 0, 1, true, *t, pl.C, x, (const int32_t*)cand, K_top, refined, done,
                       out_logits, out_ids);
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
    return pq_launch(ctx, t, x, out, t->M, B, pl, (unsigned long long*)((char*)base + PQ_COUNTER_BYTES), (unsigned int*)base);
}
