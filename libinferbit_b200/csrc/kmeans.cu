// k-means assign / accumulate / update.
//
// assign: nearest centroid by the direct squared distance, evaluated in exactly the order and with
// exactly the roundings of the reference's x86-64 Release binary (multiply and add rounded
// separately for dimensions below 4*floor(D/4), fused for the remaining D%4), strict '<' so the
// lowest index wins ties. Codes are therefore bit-identical to the reference, not "close".
//   assign_exact_kernel   every distance in that exact form (CUDA cores).
//   assign_filter_kernel  (D == 8, K % 8 == 0) TF32 tensor-core scores x.c - |c|^2/2 for all K
//                         centroids per 16-point tile, best / second-best tracked in registers; a
//                         point whose margin exceeds a rigorous error bound takes the tensor-core
//                         winner, every other point is re-evaluated in the exact form. Same codes,
//                         several times fewer issue slots.
// accumulate: per-cluster sums / counts / inertia with a fixed order of additions (no atomics):
// each warp adds its points in index order into a private shared-memory table, warps and blocks are
// then combined in index order.
#include "common.cuh"
#include "kmeans_ref.cuh"
#include <stdlib.h>
#include <stdint.h>

namespace {

constexpr int KM_MAX_D = 32;

// One thread per point, centroids broadcast from shared memory.
template <int DT>
__global__ void __launch_bounds__(256) assign_exact_kernel(const float* __restrict__ X, long N, int D, const float* __restrict__ C, int K,
                                                           int32_t* __restrict__ idx, float* __restrict__ dist,
                                                           const int32_t* __restrict__ todo, const int* __restrict__ n_todo) {
    extern __shared__ __align__(16) float cs[];       // [K][D]
    pdl_launch_dependents();
    pdl_wait();
    const int d_all = DT > 0 ? DT : D;
    for (int i = threadIdx.x; i < K * d_all; i += blockDim.x) cs[i] = C[i];
    __syncthreads();
    const long total = todo ? (long)__ldcg(n_todo) : N;    // written by the kernel just ahead: read past L1, not as a read-only load
    for (long w = (long)blockIdx.x * blockDim.x + threadIdx.x; w < total; w += (long)gridDim.x * blockDim.x) {
        const long i = todo ? (long)todo[w] : w;
        float x[DT > 0 ? DT : KM_MAX_D];
        if (DT > 0 && DT % 4 == 0) {
#pragma unroll
            for (int d = 0; d < DT; d += 4) {
                float4 v = *reinterpret_cast<const float4*>(X + (size_t)i * DT + d);
                x[d] = v.x; x[d + 1] = v.y; x[d + 2] = v.z; x[d + 3] = v.w;
            }
        } else {
#pragma unroll
            for (int d = 0; d < (DT > 0 ? DT : KM_MAX_D); d++) if (d < d_all) x[d] = X[(size_t)i * d_all + d];
        }
        float best = ref_sqdist<DT>(x, cs, D);
        int arg = 0;
        for (int k = 1; k < K; k++) {
            const float dk = ref_sqdist<DT>(x, cs + (size_t)k * d_all, D);
            if (dk < best) { best = dk; arg = k; }
        }
        idx[i] = arg;
        if (dist) dist[i] = best;
    }
}

// ── tensor-core filter (D == 8, K a multiple of 8) ──────────────────────────────────────
// Scores s_k = x.c_k - |c_k|^2/2 (the nearest centroid maximises s_k) come from TF32 tensor-core MMAs,
// m16n8k8: one MMA covers 16 points x 8 centroids with the whole D = 8 contraction. Both operands are
// split into two TF32 terms (x = xh + xl, c = ch + cl) and three MMAs (xh.ch + xh.cl + xl.ch) give the
// dot product to about 2^-21 |x||c|; -|c|^2/2 is the accumulator's initial value. Each lane keeps the
// best and second-best score of its rows; after a 4-lane merge a row whose margin exceeds
//   2^-16 (|x|^2 + max|c|^2)   (> twice the score error plus the FP32 rounding of the reference's own
//                                distances, see below)
// takes the tensor-core winner: then the exact distances of the reference also order that way, so the
// code is the reference's. Every other row (near ties, NaN/Inf) is evaluated in the exact form by the
// whole warp, lowest index winning ties. The reported distance is always the exact-form one.
// Bound: |s_k - true| <= 2^-18 |x||c_k| <= 2^-19 (|x|^2+|c|^2) (dropped xl.cl term, TF32 rounding of the low
// terms, FP32 accumulation of 24 products); true squared distances differ by twice
// the score gap; the reference's FP32 distance errs by < 12 * 2^-24 * d <= 2^-19.4 (|x|^2+|c|^2).
__device__ __forceinline__ uint32_t to_tf32(float v) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
    return r;
}
__device__ __forceinline__ void mma_tf32(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void top2_push(float s, int k, float& m1, float& m2, int& i1) {
    m2 = fmaxf(m2, fminf(m1, s));
    i1 = s > m1 ? k : i1;
    m1 = fmaxf(m1, s);
}

// Shared memory: B fragments [K/8][32] float4 (ch_t, ch_t+4, cl_t, cl_t+4 of centroid 8j+g) |
// -|c|^2/2 [K] | exact centroids [K][8] | max |c|^2 [1].
__global__ void __launch_bounds__(256) assign_filter_kernel(const float* __restrict__ X, long N, const float* __restrict__ C, int K,
                                                            int32_t* __restrict__ idx, float* __restrict__ dist) {
    extern __shared__ __align__(16) float fs[];
    float4* bfrag = reinterpret_cast<float4*>(fs);  // (K/8) * 32 float4 = K * 16 floats
    float* nh = fs + (size_t)K * 16;
    pdl_launch_dependents();
    pdl_wait();
    float* cex = nh + K;
    float* cmax2 = cex + (size_t)K * 8;
    const int tid = threadIdx.x, lane = tid & 31, g = lane >> 2, t = lane & 3;
    for (int e = tid; e < K * 8; e += blockDim.x) cex[e] = C[e];
    __syncthreads();
    for (int e = tid; e < (K / 8) * 32; e += blockDim.x) {
        const int j = e >> 5, l = e & 31, gg = l >> 2, tt = l & 3;
        const float c0 = cex[(8 * j + gg) * 8 + tt], c1 = cex[(8 * j + gg) * 8 + tt + 4];
        const uint32_t h0 = to_tf32(c0), h1 = to_tf32(c1);
        const uint32_t l0 = to_tf32(c0 - __uint_as_float(h0)), l1 = to_tf32(c1 - __uint_as_float(h1));
        bfrag[e] = make_float4(__uint_as_float(h0), __uint_as_float(h1), __uint_as_float(l0), __uint_as_float(l1));
    }
    float mx = 0.0f;
    for (int k = tid; k < K; k += blockDim.x) {
        float n = 0.0f;
#pragma unroll
        for (int d = 0; d < 8; d++) n = fmaf(cex[k * 8 + d], cex[k * 8 + d], n);
        nh[k] = -0.5f * n;
        mx = fmaxf(mx, n);
    }
    mx = warp_max(mx);
    if (tid == 0) *cmax2 = 0.0f;
    __syncthreads();
    if (lane == 0) atomicMax(reinterpret_cast<int*>(cmax2), __float_as_int(mx));    // non-negative floats order like ints
    __syncthreads();
    const float cm2 = *cmax2;

    const long ntile = (N + 15) / 16;
    const long wglobal = (long)blockIdx.x * (blockDim.x >> 5) + (tid >> 5), wstride = (long)gridDim.x * (blockDim.x >> 5);
    for (long tile = wglobal; tile < ntile; tile += wstride) {
        const long p0 = tile * 16;
        const long r0 = min(p0 + g, N - 1), r1 = min(p0 + g + 8, N - 1);     // rows past the end repeat the last point
        const float x00 = X[r0 * 8 + t], x01 = X[r0 * 8 + t + 4], x10 = X[r1 * 8 + t], x11 = X[r1 * 8 + t + 4];
        const uint32_t ah0 = to_tf32(x00), ah1 = to_tf32(x10), ah2 = to_tf32(x01), ah3 = to_tf32(x11);
        const uint32_t al0 = to_tf32(x00 - __uint_as_float(ah0)), al1 = to_tf32(x10 - __uint_as_float(ah1));
        const uint32_t al2 = to_tf32(x01 - __uint_as_float(ah2)), al3 = to_tf32(x11 - __uint_as_float(ah3));
        float xn0 = fmaf(x00, x00, x01 * x01), xn1 = fmaf(x10, x10, x11 * x11);
        xn0 += __shfl_xor_sync(0xffffffffu, xn0, 1); xn0 += __shfl_xor_sync(0xffffffffu, xn0, 2);
        xn1 += __shfl_xor_sync(0xffffffffu, xn1, 1); xn1 += __shfl_xor_sync(0xffffffffu, xn1, 2);
        float m1a = -INFINITY, m2a = -INFINITY, m1b = -INFINITY, m2b = -INFINITY;
        int ia = 0, ib = 0;
        for (int j = 0; j < K / 8; j++) {
            const float4 bf = bfrag[j * 32 + lane];
            const float2 ni = *reinterpret_cast<const float2*>(nh + 8 * j + 2 * t);
            float c[4] = { ni.x, ni.y, ni.x, ni.y };
            const uint32_t bh0 = __float_as_uint(bf.x), bh1 = __float_as_uint(bf.y), bl0 = __float_as_uint(bf.z), bl1 = __float_as_uint(bf.w);
            mma_tf32(c, al0, al1, al2, al3, bh0, bh1);
            mma_tf32(c, ah0, ah1, ah2, ah3, bl0, bl1);
            mma_tf32(c, ah0, ah1, ah2, ah3, bh0, bh1);
            const int k0 = 8 * j + 2 * t;
            top2_push(c[0], k0, m1a, m2a, ia); top2_push(c[1], k0 + 1, m1a, m2a, ia);
            top2_push(c[2], k0, m1b, m2b, ib); top2_push(c[3], k0 + 1, m1b, m2b, ib);
        }
        // merge the four lanes of a row
#pragma unroll
        for (int o = 1; o <= 2; o <<= 1) {
            float om1 = __shfl_xor_sync(0xffffffffu, m1a, o), om2 = __shfl_xor_sync(0xffffffffu, m2a, o);
            int oi = __shfl_xor_sync(0xffffffffu, ia, o);
            m2a = fmaxf(fmaxf(m2a, om2), fminf(m1a, om1));
            if (om1 > m1a || (om1 == m1a && oi < ia)) ia = oi;
            m1a = fmaxf(m1a, om1);
            om1 = __shfl_xor_sync(0xffffffffu, m1b, o); om2 = __shfl_xor_sync(0xffffffffu, m2b, o);
            oi = __shfl_xor_sync(0xffffffffu, ib, o);
            m2b = fmaxf(fmaxf(m2b, om2), fminf(m1b, om1));
            if (om1 > m1b || (om1 == m1b && oi < ib)) ib = oi;
            m1b = fmaxf(m1b, om1);
        }
        const float marg0 = 1.52587890625e-5f * (xn0 + cm2), marg1 = 1.52587890625e-5f * (xn1 + cm2);
        const bool sure0 = (m1a - m2a) > marg0, sure1 = (m1b - m2b) > marg1;   // false for NaN / Inf as well
        // lanes 0..15 finish one row each: row l's result lives in the quad of g = l & 7 (second half: rows 8..15)
        const int srcl = (lane & 7) * 4;
        const int wi_a = __shfl_sync(0xffffffffu, ia, srcl), wi_b = __shfl_sync(0xffffffffu, ib, srcl);
        const bool s_a = __shfl_sync(0xffffffffu, (int)sure0, srcl), s_b = __shfl_sync(0xffffffffu, (int)sure1, srcl);
        const bool second = (lane & 8) != 0;
        int win = second ? wi_b : wi_a;
        bool sure = second ? s_b : s_a;
        const long myp = p0 + (lane & 15);
        const bool have = lane < 16 && myp < N;
        float xr[8];
        if (have) {
            const float4 u = *reinterpret_cast<const float4*>(X + myp * 8), v = *reinterpret_cast<const float4*>(X + myp * 8 + 4);
            xr[0] = u.x; xr[1] = u.y; xr[2] = u.z; xr[3] = u.w; xr[4] = v.x; xr[5] = v.y; xr[6] = v.z; xr[7] = v.w;
        } else {
#pragma unroll
            for (int d = 0; d < 8; d++) xr[d] = 0.0f;
        }
        float best = have ? ref_sqdist<8>(xr, cex + win * 8, 8) : 0.0f;
        // rows the filter could not decide: the whole warp evaluates all centroids exactly
        unsigned todo = __ballot_sync(0xffffffffu, have && !sure);
        while (todo) {
            const int rl = __ffs(todo) - 1;
            todo &= todo - 1;
            float xq[8];
#pragma unroll
            for (int d = 0; d < 8; d++) xq[d] = __shfl_sync(0xffffffffu, xr[d], rl);
            float bd = INFINITY; int bk = 0x7fffffff;
            for (int k = lane; k < K; k += 32) {
                const float dk = ref_sqdist<8>(xq, cex + k * 8, 8);
                if (dk < bd) { bd = dk; bk = k; }
            }
            // lexicographic (distance, index) minimum: the reference's strict '<' scan keeps the lowest index
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float od = __shfl_xor_sync(0xffffffffu, bd, o);
                const int ok = __shfl_xor_sync(0xffffffffu, bk, o);
                if (od < bd || (od == bd && ok < bk)) { bd = od; bk = ok; }
            }
            if (lane == rl) {
                if (bk == 0x7fffffff) { bk = 0; bd = ref_sqdist<8>(xr, cex, 8); }   // every distance NaN: centroid 0 (the reference's seed)
                win = bk; best = bd;
            }
        }
        if (have) { idx[myp] = win; if (dist) dist[myp] = best; }
    }
}

// ── deterministic accumulation ──────────────────────────────────────────────────────────
// Block b owns points [b*chunk, (b+1)*chunk); warp w of the block owns a contiguous sub-range and
// adds its points one after another (lanes = dimensions), so each table entry sees its points in
// index order. Tables: sums [warps][K*D] float, counts [warps][K] int. Block result = warp tables
// added in warp order; written to part_* [gridDim.x][...]. Inertia: per-thread double partials,
// tree-reduced in a fixed pattern.
__global__ void __launch_bounds__(256) accumulate_kernel(const float* __restrict__ X, long N, int D, int K,
                                                         const int32_t* __restrict__ idx, const float* __restrict__ dist,
                                                         long chunk, float* __restrict__ part_sums, int32_t* __restrict__ part_counts,
                                                         double* __restrict__ part_inertia) {
    extern __shared__ __align__(16) unsigned char km_smem[];
    __shared__ double dred[8];
    const int nwarp = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* wsum = reinterpret_cast<float*>(km_smem);                            // [nwarp][K*D]
    int* wcnt = reinterpret_cast<int*>(wsum + (size_t)nwarp * K * D);           // [nwarp][K]
    pdl_launch_dependents();
    pdl_wait();
    for (int i = threadIdx.x; i < nwarp * K * D; i += blockDim.x) wsum[i] = 0.0f;
    for (int i = threadIdx.x; i < nwarp * K; i += blockDim.x) wcnt[i] = 0;
    __syncthreads();
    const long b0 = (long)blockIdx.x * chunk;
    long b1 = b0 + chunk; if (b1 > N) b1 = N;
    const long per = (b1 - b0 + nwarp - 1) / nwarp;
    long p0 = b0 + (long)warp * per, p1 = p0 + per; if (p1 > b1) p1 = b1;
    float* ms = wsum + (size_t)warp * K * D;
    int* mc = wcnt + (size_t)warp * K;
    double inert = 0.0;
    // points of this warp, 32 at a time: the warp stages their coordinates in shared memory with
    // coalesced loads, lane l fetches the code (and distance) of point p+l, then the warp walks the
    // 32 points in order with lanes acting as dimensions
    float* stage = reinterpret_cast<float*>(wcnt + (size_t)nwarp * K) + (size_t)warp * 32 * D;   // [32][D]
    if ((D & 3) == 0 && 32 % (D >> 2) == 0 && ((uintptr_t)X & 15) == 0 && ((uintptr_t)stage & 15) == 0) {
        // D/4 lanes per point (one float4 each), 32/(D/4) points per step. Points of a step that share a
        // cluster are applied in rounds: a point goes in round r when r lower points of the step have its
        // cluster, so every table entry still sees its points in index order. The next 32 points are
        // fetched while the current ones are applied.
        const int lpp = D >> 2, pps = 32 / lpp, q = lane / lpp, part = lane - q * lpp;
        float4* stage4 = reinterpret_cast<float4*>(stage);
        const float4* X4 = reinterpret_cast<const float4*>(X);
        int code_n = 0; float dist_n = 0.0f; float4 xn[KM_MAX_D / 4];
        auto fetch = [&](long p) {
            const long mine = p + lane;
            code_n = mine < p1 ? idx[mine] : 0;
            dist_n = (dist && mine < p1) ? dist[mine] : 0.0f;
            const long lim = (p1 - p) * lpp;                      // float4s that exist
#pragma unroll
            for (int u = 0; u < KM_MAX_D / 4; u++) {
                const int e = lane + 32 * u;
                xn[u] = (u < lpp && e < lim) ? X4[(size_t)p * lpp + e] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
        };
        if (p0 < p1) fetch(p0);
        for (long p = p0; p < p1; p += 32) {
            const int n = (int)((p1 - p) < 32 ? (p1 - p) : 32);
            const int code = code_n;
            inert += (double)dist_n;
            __syncwarp();                                         // the previous pass's reads of the stage are done
#pragma unroll
            for (int u = 0; u < KM_MAX_D / 4; u++) if (u < lpp) stage4[lane + 32 * u] = xn[u];
            if (p + 32 < p1) fetch(p + 32);
            __syncwarp();
            for (int j = 0; j < n; j += pps) {
                const int pt = j + q;
                const bool act = pt < n;
                const int k = __shfl_sync(0xffffffffu, code, act ? pt : j);
                const unsigned same = __match_any_sync(0xffffffffu, act ? k : -1 - lane);
                const int rank = __popc(same & ((1u << lane) - 1u)) / lpp;
                const int rounds = __reduce_max_sync(0xffffffffu, act ? rank : 0);
                for (int r = 0; r <= rounds; r++) {
                    if (act && rank == r) {
                        float4* dst = reinterpret_cast<float4*>(ms + (size_t)k * D) + part;
                        const float4 v = stage4[pt * lpp + part];
                        float4 a = *dst;
                        a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
                        *dst = a;
                        if (part == 0) mc[k] += 1;
                    }
                    __syncwarp();
                }
            }
        }
    } else
    for (long p = p0; p < p1; p += 32) {
        const long mine = p + lane;
        const int n = (int)((p1 - p) < 32 ? (p1 - p) : 32);
        const int code = mine < p1 ? idx[mine] : 0;
        if (dist && mine < p1) inert += (double)dist[mine];
        for (int e = lane; e < n * D; e += 32) stage[e] = X[(size_t)p * D + e];
        __syncwarp();
        // 32/D points per step, one lane group per point. Points of a step that share a cluster are
        // applied one after another, so every table entry still sees its points in index order.
        const int gpw = 32 / D, q = lane / D, d = lane - q * D;
        for (int j = 0; j < n; j += gpw) {
            const int mine_j = j + q;
            const bool act = q < gpw && mine_j < n;
            const int k = __shfl_sync(0xffffffffu, code, act ? mine_j : j);
            bool clash = false;
            // compare my cluster with those of the lower groups
            for (int o = 0; o < gpw - 1; o++) {
                const int ko = __shfl_sync(0xffffffffu, code, min(j + o, n - 1));
                if (act && o < q && ko == k) clash = true;
            }
            const bool any = __any_sync(0xffffffffu, clash);
            if (!any) {
                if (act) { ms[(size_t)k * D + d] += stage[mine_j * D + d]; if (d == 0) mc[k] += 1; }
                __syncwarp();
            } else {
                for (int o = 0; o < gpw; o++) {
                    if (act && q == o) { ms[(size_t)k * D + d] += stage[mine_j * D + d]; if (d == 0) mc[k] += 1; }
                    __syncwarp();
                }
            }
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < K * D; e += blockDim.x) {
        float s = wsum[e];
        for (int w = 1; w < nwarp; w++) s += wsum[(size_t)w * K * D + e];
        part_sums[(size_t)blockIdx.x * K * D + e] = s;
    }
    for (int e = threadIdx.x; e < K; e += blockDim.x) {
        int s = wcnt[e];
        for (int w = 1; w < nwarp; w++) s += wcnt[(size_t)w * K + e];
        part_counts[(size_t)blockIdx.x * K + e] = s;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) inert += __shfl_xor_sync(0xffffffffu, inert, o);
    if (lane == 0) dred[warp] = inert;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (int w = 0; w < nwarp; w++) t += dred[w];
        part_inertia[blockIdx.x] = t;
    }
}

// Adds the per-block partial tables. A block of 256 threads owns 32 columns (table entries): thread
// (g, c) adds partials g, g + 8, ... of column c with its loads in flight eight at a time, then the
// eight group sums are combined in a fixed order. Blocks [0, nS) do the sums (in double), [nS, nS + nC)
// the counts, the last one the inertia.
// With ex.gp.world > 0 the totals also go into this rank's slot of the exchange area (sums, then counts, then the
// inertia); the last block copies the slot into every peer's window and publishes: every rank then adds the slots up.
__device__ __forceinline__ size_t exch_counts_off(int KD) { return (size_t)KD * sizeof(float); }
__device__ __forceinline__ size_t exch_inertia_off(int KD, int K) { return ((size_t)KD * sizeof(float) + (size_t)K * sizeof(int32_t) + 7) & ~(size_t)7; }
template <typename T>
__device__ __forceinline__ void exch_store(const ExchSlots& ex, size_t byte_off, T v) {       // into this rank's own window
    *reinterpret_cast<T*>(ex.gp.peer[ex.gp.rank] + ex.off + (size_t)ex.gp.rank * ex.slot + byte_off) = v;
}

__global__ void __launch_bounds__(256) accumulate_finish_kernel(const float* __restrict__ part_sums, const int32_t* __restrict__ part_counts,
                                                                const double* __restrict__ part_inertia, int nblocks, int KD, int K,
                                                                float* __restrict__ sums, int32_t* __restrict__ counts, double* __restrict__ inertia,
                                                                const ExchSlots ex) {
    __shared__ double dsh[8][32];
    __shared__ int ish[8][32];
    pdl_launch_dependents();
    pdl_wait();
    const int c = threadIdx.x & 31, g = threadIdx.x >> 5;
    const int nS = (KD + 31) / 32, nC = (K + 31) / 32;
    if ((int)blockIdx.x < nS) {
        const int e = blockIdx.x * 32 + c;
        double s = 0.0;
        if (e < KD) {
#pragma unroll 8
            for (int b = g; b < nblocks; b += 8) s += (double)part_sums[(size_t)b * KD + e];
        }
        dsh[g][c] = s;
        __syncthreads();
        if (g == 0 && e < KD) {
            const float v = (float)(((dsh[0][c] + dsh[1][c]) + (dsh[2][c] + dsh[3][c])) + ((dsh[4][c] + dsh[5][c]) + (dsh[6][c] + dsh[7][c])));
            sums[e] = v;
            if (ex.gp.world) exch_store(ex, (size_t)e * sizeof(float), v);
        }
    } else if ((int)blockIdx.x < nS + nC) {
        const int e = (blockIdx.x - nS) * 32 + c;
        int s = 0;
        if (e < K) {
#pragma unroll 8
            for (int b = g; b < nblocks; b += 8) s += part_counts[(size_t)b * K + e];
        }
        ish[g][c] = s;
        __syncthreads();
        if (g == 0 && e < K) {
            const int v = ish[0][c] + ish[1][c] + ish[2][c] + ish[3][c] + ish[4][c] + ish[5][c] + ish[6][c] + ish[7][c];
            counts[e] = v;
            if (ex.gp.world) exch_store(ex, exch_counts_off(KD) + (size_t)e * sizeof(int32_t), v);
        }
    } else if (inertia || ex.gp.world) {
        double s = 0.0;
#pragma unroll 4
        for (int b = threadIdx.x; b < nblocks; b += 256) s += part_inertia[b];
        // fixed-order tree over the 256 threads
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (c == 0) dsh[0][g] = s;
        __syncthreads();
        if (threadIdx.x == 0) {
            const double v = ((dsh[0][0] + dsh[0][1]) + (dsh[0][2] + dsh[0][3])) + ((dsh[0][4] + dsh[0][5]) + (dsh[0][6] + dsh[0][7]));
            if (inertia) *inertia = v;
            if (ex.gp.world) exch_store(ex, exch_inertia_off(KD, K), v);
        }
    }
    if (ex.gp.world) {                                        // the whole slot goes to the peers in one piece
        const int j = push_arrive(ex.gp);
        if (j >= 0) {
            const size_t at = ex.off + (size_t)ex.gp.rank * ex.slot;
            const int words = (int)((exch_inertia_off(KD, K) + 8 + 15) / 16) * 4;
            push_span(ex.gp, j, push_count(ex.gp), reinterpret_cast<const float*>(ex.gp.peer[ex.gp.rank] + at), at, words, 1, 0);
            push_finish(ex.gp);
        }
    }
}

// The all-reduce of a sharded iteration, done by the consumer: waits for the peers' slots of the exchange area, adds the
// ranks' tables in rank order (the same order, hence the same bits, on every rank) into sums, counts and inertia.
__global__ void __launch_bounds__(1024) exchange_sum_kernel(const ExchSlots ex, const GatherWait gw, int KD, int K,
                                                            float* __restrict__ sums, int32_t* __restrict__ counts, double* __restrict__ inertia) {
    pdl_launch_dependents();
    pdl_wait();
    gather_wait(gw);
    const char* base = ex.gp.peer[ex.gp.rank] + ex.off;
    for (int e = threadIdx.x; e < KD; e += blockDim.x) {
        float s = 0.0f;
        for (int r = 0; r < ex.gp.world; r++) s += *reinterpret_cast<const volatile float*>(base + (size_t)r * ex.slot + (size_t)e * sizeof(float));
        sums[e] = s;
    }
    for (int e = threadIdx.x; e < K; e += blockDim.x) {
        int s = 0;
        for (int r = 0; r < ex.gp.world; r++) s += *reinterpret_cast<const volatile int*>(base + (size_t)r * ex.slot + exch_counts_off(KD) + (size_t)e * sizeof(int32_t));
        counts[e] = s;
    }
    if (threadIdx.x == 0 && inertia) {
        double s = 0.0;
        for (int r = 0; r < ex.gp.world; r++) s += *reinterpret_cast<const volatile double*>(base + (size_t)r * ex.slot + exch_inertia_off(KD, K));
        *inertia = s;
    }
}

// c = sum * (1/count) with the reference's two roundings; empty clusters stay; shift = sum dv^2.
__global__ void __launch_bounds__(1024) update_kernel(float* __restrict__ C, int K, int D, const float* __restrict__ sums,
                                                      const int32_t* __restrict__ counts, float* __restrict__ shift) {
    __shared__ float red[32];
    pdl_launch_dependents();
    pdl_wait();
    float local = 0.0f;
    for (int e = threadIdx.x; e < K * D; e += blockDim.x) {
        const int k = e / D;
        const int n = counts[k];
        if (n > 0) {
            const float inv = __fdiv_rn(1.0f, (float)n);
            const float nv = __fmul_rn(sums[e], inv);
            const float dv = nv - C[e];
            local = fmaf(dv, dv, local);
            C[e] = nv;
        }
    }
    local = warp_sum(local);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = local;
    __syncthreads();
    if (threadIdx.x < 32) {
        float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.0f;
        t = warp_sum(t);
        if (threadIdx.x == 0 && shift) *shift = t;
    }
}

int assign_exact_launch(ibcu_ctx* ctx, const float* X, long N, int D, const float* C, int K, int32_t* idx, float* dist,
                        const int32_t* todo, const int* n_todo, long work) {
    size_t smem = (size_t)K * D * sizeof(float);
    long blocks = (work + 255) / 256;
    long cap = (long)ctx->sm_count * 8;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
#define KM_LAUNCH(DT) do { \
        if (smem > 48 * 1024) IBCU_CUDA(ctx, cudaFuncSetAttribute(assign_exact_kernel<DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        return ibcu_launch(ctx, assign_exact_kernel<DT>, dim3((unsigned)blocks), dim3(256), smem, 1, true, X, N, D, C, K, idx, dist, todo, n_todo); \
    } while (0)
    switch (D) {
        case 2: KM_LAUNCH(2);
        case 4: KM_LAUNCH(4);
        case 8: KM_LAUNCH(8);
        case 16: KM_LAUNCH(16);
        default: KM_LAUNCH(0);
    }
#undef KM_LAUNCH
}

}  // namespace

int ibcu_kmeans_assign_tc(ibcu_ctx* ctx, const float* X, long N, const float* C, int K, int32_t* idx, float* dist);   // kmeans_tc.cu
int ibcu_kmeans_assign_accumulate_tc(ibcu_ctx* ctx, const float* X, long N, const float* C, int K, int32_t* idx, float* dist,
                                     float* part_sums, int32_t* part_counts, double* part_inertia, int nblocks);

extern "C" void ibcu_kmeans_set_path(ibcu_ctx* ctx, int path) { if (ctx) ctx->kmeans_path = path; }

extern "C" int ibcu_kmeans_assign(ibcu_ctx* ctx, const float* X, long N, int D, const float* C, int K,
                                  int32_t* idx, float* dist) {
    IBCU_CHECK_CTX(ctx);
    IBCU_REQUIRE(ctx, X && C && idx, "ibcu_kmeans_assign: null pointer");
    IBCU_REQUIRE(ctx, N > 0 && D >= 1 && D <= KM_MAX_D && K >= 1 && K <= 1024, "ibcu_kmeans_assign: N=%ld D=%d K=%d out of range", N, D, K);
    IBCU_REQUIRE(ctx, (size_t)K * D * sizeof(float) <= 128 * 1024, "ibcu_kmeans_assign: K*D=%d too large", K * D);
    // D == 8: scores on the tensor cores as a filter, exact re-evaluation of the candidates. The tcgen05 kernel takes
    // K a multiple of 64 up to 256; other multiples of 8 take the register-operand (mma.sync) filter.
    if (D == 8 && ctx->kmeans_path != IBCU_KMEANS_EXACT && ((uintptr_t)X & 15) == 0) {
        if (ctx->kmeans_path != IBCU_KMEANS_MMA_SYNC) {
            const int rc = ibcu_kmeans_assign_tc(ctx, X, N, C, K, idx, dist);
            if (rc != IBCU_ERR_STATE) return rc;
        }
    }
    if (D == 8 && K % 8 == 0 && K >= 8 && ctx->kmeans_path != IBCU_KMEANS_EXACT && ((uintptr_t)X & 15) == 0) {
        const size_t smem = ((size_t)K * 16 + K + (size_t)K * 8 + 4) * sizeof(float);
        if (smem > 48 * 1024) IBCU_CUDA(ctx, cudaFuncSetAttribute(assign_filter_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        long tiles = (N + 15) / 16;
        long blocks = (tiles + 7) / 8;
        const long cap = (long)ctx->sm_count * 6;
        if (blocks > cap) blocks = cap;
        return ibcu_launch(ctx, assign_filter_kernel, dim3((unsigned)blocks), dim3(256), smem, 1, true, X, N, C, K, idx, dist);
    }
    return assign_exact_launch(ctx, X, N, D, C, K, idx, dist, nullptr, nullptr, N);
}

static int kmeans_accumulate(ibcu_ctx* ctx, const float* X, long N, int D, int K, const int32_t* idx, const float* dist,
                             float* sums, int32_t* counts, double* inertia, const ExchSlots& ex) {
    IBCU_CHECK_CTX(ctx);
    IBCU_REQUIRE(ctx, X && idx && sums && counts, "ibcu_kmeans_accumulate: null pointer");
    IBCU_REQUIRE(ctx, N > 0 && D >= 1 && D <= KM_MAX_D && K >= 1 && K <= 1024, "ibcu_kmeans_accumulate: N=%ld D=%d K=%d out of range", N, D, K);
    // warps per block limited by the shared-memory tables
    const size_t per_warp = (size_t)K * D * sizeof(float) + (size_t)K * sizeof(int) + (size_t)32 * D * sizeof(float);
    int nwarp = (int)((160 * 1024) / per_warp);
    if (nwarp > 8) nwarp = 8;
    IBCU_REQUIRE(ctx, nwarp >= 1, "ibcu_kmeans_accumulate: K*D=%d does not fit shared memory", K * D);
    const size_t smem = per_warp * nwarp;
    // a fixed function of N only, so results do not depend on the machine's SM count
    long chunk = 16384;
    long nblocks = (N + chunk - 1) / chunk;
    if (nblocks > 2048) { nblocks = 2048; chunk = (N + nblocks - 1) / nblocks; nblocks = (N + chunk - 1) / chunk; }
    const size_t KD = (size_t)K * D;
    size_t need = (size_t)nblocks * (KD * sizeof(float) + K * sizeof(int32_t) + sizeof(double)) + 64;
    int rc = ibcu_reserve(ctx, &ctx->scratch, &ctx->scratch_bytes, need);
    if (rc) return rc;
    double* part_inertia = (double*)ctx->scratch;
    float* part_sums = (float*)(part_inertia + ((nblocks + 1) & ~1L));
    int32_t* part_counts = (int32_t*)(part_sums + (size_t)nblocks * KD);
    if (smem > 48 * 1024) IBCU_CUDA(ctx, cudaFuncSetAttribute(accumulate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    rc = ibcu_launch(ctx, accumulate_kernel, dim3((unsigned)nblocks), dim3(nwarp * 32), smem, 1, true,
                     X, N, D, K, idx, dist, chunk, part_sums, part_counts, part_inertia);
    if (rc) return rc;
    int fin_blocks = (int)((KD + 31) / 32) + (K + 31) / 32 + 1;
    return ibcu_launch(ctx, accumulate_finish_kernel, dim3(fin_blocks), dim3(256), 0, 1, true,
                       (const float*)part_sums, (const int32_t*)part_counts, (const double*)part_inertia, (int)nblocks, (int)KD, K,
                       sums, counts, inertia, ex);
}

extern "C" int ibcu_kmeans_accumulate(ibcu_ctx* ctx, const float* X, long N, int D, int K,
                                      const int32_t* idx, const float* dist,
                                      float* sums, int32_t* counts, double* inertia) {
    ExchSlots none;
    memset(&none, 0, sizeof none);
    return kmeans_accumulate(ctx, X, N, D, K, idx, dist, sums, counts, inertia, none);
}

extern "C" int ibcu_kmeans_update(ibcu_ctx* ctx, float* C, int K, int D, const float* sums,
                                  const int32_t* counts, float* shift) {
    IBCU_CHECK_CTX(ctx);
    IBCU_REQUIRE(ctx, C && sums && counts && K >= 1 && D >= 1, "ibcu_kmeans_update: bad arguments");
    return ibcu_launch(ctx, update_kernel, dim3(1), dim3(1024), 0, 1, true, C, K, D, sums, counts, shift);
}

extern "C" int ibcu_kmeans_lloyd_iter(ibcu_ctx* ctx, const float* X, long N, int D, float* C, int K,
                                      int32_t* idx, float* dist, float* sums, int32_t* counts, double* inertia) {
    IBCU_CHECK_CTX(ctx);
    IBCU_REQUIRE(ctx, dist, "ibcu_kmeans_lloyd_iter: dist buffer required");
    IBCU_REQUIRE(ctx, X && C && idx && sums && counts && N > 0 && D >= 1 && D <= KM_MAX_D && K >= 1 && K <= 1024, "ibcu_kmeans_lloyd_iter: bad arguments");
    int rc = IBCU_OK;
    // One exchange per iteration. Through the peer window: the kernel that finishes this rank's tables stores them into
    // every rank's exchange area and publishes, the next kernel waits for the peers' and adds the tables in rank order.
    // Without a window: the three all-reduces as one grouped NCCL call.
    ExchSlots ex;
    memset(&ex, 0, sizeof ex);
    const size_t slot_bytes = (size_t)K * D * sizeof(float) + (size_t)K * sizeof(int32_t) + 16;
    const int windowed = ctx->world > 1 && !ctx->capturing ? ibcu_exchange_begin(ctx, slot_bytes, &ex) : 0;
    if (!windowed) memset(&ex, 0, sizeof ex);
    // D == 8 on the tensor-memory kernel: the assignment kernel's epilogue adds the points into per-block tables as it
    // goes, so the accumulate pass costs no second read of X and no launch; only the per-block tables are left to add up
    bool fused = false;
    if (D == 8 && ctx->kmeans_path == IBCU_KMEANS_AUTO && ((uintptr_t)X & 15) == 0 && K >= 64 && K <= 256 && (K & 63) == 0) {
        const long ntile = (N + 127) / 128;
        const int nblocks = (int)(ntile < ctx->sm_count ? ntile : ctx->sm_count);
        const size_t KD = (size_t)K * D;
        const size_t need = (size_t)nblocks * (KD * sizeof(float) + K * sizeof(int32_t) + sizeof(double)) + 64;
        rc = ibcu_reserve(ctx, &ctx->scratch, &ctx->scratch_bytes, need);
        if (rc) return rc;
        double* part_inertia = (double*)ctx->scratch;
        float* part_sums = (float*)(part_inertia + ((nblocks + 1) & ~1));
        int32_t* part_counts = (int32_t*)(part_sums + (size_t)nblocks * KD);
        rc = ibcu_kmeans_assign_accumulate_tc(ctx, X, N, C, K, idx, dist, part_sums, part_counts, part_inertia, nblocks);
        if (rc == IBCU_OK) {
            fused = true;
            const int fin_blocks = (int)((KD + 31) / 32) + (K + 31) / 32 + 1;
            rc = ibcu_launch(ctx, accumulate_finish_kernel, dim3(fin_blocks), dim3(256), 0, 1, true,
                             (const float*)part_sums, (const int32_t*)part_counts, (const double*)part_inertia, nblocks, (int)KD, K,
                             sums, counts, inertia, ex);
            if (rc) return rc;
        } else if (rc != IBCU_ERR_STATE) return rc;
    }
    if (!fused) {
        rc = ibcu_kmeans_assign(ctx, X, N, D, C, K, idx, dist);
        if (rc) return rc;
        rc = kmeans_accumulate(ctx, X, N, D, K, idx, dist, sums, counts, inertia, ex);
        if (rc) return rc;
    }
    if (windowed) {
        ctx->gather_pending = 1;
        GatherWait gw;
        ibcu_take_gather_wait(ctx, &gw);
        rc = ibcu_launch(ctx, exchange_sum_kernel, dim3(1), dim3(1024), 0, 1, true, ex, gw, K * D, K, sums, counts, inertia);
        if (rc) return rc;
    } else if (ctx->world > 1) {
        if ((rc = ibcu_allreduce_kmeans(ctx, sums, (size_t)K * D, counts, (size_t)K, inertia))) return rc;
    }
    return ibcu_kmeans_update(ctx, C, K, D, sums, counts, nullptr);
}
