// k-means assignment for D == 8 on the fifth-generation tensor cores (tcgen05.mma, accumulators in TMEM).
//
// Scores s_k = x.c_k - |c_k|^2 / 2 (the nearest centroid maximises s_k) for a tile of 128 points against up to
// 256 centroids are one accumulator tile in tensor memory. x and c are split into two TF32 terms each
// (x = xh + xl, c = ch + cl); one tile is four tcgen05.mma steps of K = 8:
//     xh.ch  +  xl.ch  +  xh.cl  +  [1 1 1 0 0 0 0 0] . [nh0 nh1 nh2 0 0 0 0 0]
// where nh0 + nh1 + nh2 = -|c|^2 / 2 split into three TF32 terms, so the bias rides in the contraction.
// Operands sit in shared memory in the canonical K-major layout without swizzle (8 rows x 16 bytes core
// matrices); the centroid operand is built once per block, the point operand per tile by a loader warp
// (four loader warps: cp.async ring of raw tiles, split into the two TF32 terms). One thread issues the MMAs; two
// accumulator tiles (2 x 256 of the 512 TMEM columns) alternate, so the tensor cores fill one while eight
// epilogue warps drain the other with tcgen05.ld (32x32b: a thread owns one point, i.e. one row).
//
// The scores only FILTER. A thread reduces its row to the best and second-best maxima over groups of 8
// centroids (three-input max). If the best group leads by more than 2^-14 (|x|^2 + max |c|^2) - far above
// the error of the split product and of the reference's own FP32 distances - the reference's nearest
// centroid lies in that group, and its 8 centroids are evaluated in the reference binary's exact order and
// rounding, lowest index winning ties. Otherwise (near ties, NaN, Inf) the warp evaluates all centroids in
// that exact form. Codes and distances are therefore bit-identical to the reference, as with the other
// assignment kernels.
//
// Every wait (mbarrier) is bounded: when one runs out the block raises a flag in shared memory, every role
// leaves its loop, tensor memory is released and a host-visible error word is set; nothing spins for ever.
#include "common.cuh"
#include "tc_common.cuh"
#include "kmeans_ref.cuh"

namespace {

constexpr int TC_TILE = 128;                 // points per accumulator tile
constexpr int TC_STAGES = 4;                 // raw / operand tiles in flight
constexpr int TC_EPI_WARPS = 8;              // warps 0..7 drain accumulators; warps 8..11 load points (32 rows of every tile each); warp 12 issues MMAs
constexpr int TC_LOAD_WARPS = 4;
constexpr int TC_MMA_WARP = TC_EPI_WARPS + TC_LOAD_WARPS;
constexpr int TC_THREADS = (TC_MMA_WARP + 1) * 32;
constexpr int TC_A_CHUNK = 16 * 128;         // one 16-byte K chunk of 128 rows: 16 core matrices of 128 bytes
constexpr int TC_A_STAGE = 4 * TC_A_CHUNK;   // xh (two chunks), xl (two chunks)
constexpr int TC_RAW_STAGE = TC_TILE * 32;   // 128 points x 8 floats

__device__ __forceinline__ uint32_t tf32_of(float v) { uint32_t r; asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v)); return r; }
__device__ __forceinline__ void mma_tf32_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
                 :: "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ float max3(float a, float b, float c) { float r; asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c)); return r; }

// two FP32 lanes per instruction (round to nearest, each lane rounded like the scalar operation)
__device__ __forceinline__ unsigned long long pack2(float lo, float hi) { unsigned long long r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi)); return r; }
__device__ __forceinline__ void unpack2(unsigned long long v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ unsigned long long sub2(unsigned long long a, unsigned long long b) { unsigned long long r; asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b)); return r; }
__device__ __forceinline__ unsigned long long mul2(unsigned long long a, unsigned long long b) { unsigned long long r; asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b)); return r; }

constexpr int TC_GROUP_STRIDE = 64 + 4;      // floats per group of 8 centroids in the group table: the 4-float skew spreads groups over the banks

struct TcShared {
    unsigned long long full_a[TC_STAGES], empty_a[TC_STAGES];     // loader -> MMA, MMA -> loader
    unsigned long long full_acc[2], empty_acc[2];                  // MMA -> epilogue, epilogue -> MMA
    unsigned long long drained;                                    // every MMA of the block has completed
    uint32_t tmem_base;
    int abort_flag;
    unsigned cmax2_bits;
    double inert[TC_EPI_WARPS];
};

// Best and second-best of the maxima over groups of 8 scores, kept by four independent trackers (tracker q sees groups
// q, q + 4, ...) so that the four dependency chains interleave; top2_merge joins two trackers.
struct Top2 { float m1, m2; int g1; };
__device__ __forceinline__ void top2_groups(const uint32_t* r, int gid0, Top2* t) {
#pragma unroll
    for (int q = 0; q < 4; q++) {
        const float* v = reinterpret_cast<const float*>(r) + 8 * q;
        float g = max3(v[0], v[1], v[2]);
        g = max3(g, v[3], v[4]);
        g = max3(g, v[5], v[6]);
        g = fmaxf(g, v[7]);
        t[q].m2 = fmaxf(t[q].m2, fminf(t[q].m1, g));
        t[q].g1 = g > t[q].m1 ? gid0 + q : t[q].g1;
        t[q].m1 = fmaxf(t[q].m1, g);
    }
}
__device__ __forceinline__ Top2 top2_merge(const Top2& a, const Top2& b) {
    Top2 r;
    r.m2 = fmaxf(fmaxf(a.m2, b.m2), fminf(a.m1, b.m1));
    r.g1 = (b.m1 > a.m1 || (b.m1 == a.m1 && b.g1 < a.g1)) ? b.g1 : a.g1;
    r.m1 = fmaxf(a.m1, b.m1);
    return r;
}

// Dynamic shared memory: centroid operand [ch | cl | bias][2 chunks][K rows x 16 B] | constant point chunk pair
// (1 1 1 0 / 0 0 0 0 per row) | TC_STAGES point operands (xh, xl) | TC_STAGES raw point tiles | exact centroids [K][8] |
// the same centroids by group [K/8][8 dims][8] | TcShared
// ACC: the epilogue warps also add every point into the table of its cluster (a table of K x 8 sums and K counts per warp
// in shared memory, points of a warp in index order: equal clusters among its 32 points take turns), and the block leaves
// the sum of its eight tables, its counts and its share of the inertia in part_*[blockIdx.x]: the accumulate pass over X of
// a Lloyd iteration then needs no kernel and no second read of X. The order of the adds is fixed by the grid.
template <bool ACC>
__global__ void __launch_bounds__(TC_THREADS, 1) assign_tc_kernel(const float* __restrict__ X, long N, const float* __restrict__ C, int K,
                                                                  int32_t* __restrict__ idx, float* __restrict__ dist, int* __restrict__ err,
                                                                  float* __restrict__ part_sums, int32_t* __restrict__ part_counts,
                                                                  double* __restrict__ part_inertia) {
    extern __shared__ __align__(1024) unsigned char tc_smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t b_chunk = (uint32_t)K * 16u, b_piece = 2u * b_chunk;
    unsigned char* sB = tc_smem;
    unsigned char* sAug = sB + 3 * b_piece;
    unsigned char* sA = sAug + 2 * TC_A_CHUNK;
    unsigned char* sRaw = sA + TC_STAGES * TC_A_STAGE;
    float* cex = reinterpret_cast<float*>(sRaw + TC_STAGES * TC_RAW_STAGE);     // [K][8] as given
    float* cgrp = cex + (size_t)K * 8;                                           // [K / 8 groups][8 dims][8 centroids], groups TC_GROUP_STRIDE apart
    float* wtab = cgrp + (size_t)(K / 8) * TC_GROUP_STRIDE;                      // ACC: [8 warps][K][8] sums, then [8][K] counts
    int* wcnt = reinterpret_cast<int*>(wtab + (ACC ? (size_t)TC_EPI_WARPS * K * 8 : 0));
    TcShared* sh = reinterpret_cast<TcShared*>(wcnt + (ACC ? (size_t)TC_EPI_WARPS * K : 0));
    volatile int* abort_flag = &sh->abort_flag;
    pdl_launch_dependents();

    if (tid == 0) {
        for (int s = 0; s < TC_STAGES; s++) { mbar_init(smem_u32(&sh->full_a[s]), TC_LOAD_WARPS); mbar_init(smem_u32(&sh->empty_a[s]), 1); }
        for (int b = 0; b < 2; b++) { mbar_init(smem_u32(&sh->full_acc[b]), 1); mbar_init(smem_u32(&sh->empty_acc[b]), 4); }
        mbar_init(smem_u32(&sh->drained), 1);
        sh->abort_flag = 0;
        sh->cmax2_bits = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == TC_MMA_WARP) {               // all 512 columns of tensor memory: two accumulator tiles of up to 256 columns
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(&sh->tmem_base)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    pdl_wait();

    // ── centroids: exact copy, the three operand pieces, max |c|^2 ──
    for (int e = tid; e < K * 8; e += TC_THREADS) {
        const float c = C[e];
        const int k = e >> 3, d = e & 7;
        cex[e] = c;
        cgrp[(k >> 3) * TC_GROUP_STRIDE + d * 8 + (k & 7)] = c;
    }
    if (ACC) {
        for (int e = tid; e < TC_EPI_WARPS * K * 8; e += TC_THREADS) wtab[e] = 0.0f;
        for (int e = tid; e < TC_EPI_WARPS * K; e += TC_THREADS) wcnt[e] = 0;
    }
    for (int e = tid; e < 128; e += TC_THREADS) {             // constant chunk pair of the point operand: row e = (1 1 1 0 | 0 0 0 0)
        const uint32_t one = tf32_of(1.0f);
        *reinterpret_cast<uint4*>(sAug + (e >> 3) * 128 + (e & 7) * 16) = make_uint4(one, one, one, 0u);
        *reinterpret_cast<uint4*>(sAug + TC_A_CHUNK + (e >> 3) * 128 + (e & 7) * 16) = make_uint4(0u, 0u, 0u, 0u);
    }
    __syncthreads();
    unsigned cm_bits = 0u;
    for (int n = tid; n < K; n += TC_THREADS) {
        uint32_t h[8], l[8];
        float nn = 0.0f;
#pragma unroll
        for (int d = 0; d < 8; d++) {
            const float c = cex[n * 8 + d];
            h[d] = tf32_of(c);
            l[d] = tf32_of(c - __uint_as_float(h[d]));
            nn = fmaf(c, c, nn);
        }
        cm_bits = max(cm_bits, __float_as_uint(nn));         // nn >= 0 or NaN: NaN and Inf sort above everything finite
        const float nh = -0.5f * nn;
        const uint32_t n0 = tf32_of(nh);
        const float r1 = nh - __uint_as_float(n0);
        const uint32_t n1 = tf32_of(r1);
        const uint32_t n2 = tf32_of(r1 - __uint_as_float(n1));
        const uint32_t row = (uint32_t)(n >> 3) * 128u + (uint32_t)(n & 7) * 16u;
        *reinterpret_cast<uint4*>(sB + row) = make_uint4(h[0], h[1], h[2], h[3]);
        *reinterpret_cast<uint4*>(sB + b_chunk + row) = make_uint4(h[4], h[5], h[6], h[7]);
        *reinterpret_cast<uint4*>(sB + b_piece + row) = make_uint4(l[0], l[1], l[2], l[3]);
        *reinterpret_cast<uint4*>(sB + b_piece + b_chunk + row) = make_uint4(l[4], l[5], l[6], l[7]);
        *reinterpret_cast<uint4*>(sB + 2 * b_piece + row) = make_uint4(n0, n1, n2, 0u);
        *reinterpret_cast<uint4*>(sB + 2 * b_piece + b_chunk + row) = make_uint4(0u, 0u, 0u, 0u);
    }
    cm_bits = __reduce_max_sync(0xffffffffu, cm_bits);
    if (lane == 0) atomicMax(&sh->cmax2_bits, cm_bits);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // the operands written above are read by the tensor cores
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = sh->tmem_base;
    const float cm2 = __uint_as_float(sh->cmax2_bits);

    const long ntile = (N + TC_TILE - 1) / TC_TILE;
    const long n_my = (long)blockIdx.x < ntile ? (ntile - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;      // tiles blockIdx.x + i gridDim.x

    if (warp >= TC_EPI_WARPS && warp < TC_MMA_WARP) {
        // ── loaders: warp lw owns rows 32 lw .. + 31 of every tile: raw rows by cp.async (TC_STAGES - 1 tiles ahead), then the
        //    two TF32 terms into the operand stage ──
        const int lw = warp - TC_EPI_WARPS;
        auto issue = [&](long i) {
            if (i < n_my) {
                const long p0 = (blockIdx.x + i * gridDim.x) * TC_TILE + 32 * lw;
                const uint32_t dst = smem_u32(sRaw + (i % TC_STAGES) * TC_RAW_STAGE + lw * 1024);
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    const int e = lane + 32 * j;                     // 16-byte piece e of this warp's 1 KB: point e / 2, half e % 2
                    const long pt = p0 + (e >> 1);
                    const int nbytes = pt < N ? 16 : 0;              // points past the end read as zeros
                    const float* src = X + (pt < N ? pt : 0) * 8 + (e & 1) * 4;
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"(dst + e * 16), "l"(src), "r"(nbytes) : "memory");
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        for (int i = 0; i < TC_STAGES - 1; i++) issue(i);
        for (long i = 0; i < n_my; i++) {
            const int s = (int)(i % TC_STAGES);
            __syncwarp();                                            // the raw rows about to be refilled have been read by every lane
            issue(i + TC_STAGES - 1);
            asm volatile("cp.async.wait_group %0;" :: "n"(TC_STAGES - 1) : "memory");
            __syncwarp();
            if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&sh->empty_a[s]), (uint32_t)(((i / TC_STAGES) & 1) ^ 1), abort_flag, 1))) break;   // the whole warp leaves or stays
            const unsigned char* raw = sRaw + s * TC_RAW_STAGE;
            unsigned char* dstA = sA + s * TC_A_STAGE;
            {
                const int r = 32 * lw + lane;
                const float4 a = *reinterpret_cast<const float4*>(raw + r * 32), c = *reinterpret_cast<const float4*>(raw + r * 32 + 16);
                const float v[8] = { a.x, a.y, a.z, a.w, c.x, c.y, c.z, c.w };
                uint32_t h[8], l[8];
#pragma unroll
                for (int d = 0; d < 8; d++) {
                    // xh = x cut to its TF32 bits; xl = x - xh exactly (the tensor cores read its upper bits): x.c is then
                    // short by at most 2^-20 |x||c| before the xl.cl term that is left out anyway
                    h[d] = __float_as_uint(v[d]) & 0xFFFFE000u;
                    l[d] = __float_as_uint(v[d] - __uint_as_float(h[d]));
                }
                const uint32_t row = (uint32_t)(r >> 3) * 128u + (uint32_t)(r & 7) * 16u;
                *reinterpret_cast<uint4*>(dstA + row) = make_uint4(h[0], h[1], h[2], h[3]);
                *reinterpret_cast<uint4*>(dstA + TC_A_CHUNK + row) = make_uint4(h[4], h[5], h[6], h[7]);
                *reinterpret_cast<uint4*>(dstA + 2 * TC_A_CHUNK + row) = make_uint4(l[0], l[1], l[2], l[3]);
                *reinterpret_cast<uint4*>(dstA + 3 * TC_A_CHUNK + row) = make_uint4(l[4], l[5], l[6], l[7]);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&sh->full_a[s]));
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
    } else if (warp == TC_MMA_WARP) {
        // ── MMA issue: one thread ──
        if (lane == 0) {
            const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(K >> 3) << 17) | ((uint32_t)(TC_TILE >> 4) << 24);
            const uint64_t b_h = smem_desc(smem_u32(sB), b_chunk, 128), b_l = smem_desc(smem_u32(sB + b_piece), b_chunk, 128);
            const uint64_t b_n = smem_desc(smem_u32(sB + 2 * b_piece), b_chunk, 128), a_one = smem_desc(smem_u32(sAug), TC_A_CHUNK, 128);
            bool ok = true;
            for (long i = 0; i < n_my && ok; i++) {
                const int s = (int)(i % TC_STAGES), b = (int)(i & 1);
                ok = mbar_wait(smem_u32(&sh->full_a[s]), (uint32_t)((i / TC_STAGES) & 1), abort_flag, 2) &&
                     mbar_wait(smem_u32(&sh->empty_acc[b]), (uint32_t)(((i >> 1) & 1) ^ 1), abort_flag, 3);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d = tmem_base + (uint32_t)b * 256u;
                const uint64_t a_h = smem_desc(smem_u32(sA + s * TC_A_STAGE), TC_A_CHUNK, 128);
                const uint64_t a_l = smem_desc(smem_u32(sA + s * TC_A_STAGE + 2 * TC_A_CHUNK), TC_A_CHUNK, 128);
                mma_tf32_ss(d, a_h, b_h, idesc, 0u);
                mma_tf32_ss(d, a_l, b_h, idesc, 1u);
                mma_tf32_ss(d, a_h, b_l, idesc, 1u);
                mma_tf32_ss(d, a_one, b_n, idesc, 1u);
                mma_commit(smem_u32(&sh->empty_a[s]));               // the operand stage is free once these MMAs have read it
                mma_commit(smem_u32(&sh->full_acc[b]));              // and the accumulator tile is complete
            }
            mma_commit(smem_u32(&sh->drained));
            mbar_wait(smem_u32(&sh->drained), 0u, abort_flag, 4);    // nothing of this block is left in the tensor pipe
        }
    } else {
        // ── epilogue: warp w drains accumulator tile w / 4, rows 32 (w % 4) .. + 31 ──
        const int b = warp >> 2, q = warp & 3;
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)b * 256u;
        float* mytab = wtab + (size_t)warp * K * 8;
        int* mycnt = wcnt + (size_t)warp * K;
        double inert = 0.0;
        for (long i = b; i < n_my; i += 2) {
            const long row = (blockIdx.x + i * gridDim.x) * TC_TILE + q * 32 + lane;
            const bool have = row < N;
            float xr[8];
            {
                const float4 u = have ? *reinterpret_cast<const float4*>(X + row * 8) : make_float4(0.f, 0.f, 0.f, 0.f);
                const float4 v = have ? *reinterpret_cast<const float4*>(X + row * 8 + 4) : make_float4(0.f, 0.f, 0.f, 0.f);
                xr[0] = u.x; xr[1] = u.y; xr[2] = u.z; xr[3] = u.w; xr[4] = v.x; xr[5] = v.y; xr[6] = v.z; xr[7] = v.w;
            }
            if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&sh->full_acc[b]), (uint32_t)((i >> 1) & 1), abort_flag, 5))) break;            // the whole warp leaves or stays
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            Top2 tr[4];
#pragma unroll
            for (int q = 0; q < 4; q++) { tr[q].m1 = -INFINITY; tr[q].m2 = -INFINITY; tr[q].g1 = q; }
            uint32_t ra[32], rb[32];                                 // 32 columns per load, the next load in flight while one is reduced
            tmem_ld32(taddr, ra);
            for (int c0 = 0; c0 < K; c0 += 64) {
                tmem_wait_ld(ra);
                if (c0 + 32 < K) tmem_ld32(taddr + c0 + 32, rb);
                top2_groups(ra, c0 >> 3, tr);
                if (c0 + 32 < K) {
                    tmem_wait_ld(rb);
                    if (c0 + 64 < K) tmem_ld32(taddr + c0 + 64, ra);
                    top2_groups(rb, (c0 >> 3) + 4, tr);
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&sh->empty_acc[b]));  // the tensor cores may overwrite this tile
            const Top2 top = top2_merge(top2_merge(tr[0], tr[1]), top2_merge(tr[2], tr[3]));
            const float m1 = top.m1, m2 = top.m2;
            const int g1 = top.g1;
            // the margin that makes the filter safe: false for NaN / Inf as well
            float xn = 0.0f;
#pragma unroll
            for (int d = 0; d < 8; d++) xn = fmaf(xr[d], xr[d], xn);
            const bool sure = (m1 - m2) > 6.103515625e-5f * (xn + cm2);
            // the best group in the exact form (subtract, multiply, add, each rounded, in dimension order), then ascending
            // with strict '<': the lowest index wins ties as in the reference
            int win = g1 * 8;
            float best;
            {
                const float* cg = cgrp + g1 * TC_GROUP_STRIDE;
                // subtract and multiply go two centroids at a time; the add stays scalar, because the assembler contracts
                // a packed multiply followed by a packed add into a fused multiply-add, which rounds differently
                float dk[8] = { 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f };
#pragma unroll
                for (int d = 0; d < 8; d++) {
                    const ulonglong2 ca = *reinterpret_cast<const ulonglong2*>(cg + d * 8), cb = *reinterpret_cast<const ulonglong2*>(cg + d * 8 + 4);
                    const unsigned long long xx = pack2(xr[d], xr[d]);
                    const unsigned long long c2[4] = { ca.x, ca.y, cb.x, cb.y };
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const unsigned long long v = sub2(xx, c2[j]);
                        float m0, m1;
                        unpack2(mul2(v, v), m0, m1);
                        dk[2 * j] = __fadd_rn(dk[2 * j], m0);
                        dk[2 * j + 1] = __fadd_rn(dk[2 * j + 1], m1);
                    }
                }
                best = dk[0];
#pragma unroll
                for (int j = 1; j < 8; j++) if (dk[j] < best) { best = dk[j]; win = g1 * 8 + j; }
            }
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
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {                   // lexicographic (distance, index) minimum
                    const float od = __shfl_xor_sync(0xffffffffu, bd, o);
                    const int ok = __shfl_xor_sync(0xffffffffu, bk, o);
                    if (od < bd || (od == bd && ok < bk)) { bd = od; bk = ok; }
                }
                if (lane == rl) {
                    if (bk == 0x7fffffff) { bk = 0; bd = ref_sqdist<8>(xr, cex, 8); }      // every distance NaN: centroid 0 (the reference's seed)
                    win = bk; best = bd;
                }
            }
            if (have) { idx[row] = win; if (dist) dist[row] = best; }
            if (ACC) {
                // points of the warp that share a cluster take turns in index order; different clusters go together
                const unsigned grp = __match_any_sync(0xffffffffu, have ? win : -1 - lane);
                const int rank = __popc(grp & ((1u << lane) - 1u));
                const int rounds = __reduce_max_sync(0xffffffffu, (unsigned)__popc(grp));
                for (int r = 0; r < rounds; r++) {
                    if (have && rank == r) {
                        float4* t = reinterpret_cast<float4*>(mytab + (size_t)win * 8);
                        float4 a = t[0], c = t[1];
                        a.x += xr[0]; a.y += xr[1]; a.z += xr[2]; a.w += xr[3];
                        c.x += xr[4]; c.y += xr[5]; c.z += xr[6]; c.w += xr[7];
                        t[0] = a; t[1] = c;
                        mycnt[win] += 1;
                    }
                    __syncwarp();
                }
                if (have) inert += (double)best;
            }
        }
        if (ACC) {
            // the eight tables of the block, added in warp order; every epilogue warp gets here, also after a wait ran out
            for (int o = 16; o > 0; o >>= 1) inert += __shfl_xor_sync(0xffffffffu, inert, o);
            asm volatile("bar.sync 1, %0;" :: "n"(TC_EPI_WARPS * 32) : "memory");
            for (int e = tid; e < K * 8; e += TC_EPI_WARPS * 32) {
                float v = wtab[e];
#pragma unroll
                for (int w = 1; w < TC_EPI_WARPS; w++) v += wtab[(size_t)w * K * 8 + e];
                part_sums[(size_t)blockIdx.x * K * 8 + e] = v;
            }
            for (int e = tid; e < K; e += TC_EPI_WARPS * 32) {
                int v = wcnt[e];
#pragma unroll
                for (int w = 1; w < TC_EPI_WARPS; w++) v += wcnt[(size_t)w * K + e];
                part_counts[(size_t)blockIdx.x * K + e] = v;
            }
            if (lane == 0) sh->inert[warp] = inert;
            asm volatile("bar.sync 1, %0;" :: "n"(TC_EPI_WARPS * 32) : "memory");
            if (tid == 0) {
                double t = 0.0;
                for (int w = 0; w < TC_EPI_WARPS; w++) t += sh->inert[w];
                part_inertia[blockIdx.x] = t;
            }
        }
    }
    // ── teardown: every role is out of its loop (all waits are bounded); release tensor memory ──
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == TC_MMA_WARP) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"(512u) : "memory");
    }
    if (tid == 0 && sh->abort_flag) *err = 100 + sh->abort_flag;
}

}  // namespace

// D == 8, K a multiple of 64 up to 256, 16-byte aligned X: the tensor-memory kernel. Returns IBCU_ERR_STATE without
// touching the context's error when the shape is not its own (the caller takes another kernel).
static size_t tc_smem_bytes(int K, bool acc) {
    return 1024 + (size_t)3 * 2 * K * 16 + 2 * TC_A_CHUNK + (size_t)TC_STAGES * (TC_A_STAGE + TC_RAW_STAGE) + (size_t)K * 8 * sizeof(float) +
           (size_t)(K / 8) * TC_GROUP_STRIDE * sizeof(float) + (acc ? (size_t)TC_EPI_WARPS * K * 9 * sizeof(float) : 0) + sizeof(TcShared) + 64;
}

int ibcu_kmeans_assign_tc(ibcu_ctx* ctx, const float* X, long N, const float* C, int K, int32_t* idx, float* dist) {
    if (K < 64 || K > 256 || (K & 63) || ((uintptr_t)X & 15)) return IBCU_ERR_STATE;
    const size_t smem = tc_smem_bytes(K, false);
    IBCU_CUDA(ctx, cudaFuncSetAttribute(assign_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const long ntile = (N + TC_TILE - 1) / TC_TILE;
    long blocks = ntile < ctx->sm_count ? ntile : ctx->sm_count;
    if (blocks < 1) blocks = 1;
    return ibcu_launch(ctx, assign_tc_kernel<false>, dim3((unsigned)blocks), dim3(TC_THREADS), smem, 1, true, X, N, C, K, idx, dist, ctx->kern_err,
                       (float*)nullptr, (int32_t*)nullptr, (double*)nullptr);
}

// The assignment and the accumulate pass of a Lloyd iteration in one launch: per-block partial tables go to part_* (room for
// *nblocks blocks of K * 8 sums, K counts and one inertia), which accumulate_finish_kernel then adds up. Same conditions and
// return convention as above.
int ibcu_kmeans_assign_accumulate_tc(ibcu_ctx* ctx, const float* X, long N, const float* C, int K, int32_t* idx, float* dist,
                                     float* part_sums, int32_t* part_counts, double* part_inertia, int nblocks) {
    if (K < 64 || K > 256 || (K & 63) || ((uintptr_t)X & 15)) return IBCU_ERR_STATE;
    const size_t smem = tc_smem_bytes(K, true);
    if (smem > 227 * 1024) return IBCU_ERR_STATE;
    IBCU_CUDA(ctx, cudaFuncSetAttribute(assign_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    return ibcu_launch(ctx, assign_tc_kernel<true>, dim3((unsigned)nblocks), dim3(TC_THREADS), smem, 1, true, X, N, C, K, idx, dist, ctx->kern_err,
                       part_sums, part_counts, part_inertia);
}
