// k-means assign / accumulate / update.
//
// assign: nearest centroid by the direct squared distance, evaluated in exactly the order and with
// exactly the roundings of the reference's x86-64 Release binary (multiply and add rounded
// separately for dimensions below 4*floor(D/4), fused for the remaining D%4), strict '<' so the
// lowest index wins ties. Codes are therefore bit-identical to the reference, not "close".
//   assign_exact_kernel   every distance in that exact form (CUDA cores).
//   assign_filter_kernel  (D == 8) bf16 tensor-core scores x.c - |c|^2/2 for all K centroids per
//                         16-point tile, best / second-best tracked in registers; a point whose
//                         margin exceeds a rigorous error bound takes the tensor-core winner, every
//                         other point is re-evaluated in the exact form. Same codes, ~4x fewer
//                         issue slots.
// accumulate: per-cluster sums / counts / inertia with a fixed order of additions (no atomics):
// each warp adds its points in index order into a private shared-memory table, warps and blocks are
// then combined in index order.
#include "common.cuh"

namespace {

constexpr int KM_MAX_D = 32;

template <int DT>   // DT > 0: compile-time D; DT == 0: run-time D
__device__ __forceinline__ float ref_sqdist(const float* x, const float* c, int D) {
    float s = 0.0f;
    if (DT > 0) {
#pragma unroll
        for (int d = 0; d < (DT & ~3); d++) {
            const float v = __fsub_rn(x[d], c[d]);
            s = __fadd_rn(s, __fmul_rn(v, v));
        }
#pragma unroll
        for (int d = (DT & ~3); d < DT; d++) {
            const float v = __fsub_rn(x[d], c[d]);
            s = __fmaf_rn(v, v, s);
        }
    } else {
        const int body = D & ~3;
        for (int d = 0; d < body; d++) {
            const float v = __fsub_rn(x[d], c[d]);
            s = __fadd_rn(s, __fmul_rn(v, v));
        }
        for (int d = body; d < D; d++) {
            const float v = __fsub_rn(x[d], c[d]);
            s = __fmaf_rn(v, v, s);
        }
    }
    return s;
}

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
    const long total = todo ? (long)*n_todo : N;
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
    for (long p = p0; p < p1; p += 32) {
        const long mine = p + lane;
        const int n = (int)((p1 - p) < 32 ? (p1 - p) : 32);
        const int code = mine < p1 ? idx[mine] : 0;
        if (dist && mine < p1) inert += (double)dist[mine];
        for (int e = lane; e < n * D; e += 32) stage[e] = X[(size_t)p * D + e];
        __syncwarp();
        for (int j = 0; j < n; j++) {
            const int k = __shfl_sync(0xffffffffu, code, j);
            if (lane < D) ms[(size_t)k * D + lane] += stage[j * D + lane];
            if (lane == 31) mc[k] += 1;
            __syncwarp();
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

__global__ void __launch_bounds__(256) accumulate_finish_kernel(const float* __restrict__ part_sums, const int32_t* __restrict__ part_counts,
                                                                const double* __restrict__ part_inertia, int nblocks, int KD, int K,
                                                                float* __restrict__ sums, int32_t* __restrict__ counts, double* __restrict__ inertia) {
    pdl_launch_dependents();
    pdl_wait();
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e < KD) {
        double s = 0.0;
        for (int b = 0; b < nblocks; b++) s += (double)part_sums[(size_t)b * KD + e];
        sums[e] = (float)s;
    }
    if (e < K) {
        int c = 0;
        for (int b = 0; b < nblocks; b++) c += part_counts[(size_t)b * K + e];
        counts[e] = c;
    }
    if (e == 0 && inertia) {
        double t = 0.0;
        for (int b = 0; b < nblocks; b++) t += part_inertia[b];
        *inertia = t;
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

extern "C" int ibcu_kmeans_assign(ibcu_ctx* ctx, const float* X, long N, int D, const float* C, int K,
                                  int32_t* idx, float* dist) {
    IBCU_CHECK_CTX(ctx);
    IBCU_REQUIRE(ctx, X && C && idx, "ibcu_kmeans_assign: null pointer");
    IBCU_REQUIRE(ctx, N > 0 && D >= 1 && D <= KM_MAX_D && K >= 1 && K <= 1024, "ibcu_kmeans_assign: N=%ld D=%d K=%d out of range", N, D, K);
    IBCU_REQUIRE(ctx, (size_t)K * D * sizeof(float) <= 128 * 1024, "ibcu_kmeans_assign: K*D=%d too large", K * D);
    return assign_exact_launch(ctx, X, N, D, C, K, idx, dist, nullptr, nullptr, N);
}

extern "C" int ibcu_kmeans_accumulate(ibcu_ctx* ctx, const float* X, long N, int D, int K,
                                      const int32_t* idx, const float* dist,
                                      float* sums, int32_t* counts, double* inertia) {
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
    int fin_blocks = (int)((KD + 255) / 256);
    return ibcu_launch(ctx, accumulate_finish_kernel, dim3(fin_blocks), dim3(256), 0, 1, true,
                       (const float*)part_sums, (const int32_t*)part_counts, (const double*)part_inertia, (int)nblocks, (int)KD, K,
                       sums, counts, inertia);
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
    int rc = ibcu_kmeans_assign(ctx, X, N, D, C, K, idx, dist);
    if (rc) return rc;
    rc = ibcu_kmeans_accumulate(ctx, X, N, D, K, idx, dist, sums, counts, inertia);
    if (rc) return rc;
    if (ctx->world > 1) {
        if ((rc = ibcu_allreduce_f32(ctx, sums, (size_t)K * D))) return rc;
        if ((rc = ibcu_allreduce_i32(ctx, counts, (size_t)K))) return rc;
        if (inertia && (rc = ibcu_allreduce_f64(ctx, inertia, 1))) return rc;
    }
    return ibcu_kmeans_update(ctx, C, K, D, sums, counts, nullptr);
}
