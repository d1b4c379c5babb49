// Product-quantised matvec: out[r] = row_scale[r] * sum over subspaces s of LUT_s[code[r][s]],
// LUT_s[k] = codebook_s[k] . x_s (FP32), for 1..32 activations.
//
// Data in HBM: codebooks, row scales and the two row-major code planes exactly as the reference
// holds them, plus one derived array made once per tensor by ibcu_pq_prepare: the code planes
// transposed to subspace-major order idx_t[s][row] (s = 2*chunk + side). With it a block that owns a
// slab of subspaces reads long contiguous runs of codes (128-bit loads, every byte used) instead of a
// few bytes out of every row.
//
// pq_gather_kernel: grid = (slabs of S <= 24 subspaces) x (blocks of 2048 rows). A block first puts
// the codes of its slab in flight (4 rows per thread, all S subspaces, kept in registers), then, for
// every activation in turn: finds the activation's max |x| (the reference's 1 %-of-max rule drops
// whole chunks), builds the slab's lookup table in shared memory straight from the fp16 codebooks
// (128-bit codebook loads), and walks its rows: one byte extract, one shared-memory read and one add
// per code. The codes are read from HBM once however many activations there are. Partial row sums go
// to scratch [activation][slab][row]; pq_reduce_kernel adds the slabs in slab order, applies the row
// scale and stores. No atomics, so results are run-to-run identical.
#include "common.cuh"

namespace {

constexpr int PQ_THREADS = 512;
constexpr int PQ_ROWS_PER_THREAD = 4;
constexpr int PQ_ROWS_PER_BLOCK = PQ_THREADS * PQ_ROWS_PER_THREAD;
constexpr int PQ_SMAX = 24;                 // subspaces per slab (even): their codes live in PQ_SMAX registers

// rows x C bytes  ->  2C x M_pad bytes (tile transpose through shared memory)
__global__ void __launch_bounds__(256) pq_transpose_kernel(const uint8_t* __restrict__ idx_l, const uint8_t* __restrict__ idx_r,
                                                           int M, int C, int M_pad, uint8_t* __restrict__ idx_t) {
    __shared__ uint8_t tile[64][65];
    const uint8_t* src = blockIdx.z ? idx_r : idx_l;
    const int r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
    for (int e = threadIdx.x; e < 64 * 64; e += blockDim.x) {
        const int rr = e >> 6, cc = e & 63;
        const int r = r0 + rr, c = c0 + cc;
        tile[rr][cc] = (r < M && c < C) ? src[(size_t)r * C + c] : 0;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < 64 * 64; e += blockDim.x) {
        const int cc = e >> 6, rr = e & 63;
        const int r = r0 + rr, c = c0 + cc;
        if (c < C && r < M_pad) idx_t[((size_t)(2 * c + blockIdx.z)) * M_pad + r] = tile[rr][cc];
    }
}

struct PqParams {
    int M, M_pad, N, G, K, C, S, B, nslabs;   // S = subspaces per slab
    const __half* cb_l; const __half* cb_r; long cb_stride;
    const uint8_t* idx_t;
    const float* x;                            // [B][N]
    float* partial;                            // [B][nslabs][M_pad]
};

__device__ __forceinline__ uint32_t ld_stream_u1(const void* p) {
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}

// Every global read of this kernel is issued in batches of independent loads: with one block per SM
// there are too few warps to hide one L2 round trip per loop iteration.
template <int SMAX, int BT>   // BT activations share one pass over the table: entries are BT floats wide
__global__ void __launch_bounds__(PQ_THREADS, SMAX <= 12 ? 2 : 1) pq_gather_kernel(const PqParams p) {
    extern __shared__ __align__(16) float lut[];          // [S][K][BT] (+ slack)
    __shared__ __align__(16) float xs[BT][PQ_SMAX * 16];   // activation slices of the slab
    __shared__ unsigned char live[BT][PQ_SMAX];
    __shared__ float red[BT][PQ_THREADS / 32];
    pdl_launch_dependents();
    const int half = p.G >> 1, tid = threadIdx.x;
    const int s0 = blockIdx.x * p.S;                       // even: a chunk's two subspaces share a slab
    const int ns = min(p.S, 2 * p.C - s0);
    const int row = blockIdx.y * PQ_ROWS_PER_BLOCK + tid * PQ_ROWS_PER_THREAD;
    const bool has_rows = row < p.M_pad;

    // the slab's codes for this thread's 4 rows: loaded once, before anything that depends on x
    uint32_t cd[SMAX];
#pragma unroll
    for (int i = 0; i < SMAX; i++)
        cd[i] = (has_rows && i < ns) ? ld_stream_u1(p.idx_t + (size_t)(s0 + i) * p.M_pad + row) : 0u;

    pdl_wait();
    const bool vec_cb = half == 8 && (p.cb_stride & 7) == 0 && ((uintptr_t)p.cb_l & 15) == 0 && ((uintptr_t)p.cb_r & 15) == 0;
    const bool vec_x = (p.N & 3) == 0 && ((uintptr_t)p.x & 15) == 0;
    const int kshift = (p.K & (p.K - 1)) == 0 ? __ffs(p.K) - 1 : -1;
    const int per = ns * p.K;
    for (int b0 = 0; b0 < p.B; b0 += BT) {
        const int nb = min(BT, p.B - b0);
        // max |x| of each activation
        float am[BT];
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
                    am[t] = fmaxf(am[t], fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
                }
            } else {
#pragma unroll 8
                for (int j = tid; j < p.N; j += PQ_THREADS) am[t] = fmaxf(am[t], fabsf(xb[j]));
            }
        }
#pragma unroll
        for (int t = 0; t < BT; t++) am[t] = warp_max(am[t]);
        __syncthreads();                                   // the previous pass's table reads are done
#pragma unroll
        for (int t = 0; t < BT; t++) {
            if ((tid & 31) == 0) red[t][tid >> 5] = am[t];
            // subspace s covers x[s * half, (s + 1) * half)
            if (tid < ns * half) xs[t][tid] = t < nb ? p.x[(size_t)(b0 + t) * p.N + (size_t)s0 * half + tid] : 0.0f;
        }
        __syncthreads();
        if (tid < ns * BT) {
            const int t = tid / ns, sl = tid - t * ns;
            float amax = red[t][0];
#pragma unroll
            for (int w = 1; w < PQ_THREADS / 32; w++) amax = fmaxf(amax, red[t][w]);
            bool keep = t < nb;
            if (keep && amax > 0.0f) {
                const float* xc = xs[t] + (sl & ~1) * half;  // the chunk of this subspace
                float cm = 0.0f;
                for (int i = 0; i < p.G; i++) cm = fmaxf(cm, fabsf(xc[i]));
                keep = cm >= amax * 0.01f;
            }
            live[t][sl] = keep;
        }
        __syncthreads();
        // lookup table of the slab for these activations
        if (vec_cb) {
            for (int e0 = 0; e0 < per; e0 += 4 * PQ_THREADS) {
                uint4 raw[4];
                int sls[4];
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const int e = e0 + u * PQ_THREADS + tid;
                    const int sl = kshift >= 0 ? e >> kshift : e / p.K;
                    const int k = e - sl * p.K, s = s0 + sl;
                    sls[u] = e < per ? sl : -1;
                    raw[u] = make_uint4(0, 0, 0, 0);
                    if (e < per)
                        raw[u] = *reinterpret_cast<const uint4*>(((s & 1) ? p.cb_r : p.cb_l) + (size_t)(s >> 1) * p.cb_stride + (size_t)k * 8);
                }
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    if (sls[u] < 0) continue;
                    const __half2* h = reinterpret_cast<const __half2*>(&raw[u]);
                    const float2 f0 = __half22float2(h[0]), f1 = __half22float2(h[1]), f2 = __half22float2(h[2]), f3 = __half22float2(h[3]);
                    float v[BT];
#pragma unroll
                    for (int t = 0; t < BT; t++) {
                        const float4 xa = *reinterpret_cast<const float4*>(xs[t] + sls[u] * 8);
                        const float4 xc = *reinterpret_cast<const float4*>(xs[t] + sls[u] * 8 + 4);
                        float acc = 0.0f;
                        acc = fmaf(f0.x, xa.x, acc); acc = fmaf(f0.y, xa.y, acc); acc = fmaf(f1.x, xa.z, acc); acc = fmaf(f1.y, xa.w, acc);
                        acc = fmaf(f2.x, xc.x, acc); acc = fmaf(f2.y, xc.y, acc); acc = fmaf(f3.x, xc.z, acc); acc = fmaf(f3.y, xc.w, acc);
                        v[t] = live[t][sls[u]] ? acc : 0.0f;
                    }
                    float* dst = lut + (size_t)(e0 + u * PQ_THREADS + tid) * BT;
                    if constexpr (BT == 4) *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
                    else {
#pragma unroll
                        for (int t = 0; t < BT; t++) dst[t] = v[t];
                    }
                }
            }
        } else {
            for (int e = tid; e < per; e += PQ_THREADS) {
                const int sl = e / p.K, k = e - sl * p.K, s = s0 + sl;
                const __half* ent = ((s & 1) ? p.cb_r : p.cb_l) + (size_t)(s >> 1) * p.cb_stride + (size_t)k * half;
#pragma unroll
                for (int t = 0; t < BT; t++) {
                    float acc = 0.0f;
                    if (live[t][sl])
                        for (int i = 0; i < half; i++) acc = fmaf(__half2float(ent[i]), xs[t][sl * half + i], acc);
                    lut[(size_t)e * BT + t] = acc;
                }
            }
        }
        __syncthreads();
        if (has_rows) {
            float acc[PQ_ROWS_PER_THREAD][BT];
#pragma unroll
            for (int r = 0; r < PQ_ROWS_PER_THREAD; r++)
#pragma unroll
                for (int t = 0; t < BT; t++) acc[r][t] = 0.0f;
#pragma unroll
            for (int i = 0; i < SMAX; i++) {
                if (i < ns) {
                    const float* T = lut + (size_t)i * p.K * BT;
                    const uint32_t w = cd[i];
#pragma unroll
                    for (int r = 0; r < PQ_ROWS_PER_THREAD; r++) {
                        const uint32_t code = (w >> (8 * r)) & 0xFF;
                        if constexpr (BT == 4) {
                            const float4 q = *reinterpret_cast<const float4*>(T + code * 4);
                            acc[r][0] += q.x; acc[r][1] += q.y; acc[r][2] += q.z; acc[r][3] += q.w;
                        } else {
#pragma unroll
                            for (int t = 0; t < BT; t++) acc[r][t] += T[code * BT + t];
                        }
                    }
                }
            }
#pragma unroll
            for (int t = 0; t < BT; t++) {
                if (t >= nb) continue;
                float* dst = p.partial + ((size_t)(b0 + t) * p.nslabs + blockIdx.x) * p.M_pad + row;
                *reinterpret_cast<float4*>(dst) = make_float4(acc[0][t], acc[1][t], acc[2][t], acc[3][t]);
            }
        }
    }
}

// block = 32 rows x 8 slab groups: group g adds slabs g, g + 8, ... in ascending order with all its loads in
// flight at once, then the 8 group sums are combined in a fixed tree.
__global__ void __launch_bounds__(256) pq_reduce_kernel(const float* __restrict__ partial, int nslabs, int M, int M_pad,
                                                        const __half* __restrict__ row_scale, float* __restrict__ out) {
    __shared__ float part[8][32];
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31, g = threadIdx.x >> 5;
    const int r = blockIdx.x * 32 + lane, b = blockIdx.y;
    float s = 0.0f;
    if (r < M) {
        const float* src = partial + (size_t)b * nslabs * M_pad + r;
        for (int k0 = g; k0 < nslabs; k0 += 64) {                   // eight loads in flight, added in slab order
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; u++) v[u] = k0 + 8 * u < nslabs ? src[(size_t)(k0 + 8 * u) * M_pad] : 0.0f;
#pragma unroll
            for (int u = 0; u < 8; u++) s += v[u];
        }
    }
    part[g][lane] = s;
    __syncthreads();
    if (g == 0 && r < M) {
        const float t = ((part[0][lane] + part[1][lane]) + (part[2][lane] + part[3][lane])) +
                        ((part[4][lane] + part[5][lane]) + (part[6][lane] + part[7][lane]));
        out[(size_t)b * M + r] = t * __half2float(row_scale[r]);
    }
}

// Shared launch logic of the two entry points: `scratch` must hold pq_scratch_floats() floats.
struct PqPlan { int C, S, nslabs, row_blocks; size_t floats; };

PqPlan pq_plan(const ibcu_ctx* ctx, const ibcu_pq_t* t, int B) {
    PqPlan pl;
    pl.C = t->N / t->G;
    const int nsub = 2 * pl.C;
    pl.row_blocks = (t->M_pad + PQ_ROWS_PER_BLOCK - 1) / PQ_ROWS_PER_BLOCK;
    int S = (int)(((long)nsub * pl.row_blocks + ctx->sm_count - 1) / ctx->sm_count);   // about one block per SM
    S = (S + 1) & ~1;                                      // even: both halves of a chunk in one slab
    if (S < 4) S = 4;
    if (S > PQ_SMAX) S = PQ_SMAX;
    pl.S = S;
    pl.nslabs = (nsub + S - 1) / S;
    pl.floats = (size_t)B * pl.nslabs * t->M_pad;
    return pl;
}

int pq_launch(ibcu_ctx* ctx, const ibcu_pq_t* t, const float* x, float* out, int B, const PqPlan& pl, float* scratch) {
    PqParams p;
    p.M = t->M; p.M_pad = t->M_pad; p.N = t->N; p.G = t->G; p.K = t->K; p.C = pl.C; p.S = pl.S; p.B = B; p.nslabs = pl.nslabs;
    p.cb_l = (const __half*)t->codebook_l; p.cb_r = (const __half*)t->codebook_r; p.cb_stride = t->cb_chunk_stride;
    p.idx_t = t->idx_t; p.x = x; p.partial = scratch;
    const int bt = B >= 2 ? 4 : 1;
    const size_t smem = ((size_t)pl.S * t->K + 256) * bt * sizeof(float);   // + slack: a code >= K must not leave the allocation
    const dim3 grid(pl.nslabs, pl.row_blocks), block(PQ_THREADS);
    int rc;
    if (bt == 4) {
        static bool attr_done[64];                                          // per device: the wide table needs the opt-in shared-memory size
        if (!attr_done[ctx->device & 63]) {
            IBCU_CUDA(ctx, cudaFuncSetAttribute(pq_gather_kernel<12, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (12 * 256 + 256) * 4 * 4));
            IBCU_CUDA(ctx, cudaFuncSetAttribute(pq_gather_kernel<PQ_SMAX, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (PQ_SMAX * 256 + 256) * 4 * 4));
            attr_done[ctx->device & 63] = true;
        }
        rc = pl.S <= 12 ? ibcu_launch(ctx, pq_gather_kernel<12, 4>, grid, block, smem, 1, true, p)
                        : ibcu_launch(ctx, pq_gather_kernel<PQ_SMAX, 4>, grid, block, smem, 1, true, p);
    } else {
        rc = pl.S <= 12 ? ibcu_launch(ctx, pq_gather_kernel<12, 1>, grid, block, smem, 1, true, p)
                        : ibcu_launch(ctx, pq_gather_kernel<PQ_SMAX, 1>, grid, block, smem, 1, true, p);
    }
    if (rc) return rc;
    return ibcu_launch(ctx, pq_reduce_kernel, dim3((t->M + 31) / 32, B), dim3(256), 0, 1, true,
                       (const float*)scratch, pl.nslabs, t->M, t->M_pad, (const __half*)t->row_scale, out);
}

}  // namespace

extern "C" size_t ibcu_pq_idx_t_bytes(int M, int N, int G) {
    if (M <= 0 || N <= 0 || G <= 0 || N % G) return 0;
    size_t M_pad = ((size_t)M + 15) & ~(size_t)15;
    return 2 * (size_t)(N / G) * M_pad;
}

extern "C" int ibcu_pq_prepare(ibcu_ctx* ctx, ibcu_pq_t* t, uint8_t* idx_t_out) {
    IBCU_CHECK_CTX(ctx);
    IBCU_REQUIRE(ctx, t && idx_t_out && t->idx_l && t->idx_r, "ibcu_pq_prepare: null pointer");
    IBCU_REQUIRE(ctx, t->M > 0 && t->N > 0 && t->G > 0 && (t->G & 1) == 0 && t->N % t->G == 0, "ibcu_pq_prepare: bad shape M=%d N=%d G=%d", t->M, t->N, t->G);
    IBCU_REQUIRE(ctx, ((uintptr_t)idx_t_out & 15) == 0, "ibcu_pq_prepare: idx_t_out must be 16-byte aligned");
    const int C = t->N / t->G;
    const int M_pad = (t->M + 15) & ~15;
    dim3 grid((C + 63) / 64, (M_pad + 63) / 64, 2);
    int rc = ibcu_launch(ctx, pq_transpose_kernel, grid, dim3(256), 0, 1, false, t->idx_l, t->idx_r, t->M, C, M_pad, idx_t_out);
    if (rc) return rc;
    t->idx_t = idx_t_out;
    t->M_pad = M_pad;
    return IBCU_OK;
}

extern "C" int ibcu_pq_matmul_fp32(ibcu_ctx* ctx, const ibcu_pq_t* t, const float* x, float* out, int B) {
    IBCU_CHECK_CTX(ctx);
    IBCU_REQUIRE(ctx, t && x && out, "ibcu_pq_matmul_fp32: null pointer");
    IBCU_REQUIRE(ctx, t->codebook_l && t->codebook_r && t->row_scale, "ibcu_pq_matmul_fp32: tensor has a null pointer");
    IBCU_REQUIRE(ctx, t->idx_t && t->M_pad >= t->M, "ibcu_pq_matmul_fp32: call ibcu_pq_prepare on the tensor first");
    IBCU_REQUIRE(ctx, t->M > 0 && t->N > 0 && t->G > 0 && (t->G & 1) == 0 && t->G <= 32 && t->N % t->G == 0 && t->K >= 1 && t->K <= 256,
                 "ibcu_pq_matmul_fp32: bad shape M=%d N=%d G=%d K=%d", t->M, t->N, t->G, t->K);
    IBCU_REQUIRE(ctx, B >= 1 && B <= 32, "ibcu_pq_matmul_fp32: B=%d not in 1..32", B);
    const PqPlan pl = pq_plan(ctx, t, B);
    int rc = ibcu_reserve(ctx, &ctx->scratch, &ctx->scratch_bytes, pl.floats * sizeof(float));
    if (rc) return rc;
    return pq_launch(ctx, t, x, out, B, pl, (float*)ctx->scratch);
}

// ── PQ matvec without any allocation ────────────────────────────────────────────────────
// Some callers must not (or cannot) allocate device memory at call time: code that runs inside a
// latency-critical serving loop where cudaMalloc's implicit device synchronisation is unacceptable,
// plugins that are handed a fixed memory budget by their host application, and processes whose
// allocator is owned by another runtime. For them the slab partial sums and the per-activation
// maxima live in a fixed array that is part of the library image: every GPU that loads the library
// holds PQ_STATIC_FLOATS floats (4 MiB) from load until exit, whether or not this entry point is used.
constexpr size_t PQ_STATIC_FLOATS = (size_t)1 << 20;
static __device__ __align__(256) float pq_static_scratch[PQ_STATIC_FLOATS];

// In host code `pq_static_scratch` is only a handle for the runtime, not a device address; the
// address a kernel can use is looked up once per device, with that device current.
static float* pq_static_address(ibcu_ctx* ctx) {
    static float* per_device[64];
    if (ctx->device < 0 || ctx->device >= 64) return nullptr;
    if (!per_device[ctx->device]) {
        if (cudaSetDevice(ctx->device) != cudaSuccess) return nullptr;
        float* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress((void**)&p, pq_static_scratch);
        if (e != cudaSuccess) { ibcu_fail(ctx, IBCU_ERR_CUDA, "cudaGetSymbolAddress(pq_static_scratch) failed: %s", cudaGetErrorString(e)); return nullptr; }
        per_device[ctx->device] = p;
    }
    return per_device[ctx->device];
}

extern "C" size_t ibcu_pq_noalloc_max_floats(void) { return PQ_STATIC_FLOATS; }

extern "C" int ibcu_pq_matmul_fp32_noalloc(ibcu_ctx* ctx, const ibcu_pq_t* t, const float* x, float* out, int B) {
    IBCU_CHECK_CTX(ctx);
    IBCU_REQUIRE(ctx, t && x && out, "ibcu_pq_matmul_fp32_noalloc: null pointer");
    IBCU_REQUIRE(ctx, t->codebook_l && t->codebook_r && t->row_scale, "ibcu_pq_matmul_fp32_noalloc: tensor has a null pointer");
    IBCU_REQUIRE(ctx, t->idx_t && t->M_pad >= t->M, "ibcu_pq_matmul_fp32_noalloc: call ibcu_pq_prepare on the tensor first");
    IBCU_REQUIRE(ctx, t->M > 0 && t->N > 0 && t->G > 0 && (t->G & 1) == 0 && t->G <= 32 && t->N % t->G == 0 && t->K >= 1 && t->K <= 256,
                 "ibcu_pq_matmul_fp32_noalloc: bad shape M=%d N=%d G=%d K=%d", t->M, t->N, t->G, t->K);
    IBCU_REQUIRE(ctx, B >= 1 && B <= 32, "ibcu_pq_matmul_fp32_noalloc: B=%d not in 1..32", B);
    const PqPlan pl = pq_plan(ctx, t, B);
    if (pl.floats > PQ_STATIC_FLOATS)
        return ibcu_fail(ctx, IBCU_ERR_PARAM, "ibcu_pq_matmul_fp32_noalloc: this call needs %zu floats of scratch (%d activations x %d slabs x %d padded rows), "
                         "the built-in array holds %zu; use ibcu_pq_matmul_fp32", pl.floats, B, pl.nslabs, t->M_pad, PQ_STATIC_FLOATS);
    float* base = pq_static_address(ctx);
    if (!base) return ctx->status ? ctx->status : ibcu_fail(ctx, IBCU_ERR_CUDA, "ibcu_pq_matmul_fp32_noalloc: no address for the built-in scratch on device %d", ctx->device);
    // Nothing in the array has to start at zero: the gather kernel writes every partial sum that the
    // reduce kernel reads, before it reads them.
    return pq_launch(ctx, t, x, out, B, pl, base);
}
