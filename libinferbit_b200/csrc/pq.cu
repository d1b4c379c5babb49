// Product-quantised matvec: out[r] = row_scale[r] * sum over subspaces s of LUT_s[code[r][s]],
// LUT_s[k] = codebook_s[k] . x_s (FP32), for 1..32 activations.
//
// Data in HBM: codebooks, row scales and the two row-major code planes exactly as the reference
// holds them, plus one derived array made once per tensor by ibcu_pq_prepare: the code planes
// transposed to subspace-major order idx_t[s][row] (s = 2*chunk + side). With it a block that owns a
// slab of subspaces reads long contiguous runs of codes (128-bit loads, every byte used) instead of a
// few bytes out of every row.
//
// pq_gather_kernel: grid = (slabs of S subspaces) x (blocks of rows). A block first puts its code
// loads in flight, then builds the slab's lookup table in shared memory straight from the fp16
// codebooks and the activation slice (dropping chunks under the reference's 1 %-of-max rule), then
// each thread walks 16 rows x S subspaces: one byte extract, one shared-memory read and one add per
// code. Partial row sums go to scratch [slab][row]; pq_reduce_kernel adds the slabs in slab order,
// applies the row scale and stores. No atomics, so results are run-to-run identical.
#include "common.cuh"

namespace {

constexpr int PQ_THREADS = 128;
constexpr int PQ_ROWS_PER_THREAD = 16;
constexpr int PQ_ROWS_PER_BLOCK = PQ_THREADS * PQ_ROWS_PER_THREAD;

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

// amax[b] = max |x[b]|
__global__ void __launch_bounds__(1024) pq_amax_kernel(const float* __restrict__ x, int N, float* __restrict__ amax) {
    __shared__ float red[32];
    pdl_launch_dependents();
    pdl_wait();
    const float* xb = x + (size_t)blockIdx.x * N;
    float m = 0.0f;
    for (int j = threadIdx.x; j < N; j += blockDim.x) m = fmaxf(m, fabsf(xb[j]));
    m = warp_max(m);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.0f;
        v = warp_max(v);
        if (threadIdx.x == 0) amax[blockIdx.x] = v;
    }
}

struct PqParams {
    int M, M_pad, N, G, K, C, S;          // S = subspaces per slab
    const __half* cb_l; const __half* cb_r; long cb_stride;
    const uint8_t* idx_t;
    const float* x;                        // this activation
    const float* amax;                     // its max |x|
    float* partial;                        // [nslabs][M_pad]
};

__global__ void __launch_bounds__(PQ_THREADS) pq_gather_kernel(const PqParams p) {
    extern __shared__ __align__(16) float lut[];          // [S][K]
    __shared__ float xs[32 * 16];                          // activation slice of the slab, S * G/2 <= 512
    __shared__ unsigned char live[32];
    pdl_launch_dependents();
    const int half = p.G >> 1;
    const int s0 = blockIdx.x * p.S;
    const int ns = min(p.S, 2 * p.C - s0);
    const int row = blockIdx.y * PQ_ROWS_PER_BLOCK + threadIdx.x * PQ_ROWS_PER_THREAD;
    const bool has_rows = row < p.M_pad;

    // codes of the first subspaces go in flight before anything else (they do not depend on x)
    constexpr int PF = 4;
    uint4 pre[PF];
#pragma unroll
    for (int i = 0; i < PF; i++)
        pre[i] = (has_rows && i < ns) ? ld_stream_u4(p.idx_t + (size_t)(s0 + i) * p.M_pad + row) : make_uint4(0, 0, 0, 0);

    pdl_wait();
    // activation slice + live flags
    for (int e = threadIdx.x; e < ns * half; e += PQ_THREADS) {
        const int sl = e / half, i = e - sl * half, s = s0 + sl;
        xs[e] = p.x[(size_t)(s >> 1) * p.G + (s & 1) * half + i];
    }
    if (threadIdx.x < ns) {
        const int c = (s0 + threadIdx.x) >> 1;
        const float am = *p.amax;
        bool keep = true;
        if (am > 0.0f) {
            const float thr = am * 0.01f;
            float cm = 0.0f;
            for (int i = 0; i < p.G; i++) cm = fmaxf(cm, fabsf(p.x[(size_t)c * p.G + i]));
            keep = cm >= thr;
        }
        live[threadIdx.x] = keep;
    }
    __syncthreads();
    // lookup table of the slab
    for (int e = threadIdx.x; e < ns * p.K; e += PQ_THREADS) {
        const int sl = e / p.K, k = e - sl * p.K, s = s0 + sl;
        const __half* ent = ((s & 1) ? p.cb_r : p.cb_l) + (size_t)(s >> 1) * p.cb_stride + (size_t)k * half;
        float acc = 0.0f;
        if (live[sl]) for (int i = 0; i < half; i++) acc = fmaf(__half2float(ent[i]), xs[sl * half + i], acc);
        lut[sl * p.K + k] = acc;
    }
    __syncthreads();
    if (!has_rows) return;

    float acc[PQ_ROWS_PER_THREAD];
#pragma unroll
    for (int r = 0; r < PQ_ROWS_PER_THREAD; r++) acc[r] = 0.0f;
    for (int sl = 0; sl < ns; sl += PF) {
        uint4 cur[PF];
#pragma unroll
        for (int i = 0; i < PF; i++) cur[i] = pre[i];
#pragma unroll
        for (int i = 0; i < PF; i++) {
            const int nx = sl + PF + i;
            pre[i] = nx < ns ? ld_stream_u4(p.idx_t + (size_t)(s0 + nx) * p.M_pad + row) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int i = 0; i < PF; i++) {
            if (sl + i >= ns) break;
            const float* T = lut + (size_t)(sl + i) * p.K;
            const uint32_t w[4] = { cur[i].x, cur[i].y, cur[i].z, cur[i].w };
#pragma unroll
            for (int q = 0; q < 4; q++) {
                acc[4 * q + 0] += T[w[q] & 0xFF];
                acc[4 * q + 1] += T[(w[q] >> 8) & 0xFF];
                acc[4 * q + 2] += T[(w[q] >> 16) & 0xFF];
                acc[4 * q + 3] += T[w[q] >> 24];
            }
        }
    }
    float* dst = p.partial + (size_t)blockIdx.x * p.M_pad + row;
#pragma unroll
    for (int q = 0; q < 4; q++)
        *reinterpret_cast<float4*>(dst + 4 * q) = make_float4(acc[4 * q], acc[4 * q + 1], acc[4 * q + 2], acc[4 * q + 3]);
}

__global__ void __launch_bounds__(256) pq_reduce_kernel(const float* __restrict__ partial, int nslabs, int M, int M_pad,
                                                        const __half* __restrict__ row_scale, float* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= M) return;
    float s = 0.0f;
    for (int b = 0; b < nslabs; b++) s += partial[(size_t)b * M_pad + r];
    out[r] = s * __half2float(row_scale[r]);
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
    const int C = t->N / t->G, nsub = 2 * C;
    const int row_blocks = (t->M_pad + PQ_ROWS_PER_BLOCK - 1) / PQ_ROWS_PER_BLOCK;
    // slab size: about two blocks per SM, at most 32 subspaces (32 KB of table at K = 256)
    int S = (int)(((long)nsub * row_blocks + 2L * ctx->sm_count - 1) / (2L * ctx->sm_count));
    if (S < 4) S = 4;
    if (S > 32) S = 32;
    S = (S + 3) & ~3;
    const int nslabs = (nsub + S - 1) / S;
    size_t need = (size_t)nslabs * t->M_pad * sizeof(float) + 32 * sizeof(float);
    int rc = ibcu_reserve(ctx, &ctx->scratch, &ctx->scratch_bytes, need);
    if (rc) return rc;
    float* amax = (float*)ctx->scratch;
    float* partial = amax + 32;
    int threads = t->N >= 4096 ? 1024 : 256;
    rc = ibcu_launch(ctx, pq_amax_kernel, dim3(B), dim3(threads), 0, 1, true, x, t->N, amax);
    if (rc) return rc;
    const size_t smem = ((size_t)S * t->K + 256) * sizeof(float);   // + slack: a code >= K must not leave the allocation
    for (int b = 0; b < B; b++) {
        PqParams p;
        p.M = t->M; p.M_pad = t->M_pad; p.N = t->N; p.G = t->G; p.K = t->K; p.C = C; p.S = S;
        p.cb_l = (const __half*)t->codebook_l; p.cb_r = (const __half*)t->codebook_r; p.cb_stride = t->cb_chunk_stride;
        p.idx_t = t->idx_t; p.x = x + (size_t)b * t->N; p.amax = amax + b; p.partial = partial;
        rc = ibcu_launch(ctx, pq_gather_kernel, dim3(nslabs, row_blocks), dim3(PQ_THREADS), smem, 1, true, p);
        if (rc) return rc;
        rc = ibcu_launch(ctx, pq_reduce_kernel, dim3((t->M + 255) / 256), dim3(256), 0, 1, true,
                         (const float*)partial, nslabs, t->M, t->M_pad, (const __half*)t->row_scale, out + (size_t)b * t->M);
        if (rc) return rc;
    }
    return IBCU_OK;
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
    const int C = t->N / t->G, nsub = 2 * C;
    const int row_blocks = (t->M_pad + PQ_ROWS_PER_BLOCK - 1) / PQ_ROWS_PER_BLOCK;
    int S = (int)(((long)nsub * row_blocks + 2L * ctx->sm_count - 1) / (2L * ctx->sm_count));
    if (S < 4) S = 4;
    if (S > 32) S = 32;
    S = (S + 3) & ~3;
    const int nslabs = (nsub + S - 1) / S;
    const size_t need = (size_t)nslabs * t->M_pad + 32;
    if (need > PQ_STATIC_FLOATS)
        return ibcu_fail(ctx, IBCU_ERR_PARAM, "ibcu_pq_matmul_fp32_noalloc: this tensor needs %zu floats of scratch (%d slabs x %d padded rows + 32), "
                         "the built-in array holds %zu; use ibcu_pq_matmul_fp32", need, nslabs, t->M_pad, PQ_STATIC_FLOATS);
    float* base = pq_static_address(ctx);
    if (!base) return ctx->status ? ctx->status : ibcu_fail(ctx, IBCU_ERR_CUDA, "ibcu_pq_matmul_fp32_noalloc: no address for the built-in scratch on device %d", ctx->device);
    // Nothing in the array has to start at zero: the maxima kernel writes amax[0..B) and the gather
    // kernel writes every partial sum the reduce kernel reads, before it reads them.
    float* amax = base;
    float* partial = base + 32;
    int threads = t->N >= 4096 ? 1024 : 256;
    int rc = ibcu_launch(ctx, pq_amax_kernel, dim3(B), dim3(threads), 0, 1, true, x, t->N, amax);
    if (rc) return rc;
    const size_t smem = ((size_t)S * t->K + 256) * sizeof(float);
    for (int b = 0; b < B; b++) {
        PqParams p;
        p.M = t->M; p.M_pad = t->M_pad; p.N = t->N; p.G = t->G; p.K = t->K; p.C = C; p.S = S;
        p.cb_l = (const __half*)t->codebook_l; p.cb_r = (const __half*)t->codebook_r; p.cb_stride = t->cb_chunk_stride;
        p.idx_t = t->idx_t; p.x = x + (size_t)b * t->N; p.amax = amax + b; p.partial = partial;
        rc = ibcu_launch(ctx, pq_gather_kernel, dim3(nslabs, row_blocks), dim3(PQ_THREADS), smem, 1, true, p);
        if (rc) return rc;
        rc = ibcu_launch(ctx, pq_reduce_kernel, dim3((t->M + 255) / 256), dim3(256), 0, 1, true,
                         (const float*)partial, nslabs, t->M, t->M_pad, (const __half*)t->row_scale, out + (size_t)b * t->M);
        if (rc) return rc;
    }
    return IBCU_OK;
}
