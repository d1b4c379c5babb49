// The small FP32 kernels between the linear layers of a decode step: embedding dequant, RMSNorm with
// fp16 weights, RoPE on adjacent pairs + KV-cache write, GQA attention over an FP32 cache, SiLU-mul,
// residual add, softmax. They move O(hidden) or O(context) bytes per token; the design goal is few
// launches and programmatic-dependent-launch friendliness, not bandwidth.
#include "common.cuh"

namespace {

__global__ void __launch_bounds__(256) embed_int8_kernel(const int8_t* __restrict__ embed, const __half* __restrict__ scale,
                                                         const int32_t* __restrict__ tokens, float* __restrict__ x, int hidden) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.y;
    const int tok = tokens[b];
    const float s = __half2float(scale[tok]);
    const int8_t* row = embed + (size_t)tok * hidden;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < hidden; i += gridDim.x * blockDim.x)
        x[(size_t)b * hidden + i] = (float)row[i] * s;
}

// block-wide sum, result broadcast to every thread; red must hold 32 floats
__device__ __forceinline__ float block_sum(float v, float* red) {
    v = warp_sum(v);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.0f;
    if (threadIdx.x < 32) { t = warp_sum(t); if (threadIdx.x == 0) red[0] = t; }
    __syncthreads();
    t = red[0];
    __syncthreads();
    return t;
}
__device__ __forceinline__ float block_max(float v, float* red) {
    v = warp_max(v);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : -INFINITY;
    if (threadIdx.x < 32) { t = warp_max(t); if (threadIdx.x == 0) red[0] = t; }
    __syncthreads();
    t = red[0];
    __syncthreads();
    return t;
}

template <typename WT>
__global__ void __launch_bounds__(1024) rmsnorm_kernel(float* __restrict__ out, const float* __restrict__ x,
                                                       const WT* __restrict__ w, float eps, int N) {
    __shared__ float red[32];
    pdl_launch_dependents();
    pdl_wait();
    const float* xb = x + (size_t)blockIdx.x * N;
    float* ob = out + (size_t)blockIdx.x * N;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < N; i += blockDim.x) ss = fmaf(xb[i], xb[i], ss);
    ss = block_sum(ss, red);
    const float r = 1.0f / sqrtf(ss / (float)N + eps);
    for (int i = threadIdx.x; i < N; i += blockDim.x) ob[i] = xb[i] * r * (float)w[i];
}

// One block per position b. Rotates every Q head and every K head (each K head once, as the
// reference does through the first Q head of its group), then stores K and V at cache row pos0+b.
__global__ void __launch_bounds__(256) rope_kv_write_kernel(float* __restrict__ q, float* __restrict__ k, const float* __restrict__ v,
                                                            float* __restrict__ k_cache, float* __restrict__ v_cache,
                                                            int n_heads, int n_kv, int hd, int pos0, float theta) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x, pos = pos0 + b, half = hd / 2;
    const int kv_dim = n_kv * hd;
    float* qb = q + (size_t)b * n_heads * hd;
    float* kb = k + (size_t)b * kv_dim;
    const float* vb = v + (size_t)b * kv_dim;
    const int total = (n_heads + n_kv) * half;
    for (int e = threadIdx.x; e < total; e += blockDim.x) {
        const int h = e / half, m = e - h * half;
        const float freq = 1.0f / powf(theta, (float)(2 * m) / (float)hd);
        const float ang = (float)pos * freq;
        const float c = cosf(ang), s = sinf(ang);
        float* p = h < n_heads ? qb + (size_t)h * hd + 2 * m : kb + (size_t)(h - n_heads) * hd + 2 * m;
        const float a0 = p[0], a1 = p[1];
        const float r0 = a0 * c - a1 * s, r1 = a0 * s + a1 * c;
        p[0] = r0; p[1] = r1;
        if (h >= n_heads && k_cache) {
            float* dst = k_cache + (size_t)pos * kv_dim + (size_t)(h - n_heads) * hd + 2 * m;
            dst[0] = r0; dst[1] = r1;
        }
    }
    if (v_cache && v) for (int e = threadIdx.x; e < kv_dim; e += blockDim.x) v_cache[(size_t)pos * kv_dim + e] = vb[e];
}

// One block per (query head, position b). Scores against cache rows 0..pos, max-subtracted softmax,
// weighted sum of V. Dynamic shared memory: pos_max+1 scores + 8*hd partial outputs.
__global__ void __launch_bounds__(256) attention_kernel(const float* __restrict__ q, const float* __restrict__ k_cache,
                                                        const float* __restrict__ v_cache, float* __restrict__ out,
                                                        int n_heads, int n_kv, int hd, int pos0, int score_cap) {
    extern __shared__ float sm[];
    __shared__ float red[32];
    float* sc = sm;                       // [score_cap]
    float* part = sm + score_cap;         // [8][hd]
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.x, b = blockIdx.y, pos = pos0 + b;
    const int kv_dim = n_kv * hd, kvh = h / (n_heads / n_kv);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    const float* qh = q + ((size_t)b * n_heads + h) * hd;
    const float scale = 1.0f / sqrtf((float)hd);
    for (int t = warp; t <= pos; t += nwarp) {
        const float* kt = k_cache + (size_t)t * kv_dim + (size_t)kvh * hd;
        float s = 0.0f;
        for (int d = lane; d < hd; d += 32) s = fmaf(qh[d], kt[d], s);
        s = warp_sum(s);
        if (lane == 0) sc[t] = s * scale;
    }
    __syncthreads();
    float mx = -INFINITY;
    for (int t = threadIdx.x; t <= pos; t += blockDim.x) mx = fmaxf(mx, sc[t]);
    mx = block_max(mx, red);
    float tot = 0.0f;
    for (int t = threadIdx.x; t <= pos; t += blockDim.x) { float e = expf(sc[t] - mx); sc[t] = e; tot += e; }
    tot = block_sum(tot, red);
    const float inv = 1.0f / tot;
    // each warp takes every nwarp-th position; lanes cover the head dimension
    for (int d = lane; d < hd; d += 32) {
        float a = 0.0f;
        for (int t = warp; t <= pos; t += nwarp)
            a = fmaf(sc[t] * inv, v_cache[(size_t)t * kv_dim + (size_t)kvh * hd + d], a);
        part[warp * hd + d] = a;
    }
    __syncthreads();
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float a = 0.0f;
        for (int w = 0; w < nwarp; w++) a += part[w * hd + d];
        out[((size_t)b * n_heads + h) * hd + d] = a;
    }
}

__global__ void __launch_bounds__(256) silu_mul_kernel(float* __restrict__ out, const float* __restrict__ gate,
                                                       const float* __restrict__ up, size_t n) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float g = gate[i];
        out[i] = g / (1.0f + expf(-g)) * up[i];
    }
}

__global__ void __launch_bounds__(256) add_inplace_kernel(float* __restrict__ x, const float* __restrict__ y, size_t n) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) x[i] += y[i];
}

__global__ void __launch_bounds__(256) softmax_rows_kernel(float* __restrict__ data, int N) {
    __shared__ float red[32];
    pdl_launch_dependents();
    pdl_wait();
    float* row = data + (size_t)blockIdx.x * N;
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < N; i += blockDim.x) mx = fmaxf(mx, row[i]);
    mx = block_max(mx, red);
    float tot = 0.0f;
    for (int i = threadIdx.x; i < N; i += blockDim.x) { float e = expf(row[i] - mx); row[i] = e; tot += e; }
    tot = block_sum(tot, red);
    const float inv = 1.0f / tot;
    for (int i = threadIdx.x; i < N; i += blockDim.x) row[i] *= inv;
}

int grid_for(ibcu_ctx* ctx, size_t n, int threads) {
    size_t g = (n + threads - 1) / threads;
    size_t cap = (size_t)ctx->sm_count * 8;
    return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace

extern "C" int ibcu_embed_int8(ibcu_ctx* ctx, const int8_t* embed, const uint16_t* scale, const int32_t* tokens,
                               float* x, int hidden, int B) {
    IBCU_CHECK_CTX(ctx);
    IBCU_REQUIRE(ctx, embed && scale && tokens && x && hidden > 0 && B > 0, "ibcu_embed_int8: bad arguments");
    int gx = (hidden + 255) / 256; if (gx > 16) gx = 16;
    return ibcu_launch(ctx, embed_int8_kernel, dim3(gx, B), dim3(256), 0, 1, true, embed, (const __half*)scale, tokens, x, hidden);
}

extern "C" int ibcu_rmsnorm_fp16w(ibcu_ctx* ctx, float* out, const float* x, const uint16_t* w, float eps, int N, int B) {
    IBCU_CHECK_CTX(ctx);
    IBCU_REQUIRE(ctx, out && x && w && N > 0 && B > 0, "ibcu_rmsnorm_fp16w: bad arguments");
    int threads = N >= 4096 ? 1024 : (N >= 1024 ? 512 : 128);
    return ibcu_launch(ctx, rmsnorm_kernel<__half>, dim3(B), dim3(threads), 0, 1, true, out, x, (const __half*)w, eps, N);
}

extern "C" int ibcu_rmsnorm_f32w(ibcu_ctx* ctx, float* out, const float* x, const float* w, float eps, int N, int B) {
    IBCU_CHECK_CTX(ctx);
    IBCU_REQUIRE(ctx, out && x && w && N > 0 && B > 0, "ibcu_rmsnorm_f32w: bad arguments");
    int threads = N >= 4096 ? 1024 : (N >= 1024 ? 512 : 128);
    return ibcu_launch(ctx, rmsnorm_kernel<float>, dim3(B), dim3(threads), 0, 1, true, out, x, w, eps, N);
}

extern "C" int ibcu_rope_kv_write(ibcu_ctx* ctx, float* q, float* k, const float* v, float* k_cache, float* v_cache,
                                  int n_heads, int n_kv_heads, int head_dim, int pos0, int B, float theta) {
    IBCU_CHECK_CTX(ctx);
    IBCU_REQUIRE(ctx, q && k, "ibcu_rope_kv_write: null pointer");
    IBCU_REQUIRE(ctx, n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0 && head_dim > 0 && (head_dim & 1) == 0 && pos0 >= 0 && B > 0,
                 "ibcu_rope_kv_write: bad shape heads=%d kv=%d hd=%d pos0=%d B=%d", n_heads, n_kv_heads, head_dim, pos0, B);
    return ibcu_launch(ctx, rope_kv_write_kernel, dim3(B), dim3(256), 0, 1, true, q, k, v, k_cache, v_cache,
                       n_heads, n_kv_heads, head_dim, pos0, theta);
}

extern "C" int ibcu_attention(ibcu_ctx* ctx, const float* q, const float* k_cache, const float* v_cache, float* out,
                              int n_heads, int n_kv_heads, int head_dim, int pos0, int B) {
    IBCU_CHECK_CTX(ctx);
    IBCU_REQUIRE(ctx, q && k_cache && v_cache && out, "ibcu_attention: null pointer");
    IBCU_REQUIRE(ctx, n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0 && head_dim > 0 && pos0 >= 0 && B > 0,
                 "ibcu_attention: bad shape");
    int cap = pos0 + B;
    size_t smem = ((size_t)cap + 8 * (size_t)head_dim) * sizeof(float);
    IBCU_REQUIRE(ctx, smem <= 200 * 1024, "ibcu_attention: context %d too long for one block's shared memory", cap);
    if (smem > 48 * 1024) IBCU_CUDA(ctx, cudaFuncSetAttribute(attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    return ibcu_launch(ctx, attention_kernel, dim3(n_heads, B), dim3(256), smem, 1, true, q, k_cache, v_cache, out,
                       n_heads, n_kv_heads, head_dim, pos0, cap);
}

extern "C" int ibcu_silu_mul(ibcu_ctx* ctx, float* out, const float* gate, const float* up, size_t n) {
    IBCU_CHECK_CTX(ctx);
    IBCU_REQUIRE(ctx, out && gate && up, "ibcu_silu_mul: null pointer");
    if (!n) return IBCU_OK;
    return ibcu_launch(ctx, silu_mul_kernel, dim3(grid_for(ctx, n, 256)), dim3(256), 0, 1, true, out, gate, up, n);
}

extern "C" int ibcu_add_inplace(ibcu_ctx* ctx, float* x, const float* y, size_t n) {
    IBCU_CHECK_CTX(ctx);
    IBCU_REQUIRE(ctx, x && y, "ibcu_add_inplace: null pointer");
    if (!n) return IBCU_OK;
    return ibcu_launch(ctx, add_inplace_kernel, dim3(grid_for(ctx, n, 256)), dim3(256), 0, 1, true, x, y, n);
}

extern "C" int ibcu_softmax(ibcu_ctx* ctx, float* data, int N, int rows) {
    IBCU_CHECK_CTX(ctx);
    IBCU_REQUIRE(ctx, data && N > 0 && rows > 0, "ibcu_softmax: bad arguments");
    return ibcu_launch(ctx, softmax_rows_kernel, dim3(rows), dim3(256), 0, 1, true, data, N);
}
