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

// Rotation of pair m of a head at position pos (src/kernels/scalar.c:140-157).
__device__ __forceinline__ void rope_pair(float a0, float a1, int m, int hd, int pos, float theta, float& r0, float& r1) {
    const float freq = 1.0f / powf(theta, (float)(2 * m) / (float)hd);
    const float ang = (float)pos * freq;
    const float c = cosf(ang), s = sinf(ang);
    r0 = a0 * c - a1 * s; r1 = a0 * s + a1 * c;
}

// grid (Q heads + K heads, B): one block per head and position, one thread per rotated pair. Each K
// head is rotated once (the reference does it through the first Q head of its group) and stored,
// with its V row, at cache row pos0 + b.
__global__ void __launch_bounds__(128) rope_kv_write_kernel(float* __restrict__ q, float* __restrict__ k, const float* __restrict__ v,
                                                            float* __restrict__ k_cache, float* __restrict__ v_cache,
                                                            int n_heads, int n_kv, int hd, int pos0, float theta) {
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.x, b = blockIdx.y, pos = pos0 + b, half = hd / 2;
    const int kv_dim = n_kv * hd;
    const bool is_k = h >= n_heads;
    float* p = is_k ? k + (size_t)b * kv_dim + (size_t)(h - n_heads) * hd : q + (size_t)b * n_heads * hd + (size_t)h * hd;
    for (int m = threadIdx.x; m < half; m += blockDim.x) {
        float r0, r1;
        rope_pair(p[2 * m], p[2 * m + 1], m, hd, pos, theta, r0, r1);
        p[2 * m] = r0; p[2 * m + 1] = r1;
        if (is_k && k_cache) {
            float* dst = k_cache + (size_t)pos * kv_dim + (size_t)(h - n_heads) * hd + 2 * m;
            dst[0] = r0; dst[1] = r1;
        }
    }
    if (is_k && v_cache && v) {
        const float* vb = v + (size_t)b * kv_dim + (size_t)(h - n_heads) * hd;
        float* dst = v_cache + (size_t)pos * kv_dim + (size_t)(h - n_heads) * hd;
        for (int e = threadIdx.x; e < hd; e += blockDim.x) dst[e] = vb[e];
    }
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

// ── split attention for decode ──────────────────────────────────────────────────────────
// attn_partial_kernel: grid (kv heads, position chunks, B). A block owns one KV head, so the K and V
// rows it reads serve all query heads of the group, and one chunk of cache positions. Thread t of the
// block scores position t of the chunk for every query head of the group (K row read as float4s, the
// query heads broadcast from shared memory), the block forms the chunk-local softmax weights, then
// thread d accumulates dimension d of the weighted V sum. Chunk results (max, sum, weighted sum) go to
// scratch; attn_combine_kernel merges the chunks of a head with the usual max/sum rescaling.
// With k_new set the kernel is the whole attention step of a decode layer: q and k_new / v_new are
// the raw projections of positions pos0..pos0+B-1; the queries are rotated as they are loaded, tile
// rows of those positions are built from k_new / v_new (rotated) instead of being read from the cache,
// and the block whose own position is such a row also stores it in the cache. No block reads a cache
// row that another block of the same launch writes.
constexpr int ATT_GMAX = 8;          // query heads per KV head handled by the split path
constexpr int ATT_T = 128;           // threads = positions per chunk

__global__ void __launch_bounds__(ATT_T) attn_partial_kernel(const float* __restrict__ q, const float* __restrict__ k_cache,
                                                             const float* __restrict__ v_cache, float* __restrict__ part,
                                                             int n_heads, int n_kv, int hd, int pos0, int chunk, int nsplit,
                                                             const float* __restrict__ k_new, const float* __restrict__ v_new,
                                                             float* __restrict__ k_cache_w, float* __restrict__ v_cache_w, float theta) {
    extern __shared__ __align__(16) float asm_[];
    const int group = n_heads / n_kv;
    const int ld = hd + 4;                          // padded tile rows: conflict-free float4 reads down a column of rows
    float* qs = asm_;                               // [group][hd]
    float* ps = qs + group * hd;                    // [group][ATT_T] scores, then weights
    float* red = ps + group * ATT_T;                // [group][4]
    float* kt = red + group * 4;                    // [chunk][ld]
    float* vt = kt + (size_t)chunk * ld;            // [chunk][ld]
    pdl_launch_dependents();
    pdl_wait();
    const int kvh = blockIdx.x, sp = blockIdx.y, b = blockIdx.z, pos = pos0 + b;
    const int kv_dim = n_kv * hd, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int t0 = sp * chunk, t1 = min(pos + 1, t0 + chunk), n = max(0, t1 - t0);
    // the whole K and V tile of this chunk goes in flight at once (one memory round trip)
    {
        const int per_row = hd / 4;
        const uint32_t kd = (uint32_t)__cvta_generic_to_shared(kt), vd = (uint32_t)__cvta_generic_to_shared(vt);
        const int n_old = k_new ? max(0, min(n, pos0 - t0)) : n;      // rows that are in the cache already
        for (int e = tid; e < n_old * per_row; e += ATT_T) {
            const int r = e / per_row, c = e - r * per_row;
            const size_t g = (size_t)(t0 + r) * kv_dim + (size_t)kvh * hd + 4 * c;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(kd + (r * ld + 4 * c) * 4), "l"(k_cache + g) : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(vd + (r * ld + 4 * c) * 4), "l"(v_cache + g) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    if (k_new) {
        const int half = hd / 2, r_first = max(t0, pos0);
        for (int e = tid; e < group * half; e += ATT_T) {
            const int g = e / half, m = e - g * half;
            const float* src = q + ((size_t)b * n_heads + (size_t)kvh * group + g) * hd;
            rope_pair(src[2 * m], src[2 * m + 1], m, hd, pos, theta, qs[g * hd + 2 * m], qs[g * hd + 2 * m + 1]);
        }
        for (int e = tid; e < (t1 - r_first) * half; e += ATT_T) {     // this step's K rows: rotate, use, and store the block's own
            const int rr = e / half, m = e - rr * half, t = r_first + rr;
            const float* src = k_new + (size_t)(t - pos0) * kv_dim + (size_t)kvh * hd;
            float r0, r1;
            rope_pair(src[2 * m], src[2 * m + 1], m, hd, t, theta, r0, r1);
            kt[(size_t)(t - t0) * ld + 2 * m] = r0; kt[(size_t)(t - t0) * ld + 2 * m + 1] = r1;
            if (t == pos) { float* dst = k_cache_w + (size_t)t * kv_dim + (size_t)kvh * hd + 2 * m; dst[0] = r0; dst[1] = r1; }
        }
        for (int e = tid; e < (t1 - r_first) * hd; e += ATT_T) {
            const int rr = e / hd, d = e - rr * hd, t = r_first + rr;
            const float vv = v_new[(size_t)(t - pos0) * kv_dim + (size_t)kvh * hd + d];
            vt[(size_t)(t - t0) * ld + d] = vv;
            if (t == pos) v_cache_w[(size_t)t * kv_dim + (size_t)kvh * hd + d] = vv;
        }
    } else {
        for (int e = tid; e < group * hd; e += ATT_T) qs[e] = q[((size_t)b * n_heads + (size_t)kvh * group) * hd + e];
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    const float scale = 1.0f / sqrtf((float)hd);
    float sc[ATT_GMAX];
#pragma unroll
    for (int g = 0; g < ATT_GMAX; g++) sc[g] = 0.0f;
    if (tid < n) {
        const float4* kr = reinterpret_cast<const float4*>(kt + (size_t)tid * ld);
        for (int d4 = 0; d4 < hd / 4; d4++) {
            const float4 kk = kr[d4];
#pragma unroll
            for (int g = 0; g < ATT_GMAX; g++) {
                if (g >= group) break;
                const float4 qq = *reinterpret_cast<const float4*>(qs + g * hd + 4 * d4);
                sc[g] = fmaf(qq.x, kk.x, fmaf(qq.y, kk.y, fmaf(qq.z, kk.z, fmaf(qq.w, kk.w, sc[g]))));
            }
        }
    }
    // chunk-local max and sum per query head
    float mloc[ATT_GMAX], lloc[ATT_GMAX];
#pragma unroll
    for (int g = 0; g < ATT_GMAX; g++) {
        if (g >= group) break;
        float v = tid < n ? sc[g] * scale : -INFINITY;
        sc[g] = v;
        v = warp_max(v);
        if (lane == 0) red[g * 4 + warp] = v;
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < ATT_GMAX; g++) {
        if (g >= group) break;
        mloc[g] = fmaxf(fmaxf(red[g * 4], red[g * 4 + 1]), fmaxf(red[g * 4 + 2], red[g * 4 + 3]));
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < ATT_GMAX; g++) {
        if (g >= group) break;
        const float pw = tid < n ? expf(sc[g] - mloc[g]) : 0.0f;
        ps[g * ATT_T + tid] = pw;
        const float v = warp_sum(pw);
        if (lane == 0) red[g * 4 + warp] = v;
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < ATT_GMAX; g++) {
        if (g >= group) break;
        lloc[g] = red[g * 4] + red[g * 4 + 1] + red[g * 4 + 2] + red[g * 4 + 3];
    }
    // weighted V sum: thread d owns dimension d (and d + 128, ...)
    const size_t pstride = (size_t)hd + 2;          // per (b, head, split): m, l, acc[hd]
    for (int d = tid; d < hd; d += ATT_T) {
        float acc[ATT_GMAX];
#pragma unroll
        for (int g = 0; g < ATT_GMAX; g++) acc[g] = 0.0f;
#pragma unroll 4
        for (int t = 0; t < n; t++) {
            const float vv = vt[(size_t)t * ld + d];
#pragma unroll
            for (int g = 0; g < ATT_GMAX; g++) { if (g >= group) break; acc[g] = fmaf(ps[g * ATT_T + t], vv, acc[g]); }
        }
#pragma unroll
        for (int g = 0; g < ATT_GMAX; g++) {
            if (g >= group) break;
            part[(((size_t)b * n_heads + (size_t)kvh * group + g) * nsplit + sp) * pstride + 2 + d] = acc[g];
        }
    }
    if (tid < group) {
        float* dst = part + (((size_t)b * n_heads + (size_t)kvh * group + tid) * nsplit + sp) * pstride;
        dst[0] = n > 0 ? mloc[tid] : -INFINITY;
        dst[1] = n > 0 ? lloc[tid] : 0.0f;
    }
}

__global__ void __launch_bounds__(128) attn_combine_kernel(const float* __restrict__ part, float* __restrict__ out,
                                                           int n_heads, int hd, int nsplit) {
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.x, b = blockIdx.y;
    const size_t pstride = (size_t)hd + 2;
    const float* src = part + ((size_t)b * n_heads + h) * nsplit * pstride;
    float M = -INFINITY;
    for (int s = 0; s < nsplit; s++) M = fmaxf(M, src[s * pstride]);
    float L = 0.0f;
    for (int s = 0; s < nsplit; s++) L += src[s * pstride + 1] * expf(src[s * pstride] - M);
    const float inv = 1.0f / L;
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float a = 0.0f;
        for (int s = 0; s < nsplit; s++) {
            const float w = src[s * pstride + 1] > 0.0f ? expf(src[s * pstride] - M) : 0.0f;
            a = fmaf(w, src[s * pstride + 2 + d], a);
        }
        out[((size_t)b * n_heads + h) * hd + d] = a * inv;
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
    const int threads = head_dim / 2 >= 128 ? 128 : (head_dim / 2 >= 64 ? 64 : 32);
    return ibcu_launch(ctx, rope_kv_write_kernel, dim3(n_heads + n_kv_heads, B), dim3(threads), 0, 1, true, q, k, v, k_cache, v_cache,
                       n_heads, n_kv_heads, head_dim, pos0, theta);
}

static bool attn_split_ok(const float* q, const float* k_cache, const float* v_cache, int n_heads, int n_kv_heads, int head_dim) {
    return n_heads / n_kv_heads <= ATT_GMAX && head_dim % 4 == 0 && head_dim <= 256 &&
           ((uintptr_t)k_cache & 15) == 0 && ((uintptr_t)v_cache & 15) == 0 && ((uintptr_t)q & 15) == 0;
}

// k_new / v_new NULL: q is rotated already and the cache holds rows 0..pos0+B-1. Otherwise the fused decode step.
static int attention_split(ibcu_ctx* ctx, const float* q, float* k_cache, float* v_cache, float* out,
                           int n_heads, int n_kv_heads, int head_dim, int pos0, int B, const float* k_new, const float* v_new, float theta) {
    const int group = n_heads / n_kv_heads;
    {
        // split path: chunks of up to 128 cache positions per block, merged by a second small kernel
        const int cap = pos0 + B;
        int nsplit = (cap + ATT_T - 1) / ATT_T;
        const int want = (2 * ctx->sm_count) / (n_kv_heads * B);      // enough blocks to cover the machine
        int chunk = ATT_T;
        if (nsplit < want) { chunk = (cap + want - 1) / want; if (chunk < 32) chunk = 32; chunk = (chunk + 3) & ~3; nsplit = (cap + chunk - 1) / chunk; }
        const size_t pbytes = (size_t)B * n_heads * nsplit * (head_dim + 2) * sizeof(float);
        int rc = ibcu_reserve(ctx, &ctx->scratch, &ctx->scratch_bytes, pbytes);
        if (rc) return rc;
        const size_t smem = ((size_t)group * head_dim + (size_t)group * ATT_T + group * 4 + 2 * (size_t)chunk * (head_dim + 4)) * sizeof(float);
        if (smem > 48 * 1024) IBCU_CUDA(ctx, cudaFuncSetAttribute(attn_partial_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        rc = ibcu_launch(ctx, attn_partial_kernel, dim3(n_kv_heads, nsplit, B), dim3(ATT_T), smem, 1, true,
                         q, (const float*)k_cache, (const float*)v_cache, (float*)ctx->scratch, n_heads, n_kv_heads, head_dim, pos0, chunk, nsplit,
                         k_new, v_new, k_cache, v_cache, theta);
        if (rc) return rc;
        return ibcu_launch(ctx, attn_combine_kernel, dim3(n_heads, B), dim3(128), 0, 1, true,
                           (const float*)ctx->scratch, out, n_heads, head_dim, nsplit);
    }
}

extern "C" int ibcu_attention(ibcu_ctx* ctx, const float* q, const float* k_cache, const float* v_cache, float* out,
                              int n_heads, int n_kv_heads, int head_dim, int pos0, int B) {
    IBCU_CHECK_CTX(ctx);
    IBCU_REQUIRE(ctx, q && k_cache && v_cache && out, "ibcu_attention: null pointer");
    IBCU_REQUIRE(ctx, n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0 && head_dim > 0 && pos0 >= 0 && B > 0,
                 "ibcu_attention: bad shape");
    if (attn_split_ok(q, k_cache, v_cache, n_heads, n_kv_heads, head_dim))
        return attention_split(ctx, q, (float*)k_cache, (float*)v_cache, out, n_heads, n_kv_heads, head_dim, pos0, B, nullptr, nullptr, 0.0f);
    int cap = pos0 + B;
    size_t smem = ((size_t)cap + 8 * (size_t)head_dim) * sizeof(float);
    IBCU_REQUIRE(ctx, smem <= 200 * 1024, "ibcu_attention: context %d too long for one block's shared memory", cap);
    if (smem > 48 * 1024) IBCU_CUDA(ctx, cudaFuncSetAttribute(attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    return ibcu_launch(ctx, attention_kernel, dim3(n_heads, B), dim3(256), smem, 1, true, q, k_cache, v_cache, out,
                       n_heads, n_kv_heads, head_dim, pos0, cap);
}

extern "C" int ibcu_attention_decode(ibcu_ctx* ctx, float* q, float* k, const float* v, float* k_cache, float* v_cache, float* out,
                                     int n_heads, int n_kv_heads, int head_dim, int pos0, int B, float theta) {
    IBCU_CHECK_CTX(ctx);
    IBCU_REQUIRE(ctx, q && k && v && k_cache && v_cache && out, "ibcu_attention_decode: null pointer");
    IBCU_REQUIRE(ctx, n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0 && head_dim > 0 && (head_dim & 1) == 0 && pos0 >= 0 && B > 0,
                 "ibcu_attention_decode: bad shape heads=%d kv=%d hd=%d pos0=%d B=%d", n_heads, n_kv_heads, head_dim, pos0, B);
    if (attn_split_ok(q, k_cache, v_cache, n_heads, n_kv_heads, head_dim))
        return attention_split(ctx, q, k_cache, v_cache, out, n_heads, n_kv_heads, head_dim, pos0, B, k, v, theta);
    // shapes the split kernel does not take: the two steps one after the other
    int rc = ibcu_rope_kv_write(ctx, q, k, v, k_cache, v_cache, n_heads, n_kv_heads, head_dim, pos0, B, theta);
    if (rc) return rc;
    return ibcu_attention(ctx, q, k_cache, v_cache, out, n_heads, n_kv_heads, head_dim, pos0, B);
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
