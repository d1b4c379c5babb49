// The small FP32 kernels between the linear layers of a decode step: embedding dequant, RMSNorm with
// fp16 weights, RoPE on adjacent pairs + KV-cache write, GQA attention over an FP32 cache, SiLU-mul,
// residual add, softmax. They move O(hidden) or O(context) bytes per token; the design goal is few
// launches and programmatic-dependent-launch friendliness, not bandwidth.
#include "common.cuh"

namespace {

// BITS 8: INT8 rows; 4: two columns per byte, low nibble first, bias 8; 16: fp16 rows (scale unused)
template <int BITS>
__global__ void __launch_bounds__(256) embed_rows_kernel(const void* __restrict__ embed, const __half* __restrict__ scale,
                                                         const int32_t* __restrict__ tokens, float* __restrict__ x, int hidden) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.y;
    const int tok = __ldcg(tokens + b);             // past L1 and not as a read-only load: a kernel just ahead may have written it, and this one starts before that one ends
    const float s = BITS == 16 ? 1.0f : __half2float(scale[tok]);
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < hidden; i += gridDim.x * blockDim.x) {
        float v;
        if (BITS == 8) v = (float)reinterpret_cast<const int8_t*>(embed)[(size_t)tok * hidden + i] * s;
        else if (BITS == 16) v = __half2float(reinterpret_cast<const __half*>(embed)[(size_t)tok * hidden + i]);
        else {
            const uint8_t byte = reinterpret_cast<const uint8_t*>(embed)[(size_t)tok * (hidden / 2) + (i >> 1)];
            v = (float)((int)((i & 1) ? (byte >> 4) : (byte & 15)) - 8) * s;
        }
        x[(size_t)b * hidden + i] = v;
    }
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
// attn_partial_kernel: grid (kv heads, position chunks, B), one warp per query head of the group. A
// block owns one KV head, so the K and V rows it stages in shared memory serve all query heads of the
// group, and one chunk of cache positions. After the tile has landed the warps do not synchronise
// again: a warp walks the chunk 32 rows at a time (lane = row for the scores, lane = dimension for the
// weighted V sum) keeping a running max / sum / accumulator. Chunk results (max, sum, weighted sum) go to
// scratch rows of hd + 4 floats; attn_combine_kernel merges the chunks of a head with the usual
// max/sum rescaling.
// With k_new set the kernel is the whole attention step of a decode layer: q and k_new / v_new are
// the raw projections of positions pos0..pos0+B-1; the queries are rotated as they are loaded, tile
// rows of those positions are built from k_new / v_new (rotated) instead of being read from the cache,
// and the block whose own position is such a row also stores it in the cache. No block reads a cache
// row that another block of the same launch writes.
constexpr int ATT_GMAX = 8;          // query heads per KV head handled by the split path (warps per block)
constexpr int ATT_CHUNK = 128;       // most cache positions per block

// How `cap` cache positions are cut into chunks: chunks of at most chunk_cap positions, shorter ones
// (at least 32, a multiple of 4) when that still leaves `want` blocks to cover the machine.
__host__ __device__ __forceinline__ void att_plan(int cap, int want, int chunk_cap, int& chunk, int& nsplit) {
    chunk = chunk_cap;
    nsplit = (cap + chunk - 1) / chunk;
    if (nsplit < want) {
        chunk = (cap + want - 1) / want;
        if (chunk < 32) chunk = 32;
        chunk = (chunk + 3) & ~3;
        if (chunk > chunk_cap) chunk = chunk_cap;
        nsplit = (cap + chunk - 1) / chunk;
    }
}

__global__ void __launch_bounds__(32 * ATT_GMAX) attn_partial_kernel(const float* __restrict__ q, const float* __restrict__ k_cache,
                                                             const float* __restrict__ v_cache, float* __restrict__ part,
                                                             int n_heads, int n_kv, int hd, int pos0, int chunk, int nsplit,
                                                             const float* __restrict__ k_new, const float* __restrict__ v_new,
                                                             float* __restrict__ k_cache_w, float* __restrict__ v_cache_w, float theta,
                                                             const int* __restrict__ pos0_ptr, int want, int chunk_cap, const GatherWait gw) {
    extern __shared__ __align__(16) float asm_[];
    const int group = n_heads / n_kv;               // = warps in the block
    const int ld = hd + 4;                          // padded tile rows: conflict-free float4 reads down a column of rows
    float* qs = asm_;                               // [group][hd]
    float* ps = qs + group * hd;                    // [group][32]
    float* kt = ps + group * 32;                    // [chunk_cap][ld]
    float* vt = kt + (size_t)chunk_cap * ld;        // [chunk_cap][ld]
    pdl_launch_dependents();
    pdl_wait();
    gather_wait(gw);                                // q, k, v may be rows that peers pushed
    if (pos0_ptr) {                                 // position read on the device: the same launch serves every position
        pos0 = __ldcg(pos0_ptr);
        att_plan(pos0 + (int)gridDim.z, want, chunk_cap, chunk, nsplit);
    }
    const int kvh = blockIdx.x, sp = blockIdx.y, b = blockIdx.z, pos = pos0 + b;
    if (sp >= nsplit) return;                       // the grid is sized for the longest context
    const int kv_dim = n_kv * hd, tid = threadIdx.x, lane = tid & 31, g = tid >> 5, nth = blockDim.x;
    const int t0 = sp * chunk, t1 = min(pos + 1, t0 + chunk), n = max(0, t1 - t0);
    // the K and V rows of this chunk that the cache holds go in flight at once (one memory round trip)
    {
        const int per_row = hd / 4;
        const uint32_t kd = (uint32_t)__cvta_generic_to_shared(kt), vd = (uint32_t)__cvta_generic_to_shared(vt);
        const int n_old = k_new ? max(0, min(n, pos0 - t0)) : n;
        for (int e = tid; e < n_old * per_row; e += nth) {
            const int r = e / per_row, c = e - r * per_row;
            const size_t go = (size_t)(t0 + r) * kv_dim + (size_t)kvh * hd + 4 * c;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(kd + (r * ld + 4 * c) * 4), "l"(k_cache + go) : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(vd + (r * ld + 4 * c) * 4), "l"(v_cache + go) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    const float* qh = q + ((size_t)b * n_heads + (size_t)kvh * group + g) * hd;
    if (k_new) {
        const int half = hd / 2, r_first = max(t0, pos0);
        for (int m = lane; m < half; m += 32)
            rope_pair(qh[2 * m], qh[2 * m + 1], m, hd, pos, theta, qs[g * hd + 2 * m], qs[g * hd + 2 * m + 1]);
        for (int e = tid; e < (t1 - r_first) * half; e += nth) {       // this step's K rows: rotate, use, and store the block's own
            const int rr = e / half, m = e - rr * half, t = r_first + rr;
            const float* src = k_new + (size_t)(t - pos0) * kv_dim + (size_t)kvh * hd;
            float r0, r1;
            rope_pair(src[2 * m], src[2 * m + 1], m, hd, t, theta, r0, r1);
            kt[(size_t)(t - t0) * ld + 2 * m] = r0; kt[(size_t)(t - t0) * ld + 2 * m + 1] = r1;
            if (t == pos) { float* dst = k_cache_w + (size_t)t * kv_dim + (size_t)kvh * hd + 2 * m; dst[0] = r0; dst[1] = r1; }
        }
        for (int e = tid; e < (t1 - r_first) * hd; e += nth) {
            const int rr = e / hd, d = e - rr * hd, t = r_first + rr;
            const float vv = v_new[(size_t)(t - pos0) * kv_dim + (size_t)kvh * hd + d];
            vt[(size_t)(t - t0) * ld + d] = vv;
            if (t == pos) v_cache_w[(size_t)t * kv_dim + (size_t)kvh * hd + d] = vv;
        }
    } else {
        for (int d = lane; d < hd; d += 32) qs[g * hd + d] = qh[d];
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    const float scale = 1.0f / sqrtf((float)hd);
    const float4* q4 = reinterpret_cast<const float4*>(qs + g * hd);
    const int hd4 = hd / 4, ld4 = ld / 4;
    const float4* vt4 = reinterpret_cast<const float4*>(vt);
    float* pwarp = ps + g * 32;                      // this warp's weights of the current 32 rows
    float m_run = -INFINITY, l_run = 0.0f;
    float4 acc[2];                                   // lane owns dimensions 4*lane..4*lane+3 (and 128 + those when hd > 128)
    acc[0] = acc[1] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    const bool own0 = lane < hd4, own1 = lane + 32 < hd4;
    for (int r0 = 0; r0 < n; r0 += 32) {
        const int row = r0 + lane;
        float sc = -INFINITY;
        if (row < n) {
            const float4* kr = reinterpret_cast<const float4*>(kt + (size_t)row * ld);
            float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;           // four chains: the sum order is fixed, the latency a quarter
#pragma unroll 8
            for (int d4 = 0; d4 < hd4; d4++) {
                const float4 kk = kr[d4], qq = q4[d4];
                s0 = fmaf(qq.x, kk.x, s0); s1 = fmaf(qq.y, kk.y, s1); s2 = fmaf(qq.z, kk.z, s2); s3 = fmaf(qq.w, kk.w, s3);
            }
            sc = ((s0 + s1) + (s2 + s3)) * scale;
        }
        const float m_new = fmaxf(m_run, warp_max(sc));
        const float pw = row < n ? expf(sc - m_new) : 0.0f;
        const float corr = m_run == -INFINITY ? 0.0f : expf(m_run - m_new);
        l_run = l_run * corr + warp_sum(pw);
        m_run = m_new;
        __syncwarp();
        pwarp[lane] = pw;
        __syncwarp();
        acc[0].x *= corr; acc[0].y *= corr; acc[0].z *= corr; acc[0].w *= corr;
        acc[1].x *= corr; acc[1].y *= corr; acc[1].z *= corr; acc[1].w *= corr;
        const int cnt = min(32, n - r0);
        const float4* vrow = vt4 + (size_t)r0 * ld4 + lane;
#pragma unroll 8
        for (int t = 0; t < cnt; t++) {
            const float pt = pwarp[t];
            if (own0) { const float4 v = vrow[(size_t)t * ld4]; acc[0].x = fmaf(pt, v.x, acc[0].x); acc[0].y = fmaf(pt, v.y, acc[0].y); acc[0].z = fmaf(pt, v.z, acc[0].z); acc[0].w = fmaf(pt, v.w, acc[0].w); }
            if (own1) { const float4 v = vrow[(size_t)t * ld4 + 32]; acc[1].x = fmaf(pt, v.x, acc[1].x); acc[1].y = fmaf(pt, v.y, acc[1].y); acc[1].z = fmaf(pt, v.z, acc[1].z); acc[1].w = fmaf(pt, v.w, acc[1].w); }
        }
    }
    float* dst = part + (((size_t)b * n_heads + (size_t)kvh * group + g) * gridDim.y + sp) * (size_t)(hd + 4);
    if (own0) *reinterpret_cast<float4*>(dst + 4 + 4 * lane) = acc[0];
    if (own1) *reinterpret_cast<float4*>(dst + 4 + 4 * (lane + 32)) = acc[1];
    if (lane == 0) { dst[0] = m_run; dst[1] = l_run; }
}

// grid (query heads, B): merges the chunk results of one head. All of them are loaded at once, as float4s.
constexpr int ATT_CMB_V = 8;
__global__ void __launch_bounds__(128) attn_combine_kernel(const float* __restrict__ part, float* __restrict__ out,
                                                           int n_heads, int hd, int nsplit, int part_rows,
                                                           const int* __restrict__ pos0_ptr, int want, int chunk_cap) {
    extern __shared__ __align__(16) float cs[];      // the head's chunk results: [nsplit][hd + 4], then weights [nsplit]
    pdl_launch_dependents();
    pdl_wait();
    if (pos0_ptr) { int chunk; att_plan(__ldcg(pos0_ptr) + (int)gridDim.y, want, chunk_cap, chunk, nsplit); }
    const int h = blockIdx.x, b = blockIdx.y;
    const int pstride = hd + 4, total = nsplit * pstride, total4 = total / 4;
    const float4* src = reinterpret_cast<const float4*>(part + ((size_t)b * n_heads + h) * (size_t)part_rows * pstride);
    float4* cs4 = reinterpret_cast<float4*>(cs);
    float* wgt = cs + total;
    for (int e0 = 0; e0 < total4; e0 += ATT_CMB_V * 128) {
        float4 tmp[ATT_CMB_V];
#pragma unroll
        for (int u = 0; u < ATT_CMB_V; u++) { const int e = e0 + u * 128 + threadIdx.x; if (e < total4) tmp[u] = src[e]; }
#pragma unroll
        for (int u = 0; u < ATT_CMB_V; u++) { const int e = e0 + u * 128 + threadIdx.x; if (e < total4) cs4[e] = tmp[u]; }
    }
    __syncthreads();
    float M = -INFINITY;
    for (int s = 0; s < nsplit; s++) M = fmaxf(M, cs[s * pstride]);
    for (int s = threadIdx.x; s < nsplit; s += blockDim.x) wgt[s] = cs[s * pstride + 1] > 0.0f ? expf(cs[s * pstride] - M) : 0.0f;
    __syncthreads();
    float L = 0.0f;
    for (int s = 0; s < nsplit; s++) L = fmaf(cs[s * pstride + 1], wgt[s], L);
    const float inv = 1.0f / L;
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float a = 0.0f;
        for (int s = 0; s < nsplit; s++) a = fmaf(wgt[s], cs[s * pstride + 4 + d], a);
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

// grid (parts, B): silu(gate) * up over one column range of one row, and the largest magnitude written
__global__ void __launch_bounds__(256) silu_mul_amax_kernel(float* __restrict__ out, const float* __restrict__ gate, const float* __restrict__ up,
                                                            int N, int chunk, float* __restrict__ amax, const GatherWait gw) {
    __shared__ float red[32];
    pdl_launch_dependents();
    pdl_wait();
    gather_wait(gw);                                // gate and up may be rows that peers pushed
    const int p = blockIdx.x, b = blockIdx.y;
    const size_t base = (size_t)b * N;
    const int c1 = min(N, (p + 1) * chunk);
    float mx = 0.0f;
#pragma unroll 4
    for (int i = p * chunk + threadIdx.x; i < c1; i += blockDim.x) {
        const float g = gate[base + i];
        const float h = g / (1.0f + expf(-g)) * up[base + i];
        out[base + i] = h;
        mx = fmaxf(mx, fabsf(h));
    }
    mx = block_max(mx, red);
    if (threadIdx.x == 0) amax[(size_t)b * gridDim.x + p] = mx;
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

extern "C" int ibcu_embed_rows(ibcu_ctx* ctx, const void* embed, const uint16_t* scale, const int32_t* tokens,
                               float* x, int hidden, int B, int bits) {
    IBCU_CHECK_CTX(ctx);
    IBCU_REQUIRE(ctx, embed && tokens && x && hidden > 0 && B > 0, "ibcu_embed_rows: bad arguments");
    IBCU_REQUIRE(ctx, bits == 16 || (scale && (bits == 8 || (bits == 4 && (hidden & 1) == 0))), "ibcu_embed_rows: bits=%d (8 or 4 with row scales, or 16)", bits);
    int gx = (hidden + 255) / 256; if (gx > 16) gx = 16;
    const dim3 grid(gx, B), block(256);
    if (bits == 8) return ibcu_launch(ctx, embed_rows_kernel<8>, grid, block, 0, 1, true, embed, (const __half*)scale, tokens, x, hidden);
    if (bits == 4) return ibcu_launch(ctx, embed_rows_kernel<4>, grid, block, 0, 1, true, embed, (const __half*)scale, tokens, x, hidden);
    return ibcu_launch(ctx, embed_rows_kernel<16>, grid, block, 0, 1, true, embed, (const __half*)scale, tokens, x, hidden);
}
extern "C" int ibcu_embed_int8(ibcu_ctx* ctx, const int8_t* embed, const uint16_t* scale, const int32_t* tokens,
                               float* x, int hidden, int B) {
    return ibcu_embed_rows(ctx, embed, scale, tokens, x, hidden, B, 8);
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
// pos0_dev NULL: the position is the argument pos0 and the grid is cut for it. Otherwise the position is read
// on the device and the grid, shared memory and scratch are sized for max_ctx positions, so that one
// captured launch serves every position up to max_ctx - B.
static int attention_split(ibcu_ctx* ctx, const float* q, float* k_cache, float* v_cache, float* out,
                           int n_heads, int n_kv_heads, int head_dim, int pos0, int B, const float* k_new, const float* v_new, float theta,
                           const int* pos0_dev, int max_ctx) {
    const int group = n_heads / n_kv_heads;
    // Enough blocks to cover the machine several times over: a block's shared memory grows with its chunk of positions (two
    // tiles of chunk x head_dim floats), so short chunks let several blocks share an SM; with B activations every chunk
    // is staged by B blocks, which long chunks would serialise into waves of one block per SM. (One block serving all B
    // activations from one staged tile was measured slower: the activations then run one after the other in each warp.)
    int want = (6 * ctx->sm_count) / (n_kv_heads * B);
    if (want < 1) want = 1;
    int chunk, nsplit, grid_y, chunk_cap = ATT_CHUNK;
    if (pos0_dev) {
        int c_lo, n_lo;
        att_plan(B, want, ATT_CHUNK, c_lo, n_lo);              // shortest context
        att_plan(max_ctx, want, ATT_CHUNK, chunk, nsplit);     // longest context: most chunks, longest chunks
        grid_y = nsplit > n_lo ? nsplit : n_lo;
        if (want > grid_y) grid_y = want;
        chunk_cap = chunk;
        if (chunk_cap < 32) chunk_cap = 32;
    } else {
        att_plan(pos0 + B, want, ATT_CHUNK, chunk, nsplit);
        grid_y = nsplit;
        chunk_cap = chunk;
    }
    const size_t pbytes = (size_t)B * n_heads * grid_y * (head_dim + 4) * sizeof(float);
    int rc = ibcu_reserve(ctx, &ctx->scratch, &ctx->scratch_bytes, pbytes);
    if (rc) return rc;
    const size_t smem = ((size_t)group * head_dim + group * 32 + 2 * (size_t)chunk_cap * (head_dim + 4)) * sizeof(float);
    if (smem > 48 * 1024) IBCU_CUDA(ctx, cudaFuncSetAttribute(attn_partial_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    GatherWait gw;
    ibcu_take_gather_wait(ctx, &gw);
    rc = ibcu_launch(ctx, attn_partial_kernel, dim3(n_kv_heads, grid_y, B), dim3(32 * group), smem, 1, true,
                     q, (const float*)k_cache, (const float*)v_cache, (float*)ctx->scratch, n_heads, n_kv_heads, head_dim, pos0, chunk, nsplit,
                     k_new, v_new, k_cache, v_cache, theta, pos0_dev, want, chunk_cap, gw);
    if (rc) return rc;
    const size_t csmem = ((size_t)grid_y * (head_dim + 4) + grid_y) * sizeof(float);
    IBCU_REQUIRE(ctx, csmem <= 200 * 1024, "ibcu_attention: %d chunks of cache positions are more than the merge step holds", grid_y);
    if (csmem > 48 * 1024) IBCU_CUDA(ctx, cudaFuncSetAttribute(attn_combine_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)csmem));
    return ibcu_launch(ctx, attn_combine_kernel, dim3(n_heads, B), dim3(128), csmem, 1, true,
                       (const float*)ctx->scratch, out, n_heads, head_dim, nsplit, grid_y, pos0_dev, want, chunk_cap);
}

extern "C" int ibcu_attention(ibcu_ctx* ctx, const float* q, const float* k_cache, const float* v_cache, float* out,
                              int n_heads, int n_kv_heads, int head_dim, int pos0, int B) {
    IBCU_CHECK_CTX(ctx);
    IBCU_REQUIRE(ctx, q && k_cache && v_cache && out, "ibcu_attention: null pointer");
    IBCU_REQUIRE(ctx, n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0 && head_dim > 0 && pos0 >= 0 && B > 0,
                 "ibcu_attention: bad shape");
    if (attn_split_ok(q, k_cache, v_cache, n_heads, n_kv_heads, head_dim))
        return attention_split(ctx, q, (float*)k_cache, (float*)v_cache, out, n_heads, n_kv_heads, head_dim, pos0, B, nullptr, nullptr, 0.0f, nullptr, 0);
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
        return attention_split(ctx, q, k_cache, v_cache, out, n_heads, n_kv_heads, head_dim, pos0, B, k, v, theta, nullptr, 0);
    // shapes the split kernel does not take: the two steps one after the other
    int rc = ibcu_rope_kv_write(ctx, q, k, v, k_cache, v_cache, n_heads, n_kv_heads, head_dim, pos0, B, theta);
    if (rc) return rc;
    return ibcu_attention(ctx, q, k_cache, v_cache, out, n_heads, n_kv_heads, head_dim, pos0, B);
}

extern "C" int ibcu_attention_decode_at(ibcu_ctx* ctx, float* q, float* k, const float* v, float* k_cache, float* v_cache, float* out,
                                        int n_heads, int n_kv_heads, int head_dim, const int* pos0_dev, int max_ctx, int B, float theta) {
    IBCU_CHECK_CTX(ctx);
    IBCU_REQUIRE(ctx, q && k && v && k_cache && v_cache && out && pos0_dev, "ibcu_attention_decode_at: null pointer");
    IBCU_REQUIRE(ctx, n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0 && head_dim > 0 && (head_dim & 1) == 0 && B > 0 && max_ctx >= B,
                 "ibcu_attention_decode_at: bad shape heads=%d kv=%d hd=%d max_ctx=%d B=%d", n_heads, n_kv_heads, head_dim, max_ctx, B);
    IBCU_REQUIRE(ctx, attn_split_ok(q, k_cache, v_cache, n_heads, n_kv_heads, head_dim),
                 "ibcu_attention_decode_at: needs at most %d query heads per KV head, head_dim a multiple of 4 up to 256 and 16-byte aligned buffers", ATT_GMAX);
    return attention_split(ctx, q, k_cache, v_cache, out, n_heads, n_kv_heads, head_dim, 0, B, k, v, theta, pos0_dev, max_ctx);
}

extern "C" int ibcu_silu_mul_amax(ibcu_ctx* ctx, float* out, const float* gate, const float* up, int N, int B, float* amax, int parts) {
    IBCU_CHECK_CTX(ctx);
    IBCU_REQUIRE(ctx, out && gate && up && amax && N > 0 && B > 0 && parts > 0, "ibcu_silu_mul_amax: bad arguments");
    const int chunk = (N + parts - 1) / parts;
    GatherWait gw;
    ibcu_take_gather_wait(ctx, &gw);
    return ibcu_launch(ctx, silu_mul_amax_kernel, dim3(parts, B), dim3(256), 0, 1, true, out, gate, up, N, chunk, amax, gw);
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
