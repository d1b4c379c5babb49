// PQ-compressed KV cache, the encode step of one vector (src/pq_decode.c:5008-5066, inside the session's decode step):
// scale = max|v| / 7 (at least 1e-12), the vector divided by it, and for every chunk of G values the nearest entry of
// the left codebook to its first half and of the right codebook to its second half: squared distance accumulated in
// dimension order, strict '<' (the first of equal entries wins). The codes of a vector are stored as [C left | C right].
// This is the second consumer of the nearest-centroid search next to the k-means assignment; the search space is K1
// entries of G/2 values per half chunk.
#include "common.cuh"

namespace {

// grid (2 C, vectors): block (h, v) encodes half chunk h of vector v; thread k holds codebook entry k.
__global__ void __launch_bounds__(256) pqkv_encode_kernel(const float* __restrict__ vec, int dim, int G, int C, int K1,
                                                          const __half* __restrict__ cb_l, const __half* __restrict__ cb_r,
                                                          uint8_t* __restrict__ idx, float* __restrict__ scale_out) {
    __shared__ float red[8];
    __shared__ float xs[16];
    __shared__ float best_d[8];
    __shared__ int best_k[8];
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.x, v = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int half = G / 2, c = h < C ? h : h - C, side = h < C ? 0 : 1;
    const float* x = vec + (size_t)v * dim;
    float m = 1e-12f;                                         // the reference starts its maximum there
    for (int j = tid; j < dim; j += 256) m = fmaxf(m, fabsf(x[j]));
    m = warp_max(m);
    if (lane == 0) red[warp] = m;
    __syncthreads();
    m = red[0];
#pragma unroll
    for (int w = 1; w < 8; w++) m = fmaxf(m, red[w]);
    float s = __fdiv_rn(m, 7.0f);
    if (s < 1e-12f) s = 1e-12f;
    const float inv = __fdiv_rn(1.0f, s);
    if (tid < half) xs[tid] = __fmul_rn(x[c * G + side * half + tid], inv);
    if (h == 0 && tid == 0) scale_out[v] = s;
    __syncthreads();
    float d = 3.0e38f;
    if (tid < K1) {
        const __half* e = (side ? cb_r : cb_l) + (size_t)tid * half;
        d = 0.0f;
        for (int j = 0; j < half; j++) {
            const float ed = xs[j] - __half2float(e[j]);
            d = fmaf(ed, ed, d);
        }
    }
    // the smallest distance, the lowest index among equals; an entry wins only below the reference's start value 1e30
    int k = tid;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float od = __shfl_xor_sync(0xffffffffu, d, o);
        const int ok = __shfl_xor_sync(0xffffffffu, k, o);
        if (od < d || (od == d && ok < k)) { d = od; k = ok; }
    }
    if (lane == 0) { best_d[warp] = d; best_k[warp] = k; }
    __syncthreads();
    if (tid == 0) {
        float bd = best_d[0]; int bk = best_k[0];
        for (int w = 1; w < 8; w++) if (best_d[w] < bd || (best_d[w] == bd && best_k[w] < bk)) { bd = best_d[w]; bk = best_k[w]; }
        idx[(size_t)v * 2 * C + h] = (uint8_t)(bd < 1e30f ? bk : 0);
    }
}

}  // namespace

extern "C" int ibcu_pqkv_encode(ibcu_ctx* ctx, const float* vec, int dim, int n_vec, int G, int K1,
                                const uint16_t* cb_l, const uint16_t* cb_r, uint8_t* idx, float* scale) {
    IBCU_CHECK_CTX(ctx);
    IBCU_REQUIRE(ctx, vec && cb_l && cb_r && idx && scale, "ibcu_pqkv_encode: null pointer");
    IBCU_REQUIRE(ctx, dim > 0 && n_vec > 0 && G >= 2 && G <= 32 && (G & 1) == 0 && dim % G == 0 && K1 >= 1 && K1 <= 256,
                 "ibcu_pqkv_encode: dim=%d G=%d K1=%d out of range", dim, G, K1);
    const int C = dim / G;
    return ibcu_launch(ctx, pqkv_encode_kernel, dim3(2 * C, n_vec), dim3(256), 0, 1, true, vec, dim, G, C, K1,
                       (const __half*)cb_l, (const __half*)cb_r, idx, scale);
}
