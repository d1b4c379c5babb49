// INT4 weights x INT8 activations (the reference's default route for INT4 linears): activations are
// quantised per 128-column group on the device, group dot products are exact int32, and the per-row
// FP32 accumulation over groups runs in group order with separately rounded multiply and add, so the
// results equal the reference's scalar kernel bit for bit.
#include "common.cuh"

namespace {

// one warp per (activation, group of 128)
__global__ void __launch_bounds__(256) quantize_g128_kernel(const float* __restrict__ x, int8_t* __restrict__ q, float* __restrict__ sa,
                                                            int N, int groups, int total) {
    pdl_launch_dependents();
    pdl_wait();
    const int wid = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (wid >= total) return;
    const int b = wid / groups, g = wid - b * groups;
    const int lo = g * 128, hi = min(lo + 128, N);
    const float* xb = x + (size_t)b * N;
    float v[4];
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int j = lo + lane + 32 * i;
        v[i] = j < hi ? xb[j] : 0.0f;
        amax = fmaxf(amax, fabsf(v[i]));
    }
    amax = warp_max(amax);
    float scale, inv = 0.0f;
    const bool dead = amax < 1e-10f;
    if (dead) scale = 1e-10f;
    else { scale = __fdiv_rn(amax, 127.0f); inv = __fdiv_rn(1.0f, scale); }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int j = lo + lane + 32 * i;
        if (j >= hi) continue;
        int qi = 0;
        if (!dead) {
            qi = __float2int_rz(__fadd_rn(__fmul_rn(v[i], inv), v[i] >= 0.0f ? 0.5f : -0.5f));
            qi = max(-127, min(127, qi));
        }
        q[(size_t)b * N + j] = (int8_t)qi;
    }
    if (lane == 0) sa[(size_t)b * groups + g] = scale;
}

// one warp per output row; lanes split each 128-column group (4 columns = 2 weight bytes per lane)
__global__ void __launch_bounds__(256) w4a8_kernel(const uint8_t* __restrict__ w, const void* __restrict__ scales, int scales_fp32,
                                                   float* __restrict__ out, int M, int out_stride, int epilogue,
                                                   const int8_t* __restrict__ xq, const float* __restrict__ sa, int N, int B) {
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= M) return;
    const int groups = (N + 127) / 128;
    const uint8_t* wr = w + (size_t)row * (N / 2);
    const float sw = scales_fp32 ? reinterpret_cast<const float*>(scales)[row]
                                 : __half2float(reinterpret_cast<const __half*>(scales)[row]);
    for (int b = 0; b < B; b++) {
        const int8_t* xb = xq + (size_t)b * N;
        float acc = 0.0f;
        for (int g = 0; g < groups; g++) {
            const int j = g * 128 + 4 * lane;
            int dot = 0;
#pragma unroll
            for (int u = 0; u < 2; u++) {
                const int jj = j + 2 * u;
                if (jj < N) {
                    const uint8_t byte = wr[jj >> 1];
                    dot += ((int)(byte & 15) - 8) * (int)xb[jj];
                    if (jj + 1 < N) dot += ((int)(byte >> 4) - 8) * (int)xb[jj + 1];
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
            acc = __fadd_rn(acc, __fmul_rn((float)dot, sa[(size_t)b * groups + g]));
        }
        if (lane == 0) {
            const float y = __fmul_rn(acc, sw);
            float* o = out + (size_t)b * out_stride + row;
            *o = epilogue == IBCU_EPI_ADD ? *o + y : y;
        }
    }
}

}  // namespace

extern "C" int ibcu_quantize_input_int8_g128(ibcu_ctx* ctx, const float* x, int8_t* q, float* sa, int N, int B) {
    IBCU_CHECK_CTX(ctx);
    IBCU_REQUIRE(ctx, x && q && sa && N > 0 && B > 0, "ibcu_quantize_input_int8_g128: bad arguments");
    const int groups = (N + 127) / 128, total = groups * B;
    return ibcu_launch(ctx, quantize_g128_kernel, dim3((total + 7) / 8), dim3(256), 0, 1, true, x, q, sa, N, groups, total);
}

extern "C" int ibcu_linear_w4a8(ibcu_ctx* ctx, const ibcu_linear_t* t, const int8_t* xq, const float* sa, int N, int B) {
    IBCU_CHECK_CTX(ctx);
    IBCU_REQUIRE(ctx, t && t->w && t->scales && t->out && xq && sa, "ibcu_linear_w4a8: null pointer");
    IBCU_REQUIRE(ctx, N > 0 && (N & 1) == 0 && B >= 1 && B <= 32 && t->M >= 0 && t->out_stride >= t->M, "ibcu_linear_w4a8: bad shape");
    if (t->M == 0) return IBCU_OK;
    return ibcu_launch(ctx, w4a8_kernel, dim3((t->M + 7) / 8), dim3(256), 0, 1, true, (const uint8_t*)t->w, t->scales, t->scales_fp32,
                       t->out, t->M, t->out_stride, t->epilogue, xq, sa, N, B);
}
