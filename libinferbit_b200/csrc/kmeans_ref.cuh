// The squared distance of the reference's k-means (src/pq_kmeans.c:99-106) in exactly the order and with
// exactly the roundings of its x86-64 Release binary: gcc vectorises the loop four dimensions at a time with
// an in-order reduction (multiply and add rounded separately) and contracts only the scalar remainder into
// fused multiply-adds. So dimensions below 4 * floor(D / 4) are unfused and the last D % 4 are fused.
#pragma once

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

