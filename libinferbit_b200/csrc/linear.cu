// Per-row-scaled INT4 / INT8 linear layers for 1..32 FP32 activations.
//
// Data in HBM: weights keep the reference layout bit for bit (INT8 row-major; INT4 two columns per
// byte, low nibble first, bias 8), scales are FP16 (or FP32) per output row.
//
// Arithmetic of the fast path: integer tensor cores, exactly. Every slice of an FP32 activation becomes
// a 32-bit fixed-point integer X = rint(x * 2^s) (s per slice, so that the slice maximum sits just
// under 2^30), split into four signed base-256 digits (int8 "limbs").
// linear_mma_kernel feeds the weights - INT8 bytes as they are, INT4 nibbles masked in place with
// one LOP3 per four weights - and the limbs to mma.sync.m16n8k32 (s8/u8 x s8 -> s32): every product
// and every sum is an exact integer. The four limb sums are recombined in 64-bit, converted to
// floating point once, scaled back by 2^-s and multiplied by the row scale. The result is the
// correctly rounded dot product of the weights with x rounded to 2^-32 of its slice maximum: closer
// to the true value than the reference's own FP32 running sum, and independent of summation order.
// Because a dot product is invariant under a permutation of k applied to both operands, each lane
// simply owns 16 contiguous bytes of a row; no transpose or ldmatrix is needed for the weights.
//
// Activation conversion (xconvert_*): short rows are converted by every block of linear_mma_kernel for
// itself, straight into shared memory, with all of the block's loads issued before the first is used;
// long rows once, by xprep_kernel (one block per activation and column slice), into a scratch buffer
// the blocks copy from. RMSNorm and silu(x)*x2 can be folded into the conversion; a caller that knows
// max|x| (IBCU_PRO_KNOWN_MAX) spares the blocks their reduction.
//
// Work split: linear_mma_kernel is persistent, one wave of blocks. A block is bound to one column slice,
// whose limbs it holds in shared memory, and to one tensor of the launch, of which it owns one contiguous
// run of rows; the runs are equal to within a row (blocks are allotted to the tensors in proportion to
// their rows), so every SM streams the same number of bytes. A run is walked in tiles of up to RT*16
// rows; rows a tile lacks are zero-filled without fetching anything. Weights reach shared memory through
// a cp.async ring whose stages are (tile rows) x 64*W bytes, written in row-linear order (every warp
// instruction covers contiguous bytes of one row, which is what HBM wants; lane-owns-a-row-fragment
// register loads measured 2-3 TB/s, this pattern 6+ TB/s). The W warps of a block take one 64-byte
// k-block of each stage each and meet in a shared-memory reduction per tile. When the columns are split
// over several blocks (only when a row's limbs do not fit shared memory), each writes its integer partial
// sums to scratch and linear_finalize_kernel recombines them (a fence + arrival-counter epilogue
// inside the main kernel cost ~3 us per tile and slice, a second small launch costs ~2 us once).
//
// Portable path (linear_generic_kernel): one warp per output row, plain FP32 FMAs; used for shapes
// the fast path does not take (row bytes not a multiple of 16, unaligned pointers) and by tests.
#include "common.cuh"
#include "tc_common.cuh"

bool ibcu_push_match(ibcu_ctx* ctx, float* const* outs, int n);      // comm.cu
void ibcu_push_fill(ibcu_ctx* ctx, GatherPush* gp, size_t bytes);  // bytes this launch pushes to each peer

namespace {

struct LinTensor {
    const uint8_t* w;
    const void* scales;
    float* out;
    int M, out_stride, scales_fp32, epilogue;
    int row_start;                 // first row of this tensor in the launch's concatenated row space
    int blk_start, rows_per;       // its blocks (per column slice) start at blk_start; each owns rows_per contiguous rows
    long win_off;                  // byte offset of `out` inside the peer window when the launch pushes its rows to the peers
};

struct XSource {                   // where an activation value comes from
    const float* x;                // [B][N]
    const float* x2;               // second operand of silu(x)*x2, or NULL
    const __half* norm_w;          // RMSNorm weights, or NULL
    float eps;
    int op;                        // IBCU_PRO_*
    const float* amax;             // IBCU_PRO_KNOWN_MAX: [B][n_amax] pieces of max|x[b]|
    int n_amax;
};

struct LinearParams {
    LinTensor t[4];
    int n_tensors;
    int total_rows;                // rows over all tensors
    int rowbytes;                  // bytes per weight row
    int nkb;                       // 64-byte k-blocks per row
    int N, B, ncols;               // columns, activations, limb columns (4 per activation)
    int slice_kb;                  // k-blocks per column slice (a multiple of the stage width)
    int nks;                       // column slices
    int xs_ld;                     // bytes per limb row: slice columns + pad
    const int8_t* xpack;           // [nks][ncols][xs_ld] limbs in fragment order
    const float* xscale;           // [B][nks] 2^-s of each slice
    const int* xsum;               // [B][nks][4] sum of each limb over the slice (INT4 bias term)
    int* partial;                  // [slice][B*4][total_rows] when nks > 1
    XSource xsrc;                  // FP32 source of the activations when the block converts them itself
    int fused_x;                   // 1: convert in the block, 0: limbs were prepared by xprep_kernel
    GatherWait gw;                 // the activations may be rows that peers pushed: wait for them (flags == NULL: nothing to wait for)
    GatherPush gp;                 // world > 0: this rank's output rows also go into the peers' copies (row-sharded output of a gather)
};

constexpr int LIN_LIMBS = 4;
// Row length of the reduction buffer in words. With more than one group of 8 columns the rows are padded by 4 words:
// rows then start 4 banks apart and the 128-bit reads of a (row, activation)'s four limbs never collide. One group keeps
// its 8 words (a two-way collision there costs less than the shared memory the padding would take from the ring).
__host__ __device__ constexpr int lin_rld(int ncg) { return ncg == 1 ? 8 : ncg * 8 + 4; }

// ── activation split ────────────────────────────────────────────────────────────────────
// grid (nks, B), one block per slice of one activation: X = rint(x * 2^s) with 2^s * max|x| in
// [2^29, 2^30), then X = d0 + 256 d1 + 65536 d2 + 2^24 d3 with every digit in [-128, 127].
// Eight columns at a time: INT8 consumers get them in natural order, INT4 consumers as
// c0,c2,c4,c6,c1,c3,c5,c7 (low nibbles of four bytes, then high nibbles).

// four consecutive transformed activation values starting at column j of activation row xb
__device__ __forceinline__ float4 xsrc_load4(const XSource& s, const float* xb, const float* x2b, int col, float r) {
    float4 v = *reinterpret_cast<const float4*>(xb + col);
    if (s.op == IBCU_PRO_RMSNORM) {
        const __half2 w01 = *reinterpret_cast<const __half2*>(s.norm_w + col), w23 = *reinterpret_cast<const __half2*>(s.norm_w + col + 2);
        v.x = v.x * r * __low2float(w01); v.y = v.y * r * __high2float(w01);
        v.z = v.z * r * __low2float(w23); v.w = v.w * r * __high2float(w23);
    } else if (s.op == IBCU_PRO_SILU_MUL) {
        const float4 u = *reinterpret_cast<const float4*>(x2b + col);
        v.x = v.x / (1.0f + expf(-v.x)) * u.x; v.y = v.y / (1.0f + expf(-v.y)) * u.y;
        v.z = v.z / (1.0f + expf(-v.z)) * u.z; v.w = v.w / (1.0f + expf(-v.w)) * u.w;
    }
    return v;
}

// Balanced base-256 digits of eight fixed-point values, as limb words. With Y = X + 0x00808080 the
// unsigned bytes u_l of Y satisfy X = sum (u_l - 128) 256^l (l < 3) + (Y >> 24) 2^24, and u_l - 128 as
// a signed byte is u_l ^ 0x80: so the four digits of X are the four bytes of Y ^ 0x00808080. Two 4x4
// byte transposes turn eight such words into limb-major words; bit 0 of perm8 picks the INT4 column order of the
// mma.sync kernel, any non-zero perm8 also asks for the limb sums (perm8 == 2: natural order with sums).
__device__ __forceinline__ void transpose4x4_bytes(uint32_t a, uint32_t b, uint32_t c, uint32_t d, uint32_t* o) {
    const uint32_t t0 = __byte_perm(a, b, 0x5140), t1 = __byte_perm(a, b, 0x7362);
    const uint32_t t2 = __byte_perm(c, d, 0x5140), t3 = __byte_perm(c, d, 0x7362);
    o[0] = __byte_perm(t0, t2, 0x5410); o[1] = __byte_perm(t0, t2, 0x7632);
    o[2] = __byte_perm(t1, t3, 0x5410); o[3] = __byte_perm(t1, t3, 0x7632);
}
__device__ __forceinline__ void limbs8(const int* X, int perm8, uint2* pk, int* lsum) {
    uint32_t D[8], lo[4], hi[4];
#pragma unroll
    for (int i = 0; i < 8; i++) D[i] = ((uint32_t)X[i] + 0x00808080u) ^ 0x00808080u;
    if (perm8 & 1) { transpose4x4_bytes(D[0], D[2], D[4], D[6], lo); transpose4x4_bytes(D[1], D[3], D[5], D[7], hi); }
    else       { transpose4x4_bytes(D[0], D[1], D[2], D[3], lo); transpose4x4_bytes(D[4], D[5], D[6], D[7], hi); }
#pragma unroll
    for (int l = 0; l < LIN_LIMBS; l++) {
        pk[l] = make_uint2(lo[l], hi[l]);
        lsum[l] = __dp4a((int)lo[l], 0x01010101, __dp4a((int)hi[l], 0x01010101, lsum[l]));
    }
}

// Converts columns [c0, c0 + slice_cols) of activation b to limbs. Called by every thread of a block
// (it synchronises); dst_b is the [LIN_LIMBS][xs_ld] limb block of this activation and slice, in
// global or shared memory. Thread 0 stores 2^-s to *back_out, threads 0..3 the limb sums to sum_out.
struct XScratch { float red[32]; int sred[32][LIN_LIMBS]; float mul, r; };

__device__ __forceinline__ void xconvert(const XSource& src, int N, int b, int c0, int slice_cols, int8_t* dst_b, int xs_ld,
                                         int perm8, XScratch& sc, float* back_out, int* sum_out) {
    const int nth = blockDim.x, nwarp = nth >> 5;
    const int valid = max(0, min(slice_cols, N - c0));       // N and c0 are multiples of 16
    const float* xrow = src.x + (size_t)b * N;
    const float* xb = xrow + c0;
    const float* x2b = src.x2 ? src.x2 + (size_t)b * N + c0 : nullptr;
    float r = 1.0f;
    if (src.op == IBCU_PRO_RMSNORM) {                         // 1/sqrt(mean(x^2) + eps) over the whole row (src/kernels/scalar.c:126-138)
        float ss = 0.0f;
        for (int j = threadIdx.x * 4; j < N; j += nth * 4) {
            const float4 v = *reinterpret_cast<const float4*>(xrow + j);
            ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
        }
        ss = warp_sum(ss);
        __syncthreads();
        if ((threadIdx.x & 31) == 0) sc.red[threadIdx.x >> 5] = ss;
        __syncthreads();
        if (threadIdx.x == 0) {
            float t = 0.0f;
            for (int w = 0; w < nwarp; w++) t += sc.red[w];
            sc.r = 1.0f / sqrtf(t / (float)N + src.eps);
        }
        __syncthreads();
        r = sc.r;
    }
    XSource sl = src;
    sl.norm_w = src.norm_w ? src.norm_w + c0 : nullptr;
    float amax = 0.0f;
    for (int j = threadIdx.x * 4; j < valid; j += nth * 4) {
        const float4 v = xsrc_load4(sl, xb, x2b, j, r);
        amax = fmaxf(fmaxf(amax, fmaxf(fabsf(v.x), fabsf(v.y))), fmaxf(fabsf(v.z), fabsf(v.w)));
    }
    amax = warp_max(amax);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) sc.red[threadIdx.x >> 5] = amax;
    __syncthreads();
    if (threadIdx.x == 0) {
        float v = sc.red[0];
        for (int w = 1; w < nwarp; w++) v = fmaxf(v, sc.red[w]);
        const int e = (int)((__float_as_uint(v) >> 23) & 0xFF);      // v in [2^(e-127), 2^(e-126))
        int sh = (v > 0.0f && e != 255) ? 156 - e : 0;               // 2^sh * v in [2^29, 2^30)
        sh = max(-126, min(126, sh));
        sc.mul = __uint_as_float((uint32_t)(127 + sh) << 23);
        *back_out = __uint_as_float((uint32_t)(127 - sh) << 23);
    }
    __syncthreads();
    const float mul = sc.mul;
    int lsum[LIN_LIMBS] = {0, 0, 0, 0};
    for (int j = threadIdx.x * 8; j < slice_cols; j += nth * 8) {
        int X[8];
        if (j < valid) {
            const float4 a = xsrc_load4(sl, xb, x2b, j, r), c = xsrc_load4(sl, xb, x2b, j + 4, r);
            X[0] = __float2int_rn(a.x * mul); X[1] = __float2int_rn(a.y * mul); X[2] = __float2int_rn(a.z * mul); X[3] = __float2int_rn(a.w * mul);
            X[4] = __float2int_rn(c.x * mul); X[5] = __float2int_rn(c.y * mul); X[6] = __float2int_rn(c.z * mul); X[7] = __float2int_rn(c.w * mul);
        } else {
#pragma unroll
            for (int i = 0; i < 8; i++) X[i] = 0;
        }
        uint2 pk[LIN_LIMBS];
        limbs8(X, perm8, pk, lsum);
#pragma unroll
        for (int l = 0; l < LIN_LIMBS; l++) *reinterpret_cast<uint2*>(dst_b + (size_t)l * xs_ld + j) = pk[l];
    }
#pragma unroll
    for (int l = 0; l < LIN_LIMBS; l++) {
        int v = lsum[l];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if ((threadIdx.x & 31) == 0) sc.sred[threadIdx.x >> 5][l] = v;
    }
    __syncthreads();
    if (threadIdx.x < LIN_LIMBS) {
        int v = 0;
        for (int w = 0; w < nwarp; w++) v += sc.sred[w][threadIdx.x];
        sum_out[threadIdx.x] = v;
    }
}

// The same conversion with the whole slice held in registers (up to V float4 per thread): every global
// load of the block is issued before the first one is used, so the block pays one memory round trip
// instead of one per loop iteration. Values, digits and sums are those of xconvert.
template <int V>
__device__ __forceinline__ void xconvert_regs(const XSource& src, int N, int b, int c0, int slice_cols, int8_t* dst_b, int xs_ld,
                                              int perm8, XScratch& sc, float* back_out, int* sum_out) {
    constexpr int P = V / 2;                                  // groups of 8 columns per thread
    const int nth = blockDim.x, nwarp = nth >> 5;
    const int valid = max(0, min(slice_cols, N - c0));       // N and c0 are multiples of 16
    const float* xrow = src.x + (size_t)b * N;
    const float* xb = xrow + c0;
    float4 va[P], vc[P];
#pragma unroll
    for (int i = 0; i < P; i++) {
        const int j = (threadIdx.x + i * nth) * 8;
        va[i] = vc[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (j < valid) { va[i] = *reinterpret_cast<const float4*>(xb + j); vc[i] = *reinterpret_cast<const float4*>(xb + j + 4); }
    }
    if (src.op == IBCU_PRO_SILU_MUL) {
        const float* x2b = src.x2 + (size_t)b * N + c0;
        float4 ua[P], uc[P];
#pragma unroll
        for (int i = 0; i < P; i++) {
            const int j = (threadIdx.x + i * nth) * 8;
            ua[i] = uc[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (j < valid) { ua[i] = *reinterpret_cast<const float4*>(x2b + j); uc[i] = *reinterpret_cast<const float4*>(x2b + j + 4); }
        }
#pragma unroll
        for (int i = 0; i < P; i++) {
            float4& a = va[i]; float4& c = vc[i];
            a.x = a.x / (1.0f + expf(-a.x)) * ua[i].x; a.y = a.y / (1.0f + expf(-a.y)) * ua[i].y;
            a.z = a.z / (1.0f + expf(-a.z)) * ua[i].z; a.w = a.w / (1.0f + expf(-a.w)) * ua[i].w;
            c.x = c.x / (1.0f + expf(-c.x)) * uc[i].x; c.y = c.y / (1.0f + expf(-c.y)) * uc[i].y;
            c.z = c.z / (1.0f + expf(-c.z)) * uc[i].z; c.w = c.w / (1.0f + expf(-c.w)) * uc[i].w;
        }
    } else if (src.op == IBCU_PRO_RMSNORM) {                  // 1/sqrt(mean(x^2) + eps) over the whole row (src/kernels/scalar.c:126-138)
        __half2 w[P][4];
        const bool w16 = ((uintptr_t)(src.norm_w + c0) & 15) == 0;
#pragma unroll
        for (int i = 0; i < P; i++) {
            const int j = (threadIdx.x + i * nth) * 8;
            if (j < valid && w16) {
                const uint4 raw = *reinterpret_cast<const uint4*>(src.norm_w + c0 + j);
                w[i][0] = *reinterpret_cast<const __half2*>(&raw.x); w[i][1] = *reinterpret_cast<const __half2*>(&raw.y);
                w[i][2] = *reinterpret_cast<const __half2*>(&raw.z); w[i][3] = *reinterpret_cast<const __half2*>(&raw.w);
            } else {
#pragma unroll
                for (int q = 0; q < 4; q++)
                    w[i][q] = j < valid ? *reinterpret_cast<const __half2*>(src.norm_w + c0 + j + 2 * q) : __floats2half2_rn(0.0f, 0.0f);
            }
        }
        float ss = 0.0f;
        if (c0 == 0 && valid == N) {
#pragma unroll
            for (int i = 0; i < P; i++) {
                ss = fmaf(va[i].x, va[i].x, fmaf(va[i].y, va[i].y, fmaf(va[i].z, va[i].z, fmaf(va[i].w, va[i].w, ss))));
                ss = fmaf(vc[i].x, vc[i].x, fmaf(vc[i].y, vc[i].y, fmaf(vc[i].z, vc[i].z, fmaf(vc[i].w, vc[i].w, ss))));
            }
        } else {
            for (int j = threadIdx.x * 4; j < N; j += nth * 4) {
                const float4 v = *reinterpret_cast<const float4*>(xrow + j);
                ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
            }
        }
        ss = warp_sum(ss);
        __syncthreads();
        if ((threadIdx.x & 31) == 0) sc.red[threadIdx.x >> 5] = ss;
        __syncthreads();
        float t = 0.0f;
        for (int q = 0; q < nwarp; q++) t += sc.red[q];       // every thread adds in the same order: no broadcast step
        const float r = 1.0f / sqrtf(t / (float)N + src.eps);
#pragma unroll
        for (int i = 0; i < P; i++) {
            va[i].x = va[i].x * r * __low2float(w[i][0]); va[i].y = va[i].y * r * __high2float(w[i][0]);
            va[i].z = va[i].z * r * __low2float(w[i][1]); va[i].w = va[i].w * r * __high2float(w[i][1]);
            vc[i].x = vc[i].x * r * __low2float(w[i][2]); vc[i].y = vc[i].y * r * __high2float(w[i][2]);
            vc[i].z = vc[i].z * r * __low2float(w[i][3]); vc[i].w = vc[i].w * r * __high2float(w[i][3]);
        }
    }
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < P; i++) {
        amax = fmaxf(fmaxf(amax, fmaxf(fabsf(va[i].x), fabsf(va[i].y))), fmaxf(fabsf(va[i].z), fabsf(va[i].w)));
        amax = fmaxf(fmaxf(amax, fmaxf(fabsf(vc[i].x), fabsf(vc[i].y))), fmaxf(fabsf(vc[i].z), fabsf(vc[i].w)));
    }
    amax = warp_max(amax);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) sc.red[threadIdx.x >> 5] = amax;
    __syncthreads();
    float vmax = sc.red[0];
    for (int q = 1; q < nwarp; q++) vmax = fmaxf(vmax, sc.red[q]);
    const int e = (int)((__float_as_uint(vmax) >> 23) & 0xFF);       // vmax in [2^(e-127), 2^(e-126))
    int sh = (vmax > 0.0f && e != 255) ? 156 - e : 0;                // 2^sh * vmax in [2^29, 2^30)
    sh = max(-126, min(126, sh));
    const float mul = __uint_as_float((uint32_t)(127 + sh) << 23);
    if (threadIdx.x == 0) *back_out = __uint_as_float((uint32_t)(127 - sh) << 23);
    int lsum[LIN_LIMBS] = {0, 0, 0, 0};
#pragma unroll
    for (int i = 0; i < P; i++) {
        const int j = (threadIdx.x + i * nth) * 8;
        if (j >= slice_cols) continue;
        int X[8];
        X[0] = __float2int_rn(va[i].x * mul); X[1] = __float2int_rn(va[i].y * mul); X[2] = __float2int_rn(va[i].z * mul); X[3] = __float2int_rn(va[i].w * mul);
        X[4] = __float2int_rn(vc[i].x * mul); X[5] = __float2int_rn(vc[i].y * mul); X[6] = __float2int_rn(vc[i].z * mul); X[7] = __float2int_rn(vc[i].w * mul);
        uint2 pk[LIN_LIMBS];
        limbs8(X, perm8, pk, lsum);
#pragma unroll
        for (int l = 0; l < LIN_LIMBS; l++) *reinterpret_cast<uint2*>(dst_b + (size_t)l * xs_ld + j) = pk[l];
    }
    if (!perm8) return;                                       // the limb sums only remove the nibble bias of INT4 weights
#pragma unroll
    for (int l = 0; l < LIN_LIMBS; l++) {
        int v = lsum[l];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if ((threadIdx.x & 31) == 0) sc.sred[threadIdx.x >> 5][l] = v;
    }
    __syncthreads();
    if (threadIdx.x < LIN_LIMBS) {
        int v = 0;
        for (int q = 0; q < nwarp; q++) v += sc.sred[q][threadIdx.x];
        sum_out[threadIdx.x] = v;
    }
}

// The conversion when the caller knows max|x[b]| (IBCU_PRO_KNOWN_MAX): no reduction before the digits, so
// rows of any length stream through in one pass, four groups of 8 columns in flight per thread.
__device__ __forceinline__ void xconvert_known(const XSource& src, int N, int b, int c0, int slice_cols, int8_t* dst_b, int xs_ld,
                                               int perm8, XScratch& sc, float* back_out, int* sum_out) {
    const int nth = blockDim.x, nwarp = nth >> 5;
    const int valid = max(0, min(slice_cols, N - c0));
    const float* xb = src.x + (size_t)b * N + c0;
    float vmax = 0.0f;
    for (int q = 0; q < src.n_amax; q++) vmax = fmaxf(vmax, src.amax[(size_t)b * src.n_amax + q]);
    const int e = (int)((__float_as_uint(vmax) >> 23) & 0xFF);
    int sh = (vmax > 0.0f && e != 255) ? 156 - e : 0;
    sh = max(-126, min(126, sh));
    const float mul = __uint_as_float((uint32_t)(127 + sh) << 23);
    if (threadIdx.x == 0) *back_out = __uint_as_float((uint32_t)(127 - sh) << 23);
    int lsum[LIN_LIMBS] = {0, 0, 0, 0};
    constexpr int U = 4;
    for (int j0 = threadIdx.x * 8; j0 < slice_cols; j0 += nth * 8 * U) {
        float4 va[U], vc[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int j = j0 + u * nth * 8;
            va[u] = vc[u] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (j < valid) { va[u] = *reinterpret_cast<const float4*>(xb + j); vc[u] = *reinterpret_cast<const float4*>(xb + j + 4); }
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int j = j0 + u * nth * 8;
            if (j >= slice_cols) continue;
            int X[8];
            X[0] = __float2int_rn(va[u].x * mul); X[1] = __float2int_rn(va[u].y * mul); X[2] = __float2int_rn(va[u].z * mul); X[3] = __float2int_rn(va[u].w * mul);
            X[4] = __float2int_rn(vc[u].x * mul); X[5] = __float2int_rn(vc[u].y * mul); X[6] = __float2int_rn(vc[u].z * mul); X[7] = __float2int_rn(vc[u].w * mul);
            uint2 pk[LIN_LIMBS];
            limbs8(X, perm8, pk, lsum);
#pragma unroll
            for (int l = 0; l < LIN_LIMBS; l++) *reinterpret_cast<uint2*>(dst_b + (size_t)l * xs_ld + j) = pk[l];
        }
    }
    if (!perm8) return;                                       // the limb sums only remove the nibble bias of INT4 weights
#pragma unroll
    for (int l = 0; l < LIN_LIMBS; l++) {
        int v = lsum[l];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if ((threadIdx.x & 31) == 0) sc.sred[threadIdx.x >> 5][l] = v;
    }
    __syncthreads();
    if (threadIdx.x < LIN_LIMBS) {
        int v = 0;
        for (int q = 0; q < nwarp; q++) v += sc.sred[q][threadIdx.x];
        sum_out[threadIdx.x] = v;
    }
}

constexpr int XREG_V = 8;                                     // 32 columns per thread in registers
__device__ __forceinline__ void xconvert_any(const XSource& src, int N, int b, int c0, int slice_cols, int8_t* dst_b, int xs_ld,
                                             int perm8, XScratch& sc, float* back_out, int* sum_out, int xregs = 1) {
    if (src.op == IBCU_PRO_KNOWN_MAX) { xconvert_known(src, N, b, c0, slice_cols, dst_b, xs_ld, perm8, sc, back_out, sum_out); return; }
    if (xregs && slice_cols <= XREG_V * 4 * (int)blockDim.x) xconvert_regs<XREG_V>(src, N, b, c0, slice_cols, dst_b, xs_ld, perm8, sc, back_out, sum_out);
    else xconvert(src, N, b, c0, slice_cols, dst_b, xs_ld, perm8, sc, back_out, sum_out);
}

// grid (nks, B): the conversion as a kernel of its own, used when doing it inside every block of the
// main kernel would cost more than a launch (several activations, long rows, the SiLU prologue).
template <int T>
__global__ void __launch_bounds__(T) xprep_kernel(const XSource src, int N, int slice_cols, int xs_ld, int perm8,
                                                     int nks, int xregs, int8_t* __restrict__ xpack, float* __restrict__ xscale, int* __restrict__ xsum,
                                                     const GatherWait gw) {
    __shared__ XScratch sc;
    pdl_launch_dependents();
    pdl_wait();
    gather_wait(gw);
    const int ks = blockIdx.x, b = blockIdx.y;
    int8_t* dst = xpack + ((size_t)ks * (gridDim.y * LIN_LIMBS) + (size_t)b * LIN_LIMBS) * xs_ld;
    xconvert_any(src, N, b, ks * slice_cols, slice_cols, dst, xs_ld, perm8, sc, xscale + b * nks + ks, xsum + ((size_t)b * nks + ks) * LIN_LIMBS, xregs);
}

__device__ __forceinline__ void imma_s8(int* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void imma_u8(int* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t u4_get(const uint4& v, int i) { return i == 0 ? v.x : (i == 1 ? v.y : (i == 2 ? v.z : v.w)); }

// ── fast path ───────────────────────────────────────────────────────────────────────────
// BITS: 4 or 8. NCG: groups of 8 MMA columns (ceil(4B/8)). RT: 16-row MMA tiles per tile of rows.
// W: warps per block. STAGES: shared-memory ring depth.
// MMA operands (m16n8k32, lane = 4g + t): A regs a0/a2 = row g, a1/a3 = row g+8, four bytes of k each;
// B regs b0/b1 = column g. INT8: a 16-byte lane chunk is four words w0..w3 -> two MMAs (w0,w1), (w2,w3)
// against 16 consecutive limb bytes. INT4: a raw word holds eight nibbles; raw & 0x0F0F0F0F are
// columns c0,c2,c4,c6 and raw & 0xF0F0F0F0 are 16 x columns c1,c3,c5,c7, so low and high nibbles go to
// separate accumulators (the high one is divided by 16 at the end, exactly) and no shift is needed.
// The nibble bias of 8 is removed once per output as 8 * (sum of the limb over the slice).
// Dynamic shared memory: stage ring [STAGES][R][LIN_LD] | reduction buffer [W][R][NCG*8] ints (x2 for
// INT4) | limbs [ncols][xs_ld] | scale-back factors [32] | limb sums [32][4].
__host__ __device__ constexpr int lin_sk(int W) { return W * 64; }                // bytes per row per stage: one 64-byte k-block per warp
__host__ __device__ constexpr int lin_ld(int W) { return W * 64 + 64; }           // padded row stride: conflict-free fragment reads

__device__ __forceinline__ void cp_async16(uint32_t smem_dst, const void* gsrc, bool valid) {
    const int n = valid ? 16 : 0;                             // 0 source bytes -> 16 zero bytes
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"(smem_dst), "l"(gsrc), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" :: "n"(N) : "memory"); }

template <int BITS, int NCG, int RT, int W, int STAGES>
__global__ void __launch_bounds__(W * 32) linear_mma_kernel(const LinearParams p) {
    constexpr int R = RT * 16;                                // most rows per tile
    constexpr int RLD = lin_rld(NCG);                         // words per row of the reduction buffer
    constexpr int NACC = BITS == 4 ? 2 : 1;                   // INT4 keeps low- and high-nibble sums apart
    constexpr int XB = BITS == 8 ? 64 : 128;                  // limb bytes (= columns) per k-block
    constexpr int KBS = W;                                    // k-blocks per stage: one per warp
    constexpr int LIN_SK = lin_sk(W), LIN_LD = lin_ld(W);
    constexpr int CPR = LIN_SK / 16;                          // 16-byte chunks per row per stage; the block copies 8 rows per pass
    static_assert(W == 8, "8 warps");
    constexpr int STAGE_BYTES = R * LIN_LD;
    constexpr int NCP = RT * 2;                               // 16-byte chunks per thread per stage
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    pdl_launch_dependents();

    const int ks = blockIdx.x % p.nks;                        // this block's column slice, fixed
    const int cb = blockIdx.x / p.nks;                        // a block works on one tensor: a contiguous run of its rows, in tiles of up to R
    int ti = 0;
#pragma unroll
    for (int i = 1; i < 4; i++) if (i < p.n_tensors && cb >= p.t[i].blk_start) ti = i;
    const LinTensor& T = p.t[ti];
    const int row_begin = (cb - T.blk_start) * T.rows_per;
    const int row_end = min(T.M, row_begin + T.rows_per);
    const int kb_begin = ks * p.slice_kb;
    const int nk = min(p.nkb, kb_begin + p.slice_kb) - kb_begin;
    const int nst = (nk + KBS - 1) / KBS;

    unsigned char* ring = smem_raw;
    int* red = reinterpret_cast<int*>(smem_raw + STAGES * STAGE_BYTES);
    int8_t* xs = reinterpret_cast<int8_t*>(smem_raw + STAGES * STAGE_BYTES + NACC * W * R * RLD * 4);
    float* s_back = reinterpret_cast<float*>(xs + (((size_t)p.ncols * p.xs_ld + 15) & ~(size_t)15));
    int* s_xsum = reinterpret_cast<int*>(s_back + 32);

    // ── producer side: thread owns chunk column cc of rows pr + 8i of every stage ──
    const int cc = threadIdx.x % CPR, pr = threadIdx.x / CPR;
    const uint32_t ring_u32 = (uint32_t)__cvta_generic_to_shared(ring) + pr * LIN_LD + cc * 16;
    const uint8_t* src[NCP];
    // A tile is up to R consecutive rows; rows of the tile that do not exist are zero-filled.
    int pf_row = row_begin, pf_rows = 0, pf_it = 0, pf_slot = 0;
    unsigned pf_mask = 0;                                     // bit i: row pr + 8i exists in the tile
    auto pf_setup = [&]() {                                   // row pointers for the tile at pf_row
        pf_rows = min(R, row_end - pf_row);
        const int r0 = pr;
        pf_mask = 0;
#pragma unroll
        for (int i = 0; i < NCP; i++) {
            const bool has = r0 + 8 * i < pf_rows;
            pf_mask |= has ? 1u << i : 0u;
            src[i] = T.w + (size_t)(pf_row + (has ? r0 + 8 * i : 0)) * p.rowbytes + (size_t)kb_begin * 64 + cc * 16;
        }
    };
    auto pf_issue = [&]() {                                   // next stage of the prefetch stream, if any
        if (pf_row < row_end) {
            const bool valid = (kb_begin + pf_it * KBS) * 64 + cc * 16 < p.rowbytes && pf_it * KBS + (cc >> 2) < nk;
            const uint32_t d = ring_u32 + pf_slot * STAGE_BYTES;
#pragma unroll
            for (int i = 0; i < NCP; i++) {
                const bool v = valid && ((pf_mask >> i) & 1u);
                cp_async16(d + i * 8 * LIN_LD, v ? src[i] + pf_it * LIN_SK : src[i], v);
            }
            pf_slot = pf_slot + 1 == STAGES ? 0 : pf_slot + 1;
            if (++pf_it == nst) { pf_it = 0; pf_row += pf_rows; if (pf_row < row_end) pf_setup(); }
        }
        cp_async_commit();
    };
    if (pf_row < row_end) pf_setup();
#pragma unroll
    for (int s = 0; s < STAGES - 1; s++) pf_issue();          // weights first: they do not depend on x
    pdl_wait();
    const unsigned recv_tag = gather_wait(p.gw);             // not 0: this launch received a tagged gather; its own pushes then carry the next tag

    // ── this slice's limbs, scale-back factors and limb sums ──
    if (p.fused_x) {
        __shared__ XScratch xsc;
        for (int b = 0; b < p.B; b++)
            xconvert_any(p.xsrc, p.N, b, kb_begin * XB, p.slice_kb * XB, xs + (size_t)b * LIN_LIMBS * p.xs_ld, p.xs_ld, BITS == 4 ? 1 : 0,
                         xsc, s_back + b, s_xsum + b * LIN_LIMBS);
    } else {
        const uint4* gsrc = reinterpret_cast<const uint4*>(p.xpack + (size_t)ks * p.ncols * p.xs_ld);
        const uint32_t d0 = (uint32_t)__cvta_generic_to_shared(xs);
        const int nchunk = p.ncols * p.xs_ld / 16;
        for (int c = threadIdx.x; c < nchunk; c += W * 32) cp_async16(d0 + c * 16, gsrc + c, true);
        cp_async_commit();
        if (threadIdx.x < p.B) s_back[threadIdx.x] = p.xscale[threadIdx.x * p.nks + ks];
        if (threadIdx.x < p.B * LIN_LIMBS)
            s_xsum[threadIdx.x] = p.xsum[((size_t)(threadIdx.x / LIN_LIMBS) * p.nks + ks) * LIN_LIMBS + (threadIdx.x % LIN_LIMBS)];
    }
    cp_async_wait<0>();
    __syncthreads();

    const int8_t* xcol[NCG];
#pragma unroll
    for (int c = 0; c < NCG; c++) {
        int col = c * 8 + g;
        col = col < p.ncols ? col : 0;                        // spare MMA columns reread column 0
        xcol[c] = xs + (size_t)col * p.xs_ld + (XB / 4) * t;
    }

    int slot = 0;
    int tile_rows = 0;
    for (int row0 = row_begin; row0 < row_end; row0 += tile_rows) {
        tile_rows = min(R, row_end - row0);
        int acc[NACC][RT][NCG][4];
#pragma unroll
        for (int a = 0; a < NACC; a++)
#pragma unroll
            for (int i = 0; i < RT; i++)
#pragma unroll
                for (int c = 0; c < NCG; c++) { acc[a][i][c][0] = acc[a][i][c][1] = acc[a][i][c][2] = acc[a][i][c][3] = 0; }

        for (int it = 0; it < nst; it++) {
            cp_async_wait<STAGES - 2>();
            __syncthreads();                                  // this stage has landed for everyone; the previous one is free
            pf_issue();
            const int k = it * KBS + warp;                    // this warp's k-block within the slice
            if (k < nk) {
                const unsigned char* sw = ring + slot * STAGE_BYTES + warp * 64 + 16 * t;
                uint4 cur[RT * 2];
#pragma unroll
                for (int j = 0; j < RT * 2; j++)
                    cur[j] = *reinterpret_cast<const uint4*>(sw + ((j >> 1) * 16 + (j & 1) * 8 + g) * LIN_LD);
                if (BITS == 8) {
                    uint4 xf[NCG];
#pragma unroll
                    for (int c = 0; c < NCG; c++) xf[c] = *reinterpret_cast<const uint4*>(xcol[c] + (size_t)k * XB);
#pragma unroll
                    for (int i = 0; i < RT; i++)
#pragma unroll
                        for (int c = 0; c < NCG; c++) {
                            imma_s8(acc[0][i][c], cur[2 * i].x, cur[2 * i + 1].x, cur[2 * i].y, cur[2 * i + 1].y, xf[c].x, xf[c].y);
                            imma_s8(acc[0][i][c], cur[2 * i].z, cur[2 * i + 1].z, cur[2 * i].w, cur[2 * i + 1].w, xf[c].z, xf[c].w);
                        }
                } else {
#pragma unroll
                    for (int h = 0; h < 2; h++) {             // two raw words (16 columns... 8 each) per half
                        uint4 xf[NCG];
#pragma unroll
                        for (int c = 0; c < NCG; c++) xf[c] = *reinterpret_cast<const uint4*>(xcol[c] + (size_t)k * XB + 16 * h);
#pragma unroll
                        for (int i = 0; i < RT; i++) {
                            const uint32_t r0a = u4_get(cur[2 * i], 2 * h), r0b = u4_get(cur[2 * i], 2 * h + 1);
                            const uint32_t r1a = u4_get(cur[2 * i + 1], 2 * h), r1b = u4_get(cur[2 * i + 1], 2 * h + 1);
#pragma unroll
                            for (int c = 0; c < NCG; c++) {
                                // low nibbles of words a, b against columns c0,c2,c4,c6 of each word
                                imma_u8(acc[0][i][c], r0a & 0x0F0F0F0Fu, r1a & 0x0F0F0F0Fu, r0b & 0x0F0F0F0Fu, r1b & 0x0F0F0F0Fu, xf[c].x, xf[c].z);
                                // high nibbles (x16) against columns c1,c3,c5,c7
                                imma_u8(acc[1][i][c], r0a & 0xF0F0F0F0u, r1a & 0xF0F0F0F0u, r0b & 0xF0F0F0F0u, r1b & 0xF0F0F0F0u, xf[c].y, xf[c].w);
                            }
                        }
                    }
                }
            }
            slot = slot + 1 == STAGES ? 0 : slot + 1;
        }
        // ── tile done: every warp holds integer partial sums of all R rows over its k-blocks ──
#pragma unroll
        for (int a = 0; a < NACC; a++) {
            int* mine = red + ((size_t)a * W + warp) * R * RLD;
#pragma unroll
            for (int i = 0; i < RT; i++)
#pragma unroll
                for (int c = 0; c < NCG; c++) {
                    *reinterpret_cast<int2*>(mine + (i * 16 + g) * RLD + c * 8 + 2 * t) = make_int2(acc[a][i][c][0], acc[a][i][c][1]);
                    *reinterpret_cast<int2*>(mine + (i * 16 + g + 8) * RLD + c * 8 + 2 * t) = make_int2(acc[a][i][c][2], acc[a][i][c][3]);
                }
        }
        __syncthreads();
        const int B = p.B;
        const unsigned tag = p.gp.world ? (recv_tag ? recv_tag + 1u : tag_current(p.gp)) : 0u;
        // one thread per (row, activation): limb sums over the warps, bias, recombination
        for (int e = threadIdx.x; e < R * B; e += W * 32) {
            const int r = e % R, b = e / R;
            if (r >= tile_rows) continue;
            const int row = row0 + r;
            int limb[LIN_LIMBS];
            {                                                 // the four limbs of (row, activation) sit side by side: one 128-bit read per warp
                int4 lo = make_int4(0, 0, 0, 0);
#pragma unroll
                for (int w = 0; w < W; w++) {
                    const int4 v = *reinterpret_cast<const int4*>(red + ((size_t)w * R + r) * RLD + b * LIN_LIMBS);
                    lo.x += v.x; lo.y += v.y; lo.z += v.z; lo.w += v.w;
                }
                if (BITS == 4) {
                    int4 hi = make_int4(0, 0, 0, 0);
#pragma unroll
                    for (int w = 0; w < W; w++) {
                        const int4 v = *reinterpret_cast<const int4*>(red + ((size_t)(W + w) * R + r) * RLD + b * LIN_LIMBS);
                        hi.x += v.x; hi.y += v.y; hi.z += v.z; hi.w += v.w;
                    }
                    lo.x += (hi.x >> 4) - 8 * s_xsum[b * LIN_LIMBS + 0];
                    lo.y += (hi.y >> 4) - 8 * s_xsum[b * LIN_LIMBS + 1];
                    lo.z += (hi.z >> 4) - 8 * s_xsum[b * LIN_LIMBS + 2];
                    lo.w += (hi.w >> 4) - 8 * s_xsum[b * LIN_LIMBS + 3];
                }
                limb[0] = lo.x; limb[1] = lo.y; limb[2] = lo.z; limb[3] = lo.w;
            }
            if (p.nks == 1) {
                {
                    const long long V = (((long long)limb[3] * 256 + limb[2]) * 256 + limb[1]) * 256 + limb[0];
                    const float y = (float)((double)V * (double)s_back[b]);
                    const float sc = T.scales_fp32 ? reinterpret_cast<const float*>(T.scales)[row]
                                                   : __half2float(reinterpret_cast<const __half*>(T.scales)[row]);
                    float* o = T.out + (size_t)b * T.out_stride + row;
                    const float v = T.epilogue == IBCU_EPI_ADD ? *o + y * sc : y * sc;
                    *o = v;
                    if (p.gp.world) tag_push(p.gp, (size_t)T.win_off + ((size_t)b * T.out_stride + row) * sizeof(float), v, tag);
                }
            } else {
#pragma unroll
                for (int l = 0; l < LIN_LIMBS; l++)
                    p.partial[((size_t)ks * (B * LIN_LIMBS) + b * LIN_LIMBS + l) * p.total_rows + T.row_start + row] = limb[l];
            }
        }
    }
    cp_async_wait<0>();
}

// When the columns are split over several blocks: one thread per (row, activation) recombines the
// integer partial sums of all slices, each with its own 2^-s, in slice order.
__global__ void __launch_bounds__(256) linear_finalize_kernel(const LinearParams p) {
    pdl_launch_dependents();
    pdl_wait();
    const int B = p.B;
    const long total = (long)p.total_rows * B;
    const unsigned tag = p.gp.world ? tag_current(p.gp) : 0u;
    for (long e = (long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long)gridDim.x * blockDim.x) {
        const int vrow = (int)(e % p.total_rows);
        const int b = (int)(e / p.total_rows);
        int ti = 0;
#pragma unroll
        for (int i = 1; i < 4; i++) if (i < p.n_tensors && vrow >= p.t[i].row_start) ti = i;
        const LinTensor& T = p.t[ti];
        const int row = vrow - T.row_start;
        double y = 0.0;
        for (int k = 0; k < p.nks; k++) {
            const int* src_p = p.partial + ((size_t)k * (B * LIN_LIMBS) + b * LIN_LIMBS) * p.total_rows + vrow;
            const size_t st = p.total_rows;
            const long long V = (((long long)src_p[3 * st] * 256 + src_p[2 * st]) * 256 + src_p[st]) * 256 + src_p[0];
            y += (double)V * (double)p.xscale[b * p.nks + k];
        }
        const float sc = T.scales_fp32 ? reinterpret_cast<const float*>(T.scales)[row]
                                       : __half2float(reinterpret_cast<const __half*>(T.scales)[row]);
        float* o = T.out + (size_t)b * T.out_stride + row;
        const float v = T.epilogue == IBCU_EPI_ADD ? *o + (float)y * sc : (float)y * sc;
        *o = v;
        if (p.gp.world) tag_push(p.gp, (size_t)T.win_off + ((size_t)b * T.out_stride + row) * sizeof(float), v, tag);
    }
}

// ── portable path ───────────────────────────────────────────────────────────────────────
// One warp per output row; lanes stride over the columns; FP32 FMAs; activations straight from x.
template <int BITS>
__global__ void __launch_bounds__(256) linear_generic_kernel(LinTensor T, const float* __restrict__ x, int N, int B) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= T.M) return;
    const size_t rowbytes = BITS == 8 ? (size_t)N : (size_t)(N / 2);
    const uint8_t* wr = T.w + (size_t)row * rowbytes;
    const float sc = T.scales_fp32 ? reinterpret_cast<const float*>(T.scales)[row]
                                   : __half2float(reinterpret_cast<const __half*>(T.scales)[row]);
    for (int b = 0; b < B; b++) {
        const float* xb = x + (size_t)b * N;
        float s = 0.0f;
        if (BITS == 8) {
            for (int j = lane; j < N; j += 32) s = fmaf((float)(int8_t)wr[j], xb[j], s);
        } else {
            for (int j = 2 * lane; j < N; j += 64) {
                uint8_t v = wr[j >> 1];
                s = fmaf((float)((int)(v & 15) - 8), xb[j], s);
                if (j + 1 < N) s = fmaf((float)((int)(v >> 4) - 8), xb[j + 1], s);
            }
        }
        s = warp_sum(s);
        if (lane == 0) {
            float y = s * sc;
            float* o = T.out + (size_t)b * T.out_stride + row;
            *o = T.epilogue == IBCU_EPI_ADD ? *o + y : y;
        }
    }
}

template <int BITS, int NCG, int RT, int W, int STAGES>
int launch_mma(ibcu_ctx* ctx, const LinearParams& p, int grid, size_t smem_tail) {
    auto kern = linear_mma_kernel<BITS, NCG, RT, W, STAGES>;
    const size_t smem = (size_t)STAGES * RT * 16 * lin_ld(W) + (size_t)(BITS == 4 ? 2 : 1) * W * RT * 16 * lin_rld(NCG) * 4 + smem_tail;   // ring + reduction buffer + limbs
    if (smem > 48 * 1024) {
        static size_t allowed[64];                                 // per device, per kernel instance: raised only when a call needs more
        size_t& have = allowed[ctx->device & 63];
        if (smem > have) {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return ibcu_fail(ctx, IBCU_ERR_CUDA, "cudaFuncSetAttribute(smem=%zu): %s", smem, cudaGetErrorString(e));
            have = smem;
        }
    }
    return ibcu_launch(ctx, kern, dim3(grid), dim3(W * 32), smem, 1, true, p);
}

// ── batched path on tcgen05 (8 to 16 activations; optional) ─────────────────────────────
// With eight or more activations the four limbs of every activation make 32 to 64 MMA columns and the product is a
// small GEMM; mma.sync's integer rate then bounds the large launches. linear_tc_kernel runs the same exact arithmetic on
// the fifth-generation tensor cores: tiles of 64 weight rows are the A operand, read from shared memory (INT8 bytes as
// stored; INT4 nibbles widened to bytes by the loader warps), the limbs of a column slice are the B operand, resident in
// shared memory for the life of the block, and the s32 sums accumulate in tensor memory, two tiles in turn so that the
// epilogue of one tile overlaps the MMAs of the next.
//   warps 0-3: epilogue (tcgen05.ld, limb recombination, scale, store / partial sums)   warps 4-7: loaders   warp 8: MMA issue
// Both operands are K-major. A (weights) uses the 128-byte swizzle: a row's 128 bytes stay one line of shared memory, so a
// warp's asynchronous copy of 512 contiguous bytes of a row lands in four whole lines (copies scattered in 16-byte pieces
// were measured to reach L2 as one request per lane and fetched every sector twice). B (limbs) has no swizzle: a 16-byte K
// chunk of 8 columns is one 128-byte core matrix, the core matrices of a chunk are contiguous (SBO = 128), chunks follow
// one another (LBO = 16 x columns).
// A block is bound to one column slice; it walks the row tiles blockIdx.x / nks + j * gridDim.x / nks.
// Measured on B200 (graph replays, weights from HBM): 28672 x 4096 INT4 at 8 activations 42.8 us against 51.2 us for the
// mma.sync kernel; 32000 x 4096 INT8 at 8 activations 47.2 against 47.3 us; 4096 x 4096 INT8 at 16 activations 20.5 against
// 17.1 us (few tiles, and the split columns cost a recombination launch). The 7B step at batch 8 gains 5 % with the gate/up launch on this kernel. In-kernel time stamps: a stage of 32 KB takes
// 3.6 us from copy issue to landing with three stages in flight, so the kernel is bound by bytes in flight per SM (96 KB
// beside the 64 KB of resident limbs), not by the tensor pipe (10 % active). By default it therefore takes only the calls where it was measured ahead: INT4 tensors of
// at least 3072 rows and at most 4096 columns with 5 to 8 activations; ibcu_linear_use_tcgen05 widens or narrows that.
constexpr int LT_TILE = 64, LT_EPI_WARPS = 4, LT_LOAD_WARPS = 4, LT_MMA_WARP = 8, LT_THREADS = 9 * 32;
constexpr int LT_KCOLS = 512;                    // weight columns per pipeline step: sixteen MMAs of K = 32; a step reads 512 (INT8) or 256 (INT4) contiguous bytes of each row
constexpr int LT_CH = LT_KCOLS / 16;             // 16-byte K chunks per step
constexpr int LT_A_KBLOCK = LT_TILE * 128;       // A operand, K-major with the 128-byte swizzle: a block of 128 columns is 64 rows of 128 bytes (8 KB),
                                                 // 8-row atoms of 1 KB; chunk c of row r sits at chunk position c ^ (r % 8) of its row
constexpr int LT_A_STAGE = (LT_KCOLS / 128) * LT_A_KBLOCK;   // 32 KB: 64 rows x 512 bytes
constexpr int LT_RAW_LD = 256 + 16;              // INT4: bytes per row of a raw stage: the nibbles of a step + 16
constexpr int LT_RAW_STAGE = LT_TILE * LT_RAW_LD;
constexpr int LT_MAX_STAGES = 8;

struct LtShared {
    unsigned long long full_a[LT_MAX_STAGES], empty_a[LT_MAX_STAGES];   // loaders -> MMA, MMA -> loaders
    unsigned long long full_acc[2], empty_acc[2];                        // MMA -> epilogue, epilogue -> MMA
    unsigned long long b_full, drained;
    uint32_t tmem_base;
    int abort_flag;
    float back[32];                              // 2^-s of this slice per activation
    int xsum[32 * LIN_LIMBS];                    // limb sums of this slice (INT4 bias)
};

struct LtParams {
    LinTensor t[4];
    int n_tensors, tile_start[5];                // tiles of tensor i are [tile_start[i], tile_start[i + 1])
    int total_rows, rowbytes, N, B, NC, nks, slice_steps, total_steps, xs_ld;
    const int8_t* xpack; const float* xscale; const int* xsum;
    int* partial;
    GatherPush gp;
    int* err;
};

// shared-memory matrix descriptor, K-major with the 128-byte swizzle: 8-row atoms of 1024 bytes follow one another (SBO = 1024);
// the K offset inside the 128-byte rows is part of the start address
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void mma_i8_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
                 :: "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}

template <int BITS, int STAGES, int RAW_STAGES>
__global__ void __launch_bounds__(LT_THREADS, 1) linear_tc_kernel(const LtParams p) {
    extern __shared__ __align__(1024) unsigned char lt_smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int ks = blockIdx.x % p.nks, tile0 = blockIdx.x / p.nks, tile_step = gridDim.x / p.nks;
    const int ntiles = p.tile_start[p.n_tensors];
    const int n_my = tile0 < ntiles ? (ntiles - tile0 + tile_step - 1) / tile_step : 0;
    const int kbs = min(p.slice_steps, p.total_steps - ks * p.slice_steps);          // pipeline steps (of 128 columns) in this slice
    const long n_steps = (long)n_my * kbs;
    const uint32_t b_lbo = (uint32_t)p.NC * 16u;
    unsigned char* sB = lt_smem;                                                       // [slice chunks][NC / 8][8][16]
    unsigned char* sA = sB + (((size_t)p.slice_steps * LT_CH * b_lbo + 1023) & ~(size_t)1023);
    unsigned char* sRaw = sA + STAGES * LT_A_STAGE;
    LtShared* sh = reinterpret_cast<LtShared*>(sRaw + (BITS == 4 ? RAW_STAGES * LT_RAW_STAGE : 0));
    volatile int* abort_flag = &sh->abort_flag;
    pdl_launch_dependents();

    if (tid == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(smem_u32(&sh->full_a[s]), LT_LOAD_WARPS); mbar_init(smem_u32(&sh->empty_a[s]), 1); }
        for (int b = 0; b < 2; b++) { mbar_init(smem_u32(&sh->full_acc[b]), 1); mbar_init(smem_u32(&sh->empty_acc[b]), LT_EPI_WARPS); }
        mbar_init(smem_u32(&sh->b_full), LT_EPI_WARPS + 1);
        mbar_init(smem_u32(&sh->drained), 1);
        sh->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    const uint32_t tmem_cols = 2u * (uint32_t)p.NC;                                   // 64 or 128: a power of two, at least 32
    if (warp == LT_MMA_WARP) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(&sh->tmem_base)), "r"(tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = sh->tmem_base;

    // which tensor a tile belongs to, and its first row there
    auto tile_of = [&](int j, int& ti, int& row0) {
        const int tile = tile0 + j * tile_step;
        ti = 0;
#pragma unroll
        for (int i = 1; i < 4; i++) if (i < p.n_tensors && tile >= p.tile_start[i]) ti = i;
        row0 = (tile - p.tile_start[ti]) * LT_TILE;
    };

    if (warp >= LT_EPI_WARPS && warp < LT_MMA_WARP) {
        // ── loaders: warp lw owns rows 32 lw .. + 31 of every tile. The weights do not depend on the previous kernel:
        //    no dependency wait here. ──
        const int lw = warp - LT_EPI_WARPS;                                            // rows 16 lw .. + 15 of every tile
        constexpr int RING = BITS == 8 ? STAGES : RAW_STAGES;                          // depth of the ring the global loads land in
        bool alive = true;
        auto issue = [&](long i) {
            if (i < n_steps && alive) {
                const int j = (int)(i / kbs), kb = (int)(i - (long)j * kbs);
                int ti, row0;
                tile_of(j, ti, row0);
                const LinTensor& T = p.t[ti];
                if (BITS == 8) {
                    const int s = (int)(i % STAGES);
                    // the stage is free once the MMAs of its previous use have read it
                    if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&sh->empty_a[s]), (uint32_t)(((i / STAGES) & 1) ^ 1), abort_flag, 1))) { alive = false; }
                    if (alive) {
                        // a warp instruction copies one row's 512 bytes: whole lines of global memory into four whole (swizzled) lines of shared memory
                        const uint32_t dst0 = smem_u32(sA + s * LT_A_STAGE) + (uint32_t)(lane >> 3) * LT_A_KBLOCK;
                        const uint32_t c = lane & 7;
#pragma unroll
                        for (int u = 0; u < 16; u++) {
                            const int rr = 16 * lw + u;
                            const bool hv = row0 + rr < T.M;
                            const uint8_t* sp = T.w + (size_t)(hv ? row0 + rr : 0) * p.rowbytes + (size_t)(ks * p.slice_steps + kb) * LT_KCOLS + lane * 16;
                            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;"
                                         :: "r"(dst0 + (uint32_t)(rr >> 3) * 1024u + (uint32_t)(rr & 7) * 128u + ((c ^ (uint32_t)(rr & 7)) << 4)), "l"(sp), "r"(hv ? 16 : 0) : "memory");
                        }
                    }
                } else {
                    // the nibbles of the step: 2 rows x 256 bytes per warp instruction
                    const int piece = lane & 15;
                    const uint32_t dst0 = smem_u32(sRaw + (int)(i % RAW_STAGES) * LT_RAW_STAGE) + piece * 16;
#pragma unroll
                    for (int u = 0; u < 8; u++) {
                        const int rr = 16 * lw + 2 * u + (lane >> 4);
                        const bool hv = row0 + rr < T.M;
                        const uint8_t* sp = T.w + (size_t)(hv ? row0 + rr : 0) * p.rowbytes + (size_t)(ks * p.slice_steps + kb) * (LT_KCOLS / 2) + piece * 16;
                        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"(dst0 + (uint32_t)rr * LT_RAW_LD), "l"(sp), "r"(hv ? 16 : 0) : "memory");
                    }
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        constexpr int AHEAD = RING - 1;
        for (int i = 0; i < AHEAD; i++) issue(i);
        for (long i = 0; i < n_steps && alive; i++) {
            if (BITS == 4) __syncwarp();                                               // the raw rows about to be refilled have been read by every lane
            issue(i + AHEAD);
            asm volatile("cp.async.wait_group %0;" :: "n"(AHEAD) : "memory");
            if (BITS == 4) __syncwarp();                                               // rows copied by other lanes of the warp
            const int s = (int)(i % STAGES);
            if (BITS == 4) {
                if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&sh->empty_a[s]), (uint32_t)(((i / STAGES) & 1) ^ 1), abort_flag, 1))) break;
                // widen this row's 128 nibbles to bytes 0..15 in column order: a raw byte holds columns 2i (low) and 2i + 1 (high)
                // lane = (row, half of the row's 256 raw bytes): 8 pieces of 16 bytes -> 16 chunks of the operand stage
                const int r = 16 * lw + (lane & 15), hf = lane >> 4;
                const unsigned char* raw = sRaw + (int)(i % RAW_STAGES) * LT_RAW_STAGE + r * LT_RAW_LD + hf * 128;
                unsigned char* dst = sA + s * LT_A_STAGE + (uint32_t)(r >> 3) * 1024u + (uint32_t)(r & 7) * 128u;
                const uint32_t rx = (uint32_t)(r & 7);
                auto chunk_at = [&](int kc) { return dst + (kc >> 3) * LT_A_KBLOCK + (((uint32_t)(kc & 7) ^ rx) << 4); };   // K chunk kc of this row
#pragma unroll
                for (int q = 0; q < 8; q++) {
                    const uint4 v = *reinterpret_cast<const uint4*>(raw + q * 16);
                    const uint32_t w[4] = { v.x, v.y, v.z, v.w };
                    uint32_t o[8];
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        const uint32_t lo = w[u] & 0x0F0F0F0Fu, hi = (w[u] >> 4) & 0x0F0F0F0Fu;
                        o[2 * u] = __byte_perm(lo, hi, 0x5140);
                        o[2 * u + 1] = __byte_perm(lo, hi, 0x7362);
                    }
                    *reinterpret_cast<uint4*>(chunk_at(hf * 16 + 2 * q)) = make_uint4(o[0], o[1], o[2], o[3]);
                    *reinterpret_cast<uint4*>(chunk_at(hf * 16 + 2 * q + 1)) = make_uint4(o[4], o[5], o[6], o[7]);
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&sh->full_a[s]));
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
    } else {
        // ── everyone else: the slice's limbs into the B operand, after the kernel that made them ──
        pdl_wait();
        const int ncols = p.B * LIN_LIMBS;
        const int fill_tid = warp == LT_MMA_WARP ? LT_EPI_WARPS * 32 + lane : tid, fill_n = (LT_EPI_WARPS + 1) * 32;
        const int cgs = p.NC / 8;
        const long pieces = (long)kbs * LT_CH * p.NC;                                  // 16-byte pieces: LT_CH K chunks per step, NC columns
        const int8_t* xp = p.xpack + (size_t)ks * ncols * p.xs_ld;
        const uint32_t sB_u32 = smem_u32(sB);
        for (long e = fill_tid; e < pieces; e += fill_n) {
            // a warp instruction covers 8 columns x 4 K chunks: four 128-byte runs in shared memory, 64 contiguous bytes per
            // column in global memory. Asynchronous copies: all pieces of a thread are in flight together.
            const int c8 = (int)(e & 7), kl = (int)((e >> 3) & 3);
            const long hi = e >> 5;
            const int cg = (int)(hi % cgs), kc = (int)(hi / cgs) * 4 + kl;
            const int c = cg * 8 + c8;
            const bool have = c < ncols;
            const int8_t* src = xp + (size_t)(have ? c : 0) * p.xs_ld + (size_t)kc * 16;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"(sB_u32 + (uint32_t)kc * b_lbo + cg * 128 + c8 * 16), "l"(src), "r"(have ? 16 : 0) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        if (fill_tid < p.B) sh->back[fill_tid] = p.xscale[fill_tid * p.nks + ks];
        if (BITS == 4 && fill_tid < ncols) sh->xsum[fill_tid] = p.xsum[((size_t)(fill_tid / LIN_LIMBS) * p.nks + ks) * LIN_LIMBS + (fill_tid % LIN_LIMBS)];
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&sh->b_full));

        if (warp == LT_MMA_WARP) {
            if (lane == 0) {
                // s32 accumulate; A: unsigned bytes for widened nibbles (bias 8 removed through the limb sums), signed for INT8; B: signed limbs
                const uint32_t idesc = (2u << 4) | ((BITS == 8 ? 1u : 0u) << 7) | (1u << 10) | ((uint32_t)(p.NC >> 3) << 17) | ((uint32_t)(LT_TILE >> 4) << 24);
                bool ok = mbar_wait(smem_u32(&sh->b_full), 0u, abort_flag, 6);
                for (int j = 0; j < n_my && ok; j++) {
                    const int buf = j & 1;
                    ok = mbar_wait(smem_u32(&sh->empty_acc[buf]), (uint32_t)(((j >> 1) & 1) ^ 1), abort_flag, 3);
                    const uint32_t d = tmem_base + (uint32_t)buf * (uint32_t)p.NC;
                    for (int kb = 0; kb < kbs && ok; kb++) {
                        const long i = (long)j * kbs + kb;
                        const int s = (int)(i % STAGES);
                        ok = mbar_wait(smem_u32(&sh->full_a[s]), (uint32_t)((i / STAGES) & 1), abort_flag, 2);
                        if (!ok) break;
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                        for (int m = 0; m < LT_CH / 2; m++) {
                            const uint64_t a_desc = smem_desc_sw128(smem_u32(sA + s * LT_A_STAGE + (m >> 2) * LT_A_KBLOCK + (m & 3) * 32));
                            const uint64_t b_desc = smem_desc(smem_u32(sB + (size_t)(kb * LT_CH + 2 * m) * b_lbo), b_lbo, 128);
                            mma_i8_ss(d, a_desc, b_desc, idesc, (kb | m) ? 1u : 0u);
                        }
                        mma_commit(smem_u32(&sh->empty_a[s]));
                    }
                    if (ok) mma_commit(smem_u32(&sh->full_acc[buf]));
                }
                mma_commit(smem_u32(&sh->drained));
                mbar_wait(smem_u32(&sh->drained), 0u, abort_flag, 4);                  // nothing of this block is left in the tensor pipe
            }
        } else {
            // ── epilogue: warp q drains rows 32 q .. + 31 of every tile ──
            const int q = warp;
            const unsigned tag = p.gp.world ? tag_current(p.gp) : 0u;
            for (int j = 0; j < n_my; j++) {
                const int buf = j & 1;
                int ti, row0;
                tile_of(j, ti, row0);
                const LinTensor& T = p.t[ti];
                // a 64-row accumulator keeps row r in lane 32 (r / 16) + r % 16 of tensor memory: the first 16 lanes of every warp's quarter
                const int row = row0 + 16 * q + (lane & 15);
                const bool have = lane < 16 && row < T.M;
                if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&sh->full_acc[buf]), (uint32_t)((j >> 1) & 1), abort_flag, 5))) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)buf * (uint32_t)p.NC;
                const float sc = have ? (T.scales_fp32 ? reinterpret_cast<const float*>(T.scales)[row] : __half2float(reinterpret_cast<const __half*>(T.scales)[row])) : 0.0f;
                for (int c0 = 0; c0 < p.NC; c0 += 32) {
                    uint32_t acc[32];
                    tmem_ld32(taddr + c0, acc);
                    tmem_wait_ld(acc);
#pragma unroll
                    for (int bb = 0; bb < 8; bb++) {
                        const int b = c0 / 4 + bb;
                        if (b >= p.B || !have) continue;
                        int limb[LIN_LIMBS];
#pragma unroll
                        for (int l = 0; l < LIN_LIMBS; l++) {
                            limb[l] = (int)acc[bb * 4 + l];
                            if (BITS == 4) limb[l] -= 8 * sh->xsum[b * LIN_LIMBS + l];
                        }
                        if (p.nks == 1) {
                            const long long V = (((long long)limb[3] * 256 + limb[2]) * 256 + limb[1]) * 256 + limb[0];
                            const float y = (float)((double)V * (double)sh->back[b]);
                            float* o = T.out + (size_t)b * T.out_stride + row;
                            const float v = T.epilogue == IBCU_EPI_ADD ? *o + y * sc : y * sc;
                            *o = v;
                            if (p.gp.world) tag_push(p.gp, (size_t)T.win_off + ((size_t)b * T.out_stride + row) * sizeof(float), v, tag);
                        } else {
#pragma unroll
                            for (int l = 0; l < LIN_LIMBS; l++)
                                p.partial[((size_t)ks * (p.B * LIN_LIMBS) + b * LIN_LIMBS + l) * p.total_rows + T.row_start + row] = limb[l];
                        }
                    }
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&sh->empty_acc[buf]));              // the tensor cores may overwrite this tile
            }
        }
    }
    // ── the end: tensor memory back, a wait that ran out reported ──
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == LT_MMA_WARP) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"(tmem_cols) : "memory");
    }
    if (tid == 0 && sh->abort_flag) *p.err = 100 + sh->abort_flag;
}

template <int BITS, int STAGES, int RAW_STAGES>
int launch_tc(ibcu_ctx* ctx, const LtParams& p, int grid, size_t smem) {
    auto kern = linear_tc_kernel<BITS, STAGES, RAW_STAGES>;
    static size_t allowed[64];
    size_t& have = allowed[ctx->device & 63];
    if (smem > have) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return ibcu_fail(ctx, IBCU_ERR_CUDA, "cudaFuncSetAttribute(linear_tc_kernel, smem=%zu): %s", smem, cudaGetErrorString(e));
        have = smem;
    }
    return ibcu_launch(ctx, kern, dim3(grid), dim3(LT_THREADS), smem, 1, true, p);
}

constexpr int LT_STAGES8 = 4, LT_STAGES4 = 2, LT_RAW4 = 4;     // stages of weights in flight (INT8: operand stages; INT4: raw stages, widened into 3 operand stages)
constexpr size_t LT_B_BUDGET = 64 * 1024;                      // shared memory for the resident limbs of a column slice: the rest goes to the weight ring

// 8 to 16 activations, rows of whole 128-column steps: conversion kernel, tcgen05 kernel, and the recombination kernel when
// the columns had to be split over several blocks. Returns IBCU_ERR_STATE when the shape does not fit (the caller goes on).
int linear_tc(ibcu_ctx* ctx, const ibcu_linear_t* tensors, int n_tensors, const float* x, int N, int B, int bits,
              const ibcu_prologue_t* pro, int op) {
    const int NC = B <= 8 ? 32 : 64, ncols = B * LIN_LIMBS;
    const int total_steps = N / LT_KCOLS;
    const size_t ring = bits == 8 ? (size_t)LT_STAGES8 * LT_A_STAGE : (size_t)LT_STAGES4 * LT_A_STAGE + (size_t)LT_RAW4 * LT_RAW_STAGE;
    const size_t fixed = ring + sizeof(LtShared) + 2048;
    const size_t per_step = (size_t)NC * LT_KCOLS;                                     // B-operand bytes per step
    size_t b_budget = 227 * 1024 - fixed;
    if (b_budget > LT_B_BUDGET) b_budget = LT_B_BUDGET;
    const int max_steps = (int)(b_budget / per_step);
    if (max_steps < 2) return IBCU_ERR_STATE;
    const int nks = (total_steps + max_steps - 1) / max_steps;
    const int slice_steps = (total_steps + nks - 1) / nks;
    const size_t smem = (((size_t)slice_steps * per_step + 1023) & ~(size_t)1023) + ring + sizeof(LtShared);
    LtParams p;
    memset(&p, 0, sizeof p);
    long total_rows = 0;
    int ntiles = 0;
    for (int i = 0; i < n_tensors; i++) {
        p.t[i] = { (const uint8_t*)tensors[i].w, tensors[i].scales, tensors[i].out, tensors[i].M,
                   tensors[i].out_stride, tensors[i].scales_fp32, tensors[i].epilogue, (int)total_rows, 0, 0, -1 };
        p.tile_start[i] = ntiles;
        ntiles += (tensors[i].M + LT_TILE - 1) / LT_TILE;
        total_rows += tensors[i].M;
    }
    for (int i = n_tensors; i <= 4; i++) p.tile_start[i] = ntiles;
    if (ntiles == 0) return IBCU_OK;
    GatherWait gw;
    ibcu_take_gather_wait_x(ctx, &gw, x, (size_t)B * N * sizeof(float));
    if (pro && pro->x2) ibcu_gather_wait_mark(ctx, &gw, pro->x2, (size_t)B * N * sizeof(float));
    ibcu_gather_wait_settle(ctx, &gw);
    {
        float* outs[4];
        for (int i = 0; i < n_tensors; i++) outs[i] = tensors[i].out;
        if (ibcu_push_match(ctx, outs, n_tensors)) {
            size_t bytes = 0;
            for (int i = 0; i < n_tensors; i++) bytes += (size_t)tensors[i].M * B * sizeof(float);
            ibcu_push_fill(ctx, &p.gp, bytes);
            for (int i = 0; i < n_tensors; i++) p.t[i].win_off = (long)((const char*)tensors[i].out - ctx->win_base);
        }
    }
    const int cols = slice_steps * LT_KCOLS, xs_ld = cols + 16;
    const size_t xpack_bytes = (((size_t)nks * ncols * xs_ld) + 255) & ~(size_t)255;
    const size_t xscale_bytes = (((size_t)B * nks * sizeof(float)) + 255) & ~(size_t)255;
    int rc = ibcu_reserve(ctx, &ctx->xpack, &ctx->xpack_bytes, xpack_bytes + xscale_bytes + (size_t)B * nks * LIN_LIMBS * sizeof(int));
    if (rc) return rc;
    int8_t* xpack = (int8_t*)ctx->xpack;
    float* xscale = (float*)((char*)ctx->xpack + xpack_bytes);
    int* xsum = (int*)((char*)ctx->xpack + xpack_bytes + xscale_bytes);
    p.n_tensors = n_tensors; p.total_rows = (int)total_rows; p.rowbytes = bits == 8 ? N : N / 2; p.N = N; p.B = B; p.NC = NC;
    p.nks = nks; p.slice_steps = slice_steps; p.total_steps = total_steps; p.xs_ld = xs_ld;
    p.xpack = xpack; p.xscale = xscale; p.xsum = xsum; p.err = ctx->kern_err;
    if (nks > 1) {
        rc = ibcu_reserve(ctx, &ctx->scratch, &ctx->scratch_bytes, (size_t)total_rows * nks * B * LIN_LIMBS * sizeof(int));
        if (rc) return rc;
        p.partial = (int*)ctx->scratch;
    }
    XSource xsrc = { x, pro ? pro->x2 : nullptr, pro ? (const __half*)pro->norm_w : nullptr, pro ? pro->eps : 0.0f, op,
                     op == IBCU_PRO_KNOWN_MAX ? pro->amax : nullptr, op == IBCU_PRO_KNOWN_MAX ? pro->n_amax : 0 };
    {
        const dim3 xg(nks, B);
        const int perm8 = bits == 4 ? 2 : 0;                                           // natural column order; limb sums for the nibble bias
        const int xthreads = cols > XREG_V * 4 * 512 ? 1024 : (cols >= 2048 ? 512 : 256);
        rc = xthreads == 1024 ? ibcu_launch(ctx, xprep_kernel<1024>, xg, dim3(1024), 0, 1, true, xsrc, N, cols, xs_ld, perm8, nks, 0, xpack, xscale, xsum, gw)
           : xthreads == 512  ? ibcu_launch(ctx, xprep_kernel<512>, xg, dim3(512), 0, 1, true, xsrc, N, cols, xs_ld, perm8, nks, 1, xpack, xscale, xsum, gw)
                              : ibcu_launch(ctx, xprep_kernel<256>, xg, dim3(256), 0, 1, true, xsrc, N, cols, xs_ld, perm8, nks, 1, xpack, xscale, xsum, gw);
        if (rc) return rc;
    }
    int per_slice = ctx->sm_count / nks;                                               // one block per SM
    if (per_slice < 1) per_slice = 1;
    if (per_slice > ntiles) per_slice = ntiles;
    const int grid = per_slice * nks;
    rc = bits == 8 ? launch_tc<8, LT_STAGES8, 1>(ctx, p, grid, smem) : launch_tc<4, LT_STAGES4, LT_RAW4>(ctx, p, grid, smem);
    if (rc || nks == 1) return rc;
    LinearParams fp;
    memset(&fp, 0, sizeof fp);
    for (int i = 0; i < n_tensors; i++) fp.t[i] = p.t[i];
    fp.n_tensors = n_tensors; fp.total_rows = (int)total_rows; fp.B = B; fp.nks = nks; fp.partial = p.partial; fp.xscale = xscale; fp.gp = p.gp;
    long outs = total_rows * B;
    int fgrid = (int)((outs + 255) / 256);
    if (fgrid > 4 * ctx->sm_count) fgrid = 4 * ctx->sm_count;
    return ibcu_launch(ctx, linear_finalize_kernel, dim3(fgrid), dim3(256), 0, 1, true, fp);
}

// Eight warps and 512-byte stages; the ring is as deep as two resident blocks per SM allow.
template <int BITS, int NCG>
int dispatch_shape(ibcu_ctx* ctx, const LinearParams& p, int grid, int rt, int stages, size_t smem_tail) {
    if (rt == 2) {
        if (stages >= 6) return launch_mma<BITS, NCG, 2, 8, 6>(ctx, p, grid, smem_tail);
        return launch_mma<BITS, NCG, 2, 8, 4>(ctx, p, grid, smem_tail);
    }
    if (stages >= 8) return launch_mma<BITS, NCG, 1, 8, 8>(ctx, p, grid, smem_tail);
    return launch_mma<BITS, NCG, 1, 8, 4>(ctx, p, grid, smem_tail);
}

}  // namespace

extern "C" void ibcu_linear_force_generic(ibcu_ctx* ctx, int on) { if (ctx) ctx->force_generic = on; }
extern "C" void ibcu_linear_use_tcgen05(ibcu_ctx* ctx, int on) { if (ctx) ctx->linear_tc = on; }

extern "C" int ibcu_linear(ibcu_ctx* ctx, const ibcu_linear_t* tensors, int n_tensors,
                           const float* x, int N, int B, int bits) {
    return ibcu_linear_ex(ctx, tensors, n_tensors, x, N, B, bits, nullptr);
}

extern "C" int ibcu_linear_ex(ibcu_ctx* ctx, const ibcu_linear_t* tensors, int n_tensors,
                              const float* x, int N, int B, int bits, const ibcu_prologue_t* pro) {
    IBCU_CHECK_CTX(ctx);
    const int op = pro ? pro->op : IBCU_PRO_NONE;
    IBCU_REQUIRE(ctx, op == IBCU_PRO_NONE || (op == IBCU_PRO_RMSNORM && pro->norm_w) || (op == IBCU_PRO_SILU_MUL && pro->x2) ||
                      (op == IBCU_PRO_KNOWN_MAX && pro->amax && pro->n_amax >= 1),
                 "ibcu_linear_ex: prologue %d lacks its operand", op);
    IBCU_REQUIRE(ctx, tensors && x, "ibcu_linear: null pointer");
    IBCU_REQUIRE(ctx, n_tensors >= 1 && n_tensors <= 4, "ibcu_linear: n_tensors=%d not in 1..4", n_tensors);
    IBCU_REQUIRE(ctx, bits == 4 || bits == 8, "ibcu_linear: bits=%d (4 or 8 supported)", bits);
    IBCU_REQUIRE(ctx, B >= 1 && B <= 32, "ibcu_linear: B=%d not in 1..32", B);
    IBCU_REQUIRE(ctx, N >= 1 && (bits == 8 || (N & 1) == 0), "ibcu_linear: N=%d invalid for %d-bit rows", N, bits);
    for (int i = 0; i < n_tensors; i++) {
        IBCU_REQUIRE(ctx, tensors[i].w && tensors[i].scales && tensors[i].out, "ibcu_linear: tensor %d has a null pointer", i);
        IBCU_REQUIRE(ctx, tensors[i].M >= 0 && tensors[i].out_stride >= tensors[i].M, "ibcu_linear: tensor %d M=%d stride=%d", i, tensors[i].M, tensors[i].out_stride);
    }
    const int rowbytes = bits == 8 ? N : N / 2;
    bool fast = !ctx->force_generic && (rowbytes % 16 == 0) && ((uintptr_t)x & 15) == 0 &&
                (!pro || ((((uintptr_t)pro->x2) & 15) == 0 && (((uintptr_t)pro->norm_w) & 3) == 0));
    for (int i = 0; i < n_tensors; i++) if (((uintptr_t)tensors[i].w & 15) != 0) fast = false;

    if (!fast) {
        if (op == IBCU_PRO_RMSNORM || op == IBCU_PRO_SILU_MUL) {
            // portable path: apply the prologue with the element-wise kernels into the context's activation buffer
            int rc0 = ibcu_reserve(ctx, &ctx->xpack, &ctx->xpack_bytes, (size_t)B * N * sizeof(float));
            if (rc0) return rc0;
            float* tmp = (float*)ctx->xpack;
            rc0 = op == IBCU_PRO_RMSNORM ? ibcu_rmsnorm_fp16w(ctx, tmp, x, pro->norm_w, pro->eps, N, B)
                                         : ibcu_silu_mul(ctx, tmp, x, pro->x2, (size_t)B * N);
            if (rc0) return rc0;
            x = tmp;
        }
        for (int i = 0; i < n_tensors; i++) {
            if (tensors[i].M == 0) continue;
            LinTensor T = { (const uint8_t*)tensors[i].w, tensors[i].scales, tensors[i].out, tensors[i].M,
                            tensors[i].out_stride, tensors[i].scales_fp32, tensors[i].epilogue, 0 };
            dim3 grid((tensors[i].M + 7) / 8);
            int rc = bits == 8 ? ibcu_launch(ctx, linear_generic_kernel<8>, grid, dim3(256), 0, 1, true, T, x, N, B)
                               : ibcu_launch(ctx, linear_generic_kernel<4>, grid, dim3(256), 0, 1, true, T, x, N, B);
            if (rc) return rc;
        }
        return IBCU_OK;
    }

    if (B > 16) {
        // sixteen activations fill the eight column groups of one pass; more go in a second pass
        ibcu_linear_t part[4];
        for (int b0 = 0; b0 < B; b0 += 16) {
            for (int i = 0; i < n_tensors; i++) { part[i] = tensors[i]; part[i].out = tensors[i].out + (size_t)b0 * tensors[i].out_stride; }
            ibcu_prologue_t pp; if (pro) { pp = *pro; if (pp.x2) pp.x2 += (size_t)b0 * N; if (pp.amax) pp.amax += (size_t)b0 * pp.n_amax; }
            int rc2 = ibcu_linear_ex(ctx, part, n_tensors, x + (size_t)b0 * N, N, B - b0 < 16 ? B - b0 : 16, bits, pro ? &pp : nullptr);
            if (rc2) return rc2;
        }
        return IBCU_OK;
    }
    long rows_all = 0;
    for (int i = 0; i < n_tensors; i++) rows_all += tensors[i].M;
    // linear_tc: 0 = automatic (the tcgen05 kernel where it was measured faster: INT4 tensors of many rows whose columns need at most
    // two slices), 1 = every INT4 call it can take, 2 = INT8 calls too, -1 = never
    const bool tc_auto = ctx->linear_tc == 0 && bits == 4 && B >= 5 && B <= 8 && N <= 4096 && rows_all >= 3072;
    if (B >= 5 && N % LT_KCOLS == 0 && (tc_auto || (ctx->linear_tc > 0 && (bits == 4 || ctx->linear_tc > 1)))) {       // enough activations for a GEMM: the tcgen05 kernel
        const int rc_tc = linear_tc(ctx, tensors, n_tensors, x, N, B, bits, pro, op);
        if (rc_tc != IBCU_ERR_STATE) return rc_tc;
    }
    const int ncols = B * LIN_LIMBS;
    const int ncg = (ncols + 7) / 8 <= 1 ? 1 : ((ncols + 7) / 8 <= 2 ? 2 : ((ncols + 7) / 8 <= 4 ? 4 : 8));
    const int nkb = (rowbytes + 63) / 64;
    const int xk = bits == 8 ? 64 : 128;
    const int xpad = bits == 8 ? 64 : 16;                     // keeps limb rows of neighbouring columns on different banks
    long total_rows = 0;
    for (int i = 0; i < n_tensors; i++) total_rows += tensors[i].M;
    if (total_rows == 0) return IBCU_OK;
    // Rows are dealt out evenly: every block of the persistent grid owns one contiguous run of rows and
    // walks it in tiles of up to R = 16 or 32 rows. 32-row tiles once a block's run is longer than 16.
    const int w = 8;                                          // warps per block; two blocks share an SM
    const int rt = (ncg >= 4 || total_rows <= 16L * 2 * ctx->sm_count) ? 1 : 2;
    const int R = 16 * rt;
    LinearParams p;
    memset(&p, 0, sizeof p);
    {
        int row_start = 0;
        for (int i = 0; i < n_tensors; i++) {
            p.t[i] = { (const uint8_t*)tensors[i].w, tensors[i].scales, tensors[i].out, tensors[i].M,
                       tensors[i].out_stride, tensors[i].scales_fp32, tensors[i].epilogue, row_start, 0, 0, -1 };
            row_start += tensors[i].M;
        }
    }
    // multi-GPU: a windowed exchange may be pending (wait in the first kernel of this call), and the outputs may be this
    // rank's slices of an announced gather (every result also goes, tagged, into the peers' windows from the epilogue)
    GatherWait gw;
    ibcu_take_gather_wait_x(ctx, &gw, x, (size_t)B * N * sizeof(float));
    if (pro && pro->x2) ibcu_gather_wait_mark(ctx, &gw, pro->x2, (size_t)B * N * sizeof(float));
    ibcu_gather_wait_settle(ctx, &gw);
    {
        float* outs[4];
        for (int i = 0; i < n_tensors; i++) outs[i] = tensors[i].out;
        if (ibcu_push_match(ctx, outs, n_tensors)) {
            size_t bytes = 0;
            for (int i = 0; i < n_tensors; i++) bytes += (size_t)tensors[i].M * B * sizeof(float);
            ibcu_push_fill(ctx, &p.gp, bytes);
            for (int i = 0; i < n_tensors; i++) p.t[i].win_off = (long)((const char*)tensors[i].out - ctx->win_base);
        }
    }
    // Shared memory per block: stage ring + reduction buffer + the slice's limbs. Columns are
    // split over several blocks only when the limbs of a whole row do not fit.
    const int kbs = w;
    const int LIN_LD = lin_ld(w);
    // ring depth: the deeper ring when two blocks per SM still fit with it, else the shallower one
    const size_t red_bytes = (size_t)(bits == 4 ? 2 : 1) * w * R * lin_rld(ncg) * 4;
    const size_t whole_row_pieces = (size_t)ncols * ((size_t)nkb * xk + xpad);
    int stages = rt == 2 ? 6 : 8;
    if (2 * ((size_t)stages * R * LIN_LD + red_bytes + whole_row_pieces + 2048) > 227 * 1024) stages = 4;
    const size_t fixed_smem = (size_t)stages * R * LIN_LD + red_bytes + 1024;
    const size_t smem_cap = 200 * 1024;
    long piece_budget = (long)smem_cap - (long)fixed_smem;
    int max_slice_kb = (int)((piece_budget / ncols - xpad) / xk) / kbs * kbs;
    if (max_slice_kb < kbs) max_slice_kb = kbs;
    int slice_kb = (nkb + kbs - 1) / kbs * kbs;               // whole stages per slice
    if (slice_kb > max_slice_kb) slice_kb = max_slice_kb;
    const int nks = (nkb + slice_kb - 1) / slice_kb;
    const int xs_ld = slice_kb * xk + xpad;
    const size_t piece_smem = (((size_t)ncols * xs_ld) + 15) & ~(size_t)15;
    // persistent grid: as many blocks as fit on the machine at once, a multiple of nks, at most one per item
    int fit = (int)((227 * 1024) / (fixed_smem + piece_smem + 1024));
    if (fit < 1) fit = 1;
    if (fit > 4) fit = 4;
    const int slots = fit * ctx->sm_count;
    int per_slice = slots / nks;
    if (per_slice < 1) per_slice = 1;
    // every tensor gets blocks in proportion to its rows, and its rows are dealt out evenly among them;
    // the run length grows until all blocks are resident at once
    int rows_per_block = (int)((total_rows + per_slice - 1) / per_slice);
    if (rows_per_block < 4) rows_per_block = 4;
    int nblk;
    for (;; rows_per_block++) {
        nblk = 0;
        for (int i = 0; i < n_tensors; i++) nblk += (tensors[i].M + rows_per_block - 1) / rows_per_block;
        if (nblk <= per_slice || rows_per_block >= total_rows) break;
    }
    nblk = 0;
    for (int i = 0; i < n_tensors; i++) {
        const int n = (tensors[i].M + rows_per_block - 1) / rows_per_block;
        p.t[i].blk_start = nblk;
        p.t[i].rows_per = n ? (tensors[i].M + n - 1) / n : 0;
        nblk += n;
    }
    const int grid = nblk * nks;

    const size_t xpack_bytes = (((size_t)nks * ncols * xs_ld) + 255) & ~(size_t)255;
    const size_t xscale_bytes = (((size_t)B * nks * sizeof(float)) + 255) & ~(size_t)255;
    int rc = ibcu_reserve(ctx, &ctx->xpack, &ctx->xpack_bytes, xpack_bytes + xscale_bytes + (size_t)B * nks * LIN_LIMBS * sizeof(int));
    if (rc) return rc;
    int8_t* xpack = (int8_t*)ctx->xpack;
    float* xscale = (float*)((char*)ctx->xpack + xpack_bytes);
    int* xsum = (int*)((char*)ctx->xpack + xpack_bytes + xscale_bytes);
    p.n_tensors = n_tensors; p.total_rows = (int)total_rows; p.rowbytes = rowbytes; p.nkb = nkb; p.N = N; p.B = B; p.ncols = ncols;
    p.slice_kb = slice_kb; p.nks = nks; p.xs_ld = xs_ld;
    p.xpack = xpack; p.xscale = xscale; p.xsum = xsum;
    if (nks > 1) {
        const size_t part_bytes = (size_t)total_rows * nks * B * LIN_LIMBS * sizeof(int);
        rc = ibcu_reserve(ctx, &ctx->scratch, &ctx->scratch_bytes, part_bytes);
        if (rc) return rc;
        p.partial = (int*)ctx->scratch;
    }
    XSource xsrc = { x, pro ? pro->x2 : nullptr, pro ? (const __half*)pro->norm_w : nullptr, pro ? pro->eps : 0.0f, op,
                     op == IBCU_PRO_KNOWN_MAX ? pro->amax : nullptr, op == IBCU_PRO_KNOWN_MAX ? pro->n_amax : 0 };
    // Cheap conversions are done by every block of the main kernel for itself (no extra launch, no
    // dependency chain); expensive ones (SiLU, several activations, long rows) once, by xprep_kernel.
    int fused = (op != IBCU_PRO_SILU_MUL && (long)B * slice_kb * xk <= 8192 && nks == 1) ? 1 : 0;
    if (op == IBCU_PRO_KNOWN_MAX && nks == 1 && B <= 2) fused = 1;          // no reduction: cheap at any row length
    p.xsrc = xsrc; p.fused_x = fused;
    // 512 threads hold up to 16384 columns in registers; longer slices take 1024 threads and the looping conversion
    const int xthreads = slice_kb * xk > XREG_V * 4 * 512 ? 1024 : (slice_kb * xk >= 2048 ? 512 : 256);
    if (!fused) {
        const dim3 xg(nks, B);
        const int perm8 = bits == 4 ? 1 : 0, cols = slice_kb * xk;
        rc = xthreads == 1024 ? ibcu_launch(ctx, xprep_kernel<1024>, xg, dim3(1024), 0, 1, true, xsrc, N, cols, xs_ld, perm8, nks, 0, xpack, xscale, xsum, gw)
           : xthreads == 512  ? ibcu_launch(ctx, xprep_kernel<512>, xg, dim3(512), 0, 1, true, xsrc, N, cols, xs_ld, perm8, nks, 1, xpack, xscale, xsum, gw)
                              : ibcu_launch(ctx, xprep_kernel<256>, xg, dim3(256), 0, 1, true, xsrc, N, cols, xs_ld, perm8, nks, 1, xpack, xscale, xsum, gw);
        gw.flags = nullptr; gw.tag.n = 0;                     // the conversion kernel has waited and received; the main kernel follows it
    }
    p.gw = gw;
    if (rc) return rc;
    const size_t smem = piece_smem + 32 * sizeof(float) + 32 * LIN_LIMBS * sizeof(int);
#define IBCU_DISPATCH(BITS) \
    switch (ncg) { \
        case 1: rc = dispatch_shape<BITS, 1>(ctx, p, grid, rt, stages, smem); break; \
        case 2: rc = dispatch_shape<BITS, 2>(ctx, p, grid, rt, stages, smem); break; \
        case 4: rc = dispatch_shape<BITS, 4>(ctx, p, grid, rt, stages, smem); break; \
        default: rc = dispatch_shape<BITS, 8>(ctx, p, grid, rt, stages, smem); break; \
    }
    if (bits == 8) { IBCU_DISPATCH(8) } else { IBCU_DISPATCH(4) }
#undef IBCU_DISPATCH
    if (rc) return rc;
    if (nks == 1) return rc;
    long outs = total_rows * B;
    int fgrid = (int)((outs + 255) / 256);
    if (fgrid > 4 * ctx->sm_count) fgrid = 4 * ctx->sm_count;
    return ibcu_launch(ctx, linear_finalize_kernel, dim3(fgrid), dim3(256), 0, 1, true, p);
}

// v1: the two projections in one launch, then the element-wise kernel over gate.out.
extern "C" int ibcu_linear_gate_up_silu(ibcu_ctx* ctx, const ibcu_linear_t* gate_up, const float* x, int N, int B, int bits) {
    IBCU_CHECK_CTX(ctx);
    IBCU_REQUIRE(ctx, gate_up && gate_up[0].M == gate_up[1].M && gate_up[0].out_stride == gate_up[1].out_stride,
                 "ibcu_linear_gate_up_silu: gate and up must have equal shapes");
    IBCU_REQUIRE(ctx, gate_up[0].epilogue == IBCU_EPI_STORE && gate_up[1].epilogue == IBCU_EPI_STORE, "ibcu_linear_gate_up_silu: store epilogue only");
    int rc = ibcu_linear(ctx, gate_up, 2, x, N, B, bits);
    if (rc) return rc;
    return ibcu_silu_mul(ctx, gate_up[0].out, gate_up[0].out, gate_up[1].out,
                         (size_t)(B - 1) * gate_up[0].out_stride + gate_up[0].M);
}
