// Group-scaled INT4 matvec (the INT4 tensors of the reference's session engine, src/pq_decode.c:3474-3483 for the
// layout, :3565-3651 for the arithmetic): two columns per byte (low nibble = even column, value = nibble - 8), one FP16
// scale per row and group of G columns,
//   out[m] = sum over groups g of scale[m][g] * (sum over the group's columns of (nibble - 8) * x[col])
//          + sum over k < K_out of outl_val[m][k] * x[outl_idx[m][k]]          (optional per-row outlier columns),
// with groups whose largest |x| is at most eps * max|x| left out when eps > 0 (build_skip_mask, :3854-3882; off by
// default there). HBM-bound: N/2 bytes of weights and 2 N/G bytes of scales per row, read once.
//
// Fast kernel (N and G multiples of 32), integer arithmetic: the activation becomes 32-bit fixed point (2^sh max|x| in
// [2^29, 2^30)), split into four balanced base-256 digits per column ("limbs"), and a row's 32-column chunk is 32 dp4a
// instructions: nibbles as bytes (even columns w & 0x0F0F0F0F, odd columns (w >> 4) & 0x0F0F0F0F) times the limb words of
// the same columns, one int32 sum per limb, exact. The chunk's value sum_k 256^k a_k - 8 sum(X) goes to FP32, times the
// group's scale into the row's sum. Against FP32 FMAs on unpacked nibbles (the first form of this kernel: four
// instructions per weight, 25 us for 14336 x 4096) this is 1.7 instructions per weight.
// The limb words sit in shared memory per chunk as eight 16-byte pieces (piece 2 j + e: limbs 0..3 of the even (e = 0)
// or odd columns of the chunk's j-th group of eight), rotated by chunk % 8 so that lanes reading consecutive chunks hit
// different banks. A warp owns two rows at a time; lane l takes chunks l, l + 32, ...; weights and scales come through a
// ring of asynchronous copies per warp, STAGES - 1 steps ahead of their use. A fixed butterfly adds the lanes. Sums are ordered differently from the
// reference's scalar loop and the activation is rounded to 2^-30 of its largest magnitude: equal to the reference within
// the float bar, not bit for bit; f(2x) = 2 f(x) exactly.
#include "common.cuh"
#include <mutex>

namespace {

constexpr int I4G_THREADS = 256;
constexpr int I4G_WARPS = I4G_THREADS / 32;
constexpr int I4G_ROWS = 2;                                  // rows a warp carries through a pass over the columns
constexpr int I4G_STAGES = 4;                                // steps of a warp's ring of weights in shared memory (a power of two)

struct I4gParams {
    int M, N, G, K_out;
    const uint8_t* q; const __half* s; const uint16_t* outl_idx; const __half* outl_val;
    const float* x; float* out;
    float eps;                                               // > 0: groups with max|x| <= eps * max|x| are left out
};

__device__ __forceinline__ void transpose4x4_bytes(uint32_t a, uint32_t b, uint32_t c, uint32_t d, uint32_t* o) {
    const uint32_t t0 = __byte_perm(a, b, 0x5140), t1 = __byte_perm(a, b, 0x7362);
    const uint32_t t2 = __byte_perm(c, d, 0x5140), t3 = __byte_perm(c, d, 0x7362);
    o[0] = __byte_perm(t0, t2, 0x5410); o[1] = __byte_perm(t0, t2, 0x7632);
    o[2] = __byte_perm(t1, t3, 0x5410); o[3] = __byte_perm(t1, t3, 0x7632);
}

template <int ROWS, int STAGES>
__global__ void __launch_bounds__(I4G_THREADS) int4g_kernel(const I4gParams p) {
    extern __shared__ __align__(16) uint32_t xl[];           // [N/32 chunks][8 pieces][4 limb words], then chunk sums (float), then skip flags
    __shared__ float red[I4G_WARPS];
    __shared__ float s_mul, s_back;
    pdl_launch_dependents();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nchunk = p.N >> 5, ng = p.N / p.G, cpg = p.G >> 5;     // chunks per group
    // group of a chunk: a shift when a group is a power-of-two number of chunks (runtime divisions in the step loop cost
    // as many instructions as the dot products they index)
    const int cpg_sh = (cpg & (cpg - 1)) == 0 ? 31 - __clz(cpg) : -1;
    auto group_of = [&](int c) { return cpg_sh >= 0 ? c >> cpg_sh : c / cpg; };
    float* sxs = reinterpret_cast<float*>(xl + p.N);
    unsigned char* skip = reinterpret_cast<unsigned char*>(sxs + ((nchunk + 3) & ~3));     // keeps the ring behind it 16-byte aligned
    // ── rows: a warp walks its tiles of ROWS rows, lane l the chunks l, l + 32, ...; (tile, pass over 32 chunks) form one
    //    sequence of steps, and the weights (16 bytes per lane and row) and scales of step q + STAGES - 1 are on their way
    //    into the warp's ring in shared memory while step q is worked on ──
    const uint4* wq = reinterpret_cast<const uint4*>(p.q);
    constexpr int STAGE_WORDS = ROWS * 32 * 5;                // per row 32 lanes x (16 bytes of weights + 4 bytes holding the scale)
    uint32_t* ring = reinterpret_cast<uint32_t*>(skip + ((ng + 15) & ~15)) + (size_t)warp * STAGES * STAGE_WORDS;
    const uint32_t ring_s = (uint32_t)__cvta_generic_to_shared(ring);
    const int npass = (nchunk + 31) >> 5;
    const int tile0 = blockIdx.x * I4G_WARPS + warp, tstride = gridDim.x * I4G_WARPS;
    const int ntile = (p.M + ROWS - 1) / ROWS;
    const int my_tiles = tile0 < ntile ? (ntile - tile0 + tstride - 1) / tstride : 0;
    const int nstep = my_tiles * npass;
    int iq = 0, ipass = 0, itile = tile0;                     // the step to request next, its pass and its tile
    auto issue = [&]() {                                      // requests the next step (nothing beyond the last: an empty group keeps the count)
        const int q = iq++;
        if (q < nstep) {
            const int tile = itile, c = lane + 32 * ipass;
            if (++ipass == npass) { ipass = 0; itile += tstride; }
            const int g = group_of(c < nchunk ? c : 0);
            const bool on = c < nchunk && !(p.eps > 0.0f && skip[g]);
            const uint32_t dst = ring_s + (uint32_t)((q & (STAGES - 1)) * STAGE_WORDS) * 4u;
#pragma unroll
            for (int u = 0; u < ROWS; u++) {
                const int r = min(tile * ROWS + u, p.M - 1);  // rows past the end repeat the last one and are not stored
                const int cc = on ? c : 0;
                const unsigned nb = on ? 16u : 0u;            // a chunk that is off is filled with zeros: scale 0 times 0
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"(dst + (uint32_t)(u * 32 + lane) * 16u), "l"(wq + (size_t)r * nchunk + cc), "r"(nb) : "memory");
                const uintptr_t sa = (uintptr_t)(p.s + (size_t)r * ng + (on ? g : 0)) & ~(uintptr_t)3;
                asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" :: "r"(dst + (uint32_t)(ROWS * 32 * 4 + u * 32 + lane) * 4u), "l"(sa), "r"(on ? 4u : 0u) : "memory");
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    // weights and scales do not depend on the kernel ahead: without the skip rule the first steps are requested before the wait
    // for it, and travel while the activation is converted
    const bool early = !(p.eps > 0.0f);
    if (early) {
#pragma unroll
        for (int q = 0; q < STAGES - 1; q++) issue();
    }
    pdl_wait();
    // max |x|, then the fixed-point scale: 2^sh max|x| in [2^29, 2^30)
    float amax = 0.0f;
    for (int i = tid; i < (p.N >> 2); i += I4G_THREADS) {
        const float4 v = __ldcg(reinterpret_cast<const float4*>(p.x) + i);
        amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
    }
    amax = warp_max(amax);
    if (lane == 0) red[warp] = amax;
    __syncthreads();
    amax = red[0];
#pragma unroll
    for (int w = 1; w < I4G_WARPS; w++) amax = fmaxf(amax, red[w]);
    if (tid == 0) {
        const int e = (int)((__float_as_uint(amax) >> 23) & 0xFF);   // amax in [2^(e-127), 2^(e-126))
        int sh = (amax > 0.0f && e != 255) ? 156 - e : 0;
        sh = max(-126, min(126, sh));
        s_mul = __uint_as_float((uint32_t)(127 + sh) << 23);
        s_back = __uint_as_float((uint32_t)(127 - sh) << 23);
    }
    if (p.eps > 0.0f) {
        const float thr = p.eps * amax;
        for (int g = tid; g < ng; g += I4G_THREADS) {
            float gm = 0.0f;
            for (int j = 0; j < p.G; j++) gm = fmaxf(gm, fabsf(__ldcg(p.x + g * p.G + j)));
            skip[g] = gm <= thr;
        }
    }
    __syncthreads();
    const float mul = s_mul, back = s_back;
    for (int base = 0; base < (p.N >> 3); base += I4G_THREADS) {   // eight columns per thread: group j of chunk c. Every lane of a warp
        const int i8 = base + tid;                                   // goes round the same number of times: the shuffles below take all 32
        const bool on = i8 < (p.N >> 3);
        const int c = i8 >> 2, j = i8 & 3;
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
        if (on) { a = __ldcg(reinterpret_cast<const float4*>(p.x) + 2 * i8); b = __ldcg(reinterpret_cast<const float4*>(p.x) + 2 * i8 + 1); }
        const int X[8] = { __float2int_rn(a.x * mul), __float2int_rn(a.y * mul), __float2int_rn(a.z * mul), __float2int_rn(a.w * mul),
                           __float2int_rn(b.x * mul), __float2int_rn(b.y * mul), __float2int_rn(b.z * mul), __float2int_rn(b.w * mul) };
        uint32_t D[8], ev[4], od[4];
        long long sum = 0;
#pragma unroll
        for (int i = 0; i < 8; i++) { D[i] = ((uint32_t)X[i] + 0x00808080u) ^ 0x00808080u; sum += X[i]; }   // the four balanced digits of X as bytes
        transpose4x4_bytes(D[0], D[2], D[4], D[6], ev);      // ev[k]: limb k of columns 0, 2, 4, 6
        transpose4x4_bytes(D[1], D[3], D[5], D[7], od);
        if (on) {
            reinterpret_cast<uint4*>(xl)[c * 8 + ((2 * j + c) & 7)] = make_uint4(ev[0], ev[1], ev[2], ev[3]);
            reinterpret_cast<uint4*>(xl)[c * 8 + ((2 * j + 1 + c) & 7)] = make_uint4(od[0], od[1], od[2], od[3]);
        }
        float fs = (float)sum;                                // the four groups of a chunk sit in four neighbouring lanes
        fs += __shfl_xor_sync(0xffffffffu, fs, 1);
        fs += __shfl_xor_sync(0xffffffffu, fs, 2);
        if (on && j == 0) sxs[c] = fs;
    }
    __syncthreads();
    if (!early) {
#pragma unroll
        for (int q = 0; q < STAGES - 1; q++) issue();
    }
    float acc[ROWS];
    int pass = 0, tile = tile0, stage = 0;
    for (int q = 0; q < nstep; q++) {
        const int r0 = tile * ROWS;
        if (pass == 0) {
#pragma unroll
            for (int u = 0; u < ROWS; u++) acc[u] = 0.0f;
        }
        asm volatile("cp.async.wait_group %0;" :: "n"(STAGES - 2) : "memory");
        __syncwarp();
        const int c = lane + 32 * pass;
        const uint32_t* st = ring + stage * STAGE_WORDS;
        uint4 w[ROWS];
        float sc[ROWS];
#pragma unroll
        for (int u = 0; u < ROWS; u++) {
            w[u] = reinterpret_cast<const uint4*>(st)[u * 32 + lane];
            const uint32_t pair = st[ROWS * 32 * 4 + u * 32 + lane];
            const int r = min(r0 + u, p.M - 1);
            const bool hi = (((uintptr_t)(p.s + (size_t)r * ng + group_of(c < nchunk ? c : 0))) & 2) != 0;
            sc[u] = __half2float(__ushort_as_half((unsigned short)(hi ? pair >> 16 : pair & 0xffffu)));
        }
        __syncwarp();                                         // every lane has taken its words: the stage may be refilled
        issue();
        if (c < nchunk) {
            uint32_t xw[32];
#pragma unroll
            for (int piece = 0; piece < 8; piece++) {
                const uint4 v = reinterpret_cast<const uint4*>(xl)[c * 8 + ((piece + c) & 7)];
                xw[4 * piece] = v.x; xw[4 * piece + 1] = v.y; xw[4 * piece + 2] = v.z; xw[4 * piece + 3] = v.w;
            }
            const float m8s = -8.0f * sxs[c];
#pragma unroll
            for (int u = 0; u < ROWS; u++) {
                const uint32_t ww[4] = { w[u].x, w[u].y, w[u].z, w[u].w };
                int a[4] = { 0, 0, 0, 0 };
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int we = (int)(ww[j] & 0x0F0F0F0Fu), wo = (int)((ww[j] >> 4) & 0x0F0F0F0Fu);
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        a[k] = __dp4a(we, (int)xw[(2 * j) * 4 + k], a[k]);
                        a[k] = __dp4a(wo, (int)xw[(2 * j + 1) * 4 + k], a[k]);
                    }
                }
                const float v = fmaf((float)a[3], 16777216.0f, fmaf((float)a[2], 65536.0f, fmaf((float)a[1], 256.0f, (float)a[0])));
                acc[u] = fmaf(sc[u], v + m8s, acc[u]);       // sum (nibble - 8) X = sum nibble X - 8 sum X
            }
        }
        if (pass == npass - 1) {
#pragma unroll
            for (int u = 0; u < ROWS; u++) {
                float t = acc[u] * back;
                if (p.K_out > 0) {                            // per-row outlier columns: FP16 value times the activation of the listed column
                    const int r = min(r0 + u, p.M - 1);
                    for (int k = lane; k < p.K_out; k += 32)
                        t = fmaf(__half2float(p.outl_val[(size_t)r * p.K_out + k]), __ldcg(p.x + p.outl_idx[(size_t)r * p.K_out + k]), t);
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
                if (lane == 0 && r0 + u < p.M) p.out[r0 + u] = t;
            }
        }
        if (++pass == npass) { pass = 0; tile += tstride; }
        stage = (stage + 1) & (STAGES - 1);
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// Any N, G (even): a warp per row, lanes over the groups, columns in order inside a group; activations from global memory.
__global__ void __launch_bounds__(I4G_THREADS) int4g_generic_kernel(const I4gParams p, const unsigned char* skip) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, ng = p.N / p.G;
    for (int r = blockIdx.x * I4G_WARPS + warp; r < p.M; r += gridDim.x * I4G_WARPS) {
        const uint8_t* qrow = p.q + (size_t)r * (p.N / 2);
        float acc = 0.0f;
        for (int g = lane; g < ng; g += 32) {
            if (skip && __ldcg(skip + g)) continue;          // written by the kernel just ahead
            float gs = 0.0f;
            for (int j = 0; j < p.G; j += 2) {
                const uint32_t b = qrow[(g * p.G + j) >> 1];
                gs = fmaf((float)((int)(b & 15u) - 8), __ldcg(p.x + g * p.G + j), gs);
                gs = fmaf((float)((int)(b >> 4) - 8), __ldcg(p.x + g * p.G + j + 1), gs);
            }
            acc = fmaf(__half2float(p.s[(size_t)r * ng + g]), gs, acc);
        }
        for (int k = lane; k < p.K_out; k += 32)
            acc = fmaf(__half2float(p.outl_val[(size_t)r * p.K_out + k]), __ldcg(p.x + p.outl_idx[(size_t)r * p.K_out + k]), acc);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane == 0) p.out[r] = acc;
    }
}

// skip[g] = max|x over group g| <= eps * max|x| (one block; for the generic kernel)
__global__ void __launch_bounds__(1024) int4g_skip_kernel(const float* x, int N, int G, float eps, unsigned char* __restrict__ skip) {
    __shared__ float red[32];
    pdl_launch_dependents();
    pdl_wait();
    float m = 0.0f;
    for (int i = threadIdx.x; i < N; i += 1024) m = fmaxf(m, fabsf(__ldcg(x + i)));
    m = warp_max(m);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    m = red[0];
    for (int w = 1; w < 32; w++) m = fmaxf(m, red[w]);
    const float thr = eps * m;
    for (int g = threadIdx.x; g < N / G; g += 1024) {
        float gm = 0.0f;
        for (int j = 0; j < G; j++) gm = fmaxf(gm, fabsf(__ldcg(x + g * G + j)));
        skip[g] = gm <= thr;
    }
}

}  // namespace

extern "C" int ibcu_int4g_matmul_fp32(ibcu_ctx* ctx, const ibcu_int4g_t* t, const float* x, float* out, float eps_act_rel) {
    IBCU_CHECK_CTX(ctx);
    IBCU_REQUIRE(ctx, t && x && out && t->q && t->s, "ibcu_int4g_matmul_fp32: null pointer");
    IBCU_REQUIRE(ctx, t->M > 0 && t->N > 0 && t->G > 0 && (t->G & 1) == 0 && t->N % t->G == 0 && t->K_out >= 0 && t->N <= 65536,
                 "ibcu_int4g_matmul_fp32: bad shape M=%d N=%d G=%d K_out=%d", t->M, t->N, t->G, t->K_out);
    IBCU_REQUIRE(ctx, t->K_out == 0 || (t->outl_idx && t->outl_val), "ibcu_int4g_matmul_fp32: outlier arrays missing");
    IBCU_REQUIRE(ctx, !(eps_act_rel < 0.0f) && eps_act_rel == eps_act_rel, "ibcu_int4g_matmul_fp32: eps_act_rel must be >= 0");
    I4gParams p;
    p.M = t->M; p.N = t->N; p.G = t->G; p.K_out = t->K_out;
    p.q = t->q; p.s = (const __half*)t->s; p.outl_idx = t->outl_idx; p.outl_val = (const __half*)t->outl_val;
    p.x = x; p.out = out; p.eps = eps_act_rel;
    const size_t xbytes = (size_t)t->N * sizeof(float) + (((size_t)(t->N / 32) + 3) & ~(size_t)3) * sizeof(float) + (((size_t)(t->N / t->G) + 15) & ~(size_t)15);
    const size_t smem = xbytes + (size_t)I4G_WARPS * I4G_STAGES * I4G_ROWS * 32 * 5 * sizeof(uint32_t);
    const bool fast = (t->N & 31) == 0 && (t->G & 31) == 0 && smem <= 200 * 1024 &&
                      (((uintptr_t)t->q | (uintptr_t)x) & 15) == 0 && ((uintptr_t)t->s & 3) == 0;
    if (fast) {
        static std::once_flag once[64];                      // dynamic shared memory beyond 48 KB: opt in once per device
        cudaError_t e = cudaSuccess;
        std::call_once(once[ctx->device & 63], [&] {
            e = cudaFuncSetAttribute(int4g_kernel<I4G_ROWS, I4G_STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        });
        if (e != cudaSuccess) return ibcu_fail(ctx, IBCU_ERR_CUDA, "cudaFuncSetAttribute(int4g_kernel): %s", cudaGetErrorString(e));
        // Two rows per warp (four measured slower on both benchmark shapes: 9.1 against 6.9 us and 15.0 against 14.3 us).
        // With more tiles than two blocks per SM can take, three blocks share an SM; with fewer, the launch asks for more
        // shared memory than it needs so that at most two do and the blocks spread over the SMs (256 blocks packed three
        // to an SM: 8.3 us; two to an SM: 6.9 us).
        const size_t ring = (size_t)I4G_WARPS * I4G_STAGES * I4G_ROWS * 32 * 5 * sizeof(uint32_t);
        const size_t need = xbytes + ring;
        const int tiles = (t->M + I4G_WARPS * I4G_ROWS - 1) / (I4G_WARPS * I4G_ROWS);
        const bool crowd = tiles > 2 * ctx->sm_count && need <= 70 * 1024;
        const size_t ask = crowd ? need : (need > 100 * 1024 ? need : 100 * 1024);
        const int per_sm = crowd ? 3 : (ask <= 110 * 1024 ? 2 : 1);
        const int slots = ctx->sm_count * per_sm;
        return ibcu_launch(ctx, int4g_kernel<I4G_ROWS, I4G_STAGES>, dim3(tiles < slots ? tiles : slots), dim3(I4G_THREADS), ask, 1, true, p);
    }
    unsigned char* skip = nullptr;
    if (eps_act_rel > 0.0f) {
        int rc = ibcu_reserve(ctx, &ctx->scratch, &ctx->scratch_bytes, (size_t)(t->N / t->G) + 16);
        if (rc) return rc;
        skip = (unsigned char*)ctx->scratch;
        rc = ibcu_launch(ctx, int4g_skip_kernel, dim3(1), dim3(1024), 0, 1, true, x, t->N, t->G, eps_act_rel, skip);
        if (rc) return rc;
    }
    const int blocks = (t->M + I4G_WARPS - 1) / I4G_WARPS;
    return ibcu_launch(ctx, int4g_generic_kernel, dim3(blocks < 4 * ctx->sm_count ? blocks : 4 * ctx->sm_count), dim3(I4G_THREADS), 0, 1, true, p,
                       (const unsigned char*)skip);
}
