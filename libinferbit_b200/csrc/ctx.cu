// Context, memory, timing, graph capture and the counter-based fill kernels of the CUDA backend.
#include "common.cuh"
#include <stdarg.h>
#include <stdlib.h>

int ibcu_fail(ibcu_ctx* ctx, int code, const char* fmt, ...) {
    if (ctx && ctx->status == IBCU_OK) {
        ctx->status = code;
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(ctx->msg, sizeof ctx->msg, fmt, ap);
        va_end(ap);
    }
    return code;
}

int ibcu_reserve(ibcu_ctx* ctx, void** buf, size_t* have, size_t want) {
    if (*have >= want) return IBCU_OK;
    if (ctx->capturing) return ibcu_fail(ctx, IBCU_ERR_STATE, "scratch would have to grow to %zu bytes during graph capture; run the call once before capturing", want);
    IBCU_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (*buf) {
        bool graphs = false;
        for (int i = 0; i < IBCU_MAX_GRAPHS; i++) graphs = graphs || ctx->graphs[i];
        if (graphs) {
            if (ctx->n_retired == IBCU_MAX_RETIRED)
                return ibcu_fail(ctx, IBCU_ERR_STATE, "scratch would have to grow to %zu bytes while %d outgrown buffers are still held for "
                                 "instantiated graphs; destroy the graphs first", want, IBCU_MAX_RETIRED);
            ctx->retired[ctx->n_retired++] = *buf;
        } else IBCU_CUDA(ctx, cudaFree(*buf));
    }
    *buf = nullptr; *have = 0;
    size_t sz = (want + 255) & ~(size_t)255;
    cudaError_t e = cudaMalloc(buf, sz);
    if (e != cudaSuccess) return ibcu_fail(ctx, IBCU_ERR_NOMEM, "cudaMalloc(%zu) failed: %s", sz, cudaGetErrorString(e));
    *have = sz;
    return IBCU_OK;
}

extern "C" int ibcu_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) { cudaGetLastError(); return 0; }
    return n;
}

extern "C" int ibcu_ctx_create(int device, ibcu_ctx** out) {
    if (!out) return IBCU_ERR_PARAM;
    *out = nullptr;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || device < 0 || device >= n) { cudaGetLastError(); return IBCU_ERR_CUDA; }
    if (cudaSetDevice(device) != cudaSuccess) return IBCU_ERR_CUDA;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return IBCU_ERR_CUDA;
    if (prop.major != 10) {
        fprintf(stderr, "ibcu: device %d is sm_%d%d; this library is built for sm_100a only\n", device, prop.major, prop.minor);
        return IBCU_ERR_CUDA;
    }
    ibcu_ctx* ctx = (ibcu_ctx*)calloc(1, sizeof(ibcu_ctx));
    if (!ctx) return IBCU_ERR_NOMEM;
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    ctx->pdl = 1;
    ctx->world = 1;
    if (cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess) { free(ctx); return IBCU_ERR_CUDA; }
    for (int i = 0; i < IBCU_MAX_EVENTS; i++)
        if (cudaEventCreate(&ctx->events[i]) != cudaSuccess) { free(ctx); return IBCU_ERR_CUDA; }
    if (cudaHostAlloc((void**)&ctx->kern_err, sizeof(int), cudaHostAllocMapped) != cudaSuccess) { free(ctx); return IBCU_ERR_NOMEM; }
    *ctx->kern_err = 0;
    if (cudaHostAlloc((void**)&ctx->spin_flag, sizeof(int), cudaHostAllocMapped) == cudaSuccess) *ctx->spin_flag = 0;
    else { ctx->spin_flag = nullptr; cudaGetLastError(); }      // without the word ibcu_sync_spin is ibcu_sync
    *out = ctx;
    return IBCU_OK;
}

void ibcu_comm_destroy_internal(ibcu_ctx* ctx);

extern "C" void ibcu_ctx_destroy(ibcu_ctx* ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    // graphs first: a captured collective keeps a reference to the communicator, and destroying the
    // communicator while such a graph is alive blocks
    for (int i = 0; i < IBCU_MAX_GRAPHS; i++) if (ctx->graphs[i]) { cudaGraphExecDestroy(ctx->graphs[i]); ctx->graphs[i] = nullptr; }
    ibcu_comm_destroy_internal(ctx);
    for (int i = 0; i < IBCU_MAX_EVENTS; i++) cudaEventDestroy(ctx->events[i]);
    for (int i = 0; i < ctx->n_retired; i++) cudaFree(ctx->retired[i]);
    if (ctx->xpack) cudaFree(ctx->xpack);
    if (ctx->scratch) cudaFree(ctx->scratch);
    if (ctx->pq_acc) cudaFree(ctx->pq_acc);
    if (ctx->kern_err) cudaFreeHost(ctx->kern_err);
    if (ctx->spin_flag) cudaFreeHost(ctx->spin_flag);
    cudaStreamDestroy(ctx->stream);
    free(ctx);
}

extern "C" int ibcu_status(const ibcu_ctx* ctx) { return ctx ? ctx->status : IBCU_ERR_PARAM; }
extern "C" const char* ibcu_last_error(const ibcu_ctx* ctx) { return ctx ? ctx->msg : "null context"; }
extern "C" void ibcu_clear_error(ibcu_ctx* ctx) { if (ctx) { ctx->status = IBCU_OK; ctx->msg[0] = 0; } }
extern "C" int ibcu_device_sm_count(const ibcu_ctx* ctx) { return ctx ? ctx->sm_count : 0; }
extern "C" uint64_t ibcu_launch_count(const ibcu_ctx* ctx) { return ctx ? ctx->launches : 0; }
extern "C" void ibcu_set_pdl(ibcu_ctx* ctx, int enabled) { if (ctx) ctx->pdl = enabled ? 1 : 0; }

extern "C" int ibcu_malloc(ibcu_ctx* ctx, size_t bytes, void** dptr) {
    IBCU_CHECK_CTX(ctx);
    if (!dptr) return ibcu_fail(ctx, IBCU_ERR_PARAM, "ibcu_malloc: null out pointer");
    *dptr = nullptr;
    cudaSetDevice(ctx->device);
    cudaError_t e = cudaMalloc(dptr, bytes ? bytes : 1);
    if (e != cudaSuccess) return ibcu_fail(ctx, IBCU_ERR_NOMEM, "cudaMalloc(%zu) failed: %s", bytes, cudaGetErrorString(e));
    return IBCU_OK;
}
extern "C" int ibcu_free(ibcu_ctx* ctx, void* dptr) {
    IBCU_CHECK_CTX(ctx);
    if (!dptr) return IBCU_OK;
    if (ctx->win_base && (char*)dptr >= ctx->win_base && (char*)dptr < ctx->win_base + ctx->win_bytes) return IBCU_OK;   // window memory goes with the window
    IBCU_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    IBCU_CUDA(ctx, cudaFree(dptr));
    return IBCU_OK;
}
extern "C" int ibcu_host_alloc(ibcu_ctx* ctx, size_t bytes, void** hptr) {
    IBCU_CHECK_CTX(ctx);
    if (!hptr) return ibcu_fail(ctx, IBCU_ERR_PARAM, "ibcu_host_alloc: null out pointer");
    cudaError_t e = cudaHostAlloc(hptr, bytes ? bytes : 1, cudaHostAllocMapped | cudaHostAllocPortable);   // device-visible at the same address
    if (e != cudaSuccess) return ibcu_fail(ctx, IBCU_ERR_NOMEM, "cudaHostAlloc(%zu) failed: %s", bytes, cudaGetErrorString(e));
    return IBCU_OK;
}
extern "C" int ibcu_host_free(ibcu_ctx* ctx, void* hptr) {
    IBCU_CHECK_CTX(ctx);
    if (hptr) IBCU_CUDA(ctx, cudaFreeHost(hptr));
    return IBCU_OK;
}
extern "C" int ibcu_memcpy_h2d(ibcu_ctx* ctx, void* dst, const void* src, size_t bytes) {
    IBCU_CHECK_CTX(ctx);
    if (bytes) IBCU_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, ctx->stream));
    return IBCU_OK;
}
extern "C" int ibcu_memcpy_d2h(ibcu_ctx* ctx, void* dst, const void* src, size_t bytes) {
    IBCU_CHECK_CTX(ctx);
    { int rc = ibcu_flush_gather_wait(ctx); if (rc) return rc; }      // the source may be a gathered buffer whose peers' rows are still on their way
    if (bytes) IBCU_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    return IBCU_OK;
}
extern "C" int ibcu_memcpy_d2d(ibcu_ctx* ctx, void* dst, const void* src, size_t bytes) {
    IBCU_CHECK_CTX(ctx);
    { int rc = ibcu_flush_gather_wait(ctx); if (rc) return rc; }
    if (bytes) IBCU_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
    return IBCU_OK;
}
extern "C" int ibcu_memset(ibcu_ctx* ctx, void* dst, int byte, size_t bytes) {
    IBCU_CHECK_CTX(ctx);
    if (bytes) IBCU_CUDA(ctx, cudaMemsetAsync(dst, byte, bytes, ctx->stream));
    return IBCU_OK;
}
// what a kernel that gave up a bounded wait left behind, turned into the call's error
static int ibcu_collect_kernel_errors(ibcu_ctx* ctx) {
    if (ctx->win_err && *(volatile int*)ctx->win_err) {
        const int e = *(volatile int*)ctx->win_err;
        *(volatile int*)ctx->win_err = 0;
        return ibcu_fail(ctx, IBCU_ERR_COMM, "all-gather %d: a peer's rows did not arrive within the wait limit", e);
    }
    if (ctx->kern_err && *(volatile int*)ctx->kern_err) {
        const int e = *(volatile int*)ctx->kern_err;
        *(volatile int*)ctx->kern_err = 0;
        return ibcu_fail(ctx, IBCU_ERR_CUDA, "a kernel gave up a bounded wait (code %d): its results are not valid", e);
    }
    return ctx->status;
}

extern "C" int ibcu_sync(ibcu_ctx* ctx) {
    IBCU_CHECK_CTX(ctx);
    if (!ctx->capturing) { int rc = ibcu_flush_gather_wait(ctx); if (rc) return rc; }
    IBCU_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return ibcu_collect_kernel_errors(ctx);
}

// A one-thread kernel at the end of the stream's work writes a sequence number into a word of pinned host memory, and the
// host polls that word: the result is seen a few microseconds sooner than through the driver's wait, which matters when a
// call is a 5 us kernel between two small copies. The poll is bounded (about two seconds); after that, or when the launch
// fails, the driver's wait takes over and reports what went wrong.
__global__ void signal_kernel(volatile int* flag, int seq) {
    pdl_launch_dependents();
    pdl_wait();
    *flag = seq;
    __threadfence_system();
}
extern "C" int ibcu_sync_spin(ibcu_ctx* ctx) {
    IBCU_CHECK_CTX(ctx);
    if (ctx->capturing || !ctx->spin_flag) return ibcu_sync(ctx);
    { int rc = ibcu_flush_gather_wait(ctx); if (rc) return rc; }
    const int seq = ++ctx->spin_seq;
    if (ibcu_launch(ctx, signal_kernel, dim3(1), dim3(1), 0, 1, true, (volatile int*)ctx->spin_flag, seq) != IBCU_OK) return ibcu_sync(ctx);
    volatile int* flag = (volatile int*)ctx->spin_flag;
    for (long it = 0; it < 400L * 1000 * 1000; it++) {
        if (*flag == seq) return ibcu_collect_kernel_errors(ctx);
#if defined(__x86_64__)
        __builtin_ia32_pause();
#endif
    }
    return ibcu_sync(ctx);
}

__global__ void store_i32_kernel(int32_t* dst, int32_t value) { *dst = value; }
extern "C" int ibcu_store_i32(ibcu_ctx* ctx, int32_t* dst, int32_t value) {
    IBCU_CHECK_CTX(ctx);
    IBCU_REQUIRE(ctx, dst, "ibcu_store_i32: null pointer");
    return ibcu_launch(ctx, store_i32_kernel, dim3(1), dim3(1), 0, 1, false, dst, value);
}

// ── timing and graphs ───────────────────────────────────────────────────────────────────
extern "C" int ibcu_event_record(ibcu_ctx* ctx, int slot) {
    IBCU_CHECK_CTX(ctx);
    IBCU_REQUIRE(ctx, slot >= 0 && slot < IBCU_MAX_EVENTS, "event slot %d out of range", slot);
    { int rc = ibcu_flush_gather_wait(ctx); if (rc) return rc; }      // a timed region ends when its gathers have ended
    IBCU_CUDA(ctx, cudaEventRecord(ctx->events[slot], ctx->stream));
    return IBCU_OK;
}
extern "C" int ibcu_event_elapsed_ms(ibcu_ctx* ctx, int a, int b, float* ms) {
    IBCU_CHECK_CTX(ctx);
    IBCU_REQUIRE(ctx, ms && a >= 0 && a < IBCU_MAX_EVENTS && b >= 0 && b < IBCU_MAX_EVENTS, "bad event slots %d,%d", a, b);
    IBCU_CUDA(ctx, cudaEventSynchronize(ctx->events[b]));
    IBCU_CUDA(ctx, cudaEventElapsedTime(ms, ctx->events[a], ctx->events[b]));
    return IBCU_OK;
}
extern "C" int ibcu_graph_begin(ibcu_ctx* ctx) {
    IBCU_CHECK_CTX(ctx);
    if (ctx->capturing) return ibcu_fail(ctx, IBCU_ERR_STATE, "graph capture already in progress");
    IBCU_CUDA(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
    ctx->capturing = 1;
    return IBCU_OK;
}
extern "C" int ibcu_graph_end(ibcu_ctx* ctx, int* graph_id) {
    IBCU_CHECK_CTX(ctx);
    if (!ctx->capturing) return ibcu_fail(ctx, IBCU_ERR_STATE, "no graph capture in progress");
    ibcu_flush_gather_wait(ctx);                              // a replay is complete in itself: it ends with the wait for its last gather
    ctx->capturing = 0;
    cudaGraph_t g = nullptr;
    IBCU_CUDA(ctx, cudaStreamEndCapture(ctx->stream, &g));
    int slot = -1;
    for (int i = 0; i < IBCU_MAX_GRAPHS; i++) if (!ctx->graphs[i]) { slot = i; break; }
    if (slot < 0) { cudaGraphDestroy(g); return ibcu_fail(ctx, IBCU_ERR_STATE, "all %d graph slots in use", IBCU_MAX_GRAPHS); }
    cudaError_t e = cudaGraphInstantiate(&ctx->graphs[slot], g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) { ctx->graphs[slot] = nullptr; return ibcu_fail(ctx, IBCU_ERR_CUDA, "cudaGraphInstantiate failed: %s", cudaGetErrorString(e)); }
    if (graph_id) *graph_id = slot;
    return IBCU_OK;
}
extern "C" int ibcu_graph_launch(ibcu_ctx* ctx, int id) {
    IBCU_CHECK_CTX(ctx);
    IBCU_REQUIRE(ctx, id >= 0 && id < IBCU_MAX_GRAPHS && ctx->graphs[id], "no graph with id %d", id);
    IBCU_CUDA(ctx, cudaGraphLaunch(ctx->graphs[id], ctx->stream));
    return IBCU_OK;
}
extern "C" int ibcu_graph_destroy(ibcu_ctx* ctx, int id) {
    IBCU_CHECK_CTX(ctx);
    IBCU_REQUIRE(ctx, id >= 0 && id < IBCU_MAX_GRAPHS && ctx->graphs[id], "no graph with id %d", id);
    IBCU_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    IBCU_CUDA(ctx, cudaGraphExecDestroy(ctx->graphs[id]));
    ctx->graphs[id] = nullptr;
    bool graphs = false;
    for (int i = 0; i < IBCU_MAX_GRAPHS; i++) graphs = graphs || ctx->graphs[i];
    if (!graphs) {                                            // nothing can refer to the outgrown scratch buffers any more
        for (int i = 0; i < ctx->n_retired; i++) cudaFree(ctx->retired[i]);
        ctx->n_retired = 0;
    }
    return IBCU_OK;
}

// ── counter-based fills ─────────────────────────────────────────────────────────────────
// word w of the destination holds mix64(seed, first_word + w): a slice of a larger array gets the bytes
// the whole array would have at that place
__global__ void fill_hash_bytes_kernel(uint64_t* __restrict__ dst, size_t words, uint8_t* __restrict__ tail_dst,
                                       int tail, uint64_t seed, size_t first_word) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t w = i; w < words; w += stride) dst[w] = ibcu_mix64(seed, first_word + w);
    if (i == 0 && tail) {
        uint64_t v = ibcu_mix64(seed, first_word + words);
        for (int t = 0; t < tail; t++) tail_dst[t] = (uint8_t)(v >> (8 * t));
    }
}

extern "C" int ibcu_fill_hash_bytes_at(ibcu_ctx* ctx, void* dst, size_t bytes, uint64_t seed, size_t first_byte) {
    IBCU_CHECK_CTX(ctx);
    IBCU_REQUIRE(ctx, dst && ((uintptr_t)dst & 7) == 0, "ibcu_fill_hash_bytes: dst must be 8-byte aligned");
    IBCU_REQUIRE(ctx, (first_byte & 7) == 0, "ibcu_fill_hash_bytes_at: first_byte must be a multiple of 8");
    if (!bytes) return IBCU_OK;
    size_t words = bytes / 8;
    int tail = (int)(bytes % 8);
    int blocks = (int)((words + 255) / 256);
    if (blocks > ctx->sm_count * 16) blocks = ctx->sm_count * 16;
    if (blocks < 1) blocks = 1;
    return ibcu_launch(ctx, fill_hash_bytes_kernel, dim3(blocks), dim3(256), 0, 1, false,
                       (uint64_t*)dst, words, (uint8_t*)dst + words * 8, tail, seed, first_byte / 8);
}
extern "C" int ibcu_fill_hash_bytes(ibcu_ctx* ctx, void* dst, size_t bytes, uint64_t seed) {
    return ibcu_fill_hash_bytes_at(ctx, dst, bytes, seed, 0);
}

extern "C" void ibcu_hash_bytes_host(void* dst, size_t bytes, uint64_t seed, size_t first_byte) {
    uint8_t* d = (uint8_t*)dst;
    for (size_t i = 0; i < bytes; i++) {
        size_t g = first_byte + i;
        d[i] = (uint8_t)(ibcu_mix64(seed, g / 8) >> (8 * (g % 8)));
    }
}

// 16-bit draw -> u in [0,1) -> lo + (hi-lo)*u (multiply and add rounded separately) -> fp16 RNE.
__host__ __device__ static inline float hash_uniform(uint64_t seed, size_t i, float lo, float hi) {
    uint32_t r = (uint32_t)(ibcu_mix64(seed, i / 4) >> (16 * (i % 4))) & 0xFFFFu;
    float u = (float)r * (1.0f / 65536.0f);
#ifdef __CUDA_ARCH__
    return __fadd_rn(lo, __fmul_rn(hi - lo, u));
#else
    volatile float prod = (hi - lo) * u;
    return lo + prod;
#endif
}

__global__ void fill_hash_fp16_kernel(__half* __restrict__ dst, size_t count, uint64_t seed, float lo, float hi, size_t first) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < count; i += stride) dst[i] = __float2half_rn(hash_uniform(seed, first + i, lo, hi));
}

extern "C" int ibcu_fill_hash_fp16_uniform_at(ibcu_ctx* ctx, void* dst, size_t count, uint64_t seed, float lo, float hi, size_t first) {
    IBCU_CHECK_CTX(ctx);
    if (!count) return IBCU_OK;
    int blocks = (int)((count + 255) / 256);
    if (blocks > ctx->sm_count * 16) blocks = ctx->sm_count * 16;
    return ibcu_launch(ctx, fill_hash_fp16_kernel, dim3(blocks), dim3(256), 0, 1, false, (__half*)dst, count, seed, lo, hi, first);
}
extern "C" int ibcu_fill_hash_fp16_uniform(ibcu_ctx* ctx, void* dst, size_t count, uint64_t seed, float lo, float hi) {
    return ibcu_fill_hash_fp16_uniform_at(ctx, dst, count, seed, lo, hi, 0);
}

// FP32 values mean + std * z, z the centred sum of the four 16-bit pieces of mix64(seed, i) scaled to unit
// variance (Irwin-Hall with n = 4: bell-shaped, |z| <= 3.46)
__global__ void fill_hash_f32_normal_kernel(float* __restrict__ dst, size_t count, uint64_t seed, float mean, float std, size_t first) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < count; i += stride) {
        const uint64_t r = ibcu_mix64(seed, first + i);
        const float u = (float)((uint32_t)(r & 0xFFFF) + (uint32_t)((r >> 16) & 0xFFFF) + (uint32_t)((r >> 32) & 0xFFFF) + (uint32_t)(r >> 48)) * (1.0f / 65536.0f);
        dst[i] = mean + std * ((u - 2.0f) * 1.7320508f);
    }
}
extern "C" int ibcu_fill_hash_f32_normal_at(ibcu_ctx* ctx, float* dst, size_t count, uint64_t seed, float mean, float std, size_t first) {
    IBCU_CHECK_CTX(ctx);
    if (!count) return IBCU_OK;
    int blocks = (int)((count + 255) / 256);
    if (blocks > ctx->sm_count * 16) blocks = ctx->sm_count * 16;
    return ibcu_launch(ctx, fill_hash_f32_normal_kernel, dim3(blocks), dim3(256), 0, 1, false, dst, count, seed, mean, std, first);
}

static uint16_t host_f32_to_f16_rne(float f) {
    uint32_t x; memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    int e = (int)((x >> 23) & 255) - 112;
    uint32_t m = x & 0x7FFFFFu;
    if (e >= 31) return (uint16_t)(sign | 0x7C00u | (((x >> 23) & 255) == 255 && m ? 0x200u : 0));
    if (e <= 0) {
        if (e < -10) return (uint16_t)sign;
        m = (m | 0x800000u);
        int sh = 14 - e;
        uint32_t keep = m >> sh, rest = m & ((1u << sh) - 1), half = 1u << (sh - 1);
        if (rest > half || (rest == half && (keep & 1))) keep++;
        return (uint16_t)(sign | keep);
    }
    uint32_t keep = m >> 13, rest = m & 0x1FFFu;
    if (rest > 0x1000u || (rest == 0x1000u && (keep & 1))) keep++;
    return (uint16_t)(sign + ((uint32_t)e << 10) + keep);     // a mantissa carry bumps the exponent
}

extern "C" void ibcu_hash_fp16_uniform_host(uint16_t* dst, size_t count, uint64_t seed, float lo, float hi, size_t first) {
    for (size_t i = 0; i < count; i++) dst[i] = host_f32_to_f16_rne(hash_uniform(seed, first + i, lo, hi));
}
