// Shared definitions of the CUDA backend: context layout, error capture, launch helper with
// programmatic dependent launch, and a few device-side primitives used by several kernels.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>
#include "../../include/ibcu.h"

#define IBCU_MAX_GRAPHS 16
#define IBCU_MAX_EVENTS 16
#define IBCU_MAX_RANKS 16
#define IBCU_MAX_RETIRED 64

struct ncclComm;

struct ibcu_ctx {
    int device;
    int sm_count;
    cudaStream_t stream;
    int status;
    char msg[512];
    int pdl;                       // programmatic dependent launch between our kernels
    int force_generic;
    int kmeans_path;               // IBCU_KMEANS_*: which assignment kernel ibcu_kmeans_assign may take (tests)
    uint64_t launches;
    // scratch owned by the context, grown on demand (never shrinks)
    void*  xpack;      size_t xpack_bytes;      // activation limbs + per-slice scales and limb sums of the current linear call
    void*  scratch;    size_t scratch_bytes;    // partial sums (split-K slices, attention chunks, k-means per-block partials)
    void*  pq_acc;     size_t pq_acc_bytes;     // PQ matvec: arrival counters + fixed-point row accumulators, zero between calls
    void*  retired[IBCU_MAX_RETIRED]; int n_retired;   // outgrown scratch that an instantiated graph may still use
    cudaEvent_t events[IBCU_MAX_EVENTS];
    cudaGraphExec_t graphs[IBCU_MAX_GRAPHS];
    int capturing;
    // communicator (NULL when single GPU)
    ncclComm* comm;
    int rank, world;
    // peer window: a slab of this GPU's memory that the other ranks map and write their row slices into
    char*  win_base;   size_t win_bytes, win_used;
    char*  win_peer[IBCU_MAX_RANKS];               // win_peer[rank] == win_base
    int    win_open;                                // peers mapped so far
    int    win_enabled;
    int*   win_err;                                 // pinned, mapped: a push kernel that gave up waiting writes its epoch here
    int*   kern_err;                                // pinned, mapped, made with the context: a kernel whose bounded wait ran out writes a code here
    const void* win_last[4];                        // buffers of the previous push (a buffer is not pushed twice in a row)
};

int ibcu_fail(ibcu_ctx* ctx, int code, const char* fmt, ...);

#define IBCU_CHECK_CTX(ctx) do { if (!(ctx)) return IBCU_ERR_PARAM; } while (0)
#define IBCU_CUDA(ctx, expr) do { cudaError_t e_ = (expr); if (e_ != cudaSuccess) \
    return ibcu_fail((ctx), IBCU_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e_), __FILE__, __LINE__); } while (0)
#define IBCU_REQUIRE(ctx, cond, ...) do { if (!(cond)) return ibcu_fail((ctx), IBCU_ERR_PARAM, __VA_ARGS__); } while (0)

// Grow-only scratch. Growing reallocates, so it must not happen during stream capture. While the context
// holds instantiated graphs the outgrown buffer is kept (their kernels carry its address) until the
// last graph is destroyed.
int ibcu_reserve(ibcu_ctx* ctx, void** buf, size_t* have, size_t want);

// Launch `kernel` on the context's stream. With pdl_ok and ctx->pdl the launch carries the
// programmatic-stream-serialization attribute: the kernel may start while its predecessor drains,
// and must call pdl_wait() before touching anything the predecessor wrote.
template <typename... KArgs, typename... Args>
static inline int ibcu_launch(ibcu_ctx* ctx, void (*kernel)(KArgs...), dim3 grid, dim3 block,
                              size_t smem, int cluster_x, bool pdl_ok, Args... args) {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = ctx->stream;
    cudaLaunchAttribute attrs[2];
    int na = 0;
    if (cluster_x > 1) {
        attrs[na].id = cudaLaunchAttributeClusterDimension;
        attrs[na].val.clusterDim.x = cluster_x; attrs[na].val.clusterDim.y = 1; attrs[na].val.clusterDim.z = 1;
        na++;
    }
    if (pdl_ok && ctx->pdl) {
        attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[na].val.programmaticStreamSerializationAllowed = 1;
        na++;
    }
    cfg.attrs = attrs; cfg.numAttrs = na;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
    if (e != cudaSuccess)
        return ibcu_fail(ctx, IBCU_ERR_CUDA, "kernel launch failed: %s (grid %u,%u,%u block %u smem %zu cluster %d)",
                         cudaGetErrorString(e), grid.x, grid.y, grid.z, block.x, smem, cluster_x);
    ctx->launches++;
    return IBCU_OK;
}

// ── device helpers ──────────────────────────────────────────────────────────────────────
// Wait until every kernel this one depends on has finished and its writes are visible.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Allow the next kernel in the stream to begin launching.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// 128-bit streaming load that bypasses L1 allocation: weights and codes are read exactly once.
__device__ __forceinline__ uint4 ld_stream_u4(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ld_stream_u32(const void* p) {
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

__host__ __device__ __forceinline__ uint64_t ibcu_mix64(uint64_t seed, uint64_t ctr) {
    uint64_t z = seed + 0x9E3779B97F4A7C15ull * (ctr + 1);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
