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

// A tagged gather still to be received (n == 0: none): the plain buffers, this rank's own slice of each, and which of
// them the receiving kernel reads itself (all_mask): those are received in full by every block, the others are dealt
// out among the blocks.
struct TagDesc { size_t off; int stride, M, row0, rows; };     // plain buffer at byte offset off; [row0, row0 + rows) is this rank's own slice
struct TagParams { TagDesc d[4]; int n, B; char* base; size_t twin0; int* err; unsigned all_mask; };

struct ibcu_ctx {
    int device;
    int sm_count;
    cudaStream_t stream;
    int status;
    char msg[512];
    int pdl;                       // programmatic dependent launch between our kernels
    int force_generic;
    int linear_tc;                 // tcgen05 kernel for batched linears: 0 (default) where it was measured faster, 1 every INT4 call it can take, 2 INT8 calls too, -1 never
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
    char*  win_base;   size_t win_bytes, win_used;   // win_bytes: header + plain part (buffers); the tagged part of twice that size follows
    char*  win_peer[IBCU_MAX_RANKS];               // win_peer[rank] == win_base
    int    win_open;                                // peers mapped so far
    int    win_enabled;
    int*   win_err;                                 // pinned, mapped: a push kernel that gave up waiting writes its epoch here
    int*   spin_flag; int spin_seq;                 // pinned, mapped: the word ibcu_sync_spin's kernel writes and the host polls
    int*   kern_err;                                // pinned, mapped, made with the context: a kernel whose bounded wait ran out writes a code here
    const void* win_last[4];                        // buffers of the previous push (a buffer is not pushed twice in a row)
    // gathers announced ahead of the launches that produce their rows (ibcu_allgather_rows_prepare): the buffers, their
    // row strides, and which of them a linear launch has meanwhile pushed from its epilogue
    const char* arm_buf[4]; int arm_stride[4]; int arm_done[4]; int arm_n;
    int    gather_pending;                          // a linear launch has pushed its rows to the peers: the next kernel (or copy to the host) waits for theirs
    int    tag_pending; TagParams tag_p;            // a tagged gather whose receiving half has not been issued yet: the next linear call does it in its
                                                    // first kernel, anything else is preceded by the receiving kernel
    // exchange area inside the window (all-reduce of small tables, k-means): two buffers of world slots each, used in turn
    size_t exch_off, exch_slot; unsigned exch_turn;
};

// Window header, in units of 8 bytes: flags[r] is written by rank r (the epoch of its last finished push), then this
// rank's own epoch counter and the counter of blocks that have finished pushing in the current launch.
constexpr size_t IBCU_WIN_HEADER = 4096;
constexpr int IBCU_WIN_EPOCH_SLOT = IBCU_MAX_RANKS;
constexpr int IBCU_WIN_DONE_SLOT = IBCU_MAX_RANKS + 1;
constexpr int IBCU_WIN_GO_SLOT = IBCU_MAX_RANKS + 2;         // the epoch about to be published once every block of the pushing launch has arrived
constexpr int IBCU_WIN_TAG_SLOT = IBCU_MAX_RANKS + 3;        // number of tagged gathers this rank has received in full
constexpr int IBCU_WIN_TAG_DONE_SLOT = IBCU_MAX_RANKS + 4;   // blocks of the receiving kernel that are through
constexpr long IBCU_WIN_SPIN_LIMIT = 4L * 1000 * 1000;       // about a second of polling

// What a kernel needs to wait for the peers' rows of the gather that precedes it (flags == NULL and tag.n == 0: nothing).
struct GatherWait { const unsigned long long* flags; int world, rank; int* err; TagParams tag; };
// What a linear launch needs to store its rows into the peers' copies and to publish that it has (world == 0: no push).
struct GatherPush { char* peer[IBCU_MAX_RANKS]; unsigned long long* header; int world, rank, pushers; int* err; size_t twin0; };

// Every rank's table for a small all-reduce: rank r's copy sits at off + r * slot in every rank's window.
struct ExchSlots { GatherPush gp; size_t off, slot; };
// Next turn of the exchange area for tables of slot_bytes per rank. Returns 1 and fills *ex when the window can carry it
// (every rank mapped, area large enough or newly taken from the window), else 0: the caller uses NCCL.
int ibcu_exchange_begin(ibcu_ctx* ctx, size_t slot_bytes, ExchSlots* ex);
// sums, counts and inertia of a k-means iteration in one grouped NCCL call
int ibcu_allreduce_kmeans(ibcu_ctx* ctx, float* sums, size_t n_sums, int32_t* counts, size_t n_counts, double* inertia);

// Fills *gw when a push is pending and clears the pending state: the caller's kernel does the waiting in its prologue.
// A pending tagged gather is received by a kernel of its own first.
void ibcu_take_gather_wait(ibcu_ctx* ctx, GatherWait* gw);
// The same for a kernel that can receive a tagged gather itself (it calls gather_wait after its dependency wait and reads,
// of the gathered buffers, at most [x, x + x_bytes)): a pending tagged gather goes into *gw instead of a kernel of its own.
void ibcu_take_gather_wait_x(ibcu_ctx* ctx, GatherWait* gw, const void* x, size_t x_bytes);
// one more range the kernel reads itself; then, once all ranges are marked, the decision whether the kernel receives at all
void ibcu_gather_wait_mark(ibcu_ctx* ctx, GatherWait* gw, const void* x, size_t x_bytes);
void ibcu_gather_wait_settle(ibcu_ctx* ctx, GatherWait* gw);
// Launches a one-block kernel that does the waiting (for consumers that cannot: other kernels, copies to the host).
int ibcu_flush_gather_wait(ibcu_ctx* ctx);

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
    if (ctx->gather_pending || ctx->tag_pending) { int rc_ = ibcu_flush_gather_wait(ctx); if (rc_) return rc_; }     // this kernel does not wait by itself
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

__device__ __forceinline__ unsigned long long ld_acquire_sys_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys_u64(unsigned long long* p, unsigned long long v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" :: "l"(p), "l"(v) : "memory");
}
// Called by every thread of a block after pdl_wait(): the rows the peers pushed in the preceding gather are in place
// when it returns. The epoch to wait for is this rank's own (its last push, finished before this kernel's dependency
// wait returned). Bounded: a rank whose peers do not arrive gives up and raises the host-visible error word.
__device__ __forceinline__ uint2 ld_volatile_u2(const void* p) {       // one 8-byte load: value and tag as they were stored together
    uint2 v;
    asm volatile("ld.volatile.global.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}
// The receiving half of a tagged gather (see below), by all threads of all blocks of a kernel: polls the twins of the
// rows this rank does not own until they carry the gather's tag (bounded), copies the values into the plain buffers and,
// in the last block to finish, counts the gather. Elements of a buffer are dealt out among the blocks (blk of nblk), or
// all taken by every block when the kernel itself reads that buffer (all_mask). Returns the tag received.
__device__ __forceinline__ unsigned tag_receive(const TagParams& p, unsigned blk, unsigned nblk) {
    unsigned long long* header = reinterpret_cast<unsigned long long*>(p.base);
    const unsigned long long count = header[IBCU_WIN_TAG_SLOT];
    const unsigned tag = (unsigned)count + 1u;
    for (int i = 0; i < p.n; i++) {
        const TagDesc d = p.d[i];
        const int remote = d.M - d.rows;
        const long total = (long)p.B * remote;
        float* plain = reinterpret_cast<float*>(p.base + d.off);
        const uint2* twin = reinterpret_cast<const uint2*>(p.base + p.twin0 + 2 * (d.off - IBCU_WIN_HEADER));
        const bool all = (p.all_mask >> i) & 1u;
        const long step = (long)(all ? 1u : nblk) * blockDim.x;
        for (long e0 = (long)(all ? 0u : blk) * blockDim.x + threadIdx.x; e0 < total; e0 += 4 * step) {
            size_t idx[4];
            unsigned pending = 0;
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const long e = e0 + u * step;
                idx[u] = 0;
                if (e < total) {
                    const int b = (int)(e / remote), rr = (int)(e % remote);
                    idx[u] = (size_t)b * d.stride + (rr < d.row0 ? rr : rr + d.rows);
                    pending |= 1u << u;
                }
            }
            long it = 0;
            while (pending) {
                uint2 w[4];
#pragma unroll
                for (int u = 0; u < 4; u++) if (pending >> u & 1u) w[u] = ld_volatile_u2(twin + idx[u]);
#pragma unroll
                for (int u = 0; u < 4; u++)
                    if ((pending >> u & 1u) && w[u].y == tag) { plain[idx[u]] = __uint_as_float(w[u].x); pending &= ~(1u << u); }
                if (pending && ++it > IBCU_WIN_SPIN_LIMIT / 4) { *p.err = (int)tag; break; }       // give up: the host reports it at the next sync
            }
        }
    }
    __syncthreads();                                          // the block's own copies are in place for its own reads
    if (threadIdx.x == 0) {
        unsigned* done = reinterpret_cast<unsigned*>(header + IBCU_WIN_TAG_DONE_SLOT);
        if (atomicAdd(done, 1u) == nblk - 1) { *done = 0u; header[IBCU_WIN_TAG_SLOT] = count + 1; }
    }
    return tag;
}

// Called by every thread of every block after pdl_wait(). Returns the tag of the tagged gather it received, else 0: a
// kernel that goes on to push rows of its own must then use that tag + 1 (the count may or may not have moved yet).
__device__ __forceinline__ unsigned gather_wait(const GatherWait& g) {
    if (g.flags) {
        if ((int)threadIdx.x < g.world && (int)threadIdx.x != g.rank) {          // one thread per peer
            const unsigned long long e = g.flags[IBCU_WIN_EPOCH_SLOT];
            long it = 0;
            while (ld_acquire_sys_u64(g.flags + threadIdx.x) < e) {
                if (++it > IBCU_WIN_SPIN_LIMIT) { *g.err = (int)e; break; }
                __nanosleep(64);
            }
        }
        __syncthreads();
    }
    if (g.tag.n) {
        const unsigned nblk = gridDim.x * gridDim.y * gridDim.z;
        const unsigned blk = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
        return tag_receive(g.tag, blk, nblk);
    }
    return 0u;
}

// Tagged gather (the low-latency path of a gather whose rows a linear launch produces). The window has a second part
// of twice the size of the first: the float at byte offset off of the first part has an 8-byte twin at
// twin0 + 2 * (off - IBCU_WIN_HEADER), holding the value and a tag. The producing launch stores every result into its
// own buffer and, as {value, tag} in ONE 8-byte store, into the twin in every peer's window: no fence and no flag, the
// tag travels with the value. tag = number of tagged gathers received so far + 1, the same on every rank because every
// rank takes part in every gather; the receiving kernel (tag_unpack_kernel) polls the twins of the rows it does not own
// until they carry the tag, copies the values into the plain buffer and counts the gather. A zeroed window never
// matches (tags start at 1); the count wraps after 2^32 gathers.
__device__ __forceinline__ unsigned tag_current(const GatherPush& gp) { return (unsigned)gp.header[IBCU_WIN_TAG_SLOT] + 1u; }
__device__ __forceinline__ void tag_push(const GatherPush& gp, size_t off, float v, unsigned tag) {
    const size_t at = gp.twin0 + 2 * (off - IBCU_WIN_HEADER);
    const uint2 w = make_uint2(__float_as_uint(v), tag);
    for (int q = 0; q < gp.world; q++)
        if (q != gp.rank) asm volatile("st.volatile.global.v2.u32 [%0], {%1,%2};" :: "l"(gp.peer[q] + at), "r"(w.x), "r"(w.y) : "memory");
}

// The pushing half of a gather, at the end of the launch that produced the rows. Every block writes its results into
// this rank's own memory only; the last gp.pushers blocks to arrive (1 for a few KB, up to 16 for the large tables of a
// batched step) then copy them into the peers' windows, each its share, and the last of those to finish publishes. A
// system-scope fence in each of a few hundred blocks, every one with stores over NVLink in flight, was measured to
// spread the blocks' ends over about 8 us; a handful of fences is not.
//   const int j = push_arrive(gp);
//   if (j >= 0) { push_span(gp, j, ...); ...; push_finish(gp); }
// push_arrive is called by every thread of every block. It returns -1 in blocks that are done, and the pusher's index
// in the pushing blocks once every block of the grid has arrived. The pushing blocks that arrive before the last one
// wait for it (bounded); they are at most 16, so the blocks still to run always find room.
__device__ __forceinline__ int push_arrive(const GatherPush& gp) {
    __shared__ int s_j;
    __threadfence();                                          // this thread's results, visible to the blocks that will copy them
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned* done = reinterpret_cast<unsigned*>(gp.header + IBCU_WIN_DONE_SLOT);
        unsigned long long* go = gp.header + IBCU_WIN_GO_SLOT;
        const unsigned total = gridDim.x * gridDim.y * gridDim.z;
        const unsigned P = (unsigned)gp.pushers < total ? (unsigned)gp.pushers : total;
        const unsigned long long e = gp.header[IBCU_WIN_EPOCH_SLOT] + 1;       // the epoch this launch will publish
        const unsigned n = atomicAdd(done, 1u);
        int j = (int)n - (int)(total - P);
        if (n == total - 1) {
            asm volatile("st.release.gpu.global.u64 [%0], %1;" :: "l"(go), "l"(e) : "memory");
        } else if (j >= 0) {
            long it = 0;
            for (;;) {
                unsigned long long v;
                asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(go) : "memory");
                if (v >= e) break;
                if (++it > IBCU_WIN_SPIN_LIMIT) { *gp.err = (int)e; break; }
                __nanosleep(40);
            }
        }
        s_j = j;
    }
    __syncthreads();
    const int j = s_j;
    if (j >= 0) __threadfence();
    return j;
}
__device__ __forceinline__ int push_count(const GatherPush& gp) {
    const unsigned total = gridDim.x * gridDim.y * gridDim.z;
    return (unsigned)gp.pushers < total ? gp.pushers : (int)total;
}
// After a pushing block's copies: when the last pusher is through, this rank's epoch goes up by one and is written into
// every peer's flag word. Thread 0's system-scope fence is cumulative over the block's stores, which the barrier
// ordered before it; with several pushers the last one fences once more after it has seen the others' counts, which
// they raised after their own fences. The flag itself is then a plain (relaxed) system-scope store.
__device__ __forceinline__ void push_finish(const GatherPush& gp) {
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        unsigned* done = reinterpret_cast<unsigned*>(gp.header + IBCU_WIN_DONE_SLOT);
        const int P = push_count(gp);
        bool last = true;
        if (P > 1) {
            last = atomicAdd(done + 1, 1u) == (unsigned)P - 1;
            if (last) __threadfence_system();
        }
        if (last) {
            done[0] = 0u; done[1] = 0u;
            const unsigned long long e = gp.header[IBCU_WIN_EPOCH_SLOT] + 1;
            gp.header[IBCU_WIN_EPOCH_SLOT] = e;
            for (int q = 0; q < gp.world; q++)
                if (q != gp.rank)
                    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" :: "l"(reinterpret_cast<unsigned long long*>(gp.peer[q]) + gp.rank), "l"(e) : "memory");
        }
    }
}
// A table of `rows` spans, span r being n floats at src + r * stride (this rank's memory), into every peer's window at
// byte offset off + r * stride * 4: pusher j of P takes every P-th block-sized piece. VEC = 4 needs n, stride, src and
// off in multiples of 16 bytes. Four loads per thread are in flight before the first store.
template <int VEC>
__device__ __forceinline__ void push_table(const GatherPush& gp, int j, int P, const float* src, size_t off, int n, int rows, size_t stride) {
    const int per = n / VEC;
    const long total = (long)per * rows;
    const long step = (long)P * blockDim.x;
    for (long e0 = (long)j * blockDim.x + threadIdx.x; e0 < total; e0 += 4 * step) {
        float4 v[4];
        size_t at[4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const long e = e0 + u * step;
            if (e < total) {
                const int r = (int)(e / per), i = (int)(e % per);
                at[u] = ((size_t)r * stride + (size_t)i * VEC) * sizeof(float);
                if (VEC == 4) v[u] = __ldcg(reinterpret_cast<const float4*>(reinterpret_cast<const char*>(src) + at[u]));
                else v[u].x = __ldcg(reinterpret_cast<const float*>(reinterpret_cast<const char*>(src) + at[u]));
            }
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
            if (e0 + u * step < total) {
                for (int q = 0; q < gp.world; q++) {
                    if (q == gp.rank) continue;
                    if (VEC == 4) *reinterpret_cast<float4*>(gp.peer[q] + off + at[u]) = v[u];
                    else *reinterpret_cast<float*>(gp.peer[q] + off + at[u]) = v[u].x;
                }
            }
        }
    }
}
__device__ __forceinline__ void push_span(const GatherPush& gp, int j, int P, const float* src, size_t off, int n, int rows, size_t stride) {
    if ((((uintptr_t)src | off | (stride * sizeof(float))) & 15) == 0 && (n & 3) == 0) push_table<4>(gp, j, P, src, off, n, rows, stride);
    else push_table<1>(gp, j, P, src, off, n, rows, stride);
}

__host__ __device__ __forceinline__ uint64_t ibcu_mix64(uint64_t seed, uint64_t ctr) {
    uint64_t z = seed + 0x9E3779B97F4A7C15ull * (ctr + 1);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
