// Multi-GPU plumbing: one process per GPU over NVLink/NVSwitch. The hot path has exactly two exchange
// steps: the all-gather of row-sharded linear outputs (a push over peer memory when the ranks have
// mapped each other's windows, else NCCL) and the all-reduce of k-means centroid sums / counts (NCCL).
// Everything else is replicated.
#include "common.cuh"
#include <nccl.h>
#include <dlfcn.h>

// NCCL is bound at run time, on the first communicator call, not at link time: a process that also
// loads PyTorch must end up with exactly one libnccl.so.2 (PyTorch ships its own, newer one), and
// single-GPU users need no NCCL at all. dlopen by soname returns the copy already in the process.
namespace {
struct NcclApi {
    ncclResult_t (*GetUniqueId)(ncclUniqueId*);
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int);
    ncclResult_t (*CommDestroy)(ncclComm_t);
    const char* (*GetErrorString)(ncclResult_t);
    ncclResult_t (*GroupStart)();
    ncclResult_t (*GroupEnd)();
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t);
    ncclResult_t (*Broadcast)(const void*, void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t);
    bool ok;
};
NcclApi g_nccl;
bool nccl_load() {
    if (g_nccl.ok) return true;
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return false;
#define IBCU_SYM(field, name) *(void**)&g_nccl.field = dlsym(h, name); if (!g_nccl.field) return false;
    IBCU_SYM(GetUniqueId, "ncclGetUniqueId") IBCU_SYM(CommInitRank, "ncclCommInitRank") IBCU_SYM(CommDestroy, "ncclCommDestroy")
    IBCU_SYM(GetErrorString, "ncclGetErrorString") IBCU_SYM(GroupStart, "ncclGroupStart") IBCU_SYM(GroupEnd, "ncclGroupEnd")
    IBCU_SYM(AllGather, "ncclAllGather") IBCU_SYM(Broadcast, "ncclBroadcast") IBCU_SYM(AllReduce, "ncclAllReduce")
#undef IBCU_SYM
    g_nccl.ok = true;
    return true;
}
}  // namespace
#define ncclGetUniqueId g_nccl.GetUniqueId
#define ncclCommInitRank g_nccl.CommInitRank
#define ncclCommDestroy g_nccl.CommDestroy
#define ncclGetErrorString g_nccl.GetErrorString
#define ncclGroupStart g_nccl.GroupStart
#define ncclGroupEnd g_nccl.GroupEnd
#define ncclAllGather g_nccl.AllGather
#define ncclBroadcast g_nccl.Broadcast
#define ncclAllReduce g_nccl.AllReduce

#define IBCU_NCCL(ctx, expr) do { ncclResult_t r_ = (expr); if (r_ != ncclSuccess) \
    return ibcu_fail((ctx), IBCU_ERR_COMM, "%s failed: %s", #expr, ncclGetErrorString(r_)); } while (0)

static_assert(sizeof(ncclUniqueId) <= IBCU_COMM_ID_BYTES, "communicator id does not fit the ABI token");

void ibcu_comm_destroy_internal(ibcu_ctx* ctx) {
    if (ctx->comm && g_nccl.ok) { ncclCommDestroy((ncclComm_t)ctx->comm); ctx->comm = nullptr; }
    for (int r = 0; r < IBCU_MAX_RANKS; r++)
        if (ctx->win_peer[r] && ctx->win_peer[r] != ctx->win_base) { cudaIpcCloseMemHandle(ctx->win_peer[r]); ctx->win_peer[r] = nullptr; }
    if (ctx->win_base) { cudaFree(ctx->win_base); ctx->win_base = nullptr; }
    if (ctx->win_err) { cudaFreeHost(ctx->win_err); ctx->win_err = nullptr; }
}

extern "C" int ibcu_comm_get_id(void* id_out) {
    if (!id_out) return IBCU_ERR_PARAM;
    if (!nccl_load()) return IBCU_ERR_COMM;
    ncclUniqueId id;
    if (ncclGetUniqueId(&id) != ncclSuccess) return IBCU_ERR_COMM;
    memset(id_out, 0, IBCU_COMM_ID_BYTES);
    memcpy(id_out, &id, sizeof id);
    return IBCU_OK;
}

extern "C" int ibcu_comm_init(ibcu_ctx* ctx, const void* id, int rank, int world) {
    IBCU_CHECK_CTX(ctx);
    IBCU_REQUIRE(ctx, id && world >= 1 && rank >= 0 && rank < world, "ibcu_comm_init: rank %d of %d", rank, world);
    if (ctx->comm) return ibcu_fail(ctx, IBCU_ERR_STATE, "communicator already initialised");
    ctx->rank = rank; ctx->world = world;
    if (world == 1) return IBCU_OK;
    if (!nccl_load()) return ibcu_fail(ctx, IBCU_ERR_COMM, "libnccl.so.2 could not be loaded: %s", dlerror());
    ncclUniqueId uid;
    memcpy(&uid, id, sizeof uid);
    IBCU_CUDA(ctx, cudaSetDevice(ctx->device));
    ncclComm_t comm;
    IBCU_NCCL(ctx, ncclCommInitRank(&comm, world, uid, rank));
    ctx->comm = (ncclComm*)comm;
    return IBCU_OK;
}

extern "C" int ibcu_comm_rank(const ibcu_ctx* ctx, int* rank, int* world) {
    if (!ctx) return IBCU_ERR_PARAM;
    if (rank) *rank = ctx->rank;
    if (world) *world = ctx->world;
    return IBCU_OK;
}

// Contiguous row slices in units of `align` rows; the first (units % world) ranks get one more unit;
// the last non-empty slice absorbs the ragged tail.
extern "C" void ibcu_shard_rows(int M, int world, int rank, int align, int* row0, int* rows) {
    if (align < 1) align = 1;
    if (world < 1) world = 1;
    long units = (M + align - 1) / align;
    long base = units / world, extra = units % world;
    long u0 = rank * base + (rank < extra ? rank : extra);
    long un = base + (rank < extra ? 1 : 0);
    long r0 = u0 * align, r1 = (u0 + un) * align;
    if (r0 > M) r0 = M;
    if (r1 > M) r1 = M;
    if (row0) *row0 = (int)r0;
    if (rows) *rows = (int)(r1 - r0);
}

extern "C" int ibcu_allgather_rows(ibcu_ctx* ctx, float* buf, int M, int stride, int B, int align) {
    IBCU_CHECK_CTX(ctx);
    IBCU_REQUIRE(ctx, buf && M >= 0 && stride >= M && B >= 1, "ibcu_allgather_rows: bad arguments");
    if (ctx->world == 1 || M == 0) return IBCU_OK;
    if (!ctx->comm) return ibcu_fail(ctx, IBCU_ERR_STATE, "ibcu_allgather_rows: no communicator");
    { int rc = ibcu_flush_gather_wait(ctx); if (rc) return rc; }
    for (int j = 0; j < 4; j++) ctx->win_last[j] = nullptr;    // an NCCL gather in between ends the no-repeat rule
    ncclComm_t comm = (ncclComm_t)ctx->comm;
    int r0, rn;
    ibcu_shard_rows(M, ctx->world, 0, align, &r0, &rn);
    bool even = (long)rn * ctx->world == M;
    IBCU_NCCL(ctx, ncclGroupStart());
    for (int b = 0; b < B; b++) {
        float* base = buf + (size_t)b * stride;
        if (even) {
            IBCU_NCCL(ctx, ncclAllGather(base + (size_t)ctx->rank * rn, base, rn, ncclFloat, comm, ctx->stream));
        } else {
            for (int r = 0; r < ctx->world; r++) {
                int q0, qn;
                ibcu_shard_rows(M, ctx->world, r, align, &q0, &qn);
                if (qn > 0) IBCU_NCCL(ctx, ncclBroadcast(base + q0, base + q0, qn, ncclFloat, r, comm, ctx->stream));
            }
        }
    }
    IBCU_NCCL(ctx, ncclGroupEnd());
    return IBCU_OK;
}

// ── push all-gather over peer memory ────────────────────────────────────────────────────
// Every rank owns a window of its own HBM that the other ranks have mapped (CUDA IPC). A buffer that
// lives at the same offset in every rank's window is gathered by ONE small kernel per rank: it stores
// this rank's row slice straight into the peers' copies over NVLink (plain peer stores), publishes an
// epoch number in each peer's flag word (release, system scope) and then waits, with a limit, until
// every peer's flag in its own window has reached the same epoch. No NCCL launch, no staging copy.
// The epoch is device state, so a captured launch replays correctly.
// Window header: flags[IBCU_MAX_RANKS] (flags[r] written by rank r), then this rank's epoch counter.
constexpr size_t WIN_HEADER = IBCU_WIN_HEADER;
constexpr int WIN_EPOCH_SLOT = IBCU_WIN_EPOCH_SLOT;
constexpr long WIN_SPIN_LIMIT = IBCU_WIN_SPIN_LIMIT;

struct PushDesc { float* buf; int stride, row0, rows; };
struct PushParams {
    PushDesc d[4];
    int n, B, rank, world;
    char* base;
    char* peer[IBCU_MAX_RANKS];
    int* err;
};

__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) { return ld_acquire_sys_u64(p); }
__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) { st_release_sys_u64(p, v); }

// The waiting half of a gather whose stores were made by a linear launch, for consumers that do not wait themselves.
__global__ void __launch_bounds__(32) gather_wait_kernel(const GatherWait g) {
    pdl_launch_dependents();
    pdl_wait();
    gather_wait(g);
}

__global__ void __launch_bounds__(1024) allgather_push_kernel(const PushParams p) {
    __shared__ unsigned long long s_epoch;
    pdl_launch_dependents();
    pdl_wait();
    for (int i = 0; i < p.n; i++) {
        const PushDesc d = p.d[i];
        const size_t off0 = (size_t)((char*)d.buf - p.base);
        const bool vec = ((d.row0 | d.rows | d.stride) & 3) == 0 && (off0 & 15) == 0;
        for (int b = 0; b < p.B; b++) {
            const float* src = d.buf + (size_t)b * d.stride + d.row0;
            const size_t off = off0 + ((size_t)b * d.stride + d.row0) * sizeof(float);
            if (vec) {
                for (int e = threadIdx.x; e < d.rows / 4; e += blockDim.x) {
                    const float4 v = reinterpret_cast<const float4*>(src)[e];
                    for (int q = 0; q < p.world; q++)
                        if (q != p.rank) reinterpret_cast<float4*>(p.peer[q] + off)[e] = v;
                }
            } else {
                for (int e = threadIdx.x; e < d.rows; e += blockDim.x) {
                    const float v = src[e];
                    for (int q = 0; q < p.world; q++)
                        if (q != p.rank) reinterpret_cast<float*>(p.peer[q] + off)[e] = v;
                }
            }
        }
    }
    __threadfence_system();
    __syncthreads();
    unsigned long long* my_flags = reinterpret_cast<unsigned long long*>(p.base);
    if (threadIdx.x == 0) {
        const unsigned long long e = my_flags[WIN_EPOCH_SLOT] + 1;
        my_flags[WIN_EPOCH_SLOT] = e;
        s_epoch = e;
        for (int q = 0; q < p.world; q++)
            if (q != p.rank) st_release_sys(reinterpret_cast<unsigned long long*>(p.peer[q]) + p.rank, e);
    }
    __syncthreads();
    const unsigned long long e = s_epoch;
    if ((int)threadIdx.x < p.world && (int)threadIdx.x != p.rank) {
        long it = 0;
        while (ld_acquire_sys(my_flags + threadIdx.x) < e) {
            if (++it > WIN_SPIN_LIMIT) { *p.err = (int)e; break; }       // give up: the host reports it at the next sync
            __nanosleep(100);
        }
    }
    __syncthreads();
}

// The receiving half of a tagged gather as a kernel of its own (for consumers that cannot receive themselves).
__global__ void __launch_bounds__(256) tag_unpack_kernel(const TagParams p) {
    pdl_launch_dependents();
    pdl_wait();
    tag_receive(p, blockIdx.x, gridDim.x);
}

static int launch_tag_unpack(ibcu_ctx* ctx, const TagParams& tp) {
    long elems = 0;
    for (int i = 0; i < tp.n; i++) elems += (long)tp.B * (tp.d[i].M - tp.d[i].rows);
    long blocks = (elems + 2047) / 2048;                      // 8 elements per thread
    if (blocks < 1) blocks = 1;
    if (blocks > 64) blocks = 64;
    TagParams q = tp;
    q.all_mask = 0u;
    return ibcu_launch(ctx, tag_unpack_kernel, dim3((unsigned)blocks), dim3(256), 0, 1, true, q);
}

static void take_flags(ibcu_ctx* ctx, GatherWait* gw) {
    memset(gw, 0, sizeof *gw);
    gw->world = ctx->world; gw->rank = ctx->rank; gw->err = ctx->win_err;
    if (!ctx->gather_pending) return;
    gw->flags = reinterpret_cast<const unsigned long long*>(ctx->win_base);
    ctx->gather_pending = 0;
}

void ibcu_take_gather_wait(ibcu_ctx* ctx, GatherWait* gw) {
    if (ctx->tag_pending) {                                   // the caller's kernel cannot receive: a kernel of its own does
        ctx->tag_pending = 0;
        launch_tag_unpack(ctx, ctx->tag_p);                  // a failed launch is recorded in the context; the caller's own launch reports it
    }
    take_flags(ctx, gw);
}

void ibcu_gather_wait_mark(ibcu_ctx* ctx, GatherWait* gw, const void* x, size_t x_bytes);
void ibcu_take_gather_wait_x(ibcu_ctx* ctx, GatherWait* gw, const void* x, size_t x_bytes) {
    take_flags(ctx, gw);
    if (!ctx->tag_pending) return;
    ctx->tag_pending = 0;
    gw->tag = ctx->tag_p;
    gw->tag.all_mask = 0u;
    ibcu_gather_wait_mark(ctx, gw, x, x_bytes);              // buffers the kernel reads itself: received in full by every block
}

// After the ranges the kernel reads have been marked: every block repeating the whole receive of those buffers pays only
// while that is little work; beyond, the receiving kernel of its own is cheaper and the caller's kernel receives nothing.
void ibcu_gather_wait_settle(ibcu_ctx* ctx, GatherWait* gw) {
    long repeated = 0;
    for (int i = 0; i < gw->tag.n; i++)
        if ((gw->tag.all_mask >> i) & 1u) repeated += (long)gw->tag.B * (gw->tag.d[i].M - gw->tag.d[i].rows);
    if (repeated > 1024) {
        TagParams tp = gw->tag;
        gw->tag.n = 0;
        launch_tag_unpack(ctx, tp);
    }
}

void ibcu_gather_wait_mark(ibcu_ctx* ctx, GatherWait* gw, const void* x, size_t x_bytes) {
    for (int i = 0; i < gw->tag.n; i++) {
        const char* lo = ctx->win_base + gw->tag.d[i].off;
        const char* hi = lo + ((size_t)(gw->tag.B - 1) * gw->tag.d[i].stride + gw->tag.d[i].M) * sizeof(float);
        if ((const char*)x < hi && (const char*)x + x_bytes > lo) gw->tag.all_mask |= 1u << i;
    }
}

int ibcu_flush_gather_wait(ibcu_ctx* ctx) {
    if (ctx->tag_pending) {
        ctx->tag_pending = 0;
        const int rc = launch_tag_unpack(ctx, ctx->tag_p);
        if (rc) return rc;
    }
    if (!ctx->gather_pending) return IBCU_OK;
    GatherWait gw;
    take_flags(ctx, &gw);                                     // clears the pending state, so the launch below does not come back here
    return ibcu_launch(ctx, gather_wait_kernel, dim3(1), dim3(32), 0, 1, true, gw);
}

// For the linear kernels: do all output slices of a launch belong to buffers of an announced gather? Then the launch
// stores them into the peers' copies as well and marks those buffers done.
bool ibcu_push_match(ibcu_ctx* ctx, float* const* outs, int n) {
    if (ctx->arm_n == 0 || ctx->world <= 1) return false;
    int hit[4];
    for (int i = 0; i < n; i++) {
        hit[i] = -1;
        for (int j = 0; j < ctx->arm_n; j++) {
            const char* p = (const char*)outs[i];
            if (p >= ctx->arm_buf[j] && p < ctx->arm_buf[j] + (size_t)ctx->arm_stride[j] * sizeof(float)) hit[i] = j;
        }
        if (hit[i] < 0) return false;
    }
    for (int i = 0; i < n; i++) ctx->arm_done[hit[i]] = 1;
    return true;                                              // the caller raises gather_pending once its pushing kernel is launched
}
void ibcu_push_fill(ibcu_ctx* ctx, GatherPush* gp, size_t bytes) {
    memset(gp, 0, sizeof *gp);
    gp->world = ctx->world; gp->rank = ctx->rank;
    gp->err = ctx->win_err;
    gp->twin0 = ctx->win_bytes;
    long P = (long)(bytes / (16 * 1024));                     // one pushing block per 16 KB, at most 16
    gp->pushers = P < 1 ? 1 : P > 16 ? 16 : (int)P;
    gp->header = reinterpret_cast<unsigned long long*>(ctx->win_base);
    for (int r = 0; r < ctx->world; r++) gp->peer[r] = ctx->win_peer[r];
}

extern "C" int ibcu_window_create(ibcu_ctx* ctx, size_t bytes, void* handle_out) {
    IBCU_CHECK_CTX(ctx);
    IBCU_REQUIRE(ctx, handle_out && bytes > 0, "ibcu_window_create: bad arguments");
    static_assert(sizeof(cudaIpcMemHandle_t) <= IBCU_WINDOW_HANDLE_BYTES, "IPC handle does not fit the ABI token");
    if (ctx->win_base) return ibcu_fail(ctx, IBCU_ERR_STATE, "window already created");
    IBCU_REQUIRE(ctx, ctx->world <= IBCU_MAX_RANKS, "ibcu_window_create: %d ranks, at most %d", ctx->world, IBCU_MAX_RANKS);
    IBCU_CUDA(ctx, cudaSetDevice(ctx->device));
    // header, then the plain part that buffers are taken from, then the tagged part: an 8-byte {value, tag} twin of every float
    const size_t plain = (bytes + 255) & ~(size_t)255;
    const size_t total = WIN_HEADER + plain;
    void* base = nullptr;
    IBCU_CUDA(ctx, cudaMalloc(&base, total + 2 * plain));
    int* err_word = nullptr;
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaMemset(base, 0, total + 2 * plain);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e == cudaSuccess && !ctx->win_err) e = cudaHostAlloc((void**)&err_word, sizeof(int), cudaHostAllocMapped);
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, base);
    if (e != cudaSuccess) {                                   // nothing is kept of a window that could not be made
        cudaFree(base);
        if (err_word) cudaFreeHost(err_word);
        return ibcu_fail(ctx, IBCU_ERR_CUDA, "ibcu_window_create: %s", cudaGetErrorString(e));
    }
    if (err_word) { *err_word = 0; ctx->win_err = err_word; }
    memset(handle_out, 0, IBCU_WINDOW_HANDLE_BYTES);
    memcpy(handle_out, &h, sizeof h);
    ctx->win_base = (char*)base; ctx->win_bytes = total; ctx->win_used = WIN_HEADER;
    ctx->win_peer[ctx->rank] = ctx->win_base; ctx->win_open = 1; ctx->win_enabled = 1;
    return IBCU_OK;
}

extern "C" int ibcu_window_open(ibcu_ctx* ctx, int peer, const void* handle) {
    IBCU_CHECK_CTX(ctx);
    IBCU_REQUIRE(ctx, handle && peer >= 0 && peer < ctx->world && peer < IBCU_MAX_RANKS, "ibcu_window_open: peer %d of %d", peer, ctx->world);
    if (!ctx->win_base) return ibcu_fail(ctx, IBCU_ERR_STATE, "ibcu_window_open before ibcu_window_create");
    if (peer == ctx->rank || ctx->win_peer[peer]) return IBCU_OK;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof h);
    void* ptr = nullptr;
    IBCU_CUDA(ctx, cudaSetDevice(ctx->device));
    IBCU_CUDA(ctx, cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
    ctx->win_peer[peer] = (char*)ptr;
    ctx->win_open++;
    return IBCU_OK;
}

extern "C" int ibcu_window_alloc(ibcu_ctx* ctx, size_t bytes, void** dptr) {
    IBCU_CHECK_CTX(ctx);
    if (!dptr) return IBCU_ERR_PARAM;
    *dptr = nullptr;
    if (!ctx->win_base) return IBCU_ERR_STATE;               // not an error state of the context: callers fall back to ibcu_malloc
    const size_t need = (bytes + 255) & ~(size_t)255;
    if (ctx->win_used + need > ctx->win_bytes) return IBCU_ERR_NOMEM;
    *dptr = ctx->win_base + ctx->win_used;
    ctx->win_used += need;
    return IBCU_OK;
}

extern "C" void ibcu_window_enable(ibcu_ctx* ctx, int on) { if (ctx) ctx->win_enabled = on ? 1 : 0; }


static bool in_window(const ibcu_ctx* ctx, const void* p) {
    return ctx->win_base && (const char*)p >= ctx->win_base + WIN_HEADER && (const char*)p < ctx->win_base + ctx->win_bytes;
}

// A wait that cannot be satisfied, on one GPU: a private header whose own epoch says 1 while the flag word of a
// "peer" that does not exist stays 0. The waiting kernel must give up at its limit and raise the error word.
extern "C" int ibcu_gather_wait_probe(ibcu_ctx* ctx) {
    IBCU_CHECK_CTX(ctx);
    IBCU_CUDA(ctx, cudaSetDevice(ctx->device));
    if (!ctx->win_err) {
        IBCU_CUDA(ctx, cudaHostAlloc((void**)&ctx->win_err, sizeof(int), cudaHostAllocMapped));
        *ctx->win_err = 0;
    }
    unsigned long long host_hdr[IBCU_WIN_HEADER / 8];
    memset(host_hdr, 0, sizeof host_hdr);
    host_hdr[IBCU_WIN_EPOCH_SLOT] = 1;
    int rc = ibcu_reserve(ctx, &ctx->scratch, &ctx->scratch_bytes, IBCU_WIN_HEADER);
    if (rc) return rc;
    IBCU_CUDA(ctx, cudaMemcpyAsync(ctx->scratch, host_hdr, sizeof host_hdr, cudaMemcpyHostToDevice, ctx->stream));
    IBCU_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    GatherWait gw = { (const unsigned long long*)ctx->scratch, 2, 0, ctx->win_err };
    return ibcu_launch(ctx, gather_wait_kernel, dim3(1), dim3(32), 0, 1, true, gw);
}

extern "C" int ibcu_allgather_rows_prepare(ibcu_ctx* ctx, float* const* bufs, const int* stride, int n) {
    IBCU_CHECK_CTX(ctx);
    IBCU_REQUIRE(ctx, bufs && stride && n >= 1 && n <= 4, "ibcu_allgather_rows_prepare: bad arguments");
    ctx->arm_n = 0;
    if (ctx->world <= 1 || !ctx->win_enabled || ctx->win_open != ctx->world) return IBCU_OK;
    for (int i = 0; i < n; i++) {
        if (!in_window(ctx, bufs[i])) return IBCU_OK;
        for (int j = 0; j < 4; j++) if (ctx->win_last[j] == bufs[i]) return IBCU_OK;      // the peers may still be reading the previous gather of it
    }
    for (int i = 0; i < n; i++) { ctx->arm_buf[i] = (const char*)bufs[i]; ctx->arm_stride[i] = stride[i]; ctx->arm_done[i] = 0; }
    ctx->arm_n = n;
    return IBCU_OK;
}

extern "C" int ibcu_allgather_rows_n(ibcu_ctx* ctx, float* const* bufs, const int* M, const int* stride, int n, int B, int align) {
    IBCU_CHECK_CTX(ctx);
    IBCU_REQUIRE(ctx, bufs && M && stride && n >= 1 && n <= 4 && B >= 1, "ibcu_allgather_rows_n: bad arguments");
    if (ctx->world == 1) return IBCU_OK;
    if (ctx->arm_n) {
        // announced ahead (ibcu_allgather_rows_prepare): the linear launches that produced these rows may already have
        // stored them into the peers' copies; then only the waiting is left, and the next kernel or copy does it
        bool done = ctx->arm_n == n;
        for (int i = 0; i < n && done; i++) done = ctx->arm_buf[i] == (const char*)bufs[i] && ctx->arm_done[i];
        ctx->arm_n = 0;
        if (done) {
            // every rank's rows are on their way, tagged, to every other rank's window: receive this rank's copies
            for (int j = 0; j < 4; j++) ctx->win_last[j] = j < n ? bufs[j] : nullptr;
            TagParams tp;
            memset(&tp, 0, sizeof tp);
            tp.n = n; tp.B = B; tp.base = ctx->win_base; tp.twin0 = ctx->win_bytes; tp.err = ctx->win_err;
            for (int i = 0; i < n; i++) {
                int r0, rn;
                ibcu_shard_rows(M[i], ctx->world, ctx->rank, align, &r0, &rn);
                tp.d[i] = { (size_t)((const char*)bufs[i] - ctx->win_base), stride[i], M[i], r0, rn };
            }
            { int rc = ibcu_flush_gather_wait(ctx); if (rc) return rc; }      // an earlier gather still to be received comes first
            ctx->tag_p = tp;
            ctx->tag_pending = 1;                             // received by the next linear call in its first kernel, else by a kernel of its own
            return IBCU_OK;
        }
    }
    { int rc = ibcu_flush_gather_wait(ctx); if (rc) return rc; }
    bool push = ctx->win_enabled && ctx->win_open == ctx->world;
    for (int i = 0; i < n && push; i++) {
        push = in_window(ctx, bufs[i]);
        for (int j = 0; j < 4; j++) if (ctx->win_last[j] == bufs[i]) push = false;   // the peers may still be reading the previous gather of it
    }
    if (!push) {
        for (int j = 0; j < 4; j++) ctx->win_last[j] = nullptr;
        for (int i = 0; i < n; i++) { int rc = ibcu_allgather_rows(ctx, bufs[i], M[i], stride[i], B, align); if (rc) return rc; }
        return IBCU_OK;
    }
    PushParams p;
    memset(&p, 0, sizeof p);
    p.n = n; p.B = B; p.rank = ctx->rank; p.world = ctx->world; p.base = ctx->win_base; p.err = ctx->win_err;
    for (int r = 0; r < ctx->world; r++) p.peer[r] = ctx->win_peer[r];
    for (int i = 0; i < n; i++) {
        IBCU_REQUIRE(ctx, bufs[i] && M[i] >= 0 && stride[i] >= M[i], "ibcu_allgather_rows_n: tensor %d", i);
        int r0, rn;
        ibcu_shard_rows(M[i], ctx->world, ctx->rank, align, &r0, &rn);
        p.d[i] = { bufs[i], stride[i], r0, rn };
    }
    for (int j = 0; j < 4; j++) ctx->win_last[j] = j < n ? bufs[j] : nullptr;
    return ibcu_launch(ctx, allgather_push_kernel, dim3(1), dim3(1024), 0, 1, true, p);
}

static int allreduce(ibcu_ctx* ctx, void* buf, size_t n, ncclDataType_t ty) {
    IBCU_CHECK_CTX(ctx);
    if (ctx->world == 1 || n == 0) return IBCU_OK;
    if (!ctx->comm) return ibcu_fail(ctx, IBCU_ERR_STATE, "all-reduce requested without a communicator");
    { int rc = ibcu_flush_gather_wait(ctx); if (rc) return rc; }
    IBCU_NCCL(ctx, ncclAllReduce(buf, buf, n, ty, ncclSum, (ncclComm_t)ctx->comm, ctx->stream));
    return IBCU_OK;
}
int ibcu_allreduce_kmeans(ibcu_ctx* ctx, float* sums, size_t n_sums, int32_t* counts, size_t n_counts, double* inertia) {
    IBCU_CHECK_CTX(ctx);
    if (ctx->world == 1) return IBCU_OK;
    if (!ctx->comm) return ibcu_fail(ctx, IBCU_ERR_STATE, "all-reduce requested without a communicator");
    { int rc = ibcu_flush_gather_wait(ctx); if (rc) return rc; }
    ncclComm_t comm = (ncclComm_t)ctx->comm;
    IBCU_NCCL(ctx, ncclGroupStart());
    IBCU_NCCL(ctx, ncclAllReduce(sums, sums, n_sums, ncclFloat, ncclSum, comm, ctx->stream));
    IBCU_NCCL(ctx, ncclAllReduce(counts, counts, n_counts, ncclInt32, ncclSum, comm, ctx->stream));
    if (inertia) IBCU_NCCL(ctx, ncclAllReduce(inertia, inertia, 1, ncclDouble, ncclSum, comm, ctx->stream));
    IBCU_NCCL(ctx, ncclGroupEnd());
    return IBCU_OK;
}

// The exchange area: two buffers of `world` slots, taken from the window the first time (or when a larger slot is asked
// for). Every rank calls this at the same point of the same sequence of window allocations, so the area has the same
// offset in every window. Two buffers used in turn are enough: a rank can only write buffer t again after it has waited
// for the exchange in between, which its peers publish only after their kernels that read buffer t have finished.
int ibcu_exchange_begin(ibcu_ctx* ctx, size_t slot_bytes, ExchSlots* ex) {
    if (ctx->world <= 1 || !ctx->win_base || !ctx->win_enabled || ctx->win_open != ctx->world) return 0;
    const size_t slot = (slot_bytes + 255) & ~(size_t)255;
    if (slot > ctx->exch_slot) {
        void* area = nullptr;
        if (ibcu_window_alloc(ctx, 2 * slot * ctx->world, &area) != IBCU_OK) return 0;
        ctx->exch_off = (size_t)((char*)area - ctx->win_base);
        ctx->exch_slot = slot;
        ctx->exch_turn = 0;
    }
    ibcu_push_fill(ctx, &ex->gp, slot_bytes);
    ex->slot = ctx->exch_slot;
    ex->off = ctx->exch_off + (size_t)(ctx->exch_turn & 1u) * ctx->exch_slot * ctx->world;
    ctx->exch_turn++;
    return 1;
}

extern "C" int ibcu_allreduce_f32(ibcu_ctx* ctx, float* buf, size_t n) { return allreduce(ctx, buf, n, ncclFloat); }
extern "C" int ibcu_allreduce_i32(ibcu_ctx* ctx, int32_t* buf, size_t n) { return allreduce(ctx, buf, n, ncclInt32); }
extern "C" int ibcu_allreduce_f64(ibcu_ctx* ctx, double* buf, size_t n) { return allreduce(ctx, buf, n, ncclDouble); }
