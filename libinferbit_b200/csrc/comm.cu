// Multi-GPU plumbing: one process per GPU, NCCL over NVLink/NVSwitch. The hot path has exactly two
// exchange steps: the all-gather of row-sharded linear outputs and the all-reduce of k-means
// centroid sums / counts. Everything else is replicated.
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

static int allreduce(ibcu_ctx* ctx, void* buf, size_t n, ncclDataType_t ty) {
    IBCU_CHECK_CTX(ctx);
    if (ctx->world == 1 || n == 0) return IBCU_OK;
    if (!ctx->comm) return ibcu_fail(ctx, IBCU_ERR_STATE, "all-reduce requested without a communicator");
    IBCU_NCCL(ctx, ncclAllReduce(buf, buf, n, ty, ncclSum, (ncclComm_t)ctx->comm, ctx->stream));
    return IBCU_OK;
}
extern "C" int ibcu_allreduce_f32(ibcu_ctx* ctx, float* buf, size_t n) { return allreduce(ctx, buf, n, ncclFloat); }
extern "C" int ibcu_allreduce_i32(ibcu_ctx* ctx, int32_t* buf, size_t n) { return allreduce(ctx, buf, n, ncclInt32); }
extern "C" int ibcu_allreduce_f64(ibcu_ctx* ctx, double* buf, size_t n) { return allreduce(ctx, buf, n, ncclDouble); }
