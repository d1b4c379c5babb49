/*
 * ibcu.h — C ABI of the sm_100a CUDA backend (libibcu.so) for libinferbit's quantized-weight
 * product hot path: per-row-scaled INT4/INT8 matvec, the product-quantisation LUT + gather
 * matvec, the k-means assign/update loop, and the small element-wise kernels a decode step needs.
 *
 * Plain C: opaque context, raw device/host pointers, sizes. No CPU fallback anywhere — a call
 * either runs on the GPU or returns a negative code and records a message (ibcu_last_error).
 * All launches go to the context's stream and are asynchronous unless stated; ibcu_sync waits.
 *
 * Each entry point names the reference interface it stands in for (paths inside the reference
 * checkout, file:line).
 */
#ifndef IBCU_H
#define IBCU_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

/* Return codes follow include/inferbit.h:43-49 (0 ok, negatives for failure classes). */
#define IBCU_OK              0
#define IBCU_ERR_PARAM     (-1)   /* bad argument / unsupported shape */
#define IBCU_ERR_CUDA      (-2)   /* a CUDA runtime call or launch failed */
#define IBCU_ERR_NOMEM     (-3)
#define IBCU_ERR_COMM      (-4)   /* NCCL failure */
#define IBCU_ERR_STATE     (-5)   /* call not valid in the current state (e.g. no communicator) */

typedef struct ibcu_ctx ibcu_ctx;

/* ── context, memory, stream ─────────────────────────────────────────────────────────── */
/* The reference has one process-global kernel table (src/kernels/scalar.c:185) and one pool per
 * model (src/ibf_loader.c:543); here one context = one GPU + one stream + scratch. */
int  ibcu_ctx_create(int device, ibcu_ctx** out);
void ibcu_ctx_destroy(ibcu_ctx* ctx);
/* Sticky status: first failure since the last ibcu_clear_error (0 if none); message is
 * thread-compatible, owned by the context (src/error.c:7-22 keeps a TLS string instead). */
int         ibcu_status(const ibcu_ctx* ctx);
const char* ibcu_last_error(const ibcu_ctx* ctx);
void        ibcu_clear_error(ibcu_ctx* ctx);
int  ibcu_device_count(void);
int  ibcu_device_sm_count(const ibcu_ctx* ctx);

int  ibcu_malloc(ibcu_ctx* ctx, size_t bytes, void** dptr);
int  ibcu_free(ibcu_ctx* ctx, void* dptr);
int  ibcu_host_alloc(ibcu_ctx* ctx, size_t bytes, void** hptr);      /* pinned */
int  ibcu_host_free(ibcu_ctx* ctx, void* hptr);
int  ibcu_memcpy_h2d(ibcu_ctx* ctx, void* dst, const void* src, size_t bytes);   /* async */
int  ibcu_memcpy_d2h(ibcu_ctx* ctx, void* dst, const void* src, size_t bytes);   /* async */
int  ibcu_memcpy_d2d(ibcu_ctx* ctx, void* dst, const void* src, size_t bytes);   /* async */
int  ibcu_memset(ibcu_ctx* ctx, void* dst, int byte, size_t bytes);              /* async */
int  ibcu_sync(ibcu_ctx* ctx);
/* The same wait for callers that turn a short kernel round: a one-thread kernel writes a sequence number into pinned host
 * memory when the stream's work is done and the host polls that word (bounded; the driver's wait takes over after about two
 * seconds or when the launch fails). Returns what ibcu_sync would. */
int  ibcu_sync_spin(ibcu_ctx* ctx);
/* *dst = value on the context's stream (a one-thread kernel: the value travels as a launch argument, so
 * the host may change its own copy at once). */
int  ibcu_store_i32(ibcu_ctx* ctx, int32_t* dst, int32_t value);
/* Fill a device buffer with counter-based pseudo-random bytes: byte i = low 8 bits of
 * mix64(seed, i / 8) >> (8 * (i % 8)) (mix64 = splitmix64 finaliser). Used to build random-weight
 * models in HBM without a host copy; ibcu_hash_bytes_host computes the same bytes on the CPU. */
int  ibcu_fill_hash_bytes(ibcu_ctx* ctx, void* dst, size_t bytes, uint64_t seed);
/* The slice [first_byte, first_byte + bytes) of that stream (first_byte a multiple of 8): a rank that holds some
 * rows of a tensor gets exactly the bytes the whole tensor would have there. */
int  ibcu_fill_hash_bytes_at(ibcu_ctx* ctx, void* dst, size_t bytes, uint64_t seed, size_t first_byte);
void ibcu_hash_bytes_host(void* dst, size_t bytes, uint64_t seed, size_t first_byte);
/* fp16 values lo + (hi-lo)*u, u from the same generator (one 16-bit draw per element). */
int  ibcu_fill_hash_fp16_uniform(ibcu_ctx* ctx, void* dst, size_t count, uint64_t seed, float lo, float hi);
int  ibcu_fill_hash_fp16_uniform_at(ibcu_ctx* ctx, void* dst, size_t count, uint64_t seed, float lo, float hi, size_t first);
/* FP32 values mean + std * z with z bell-shaped of unit variance (the centred sum of four 16-bit draws), element
 * first + i of the stream; used to fill synthetic KV caches. */
int  ibcu_fill_hash_f32_normal_at(ibcu_ctx* ctx, float* dst, size_t count, uint64_t seed, float mean, float std, size_t first);
void ibcu_hash_fp16_uniform_host(uint16_t* dst, size_t count, uint64_t seed, float lo, float hi, size_t first);

/* Device timing on the context's stream (CUDA events). slot in [0,16). */
int  ibcu_event_record(ibcu_ctx* ctx, int slot);
int  ibcu_event_elapsed_ms(ibcu_ctx* ctx, int slot_start, int slot_stop, float* ms);   /* syncs on stop */
/* Stream capture into a replayable graph (one per context): begin, issue calls, end, replay. */
int  ibcu_graph_begin(ibcu_ctx* ctx);
int  ibcu_graph_end(ibcu_ctx* ctx, int* graph_id);
int  ibcu_graph_launch(ibcu_ctx* ctx, int graph_id);
int  ibcu_graph_destroy(ibcu_ctx* ctx, int graph_id);
/* Number of kernels this library has launched through this context since creation. */
uint64_t ibcu_launch_count(const ibcu_ctx* ctx);
/* Programmatic dependent launch between consecutive kernels of this library (default on). */
void ibcu_set_pdl(ibcu_ctx* ctx, int enabled);

/* ── INT4 / INT8 linear layers ───────────────────────────────────────────────────────── */
/* Stands in for ib_kernels.matmul_int4 / matmul_int8 / matmul_int8_batch
 * (src/inferbit_internal.h:199-277; scalar definitions src/kernels/scalar.c:9-41,70-84) as driven
 * by tensor_matmul / tensor_matmul_batch (src/forward.c:144-246) and ib_parallel_matmul*
 * (src/threading.c:244-258,383-394).
 *
 * Weights stay in the reference's own layout in HBM: INT8 row-major [M*N]; INT4 two columns per
 * byte, low nibble first, bias 8, row stride N/2 (src/kernels/scalar.c:17-22). Scales are the
 * per-output-row FP16 values as stored in the model file (src/forward.c:31-34), or FP32 when the
 * caller already widened them as the table contract does. */
typedef struct {
    const void* w;            /* device */
    const void* scales;       /* device, [M] */
    float*      out;          /* device, out[b*out_stride + row] */
    int M;                    /* rows of this tensor */
    int out_stride;           /* >= M; the reference's M_stride */
    int scales_fp32;          /* 0: fp16 bit patterns, 1: float */
    int epilogue;             /* IBCU_EPI_* */
} ibcu_linear_t;

#define IBCU_EPI_STORE     0  /* out  = y                                   */
#define IBCU_EPI_ADD       1  /* out += y   (residual add, src/forward.c:620-622,644-646) */

/* y_t = W_t x for n_tensors (1..4) tensors that share the activation x[B*N] (device, FP32, x[b*N+j])
 * and the bit width (4 or 8). B in 1..32 (IB_BATCH_MAX, src/inferbit_internal.h:287).
 * N must be even for bits == 4. */
int ibcu_linear(ibcu_ctx* ctx, const ibcu_linear_t* tensors, int n_tensors,
                const float* x, int N, int B, int bits);
/* Same with a transformation of the activation folded into the call (no separate launch, no
 * intermediate vector): RMSNorm with fp16 weights ahead of the q/k/v and gate/up projections
 * (src/forward.c:566-572,625-636), or silu(x)*x2 ahead of down_proj (src/forward.c:637-640). */
#define IBCU_PRO_NONE      0
#define IBCU_PRO_RMSNORM   1  /* x <- x * rsqrt(mean(x^2) + eps) * fp16(norm_w) */
#define IBCU_PRO_SILU_MUL  2  /* x <- x / (1 + exp(-x)) * x2 */
#define IBCU_PRO_KNOWN_MAX 3  /* x as it is; the caller supplies max|x[b]| in pieces (ibcu_silu_mul_amax makes them), which
                               * spares every block of the kernel its own reduction over the activation */
typedef struct {
    int op;
    const float*    x2;       /* device [B*N], IBCU_PRO_SILU_MUL */
    const uint16_t* norm_w;   /* device fp16 [N], IBCU_PRO_RMSNORM */
    float eps;
    const float*    amax;     /* device [B*n_amax], IBCU_PRO_KNOWN_MAX: max over amax[b*n_amax .. +n_amax) == max|x[b]| */
    int n_amax;
} ibcu_prologue_t;
int ibcu_linear_ex(ibcu_ctx* ctx, const ibcu_linear_t* tensors, int n_tensors,
                   const float* x, int N, int B, int bits, const ibcu_prologue_t* prologue);
/* A gate/up pair in one launch over the shared activation, followed by a second, elementwise launch that forms
 * silu(gate_y) * up_y (src/forward.c:635-637, src/kernels/scalar.c:175-181): tensors[0] = gate, tensors[1] = up,
 * equal M. Both outputs are written by the first launch; the second overwrites tensors[0].out[b*out_stride + row]
 * with the product and leaves tensors[1].out holding up_y. */
int ibcu_linear_gate_up_silu(ibcu_ctx* ctx, const ibcu_linear_t* gate_up,
                             const float* x, int N, int B, int bits);
/* Force the portable (non tensor-core) kernel for the next ibcu_linear calls; for tests. */
void ibcu_linear_force_generic(ibcu_ctx* ctx, int on);
/* A second kernel for calls with 5 to 16 activations and N a multiple of 512: the same exact arithmetic on the tcgen05
 * tensor cores, weights as the A operand from shared memory, limbs as the B operand, s32 accumulators in tensor memory.
 * on = 0 (the default): only the calls where it was measured faster than the mma.sync kernel on B200 (INT4 tensors of at
 * least 3072 rows and at most 4096 columns with 5 to 8 activations); 1: every INT4 call it can take; 2: INT8 calls as well;
 * -1: never. The choice depends on the call's shape only, so every rank of a sharded model takes the same kernel. */
void ibcu_linear_use_tcgen05(ibcu_ctx* ctx, int on);

/* W4A8 route (src/threading.c:401-432 activation quantiser, src/kernels/scalar.c:43-124 kernels):
 * x quantised per 128-column group on the device, exact int32 group dot products. */
int ibcu_quantize_input_int8_g128(ibcu_ctx* ctx, const float* x, int8_t* q, float* sa, int N, int B);
int ibcu_linear_w4a8(ibcu_ctx* ctx, const ibcu_linear_t* tensor, const int8_t* xq, const float* sa,
                     int N, int B);
/* Both steps of the reference's INT4 route for FP32 activations (tensor_matmul with IB_W4A8 on, src/forward.c:175-246):
 * the quantiser and the matvec (one launch for a single activation of up to 4096 columns, else two). Same bits as the two calls. */
int ibcu_linear_w4a8_fp32(ibcu_ctx* ctx, const ibcu_linear_t* tensor, const float* x, int N, int B);

/* ── PQ matvec ───────────────────────────────────────────────────────────────────────── */
/* Stands in for ib_pq_matmul_fp32 / _threaded / _streaming (src/pq_decode.h:189-222; body
 * src/pq_decode.c:1504-1682), including the second residual level with one-byte or 4-bit packed indices
 * (K_l2 <= 256; src/pq_decode.c:1058-1075, :1441-1496) and the int8 outlier sidecar (:1394-1409). Field
 * meanings follow ib_pq_tensor (src/pq_decode.h:39-87). All pointers are device pointers. */
typedef struct {
    int M, N, G, K;                   /* K <= 256, G even, N % G == 0, C = N / G chunks */
    const uint16_t* codebook_l;       /* fp16 [K * G/2] (shared by all chunks) */
    const uint16_t* codebook_r;
    long            cb_chunk_stride;  /* 0 = shared tables (the reference); else fp16 elements between chunk tables */
    const uint8_t*  idx_l;            /* [M * C] row-major, as in the reference */
    const uint8_t*  idx_r;
    const uint16_t* row_scale;        /* fp16 [M] */
    const uint8_t*  idx_t;            /* regrouped copy of the codes made by ibcu_pq_prepare */
    int             M_pad;
    /* production extras; all zero / NULL for a plain single-level tensor */
    int             K_l2;             /* > 0: a second residual level with K_l2 <= 256 entries per shared codebook */
    const uint16_t* codebook2_l;      /* fp16 [K_l2 * G/2] */
    const uint16_t* codebook2_r;
    const uint8_t*  idx2_l;           /* [M * C] bytes, or [M * (C+1)/2] bytes of two 4-bit indices (low nibble = even chunk) when K_l2 == 16 */
    const uint8_t*  idx2_r;
    int             n_outlier;        /* > 0: that many columns of x bypass the tables; then C = (N - n_outlier) / G */
    const int32_t*  outlier_cols;     /* [n_outlier] ascending */
    const int8_t*   outlier_sidecar;  /* [M * n_outlier] */
    const uint16_t* outlier_scale;    /* fp16 [n_outlier] */
    const int32_t*  inner_cols;       /* [N - n_outlier] the other columns, made by ibcu_pq_prepare */
} ibcu_pq_t;

/* One-off per tensor (like the reference's ib_pq_lut_cache regrouped index layout,
 * src/pq_decode.c:2687-2737): writes the codes regrouped into slabs of 32 subspaces
 * ([slab][group of 16 rows][lane][16 rows], subspace 2 * chunk + side = 32 * slab + lane, byte i of lane l holding
 * row i ^ (l >> 1) of the group) and, after them,
 * the largest codebook magnitude into idx_t_out, which must hold ibcu_pq_idx_t_bytes(M, N, G) bytes, and
 * fills t->idx_t / t->M_pad. Needs the tensor's codebooks as well as its codes. */
size_t ibcu_pq_idx_t_bytes(int M, int N, int G);
/* the same for any tensor: both levels' regrouped codes, the tail, and the list of inner columns when there are outliers */
size_t ibcu_pq_prepared_bytes(const ibcu_pq_t* t);
int    ibcu_pq_prepare(ibcu_ctx* ctx, ibcu_pq_t* t, uint8_t* idx_t_out);
/* out[b*M + r] = row_scale[r] * sum_c (TL[c][idx_l[r,c]] + TR[c][idx_r[r,c]]) for B activations
 * x[b*N + j]; applies the reference's 1 %-of-max chunk skip rule per activation. One launch; the sums of a
 * row over slabs of 32 subspaces are added as 64-bit fixed-point integers (quantum 2^-62 of a bound on the
 * row sums), so the result is the same bits from run to run. An activation that holds NaN or Inf gives NaN
 * in every output of that call. */
int    ibcu_pq_matmul_fp32(ibcu_ctx* ctx, const ibcu_pq_t* t, const float* x, float* out, int B);
/* The same with rows of out out_stride floats apart (out[b*out_stride + r]): a rank that holds a slice of the tensor's rows
 * writes it in place into the full-width result, which ibcu_allgather_rows then completes (the reference's threaded form
 * splits rows over workers the same way, src/pq_decode.c:1807-1830). */
int    ibcu_pq_matmul_fp32_strided(ibcu_ctx* ctx, const ibcu_pq_t* t, const float* x, float* out, int out_stride, int B);
/* Same result as ibcu_pq_matmul_fp32 for callers that must not allocate device memory: serving
 * loops that cannot take cudaMalloc's device-wide synchronisation, plugins living inside a fixed
 * memory budget, processes whose allocator belongs to another runtime. This entry point has no
 * counterpart in the reference (its matmul_impl mallocs its tables on every call,
 * src/pq_decode.c:1519-1680). It calls no cudaMalloc / cudaFree or any allocating routine: the row
 * accumulators and arrival counters live in an array built into the library, ibcu_pq_noalloc_max_floats()
 * four-byte words (4 MiB) held by every GPU that loads the library from load to exit. A call that needs
 * more (4096 words for counters plus 2 words per activation and padded row) is refused with IBCU_ERR_PARAM
 * and a message giving both numbers. The first call on a device looks up the array's device address; make
 * that call before any stream capture. All calls on a device share the one array and it keeps the
 * previous call's contents; the part a call uses must start at zero, so the call clears it on the stream
 * before its kernel. Two calls whose kernels may overlap on the GPU - different contexts or streams on the
 * same device - race and must be serialised by the caller. */
int    ibcu_pq_matmul_fp32_noalloc(ibcu_ctx* ctx, const ibcu_pq_t* t, const float* x, float* out, int B);
size_t ibcu_pq_noalloc_max_floats(void);

/* ib_pq_lm_head_topk (src/pq_decode.h, body src/pq_decode.c:2259-2341) on the device: first-level logits of all M rows
 * without the 1 % rule (ib_pq_matmul_fp32_l1_only, :2085-2143), the K_top rows with the largest of them, every level
 * of those rows (ib_pq_matmul_fp32_subset, :2145-2248), and out_logits[K_top] / out_ids[K_top] in descending order of the
 * full logit (equal logits: ascending row). 1 <= K_top <= min(M, 1024). Reads the row-major code planes idx_l / idx_r
 * (and idx2_l / idx2_r), which must still be resident, beside the regrouped copy. x, out_logits, out_ids: device memory. */
int ibcu_pq_lm_head_topk(ibcu_ctx* ctx, const ibcu_pq_t* t, const float* x, int K_top, float* out_logits, int32_t* out_ids);

/* PQ-compressed KV cache, encode of n_vec vectors of dim values (src/pq_decode.c:5008-5066: the K or the V row of a
 * position): scale[v] = max|vec| / 7 (at least 1e-12), and per chunk of G normalised values the nearest entry (squared
 * distance, strict '<') of the left codebook to its first half and of the right codebook to its second half.
 * idx[v * 2C + c] = left code of chunk c, idx[v * 2C + C + c] = right code; cb_l / cb_r: fp16 [K1 * G/2], K1 <= 256. */
int ibcu_pqkv_encode(ibcu_ctx* ctx, const float* vec, int dim, int n_vec, int G, int K1,
                     const uint16_t* cb_l, const uint16_t* cb_r, uint8_t* idx, float* scale);

/* ── group-scaled INT4 matvec ────────────────────────────────────────────────────────── */
/* The INT4 tensors of the reference's session engine (struct ib_int4_tensor, src/pq_decode.c:3474-3483; arithmetic of
 * int4_matmul_rows_skip, :3565-3651; skip rule of build_skip_mask, :3854-3882). The reference has these only as static
 * functions of that engine, so there is no entry point to mirror; the call below is this backend's form of them.
 * q: [M * N/2] two columns per byte, low nibble = even column, value = nibble - 8; s: fp16 [M * N/G] one scale per row
 * and group of G columns (G even, N % G == 0); optionally K_out outlier columns per row: outl_idx uint16 [M * K_out],
 * outl_val fp16 [M * K_out]. All pointers are device pointers. */
typedef struct {
    int M, N, G, K_out;
    const uint8_t*  q;
    const uint16_t* s;
    const uint16_t* outl_idx;
    const uint16_t* outl_val;
} ibcu_int4g_t;
/* out[m] = sum_g s[m][g] * sum_{j in g} (nibble(m, j) - 8) * x[j]  +  sum_k outl_val[m][k] * x[outl_idx[m][k]].
 * eps_act_rel > 0 leaves out the groups whose max|x| is at most eps_act_rel * max|x| (0 = the reference's default: none).
 * One activation. FP32 sums are ordered differently from the reference's scalar loop: equal to rounding. */
int ibcu_int4g_matmul_fp32(ibcu_ctx* ctx, const ibcu_int4g_t* t, const float* x, float* out, float eps_act_rel);

/* ── k-means ─────────────────────────────────────────────────────────────────────────── */
/* ib_kmeans_assign (src/pq_kmeans.h:70-74, src/pq_kmeans.c:399-413): idx[i] = nearest centroid of
 * X[i*D..], direct squared distance in the reference binary's rounding order, strict '<'.
 * dist (may be NULL) receives the winning distance. D <= 32, K <= 1024. */
int ibcu_kmeans_assign(ibcu_ctx* ctx, const float* X, long N, int D, const float* C, int K,
                       int32_t* idx, float* dist);
/* Which assignment kernel ibcu_kmeans_assign may take; every one gives the same codes and distances. For tests
 * and comparisons: AUTO = the fastest the shape allows (D == 8: tcgen05 tensor-core filter for K a multiple of 64
 * up to 256, else the mma.sync filter for K a multiple of 8; other shapes the exact kernel). */
#define IBCU_KMEANS_AUTO     0
#define IBCU_KMEANS_EXACT    1   /* every distance in the exact form on the CUDA cores */
#define IBCU_KMEANS_MMA_SYNC 2   /* never the tcgen05 kernel */
void ibcu_kmeans_set_path(ibcu_ctx* ctx, int path);
/* The accumulate half of pq_assign_task (src/pq_kmeans.c:183-201): sums[K*D] (FP32), counts[K],
 * inertia (double, sum of dist) over this context's N points, deterministic for a given N. */
int ibcu_kmeans_accumulate(ibcu_ctx* ctx, const float* X, long N, int D, int K,
                           const int32_t* idx, const float* dist,
                           float* sums, int32_t* counts, double* inertia);
/* Centroid move of lloyd_one_init (src/pq_kmeans.c:252-283): C[k] = sums[k] * (1/count[k]) for
 * non-empty clusters; shift (device float, may be NULL) = sum of squared moves. */
int ibcu_kmeans_update(ibcu_ctx* ctx, float* C, int K, int D, const float* sums,
                       const int32_t* counts, float* shift);
/* One Lloyd iteration = assign + accumulate (+ all-reduce of sums/counts/inertia when the context
 * has a communicator) + update. */
int ibcu_kmeans_lloyd_iter(ibcu_ctx* ctx, const float* X, long N, int D, float* C, int K,
                           int32_t* idx, float* dist, float* sums, int32_t* counts, double* inertia);

/* ── decode-step glue (ib_kernels.rmsnorm/rope/softmax/silu_mul, src/kernels/scalar.c:126-181,
 *    and the helpers of src/forward.c) ─────────────────────────────────────────────────── */
/* x[b*hidden + i] = embed[token_b*hidden + i] * fp16(scale[token_b])  (src/forward.c:94-106) */
int ibcu_embed_int8(ibcu_ctx* ctx, const int8_t* embed, const uint16_t* scale, const int32_t* tokens,
                    float* x, int hidden, int B);
/* The same for the three embedding storage forms of embedding_lookup (src/forward.c:90-135): bits 8, bits 4
 * (two columns per byte, low nibble first, bias 8) - both with fp16 row scales - and bits 16 (fp16 rows). */
int ibcu_embed_rows(ibcu_ctx* ctx, const void* embed, const uint16_t* scale, const int32_t* tokens,
                    float* x, int hidden, int B, int bits);
/* out = x * rsqrt(mean(x^2) + eps) * fp16(w), per row of B (src/forward.c:322-327). */
int ibcu_rmsnorm_fp16w(ibcu_ctx* ctx, float* out, const float* x, const uint16_t* w, float eps, int N, int B);
/* Same with FP32 weights, the form ib_kernels.rmsnorm receives (src/kernels/scalar.c:126-138). */
int ibcu_rmsnorm_f32w(ibcu_ctx* ctx, float* out, const float* x, const float* w, float eps, int N, int B);
/* RoPE on adjacent pairs for every Q head and every K head of B positions pos0+b, then the FP32
 * KV-cache write at those positions (src/forward.c:577-593, src/kernels/scalar.c:140-157).
 * k_cache / v_cache / v may be NULL: rotation only (the plain ib_kernels.rope call). */
int ibcu_rope_kv_write(ibcu_ctx* ctx, float* q, float* k, const float* v, float* k_cache, float* v_cache,
                       int n_heads, int n_kv_heads, int head_dim, int pos0, int B, float theta);
/* GQA attention of B query positions against cache rows 0..pos0+b (src/forward.c:463-504). */
int ibcu_attention(ibcu_ctx* ctx, const float* q, const float* k_cache, const float* v_cache, float* out,
                   int n_heads, int n_kv_heads, int head_dim, int pos0, int B);
/* The attention step of a decode layer in one call: what ibcu_rope_kv_write followed by ibcu_attention
 * computes for out and for the cache rows pos0..pos0+B-1 (src/forward.c:577-593 and 463-504). q and k
 * hold the raw projections and are left as they are (the reference rotates its scratch copies in
 * place; nothing reads them afterwards). */
int ibcu_attention_decode(ibcu_ctx* ctx, float* q, float* k, const float* v, float* k_cache, float* v_cache, float* out,
                          int n_heads, int n_kv_heads, int head_dim, int pos0, int B, float theta);
/* The same step with the position pos0 read from device memory when the kernels run, and grid, shared
 * memory and scratch sized for max_ctx cache rows: a launch captured into a CUDA graph then serves every
 * position of an autoregressive decode (pos0 + B <= max_ctx). Needs at most 8 query heads per KV head,
 * head_dim a multiple of 4 up to 256 and 16-byte aligned q / caches. */
int ibcu_attention_decode_at(ibcu_ctx* ctx, float* q, float* k, const float* v, float* k_cache, float* v_cache, float* out,
                             int n_heads, int n_kv_heads, int head_dim, const int* pos0_dev, int max_ctx, int B, float theta);
/* out[b] = silu(gate[b]) * up[b] over rows of N, and amax[b*parts + p] = max|out[b]| over the p-th of `parts`
 * equal column ranges: the element-wise step of the MLP (src/forward.c:637-640) shaped for IBCU_PRO_KNOWN_MAX. */
int ibcu_silu_mul_amax(ibcu_ctx* ctx, float* out, const float* gate, const float* up, int N, int B, float* amax, int parts);
int ibcu_silu_mul(ibcu_ctx* ctx, float* out, const float* gate, const float* up, size_t n);
int ibcu_add_inplace(ibcu_ctx* ctx, float* x, const float* y, size_t n);
int ibcu_softmax(ibcu_ctx* ctx, float* data, int N, int rows);

/* ── multi-GPU (one process per GPU; NCCL over NVLink/NVSwitch) ──────────────────────── */
/* The reference's only parallelism is a row-slicing thread pool (src/threading.c:220-258); the
 * same row slices are spread over GPUs here. id is an opaque 128-byte token made on rank 0 and
 * handed to every rank by the launcher. */
#define IBCU_COMM_ID_BYTES 128
int ibcu_comm_get_id(void* id_out);
int ibcu_comm_init(ibcu_ctx* ctx, const void* id, int rank, int world);
int ibcu_comm_rank(const ibcu_ctx* ctx, int* rank, int* world);
/* Rows [row0, row0+rows) of an M-row tensor owned by `rank` (contiguous, remainder to the low ranks,
 * multiples of `align` rows except for the last owner). */
void ibcu_shard_rows(int M, int world, int rank, int align, int* row0, int* rows);
/* In-place all-gather of row-sharded outputs: buf[b*stride + r], every rank owns its ibcu_shard_rows
 * slice (align as given) and receives the others. */
int ibcu_allgather_rows(ibcu_ctx* ctx, float* buf, int M, int stride, int B, int align);
/* Peer window: a slab of this GPU's memory that the other ranks of the node map (CUDA IPC) so that an
 * all-gather becomes one kernel per rank storing its row slice straight into the peers' buffers over
 * NVLink, with an epoch flag and a bounded wait, instead of an NCCL launch. Every rank calls
 * ibcu_window_create (after ibcu_comm_init) with the same size, the launcher hands the 64-byte handles
 * round, every rank calls ibcu_window_open for every peer, and buffers to be gathered are taken from
 * the window with ibcu_window_alloc in the same order on every rank (same offsets). ibcu_window_alloc
 * returns IBCU_ERR_STATE without touching the context's error when there is no window.
 * ibcu_allgather_rows_n gathers up to four such buffers in one kernel; it falls back to NCCL for
 * buffers outside the window, when not every peer is mapped, after ibcu_window_enable(ctx, 0), and for
 * a buffer that was part of the previous push (peers may still be reading it). A rank whose peers do
 * not arrive within about a second stops waiting and the next ibcu_sync returns IBCU_ERR_COMM.
 * No counterpart in the reference (its workers share one address space). */
#define IBCU_WINDOW_HANDLE_BYTES 64
int ibcu_window_create(ibcu_ctx* ctx, size_t bytes, void* handle_out);
int ibcu_window_open(ibcu_ctx* ctx, int peer_rank, const void* handle);
int ibcu_window_alloc(ibcu_ctx* ctx, size_t bytes, void** dptr);
void ibcu_window_enable(ibcu_ctx* ctx, int on);
int ibcu_allgather_rows_n(ibcu_ctx* ctx, float* const* bufs, const int* M, const int* stride, int n, int B, int align);
/* Announces the next ibcu_allgather_rows_n over these buffers ahead of the ibcu_linear* calls that produce this rank's row
 * slices of them. When the buffers lie in the peer window (and none was part of the previous push), those calls store
 * their rows into the peers' copies from the kernel's own epilogue, the last block publishes the epoch, and the gather
 * call that follows has nothing left to launch: the kernel that consumes the gathered rows (a linear, the attention step,
 * ibcu_silu_mul_amax), or a small waiting kernel ahead of any other consumer, of ibcu_memcpy_d2h and of ibcu_sync, waits
 * - with the same limit - for the peers' epochs in its prologue. Without a window the call does nothing and the gather
 * works as before. Invariant for callers: every read of a gathered buffer must be issued before the rank's next gather but
 * one of that buffer begins, and consecutive gathers must use different buffers (else the slower path is taken). */
int ibcu_allgather_rows_prepare(ibcu_ctx* ctx, float* const* bufs, const int* stride, int n);
/* For tests of the bounded wait, on one GPU and without any peer: launches the waiting kernel on a private header in which
 * one of two ranks never publishes. The kernel gives up at its limit (a second or two); the next ibcu_sync returns
 * IBCU_ERR_COMM and the context stays usable after ibcu_clear_error. */
int ibcu_gather_wait_probe(ibcu_ctx* ctx);
int ibcu_allreduce_f32(ibcu_ctx* ctx, float* buf, size_t n);
int ibcu_allreduce_i32(ibcu_ctx* ctx, int32_t* buf, size_t n);
int ibcu_allreduce_f64(ibcu_ctx* ctx, double* buf, size_t n);

#ifdef __cplusplus
}
#endif
#endif
