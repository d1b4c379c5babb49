/*
 * ib_b200.h — C host layer of the B200 backend (libib_b200.so). It mirrors, name for name and
 * argument for argument, the interfaces through which libinferbit reaches its quantized-weight
 * product kernels, and forwards them to the CUDA backend (include/ibcu.h). Plain C, host pointers.
 *
 * There is no CPU fallback: a call whose weights were not registered, or that fails on the GPU,
 * records an error (ib_b200_last_error) and leaves its outputs untouched.
 */
#ifndef IB_B200_H
#define IB_B200_H
#include <stddef.h>
#include <stdint.h>
#include "ibcu.h"
#ifdef __cplusplus
extern "C" {
#endif

/* ── process-wide backend (the reference's kernel table is process-global too,
 *    src/kernels/scalar.c:185) ─────────────────────────────────────────────────────────── */
int         ib_b200_init(int device);            /* 0 or a negative IBCU_ERR_* */
void        ib_b200_shutdown(void);
ibcu_ctx*   ib_b200_ctx(void);                   /* the context behind the table, NULL before init */
/* Sticky error of the table calls, which return void like the reference's (src/inferbit_internal.h:199-277);
 * read-once like inferbit_last_error (src/error.c:14-22). */
int         ib_b200_status(void);
const char* ib_b200_last_error(void);

/* Weights live in a read-only host mapping owned by the model (src/ibf_loader.c:471-503) and the
 * table calls only carry host pointers, so the mapping is copied to HBM once and calls translate
 * host addresses inside a registered range to device addresses by offset. */
int  ib_b200_register(const void* host_base, size_t bytes);
int  ib_b200_unregister(const void* host_base);

/* Bytes the table calls have moved since ib_b200_init: host->device (activations; row scales when first seen
 * or changed) and device->host (results). */
void ib_b200_copy_stats(unsigned long long* h2d_bytes, unsigned long long* d2h_bytes);

/* ── ib_kernels-shaped dispatch table (src/inferbit_internal.h:199-277) ─────────────── */
typedef struct {
    void (*matmul_int4)(float* out, const void* weights, const float* scales, const float* input, int M, int N);
    void (*matmul_int8)(float* out, const void* weights, const float* scales, const float* input, int M, int N);
    void (*matmul_int2)(float* out, const void* weights, const float* scales, const float* input, int M, int N);
    void (*rmsnorm)(float* out, const float* input, const float* weight, float eps, int N);
    void (*rope)(float* q, float* k, int head_dim, int pos, float theta);
    void (*softmax)(float* data, int N);
    void (*silu_mul)(float* out, const float* gate, const float* up, int N);
    void (*matmul_w4a8)(float* out, const void* weights, const float* scales_w, const int8_t* input,
                        const float* scales_a, int M, int N);
    void (*matmul_w4a8_batch)(float* out, const void* weights, const float* scales_w, const int8_t* input,
                              const float* scales_a, int M, int N, int B, int M_stride);
    void (*matmul_int8_batch)(float* out, const void* weights, const float* scales_w, const float* input,
                              int M, int N, int B, int M_stride);
} ib_b200_kernels;

/* Fill a table with the GPU entries. `table` may be the reference's own global ib_kern
 * (src/kernels/scalar.c:185): the field order above is the reference's. matmul_int2 is left as it
 * is (the 2-bit ternary kernel is outside this backend). Call again after every model load, because
 * ibf_load re-runs ib_init_kernels (src/ibf_loader.c:539-540). */
void ib_b200_install_kernels(void* table);
/* Row-sliced, pre-offset calls from pool workers (src/threading.c:220-241) are accepted: weights,
 * scales and out may point inside a tensor, and several workers may call at the same time: every
 * entry takes one process-wide lock, so concurrent calls run one after another on the device. With
 * threads <= 1 the reference makes exactly one call per linear (src/threading.c:247-252), which is
 * the mode this backend wants. */
void ib_b200_matmul_int4(float* out, const void* weights, const float* scales, const float* input, int M, int N);
void ib_b200_matmul_int8(float* out, const void* weights, const float* scales, const float* input, int M, int N);
void ib_b200_matmul_int8_batch(float* out, const void* weights, const float* scales_w, const float* input,
                               int M, int N, int B, int M_stride);
void ib_b200_matmul_w4a8(float* out, const void* weights, const float* scales_w, const int8_t* input,
                         const float* scales_a, int M, int N);
void ib_b200_matmul_w4a8_batch(float* out, const void* weights, const float* scales_w, const int8_t* input,
                               const float* scales_a, int M, int N, int B, int M_stride);
void ib_b200_rmsnorm(float* out, const float* input, const float* weight, float eps, int N);
void ib_b200_rope(float* q, float* k, int head_dim, int pos, float theta);
void ib_b200_softmax(float* data, int N);
void ib_b200_silu_mul(float* out, const float* gate, const float* up, int N);
/* ib_quantize_input_int8_g128 (src/threading.c:401-432); returns the number of groups. */
int  ib_b200_quantize_input_int8_g128(const float* input, int8_t* out_q, float* out_scales, int N);

/* ── PQ matvec (src/pq_decode.h:189-222) ─────────────────────────────────────────────── */
/* Field-for-field copy of ib_pq_tensor (src/pq_decode.h:39-87), so a pointer to the reference's
 * struct can be passed as is. */
typedef struct {
    int M, N, G, K, K_l2, n_levels, rotate, n_outlier;
    int format;
    uint16_t* codebook_l1_l; uint16_t* codebook_l1_r; uint16_t* codebook_l2_l; uint16_t* codebook_l2_r;
    uint8_t* indices_l1_l; uint8_t* indices_l1_r; uint8_t* indices_l2_l; uint8_t* indices_l2_r;
    int C, l2_idx_bytes, l2_packed_bits;
    uint16_t* row_scale;
    int32_t* outlier_cols; int8_t* outlier_sidecar; uint16_t* outlier_scale;
    void* _arena; size_t _arena_size; void* _mmap_base; size_t _mmap_size; int _owns_mmap;
} ib_b200_pq_tensor;

/* Field-for-field copies of ib_pq_raw_tensor and ib_pq_multi (src/pq_decode.h:108-131): what the multi-tensor file
 * reader fills (ib_pq_load_multi in include/inferbit_gpu.h). */
typedef struct {
    char* name; void* data; int dtype; int ndim; int shape[4]; size_t size_bytes; int _owns_data;
} ib_b200_pq_raw_tensor;
typedef struct {
    int n; char** names; ib_b200_pq_tensor* tensors; void* _mmap_base; size_t _mmap_size;
    int n_raw; ib_b200_pq_raw_tensor* raw_tensors; char* config_json;
} ib_b200_pq_multi;

/* ib_pq_matmul_fp32: out[M] = W x. One or two levels (second level: at most 256 entries, one-byte or 4-bit packed
 * indices), optional int8 outlier sidecar, formats "l1", "l2", "l1_l2" (or none, for a struct filled by hand); the
 * pyramid format and uint16 second-level indices return -1 (as the reference does for a bad argument). The tensor's
 * arrays are copied to HBM on first use and cached by the address of the struct; ib_b200_pq_release drops the copy. */
int  ib_b200_pq_matmul_fp32(const ib_b200_pq_tensor* t, const float* x, float* out);
int  ib_b200_pq_matmul_fp32_threaded(const ib_b200_pq_tensor* t, const float* x, float* out, void* pool);
int  ib_b200_pq_matmul_fp32_streaming(const ib_b200_pq_tensor* t, const float* x, float* out);
/* B activations at once, x[b*N + j] -> out[b*M + r] (the reference loops, src/pq_decode.c:5848-5851). */
int  ib_b200_pq_matmul_fp32_batch(const ib_b200_pq_tensor* t, const float* x, float* out, int B);
/* ib_pq_lm_head_topk (src/pq_decode.c:2259-2341): ids and full logits of the K_top rows with the largest first-level
 * logits, by descending full logit. Host pointers; -1 on a bad argument like the reference (K_top outside 1..M), and
 * for K_top above 1024, which this backend does not take. */
int  ib_b200_pq_lm_head_topk(const ib_b200_pq_tensor* t, const float* x, int K_top, float* out_logits, int32_t* out_token_ids);
void ib_b200_pq_release(const ib_b200_pq_tensor* t);

/* ── k-means (src/pq_kmeans.h:60-74) ─────────────────────────────────────────────────── */
/* ib_kmeans_assign; `pool` is ignored. X is copied to HBM per call unless it lies in a registered range. */
int ib_b200_kmeans_assign(const float* X, int N, int D, const float* centers, int K, int32_t* indices_out, void* pool);
/* The Lloyd loop of lloyd_one_init (src/pq_kmeans.c:232-288) from caller-given initial centroids:
 * exactly `iters` iterations when tol < 0, else the reference's two stopping rules. centers[K*D] is
 * updated in place; indices_out / inertia_out may be NULL. Returns iterations run, or < 0. */
int ib_b200_kmeans_lloyd(const float* X, int N, int D, int K, int iters, float tol,
                         float* centers, int32_t* indices_out, double* inertia_out);

/* ── decode step (ib_forward / ib_forward_positions, src/forward.c:850-939) ──────────── */
typedef struct {
    int hidden, inter, n_layers, n_heads, n_kv_heads, head_dim, vocab, max_ctx;
    float eps, theta;
    int attn_bits, mlp_bits, head_bits;      /* 8 / 4 / 8 in the benchmark configuration */
} ib_b200_model_cfg;
typedef struct ib_b200_model ib_b200_model;

enum { IB_B200_Q = 0, IB_B200_K, IB_B200_V, IB_B200_O, IB_B200_GATE, IB_B200_UP, IB_B200_DOWN, IB_B200_HEAD };

/* A model lives on one context; with a communicator on the context every linear is row-sharded over
 * the ranks (the reference's row slices, src/threading.c:220-241) and gathered after each layer op. */
ib_b200_model* ib_b200_model_create(ibcu_ctx* ctx, const ib_b200_model_cfg* cfg);
/* Same with a bit width (4 or 8) per tensor, as a model file gives them: linear_bits[layer * 7 + which] for
 * which = IB_B200_Q..IB_B200_DOWN, then linear_bits[n_layers * 7] for the head (NULL: the widths of cfg).
 * embed_bits: storage form of the embedding rows, 8, 4 or 16 (src/forward.c:90-135). */
ib_b200_model* ib_b200_model_create_bits(ibcu_ctx* ctx, const ib_b200_model_cfg* cfg, const int* linear_bits, int embed_bits);
void           ib_b200_model_free(ib_b200_model* m);
/* Random weights written straight into HBM (counter-based generator), norms near 1, KV cache
 * positions [0, kv_fill) filled with bell-shaped values of unit variance. Every tensor is a function of the
 * seed and its place in the model only: N ranks together hold exactly the model one rank would hold. */
int  ib_b200_model_fill_random(ib_b200_model* m, uint64_t seed, int kv_fill);
/* Upload one full (unsharded) tensor from host memory; each rank keeps its row slice.
 * layer is ignored for IB_B200_HEAD. w: int8 [M*N] or packed nibbles [M*N/2]; scales: fp16 [M], or NULL for
 * a tensor stored without scales (scale 1, src/forward.c:152-156). */
int  ib_b200_model_set_linear(ib_b200_model* m, int layer, int which, const void* w, const uint16_t* scales);
int  ib_b200_model_set_norms(ib_b200_model* m, int layer, const uint16_t* input_norm, const uint16_t* post_attn_norm);
/* embed: rows in the model's embedding storage form; embed_scale: fp16 [vocab] or NULL (rows used as they are). */
int  ib_b200_model_set_embedding(ib_b200_model* m, const void* embed, const uint16_t* embed_scale, const uint16_t* final_norm);
int  ib_b200_model_set_kv(ib_b200_model* m, int layer, const float* k, const float* v, int n_pos);
int  ib_b200_model_get_kv(ib_b200_model* m, int layer, float* k, float* v, int n_pos);
/* B consecutive positions pos0.. of one sequence (B == 1: forward_single_ex, src/forward.c:518-664;
 * B > 1: forward_batch, :682-846). tokens and logits are host arrays; logits [B*vocab] may be NULL.
 * The launch sequence is captured into a CUDA graph per batch size on first use and replayed for every
 * position (the position is read on the device); the call that captures runs the step eagerly first. */
int  ib_b200_forward_step(ib_b200_model* m, const int32_t* tokens, int pos0, int B, float* logits);
/* Same step, but only the last position goes through the output head: logits_last [vocab] (what ib_forward
 * keeps of a multi-token call, src/forward.c:872-901). */
int  ib_b200_forward_step_last(ib_b200_model* m, const int32_t* tokens, int pos0, int B, float* logits_last);
/* Same without host traffic: tokens already in the model's device token buffer (ib_b200_model_tokens),
 * logits left in ib_b200_model_logits. */
int    ib_b200_forward_step_device(ib_b200_model* m, int pos0, int B);
/* 0: issue the launches of a step one by one instead of replaying a graph (for per-kernel profiles). */
void   ib_b200_model_use_graph(ib_b200_model* m, int on);
void*  ib_b200_model_tokens(ib_b200_model* m);
float* ib_b200_model_logits(ib_b200_model* m);
/* Bytes of weights + scales this rank streams per decoded position. */
size_t ib_b200_model_weight_bytes(const ib_b200_model* m);

#ifdef __cplusplus
}
#endif
#endif
