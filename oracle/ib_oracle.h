/*
 * ib_oracle.h — CPU restatement of libinferbit's quantized-weight product hot path.
 *
 * TEST INFRASTRUCTURE ONLY. This is the checker the GPU kernels are compared against; it is
 * never linked, loaded or called by the product libraries (libibcu.so / libib_b200.so).
 * Every function names the reference lines it restates (paths relative to the reference
 * checkout). Parity status: PINNED — tests/test_oracle_vs_ref.py runs each function against
 * the unmodified reference library built by oracle/Makefile (oracle/_ref/libinferbit_ref.so)
 * and tests/golden/ holds outputs of that reference on seeded inputs.
 */
#ifndef IB_ORACLE_H
#define IB_ORACLE_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

/* src/forward.c:38-70, src/pq_decode.c:263-288 — exact binary16 -> binary32 widening. */
float    ibo_fp16_to_fp32(uint16_t h);
/* src/pq_decode.c:295-337 — binary32 -> binary16, round to nearest even. */
uint16_t ibo_fp32_to_fp16(float f);
void     ibo_fp16_array_to_fp32(const uint16_t* in, float* out, int n);

/* src/kernels/scalar.c:9-27 */
void ibo_matmul_int4(float* out, const uint8_t* w, const float* scales, const float* x, int M, int N);
/* src/kernels/scalar.c:29-41 */
void ibo_matmul_int8(float* out, const int8_t* w, const float* scales, const float* x, int M, int N);
/* src/kernels/scalar.c:70-84 */
void ibo_matmul_int8_batch(float* out, const int8_t* w, const float* scales, const float* x,
                           int M, int N, int B, int M_stride);
/* src/forward.c:226-233 — INT4 with FP32 activations has no batched kernel: one call per position. */
void ibo_matmul_int4_batch(float* out, const uint8_t* w, const float* scales, const float* x,
                           int M, int N, int B, int M_stride);
/* src/threading.c:401-432 */
int  ibo_quantize_input_int8_g128(const float* x, int8_t* q, float* sa, int N);
/* src/kernels/scalar.c:43-68 and :86-124 */
void ibo_matmul_w4a8(float* out, const uint8_t* w, const float* sw, const int8_t* xq,
                     const float* sa, int M, int N);
void ibo_matmul_w4a8_batch(float* out, const uint8_t* w, const float* sw, const int8_t* xq,
                           const float* sa, int M, int N, int B, int M_stride);

/* src/pq_decode.c:1504-1682 (matmul_impl) + :1441-1496 (pq_gather_rows), single level, no outliers.
 * cb_l / cb_r: K*(G/2) fp16 bit patterns shared by all chunks; idx_l / idx_r: M*C uint8, C = N/G.
 * cb_chunk_stride = 0 restates the reference (shared tables); a non-zero stride (in fp16 elements)
 * gives each chunk its own K*(G/2) table at cb + c*stride (same arithmetic, per-chunk pointer).
 * fused != 0 uses fmaf for the LUT dot products, as the reference's -mfma build does.
 * Returns 0, or -1 on a bad argument. n_skipped (may be NULL) receives the number of chunks
 * dropped by the 1 %-of-max activation rule (src/pq_decode.c:1582-1616). */
int ibo_pq_matmul_fp32(int M, int N, int G, int K,
                       const uint16_t* cb_l, const uint16_t* cb_r, long cb_chunk_stride,
                       const uint8_t* idx_l, const uint8_t* idx_r, const uint16_t* row_scale,
                       const float* x, float* out, int fused, int* n_skipped);
/* The same with a second residual level (one-byte or 4-bit-packed indices) and the outlier sidecar
 * (src/pq_decode.c:1058-1075, :1394-1409, :1441-1496, :1538-1546); NULL / 0 switch a part off. */
int ibo_pq_matmul_fp32_ex(int M, int N, int G, int K, int K_l2,
                          const uint16_t* cb1_l, const uint16_t* cb1_r, const uint16_t* cb2_l, const uint16_t* cb2_r,
                          const uint8_t* idx1_l, const uint8_t* idx1_r, const uint8_t* idx2_l, const uint8_t* idx2_r,
                          const uint16_t* row_scale, int n_outlier, const int32_t* outlier_cols,
                          const int8_t* outlier_sidecar, const uint16_t* outlier_scale,
                          const float* x, float* out, int fused);
/* src/pq_decode.c:2259-2341 (ib_pq_lm_head_topk) with its two helpers (:2085-2143 first level only, no 1 % rule;
 * :2145-2248 every level of the chosen rows): ids and logits of the K_top rows with the largest first-level
 * logits, ordered by their full logits, descending. coarse_out (may be NULL) receives the M first-level logits. */
int ibo_pq_lm_head_topk(int M, int N, int G, int K, int K_l2,
                        const uint16_t* cb1_l, const uint16_t* cb1_r, const uint16_t* cb2_l, const uint16_t* cb2_r,
                        const uint8_t* idx1_l, const uint8_t* idx1_r, const uint8_t* idx2_l, const uint8_t* idx2_r,
                        const uint16_t* row_scale, int n_outlier, const int32_t* outlier_cols,
                        const int8_t* outlier_sidecar, const uint16_t* outlier_scale,
                        const float* x, int K_top, float* out_logits, int32_t* out_ids, float* coarse_out, int fused);
/* src/pq_decode.c:3565-3651, :3854-3882 — group-scaled INT4 rows of the session engine (parity unpinned: static
 * functions there, no entry point). eps_act_rel <= 0: no group is left out (the reference's default). */
int ibo_int4g_matmul_fp32(int M, int N, int G, const uint8_t* q, const uint16_t* s, int K_out,
                          const uint16_t* outl_idx, const uint16_t* outl_val, const float* x, float* out,
                          float eps_act_rel, int fused);
/* src/pq_decode.c:5008-5066 — PQ KV cache encode of one vector (parity unpinned: no entry point in the reference). */
void ibo_pqkv_encode(const float* vec, int dim, int G, int K1, const uint16_t* cb_l, const uint16_t* cb_r,
                     uint8_t* idx, float* scale, int fused);
/* src/pq_decode.c:1103-1196 — dense W[M*N] from codes, every value rounded through fp16. */
int ibo_pq_reconstruct_fp32(int M, int N, int G, int K,
                            const uint16_t* cb_l, const uint16_t* cb_r,
                            const uint8_t* idx_l, const uint8_t* idx_r, const uint16_t* row_scale,
                            float* W);

/* src/pq_kmeans.c:99-122 — nearest centroid, direct squared distance, strict '<'.
 * fused: 0 = s + v*v with two roundings; 1 = fmaf(v, v, s); 2 = the mix the reference's x86-64
 * Release binary executes (unfused for d < 4*floor(D/4), fused for the remaining D%4 dimensions),
 * which is the mode the GPU kernel is held to. dist_out may be NULL. */
void ibo_kmeans_assign(const float* X, long N, int D, const float* C, int K,
                       int32_t* idx, float* dist_out, int fused);
/* src/pq_kmeans.c:183-201 + :249-283 — one Lloyd iteration on a single lane: assign, accumulate
 * sums/counts/inertia in point order, then move the centroids (empty cluster keeps its place).
 * sums[K*D], counts[K] are outputs; returns the centroid shift (FP32 sum of squared moves). */
float ibo_kmeans_lloyd_iter(const float* X, long N, int D, float* C, int K, int32_t* idx,
                            float* sums, int32_t* counts, double* inertia, int fused);
/* centroid move only (src/pq_kmeans.c:252-283) from given sums/counts. */
float ibo_kmeans_update(float* C, int K, int D, const float* sums, const int32_t* counts);

/* src/kernels/scalar.c:126-181 */
void ibo_rmsnorm(float* out, const float* x, const float* w, float eps, int N);
void ibo_rope(float* q, float* k, int head_dim, int pos, float theta);
void ibo_softmax(float* v, int N);
void ibo_silu_mul(float* out, const float* gate, const float* up, int N);

/* In-memory model for the decode-step restatement (src/forward.c:518-664 and :682-846).
 * Attention projections, MLP projections and the head are per-row-scaled INT8 or INT4
 * (bits = 8 / 4); the embedding is INT8 with an fp16 scale per token; norms are fp16;
 * the KV cache is FP32 (header kv bits >= 16, src/forward.c:355-361). */
typedef struct {
    const void*     w;       /* [M*N] int8 or [M*N/2] packed nibbles */
    const uint16_t* scale;   /* [M] fp16 */
    int M, N, bits;
} ibo_linear;

typedef struct {
    ibo_linear q, k, v, o, gate, up, down;
    const uint16_t* input_norm;      /* [hidden] fp16 */
    const uint16_t* post_attn_norm;  /* [hidden] fp16 */
    float* k_cache;                  /* [max_ctx * kv_dim] */
    float* v_cache;
} ibo_layer;

typedef struct {
    int hidden, inter, n_layers, n_heads, n_kv_heads, head_dim, vocab, max_ctx;
    float eps, theta;
    const int8_t*   embed;           /* [vocab*hidden] */
    const uint16_t* embed_scale;     /* [vocab] fp16 */
    const uint16_t* final_norm;      /* [hidden] fp16 */
    ibo_linear head;
    ibo_layer* layers;
} ibo_model;

/* B consecutive positions pos0..pos0+B-1 of one sequence (B == 1 is the single-token path).
 * logits: [B*vocab] or NULL. hidden_out: [B*hidden] post-final-norm hidden or NULL.
 * Returns 0, -1 on bad arguments. */
int ibo_decode_step(ibo_model* m, const int32_t* tokens, int pos0, int B,
                    float* logits, float* hidden_out);

#ifdef __cplusplus
}
#endif
#endif
