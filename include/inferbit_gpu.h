/*
 * inferbit_gpu.h — the part of libinferbit's public C API (include/inferbit.h in the reference checkout)
 * that the quantized-weight product path needs, served by the B200 backend. Same names, same argument
 * meaning, same return codes and error-string behaviour as the reference, so a program or FFI binding
 * written against the reference's libinferbit.so can load libinferbit_b200/libinferbit.so instead.
 *
 * Kept: configuration, load / free, forward, KV-cache control, model info, last error.
 * Not provided: generate / stream / speculative decoding / perplexity / calibration / conversion
 * (token-level control flow and offline tooling; they are not on the hot path and stay in the
 * reference).
 *
 * There is no CPU path: loading needs a B200; without one inferbit_load returns NULL and
 * inferbit_last_error says so.
 */
#ifndef INFERBIT_GPU_H
#define INFERBIT_GPU_H
#include <stddef.h>
#include <stdint.h>
#include "ib_b200.h"
#ifdef __cplusplus
extern "C" {
#endif
#define IBG_API __attribute__((visibility("default")))

/* include/inferbit.h:43-49 */
#define INFERBIT_OK              0
#define INFERBIT_ERROR_LOAD     -1
#define INFERBIT_ERROR_FORMAT   -2
#define INFERBIT_ERROR_MEMORY   -3
#define INFERBIT_ERROR_CONTEXT  -4
#define INFERBIT_ERROR_PARAM    -5
#define INFERBIT_ERROR_INTERNAL -6

/* Thread-local, read-once: returns NULL when no error is pending (src/error.c:7-22, include/inferbit.h:51). */
IBG_API const char* inferbit_last_error(void);

typedef struct inferbit_model  inferbit_model;     /* include/inferbit.h:55-56 */
typedef struct inferbit_config inferbit_config;

/* include/inferbit.h:60-69, src/config.c:5-41. threads is accepted and ignored (the GPU grid is the pool);
 * context_length, when positive and below the file's max_context_length, is the KV capacity and the limit
 * inferbit_forward enforces; kv_cache_dynamic is accepted (the cache is allocated up front either way);
 * native_parse makes inferbit_load fail as it does in the reference (src/model.c:25-29). */
IBG_API inferbit_config* inferbit_config_create(void);
IBG_API void             inferbit_config_free(inferbit_config* config);
IBG_API void inferbit_config_set_threads(inferbit_config* config, int threads);
IBG_API void inferbit_config_set_context_length(inferbit_config* config, int length);
IBG_API void inferbit_config_set_kv_cache_dynamic(inferbit_config* config, int dynamic);
IBG_API void inferbit_config_set_native_parse(inferbit_config* config, int enabled);
IBG_API void inferbit_config_set_native_bits(inferbit_config* config, int bits);

/* include/inferbit.h:73-74; src/model.c:20-36 (extension check), src/ibf_loader.c:351-546 (IBF-v1 reader).
 * Reads the file's header, maps the file, uploads every tensor to HBM with the bit width the header gives
 * it (4 or 8 for linear layers; 8, 4 or 16 for the embedding), allocates an FP32 KV cache (header
 * kv_cache.bits must be 16, which is what the reference's converter writes, src/convert.c:349) and drops
 * the mapping. Returns NULL on failure with the reason in inferbit_last_error. The GPU is chosen by the
 * environment variable INFERBIT_B200_DEVICE (default 0). */
IBG_API inferbit_model* inferbit_load(const char* path, const inferbit_config* config);
IBG_API void            inferbit_free(inferbit_model* model);

/* include/inferbit.h:111-117; src/generate.c:225-241, src/forward.c:850-902. Appends num_tokens positions to
 * the KV cache and writes the logits of the LAST one to out_logits[vocab_size]. Errors: INFERBIT_ERROR_PARAM
 * (NULL argument, vocab_size mismatch, token out of range), INFERBIT_ERROR_CONTEXT (cache would overflow),
 * INFERBIT_ERROR_INTERNAL (GPU failure). INT4 layers take FP32 activations (the reference's IB_W4A8=0 route). */
IBG_API int inferbit_forward(inferbit_model* model, const int32_t* tokens, int num_tokens, float* out_logits, int vocab_size);

/* include/inferbit.h:121-123, src/kv_cache.c:5-26 */
IBG_API void inferbit_kv_clear(inferbit_model* model);
IBG_API void inferbit_kv_truncate(inferbit_model* model, int length);
IBG_API int  inferbit_kv_length(const inferbit_model* model);

/* include/inferbit.h:127-135, src/model.c:98-158 */
IBG_API const char* inferbit_model_architecture(const inferbit_model* model);
IBG_API int         inferbit_model_num_layers(const inferbit_model* model);
IBG_API int         inferbit_model_hidden_size(const inferbit_model* model);
IBG_API int         inferbit_model_vocab_size(const inferbit_model* model);
IBG_API int         inferbit_model_max_context(const inferbit_model* model);
IBG_API int         inferbit_model_default_bits(const inferbit_model* model);
IBG_API size_t      inferbit_model_weight_memory(const inferbit_model* model);
IBG_API size_t      inferbit_model_kv_memory(const inferbit_model* model);
IBG_API size_t      inferbit_model_total_memory(const inferbit_model* model);

/* ── product-quantised tensors from files (src/pq_decode.h:89-135, :189, :2259) ──────────
 * The reference's loader names for its "IBF v5" files, filling the reference's own structs (ib_b200_pq_tensor and
 * ib_b200_pq_multi are field-for-field ib_pq_tensor and ib_pq_multi), and its matvec names over the GPU:
 * ib_pq_load_single reads the first tensor of a file, ib_pq_load_multi all of them with their names, the raw tensors
 * and the free-form config object (as compact JSON text); both return 0, or -1 with the output zeroed, under the
 * reference's checks (src/pq_decode.c:391-546). Arrays live in host memory owned by the struct until ib_pq_free /
 * ib_pq_multi_free, which also drop the tensor's copy in HBM. Memory-mapped opening (ib_pq_open_mmap) is not provided:
 * the arrays go to HBM on first use anyway. */
IBG_API int  ib_pq_load_single(const char* path, ib_b200_pq_tensor* out);
IBG_API void ib_pq_free(ib_b200_pq_tensor* t);
IBG_API int  ib_pq_load_multi(const char* path, ib_b200_pq_multi* out);
IBG_API void ib_pq_multi_free(ib_b200_pq_multi* m);
IBG_API const ib_b200_pq_tensor* ib_pq_multi_find(const ib_b200_pq_multi* m, const char* name);
IBG_API int  ib_pq_matmul_fp32(const ib_b200_pq_tensor* t, const float* x, float* out);
IBG_API int  ib_pq_lm_head_topk(const ib_b200_pq_tensor* t, const float* x, int K_top, float* out_logits, int32_t* out_token_ids);

#ifdef __cplusplus
}
#endif
#endif
