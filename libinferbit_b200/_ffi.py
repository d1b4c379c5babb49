"""ctypes bindings for the two product libraries, libibcu.so (CUDA backend, include/ibcu.h) and
libib_b200.so (C host layer, include/ib_b200.h).

There is no fallback: if a library is missing or a call fails, an exception is raised.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIBIBCU_PATH = os.path.join(_HERE, "libibcu.so")
LIBHOST_PATH = os.path.join(_HERE, "libib_b200.so")

c_void_pp = C.POINTER(C.c_void_p)


class LinearT(C.Structure):
    """ibcu_linear_t"""
    _fields_ = [("w", C.c_void_p), ("scales", C.c_void_p), ("out", C.c_void_p),
                ("M", C.c_int), ("out_stride", C.c_int), ("scales_fp32", C.c_int), ("epilogue", C.c_int)]


class PrologueT(C.Structure):
    """ibcu_prologue_t"""
    _fields_ = [("op", C.c_int), ("x2", C.c_void_p), ("norm_w", C.c_void_p), ("eps", C.c_float),
                ("amax", C.c_void_p), ("n_amax", C.c_int)]


class PqT(C.Structure):
    """ibcu_pq_t"""
    _fields_ = [("M", C.c_int), ("N", C.c_int), ("G", C.c_int), ("K", C.c_int),
                ("codebook_l", C.c_void_p), ("codebook_r", C.c_void_p), ("cb_chunk_stride", C.c_long),
                ("idx_l", C.c_void_p), ("idx_r", C.c_void_p), ("row_scale", C.c_void_p),
                ("idx_t", C.c_void_p), ("M_pad", C.c_int),
                ("K_l2", C.c_int), ("codebook2_l", C.c_void_p), ("codebook2_r", C.c_void_p), ("idx2_l", C.c_void_p), ("idx2_r", C.c_void_p),
                ("n_outlier", C.c_int), ("outlier_cols", C.c_void_p), ("outlier_sidecar", C.c_void_p), ("outlier_scale", C.c_void_p),
                ("inner_cols", C.c_void_p)]


class Int4gT(C.Structure):
    """ibcu_int4g_t"""
    _fields_ = [("M", C.c_int), ("N", C.c_int), ("G", C.c_int), ("K_out", C.c_int),
                ("q", C.c_void_p), ("s", C.c_void_p), ("outl_idx", C.c_void_p), ("outl_val", C.c_void_p)]


# name -> (restype, argtypes); every symbol include/ibcu.h declares
IBCU_SYMBOLS = {
    "ibcu_ctx_create": (C.c_int, [C.c_int, c_void_pp]),
    "ibcu_ctx_destroy": (None, [C.c_void_p]),
    "ibcu_status": (C.c_int, [C.c_void_p]),
    "ibcu_last_error": (C.c_char_p, [C.c_void_p]),
    "ibcu_clear_error": (None, [C.c_void_p]),
    "ibcu_device_count": (C.c_int, []),
    "ibcu_device_sm_count": (C.c_int, [C.c_void_p]),
    "ibcu_malloc": (C.c_int, [C.c_void_p, C.c_size_t, c_void_pp]),
    "ibcu_free": (C.c_int, [C.c_void_p, C.c_void_p]),
    "ibcu_host_alloc": (C.c_int, [C.c_void_p, C.c_size_t, c_void_pp]),
    "ibcu_host_free": (C.c_int, [C.c_void_p, C.c_void_p]),
    "ibcu_memcpy_h2d": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t]),
    "ibcu_memcpy_d2h": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t]),
    "ibcu_memcpy_d2d": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t]),
    "ibcu_memset": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_size_t]),
    "ibcu_sync": (C.c_int, [C.c_void_p]),
    "ibcu_sync_spin": (C.c_int, [C.c_void_p]),
    "ibcu_store_i32": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32]),
    "ibcu_fill_hash_bytes": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_uint64]),
    "ibcu_fill_hash_bytes_at": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_uint64, C.c_size_t]),
    "ibcu_fill_hash_fp16_uniform_at": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_uint64, C.c_float, C.c_float, C.c_size_t]),
    "ibcu_fill_hash_f32_normal_at": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_uint64, C.c_float, C.c_float, C.c_size_t]),
    "ibcu_hash_bytes_host": (None, [C.c_void_p, C.c_size_t, C.c_uint64, C.c_size_t]),
    "ibcu_fill_hash_fp16_uniform": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_uint64, C.c_float, C.c_float]),
    "ibcu_hash_fp16_uniform_host": (None, [C.c_void_p, C.c_size_t, C.c_uint64, C.c_float, C.c_float, C.c_size_t]),
    "ibcu_event_record": (C.c_int, [C.c_void_p, C.c_int]),
    "ibcu_event_elapsed_ms": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_float)]),
    "ibcu_graph_begin": (C.c_int, [C.c_void_p]),
    "ibcu_graph_end": (C.c_int, [C.c_void_p, C.POINTER(C.c_int)]),
    "ibcu_graph_launch": (C.c_int, [C.c_void_p, C.c_int]),
    "ibcu_graph_destroy": (C.c_int, [C.c_void_p, C.c_int]),
    "ibcu_launch_count": (C.c_uint64, [C.c_void_p]),
    "ibcu_set_pdl": (None, [C.c_void_p, C.c_int]),
    "ibcu_linear": (C.c_int, [C.c_void_p, C.POINTER(LinearT), C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int]),
    "ibcu_linear_ex": (C.c_int, [C.c_void_p, C.POINTER(LinearT), C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int, C.POINTER(PrologueT)]),
    "ibcu_linear_gate_up_silu": (C.c_int, [C.c_void_p, C.POINTER(LinearT), C.c_void_p, C.c_int, C.c_int, C.c_int]),
    "ibcu_linear_force_generic": (None, [C.c_void_p, C.c_int]),
    "ibcu_linear_use_tcgen05": (None, [C.c_void_p, C.c_int]),
    "ibcu_quantize_input_int8_g128": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int]),
    "ibcu_linear_w4a8": (C.c_int, [C.c_void_p, C.POINTER(LinearT), C.c_void_p, C.c_void_p, C.c_int, C.c_int]),
    "ibcu_linear_w4a8_fp32": (C.c_int, [C.c_void_p, C.POINTER(LinearT), C.c_void_p, C.c_int, C.c_int]),
    "ibcu_pq_idx_t_bytes": (C.c_size_t, [C.c_int, C.c_int, C.c_int]),
    "ibcu_pq_prepared_bytes": (C.c_size_t, [C.POINTER(PqT)]),
    "ibcu_pq_prepare": (C.c_int, [C.c_void_p, C.POINTER(PqT), C.c_void_p]),
    "ibcu_pq_matmul_fp32": (C.c_int, [C.c_void_p, C.POINTER(PqT), C.c_void_p, C.c_void_p, C.c_int]),
    "ibcu_pqkv_encode": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "ibcu_pq_matmul_fp32_strided": (C.c_int, [C.c_void_p, C.POINTER(PqT), C.c_void_p, C.c_void_p, C.c_int, C.c_int]),
    "ibcu_int4g_matmul_fp32": (C.c_int, [C.c_void_p, C.POINTER(Int4gT), C.c_void_p, C.c_void_p, C.c_float]),
    "ibcu_pq_lm_head_topk": (C.c_int, [C.c_void_p, C.POINTER(PqT), C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]),
    "ibcu_pq_matmul_fp32_noalloc": (C.c_int, [C.c_void_p, C.POINTER(PqT), C.c_void_p, C.c_void_p, C.c_int]),
    "ibcu_pq_noalloc_max_floats": (C.c_size_t, []),
    "ibcu_kmeans_assign": (C.c_int, [C.c_void_p, C.c_void_p, C.c_long, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]),
    "ibcu_kmeans_set_path": (None, [C.c_void_p, C.c_int]),
    "ibcu_kmeans_accumulate": (C.c_int, [C.c_void_p, C.c_void_p, C.c_long, C.c_int, C.c_int, C.c_void_p, C.c_void_p,
                                         C.c_void_p, C.c_void_p, C.c_void_p]),
    "ibcu_kmeans_update": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]),
    "ibcu_kmeans_lloyd_iter": (C.c_int, [C.c_void_p, C.c_void_p, C.c_long, C.c_int, C.c_void_p, C.c_int, C.c_void_p,
                                         C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "ibcu_embed_int8": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int]),
    "ibcu_embed_rows": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int]),
    "ibcu_rmsnorm_fp16w": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_int, C.c_int]),
    "ibcu_rmsnorm_f32w": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_int, C.c_int]),
    "ibcu_rope_kv_write": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                     C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float]),
    "ibcu_silu_mul_amax": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int]),
    "ibcu_attention_decode": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                        C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float]),
    "ibcu_attention_decode_at": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                           C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_float]),
    "ibcu_attention": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                 C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]),
    "ibcu_silu_mul": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t]),
    "ibcu_add_inplace": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t]),
    "ibcu_softmax": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int]),
    "ibcu_comm_get_id": (C.c_int, [C.c_void_p]),
    "ibcu_comm_init": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int]),
    "ibcu_comm_rank": (C.c_int, [C.c_void_p, C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "ibcu_shard_rows": (None, [C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "ibcu_allgather_rows": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int]),
    "ibcu_window_create": (C.c_int, [C.c_void_p, C.c_size_t, C.c_void_p]),
    "ibcu_window_open": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p]),
    "ibcu_window_alloc": (C.c_int, [C.c_void_p, C.c_size_t, C.POINTER(C.c_void_p)]),
    "ibcu_window_enable": (None, [C.c_void_p, C.c_int]),
    "ibcu_allgather_rows_n": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_int), C.POINTER(C.c_int), C.c_int, C.c_int, C.c_int]),
    "ibcu_allgather_rows_prepare": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_int), C.c_int]),
    "ibcu_gather_wait_probe": (C.c_int, [C.c_void_p]),
    "ibcu_allreduce_f32": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t]),
    "ibcu_allreduce_i32": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t]),
    "ibcu_allreduce_f64": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t]),
}

_libibcu = None


def load_ibcu():
    """Load libibcu.so and attach prototypes. Raises OSError if the library has not been built."""
    global _libibcu
    if _libibcu is None:
        if not os.path.exists(LIBIBCU_PATH):
            raise OSError(f"{LIBIBCU_PATH} not found: build it with `make -C libinferbit_b200` "
                          "(or __graft_entry__.build()); there is no CPU fallback")
        lib = C.CDLL(LIBIBCU_PATH, mode=C.RTLD_GLOBAL)
        for name, (res, args) in IBCU_SYMBOLS.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _libibcu = lib
    return _libibcu


class ModelCfg(C.Structure):
    """ib_b200_model_cfg"""
    _fields_ = [(n, C.c_int) for n in ("hidden", "inter", "n_layers", "n_heads", "n_kv_heads", "head_dim", "vocab", "max_ctx")] + [
        ("eps", C.c_float), ("theta", C.c_float), ("attn_bits", C.c_int), ("mlp_bits", C.c_int), ("head_bits", C.c_int)]


class HostPqTensor(C.Structure):
    """ib_b200_pq_tensor == ib_pq_tensor (src/pq_decode.h:39-87)"""
    _fields_ = [("M", C.c_int), ("N", C.c_int), ("G", C.c_int), ("K", C.c_int), ("K_l2", C.c_int),
                ("n_levels", C.c_int), ("rotate", C.c_int), ("n_outlier", C.c_int), ("format", C.c_int),
                ("codebook_l1_l", C.c_void_p), ("codebook_l1_r", C.c_void_p),
                ("codebook_l2_l", C.c_void_p), ("codebook_l2_r", C.c_void_p),
                ("indices_l1_l", C.c_void_p), ("indices_l1_r", C.c_void_p),
                ("indices_l2_l", C.c_void_p), ("indices_l2_r", C.c_void_p),
                ("C", C.c_int), ("l2_idx_bytes", C.c_int), ("l2_packed_bits", C.c_int),
                ("row_scale", C.c_void_p), ("outlier_cols", C.c_void_p), ("outlier_sidecar", C.c_void_p),
                ("outlier_scale", C.c_void_p), ("_arena", C.c_void_p), ("_arena_size", C.c_size_t),
                ("_mmap_base", C.c_void_p), ("_mmap_size", C.c_size_t), ("_owns_mmap", C.c_int)]


_MM = C.CFUNCTYPE(None, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int)


class HostKernels(C.Structure):
    """ib_b200_kernels == ib_kernels (src/inferbit_internal.h:199-277)"""
    _fields_ = [
        ("matmul_int4", _MM), ("matmul_int8", _MM), ("matmul_int2", _MM),
        ("rmsnorm", C.CFUNCTYPE(None, C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_int)),
        ("rope", C.CFUNCTYPE(None, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_float)),
        ("softmax", C.CFUNCTYPE(None, C.c_void_p, C.c_int)),
        ("silu_mul", C.CFUNCTYPE(None, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int)),
        ("matmul_w4a8", C.CFUNCTYPE(None, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int)),
        ("matmul_w4a8_batch", C.CFUNCTYPE(None, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int)),
        ("matmul_int8_batch", C.CFUNCTYPE(None, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int)),
    ]


_vp, _i, _f = C.c_void_p, C.c_int, C.c_float
HOST_SYMBOLS = {
    "ib_b200_init": (_i, [_i]),
    "ib_b200_shutdown": (None, []),
    "ib_b200_ctx": (_vp, []),
    "ib_b200_status": (_i, []),
    "ib_b200_last_error": (C.c_char_p, []),
    "ib_b200_register": (_i, [_vp, C.c_size_t]),
    "ib_b200_unregister": (_i, [_vp]),
    "ib_b200_copy_stats": (None, [C.POINTER(C.c_ulonglong), C.POINTER(C.c_ulonglong)]),
    "ib_b200_install_kernels": (None, [_vp]),
    "ib_b200_matmul_int4": (None, [_vp, _vp, _vp, _vp, _i, _i]),
    "ib_b200_matmul_int8": (None, [_vp, _vp, _vp, _vp, _i, _i]),
    "ib_b200_matmul_int8_batch": (None, [_vp, _vp, _vp, _vp, _i, _i, _i, _i]),
    "ib_b200_matmul_w4a8": (None, [_vp, _vp, _vp, _vp, _vp, _i, _i]),
    "ib_b200_matmul_w4a8_batch": (None, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i]),
    "ib_b200_rmsnorm": (None, [_vp, _vp, _vp, _f, _i]),
    "ib_b200_rope": (None, [_vp, _vp, _i, _i, _f]),
    "ib_b200_softmax": (None, [_vp, _i]),
    "ib_b200_silu_mul": (None, [_vp, _vp, _vp, _i]),
    "ib_b200_quantize_input_int8_g128": (_i, [_vp, _vp, _vp, _i]),
    "ib_b200_pq_matmul_fp32": (_i, [C.POINTER(HostPqTensor), _vp, _vp]),
    "ib_b200_pq_matmul_fp32_threaded": (_i, [C.POINTER(HostPqTensor), _vp, _vp, _vp]),
    "ib_b200_pq_matmul_fp32_streaming": (_i, [C.POINTER(HostPqTensor), _vp, _vp]),
    "ib_b200_pq_matmul_fp32_batch": (_i, [C.POINTER(HostPqTensor), _vp, _vp, _i]),
    "ib_b200_pq_lm_head_topk": (_i, [C.POINTER(HostPqTensor), _vp, _i, _vp, _vp]),
    "ib_b200_pq_release": (None, [C.POINTER(HostPqTensor)]),
    "ib_b200_kmeans_assign": (_i, [_vp, _i, _i, _vp, _i, _vp, _vp]),
    "ib_b200_kmeans_lloyd": (_i, [_vp, _i, _i, _i, _i, _f, _vp, _vp, _vp]),
    "ib_b200_model_create": (_vp, [_vp, C.POINTER(ModelCfg)]),
    "ib_b200_model_create_bits": (_vp, [_vp, C.POINTER(ModelCfg), _vp, _i]),
    "ib_b200_model_free": (None, [_vp]),
    "ib_b200_model_fill_random": (_i, [_vp, C.c_uint64, _i]),
    "ib_b200_model_set_linear": (_i, [_vp, _i, _i, _vp, _vp]),
    "ib_b200_model_set_norms": (_i, [_vp, _i, _vp, _vp]),
    "ib_b200_model_set_embedding": (_i, [_vp, _vp, _vp, _vp]),
    "ib_b200_model_set_kv": (_i, [_vp, _i, _vp, _vp, _i]),
    "ib_b200_model_get_kv": (_i, [_vp, _i, _vp, _vp, _i]),
    "ib_b200_forward_step": (_i, [_vp, _vp, _i, _i, _vp]),
    "ib_b200_forward_step_last": (_i, [_vp, _vp, _i, _i, _vp]),
    "ib_b200_forward_step_device": (_i, [_vp, _i, _i]),
    "ib_b200_model_use_graph": (None, [_vp, _i]),
    "ib_b200_model_tokens": (_vp, [_vp]),
    "ib_b200_model_logits": (_vp, [_vp]),
    "ib_b200_model_weight_bytes": (C.c_size_t, [_vp]),
}

_libhost = None


def load_host():
    """Load libib_b200.so (and libibcu.so before it). Raises OSError if it has not been built."""
    global _libhost
    if _libhost is None:
        load_ibcu()
        if not os.path.exists(LIBHOST_PATH):
            raise OSError(f"{LIBHOST_PATH} not found: build it with `make -C libinferbit_b200`")
        lib = C.CDLL(LIBHOST_PATH, mode=C.RTLD_GLOBAL)
        for name, (res, args) in HOST_SYMBOLS.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _libhost = lib
    return _libhost


FRONT_PATH = os.path.join(_HERE, "libinferbit.so")
_sz = C.c_size_t
FRONT_SYMBOLS = {
    "inferbit_last_error": (C.c_char_p, []),
    "inferbit_config_create": (_vp, []),
    "inferbit_config_free": (None, [_vp]),
    "inferbit_config_set_threads": (None, [_vp, _i]),
    "inferbit_config_set_context_length": (None, [_vp, _i]),
    "inferbit_config_set_kv_cache_dynamic": (None, [_vp, _i]),
    "inferbit_config_set_native_parse": (None, [_vp, _i]),
    "inferbit_config_set_native_bits": (None, [_vp, _i]),
    "inferbit_load": (_vp, [C.c_char_p, _vp]),
    "inferbit_free": (None, [_vp]),
    "inferbit_forward": (_i, [_vp, _vp, _i, _vp, _i]),
    "inferbit_kv_clear": (None, [_vp]),
    "inferbit_kv_truncate": (None, [_vp, _i]),
    "inferbit_kv_length": (_i, [_vp]),
    "inferbit_model_architecture": (C.c_char_p, [_vp]),
    "inferbit_model_num_layers": (_i, [_vp]),
    "inferbit_model_hidden_size": (_i, [_vp]),
    "inferbit_model_vocab_size": (_i, [_vp]),
    "inferbit_model_max_context": (_i, [_vp]),
    "inferbit_model_default_bits": (_i, [_vp]),
    "inferbit_model_weight_memory": (_sz, [_vp]),
    "inferbit_model_kv_memory": (_sz, [_vp]),
    "inferbit_model_total_memory": (_sz, [_vp]),
    "ib_pq_load_single": (_i, [C.c_char_p, _vp]),
    "ib_pq_free": (None, [_vp]),
    "ib_pq_load_multi": (_i, [C.c_char_p, _vp]),
    "ib_pq_multi_free": (None, [_vp]),
    "ib_pq_multi_find": (_vp, [_vp, C.c_char_p]),
    "ib_pq_matmul_fp32": (_i, [_vp, _vp, _vp]),
    "ib_pq_lm_head_topk": (_i, [_vp, _vp, _i, _vp, _vp]),
}

_libfront = None


def load_front():
    """Load libinferbit.so, the reference-named entry points (include/inferbit_gpu.h). Loaded with local
    symbol scope: the names are the reference's own, and a process may hold the reference library too."""
    global _libfront
    if _libfront is None:
        load_host()
        if not os.path.exists(FRONT_PATH):
            raise OSError(f"{FRONT_PATH} not found: build it with `make -C libinferbit_b200`")
        lib = C.CDLL(FRONT_PATH, mode=C.RTLD_LOCAL)
        for name, (res, args) in FRONT_SYMBOLS.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _libfront = lib
    return _libfront
