"""ctypes binding of libatlas_kernels.so (the C ABI in include/atlas_kernels.h).

This is the stand-in for the `mod ffi` block of the reference's atlas-tensor crate
(crates/atlas-tensor/src/lib.rs:17-92): thin declarations, no logic.  There is no CPU
fallback — if the library is missing or no CUDA device is present, calls raise.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "lib", "libatlas_kernels.so")

F32, BF16, INT8, INT4, F16 = 0, 1, 2, 3, 4
AUTO = -1

T_EMBED, T_FINAL_NORM, T_LM_HEAD = 0, 1, 2
T_WQ, T_WK, T_WV, T_WO, T_GATE, T_UP, T_DOWN = 10, 11, 12, 13, 14, 15, 16
T_ATTN_NORM, T_FFN_NORM, T_Q_NORM, T_K_NORM = 17, 18, 19, 20


class AtlasError(RuntimeError):
    """Counterpart of AtlasError (crates/atlas-core/src/lib.rs:12-28) for the CUDA path."""


class ModelConfigC(C.Structure):
    _fields_ = [
        ("vocab_size", C.c_int), ("d_model", C.c_int), ("n_layers", C.c_int), ("n_heads", C.c_int),
        ("n_kv_heads", C.c_int), ("ffn_hidden", C.c_int), ("max_seq_len", C.c_int),
        ("rope_theta", C.c_float), ("rms_norm_eps", C.c_float), ("sliding_window", C.c_int),
        ("rope_scaling", C.c_int), ("yarn_factor", C.c_float), ("yarn_orig_max_pos", C.c_int),
        ("yarn_attn_factor", C.c_float), ("yarn_beta_fast", C.c_float), ("yarn_beta_slow", C.c_float),
        ("post_norm", C.c_int), ("eos_token_id", C.c_int), ("kv_dtype", C.c_int),
        ("weight_format", C.c_int), ("int4_block", C.c_int), ("tp_rank", C.c_int), ("tp_world", C.c_int),
    ]


class SamplingConfigC(C.Structure):
    _fields_ = [("temperature", C.c_float), ("repetition_penalty", C.c_float), ("repetition_window", C.c_int),
                ("frequency_penalty", C.c_float), ("presence_penalty", C.c_float), ("top_p", C.c_float),
                ("top_k", C.c_int), ("min_p", C.c_float)]


class LoadStatsC(C.Structure):
    _fields_ = [("seconds", C.c_double), ("file_bytes_read", C.c_size_t), ("bytes_uploaded", C.c_size_t),
                ("peak_host_rss_bytes", C.c_size_t), ("n_tensors_used", C.c_int), ("post_norm", C.c_int),
                ("tied_lm_head", C.c_int), ("weight_format", C.c_int)]


TOKEN_CALLBACK = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_uint32)
LAYER_HOOK = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_int, C.POINTER(C.c_float), C.c_int, C.POINTER(C.c_float))

_lib = None

vp, sz, u64, ci, cf = C.c_void_p, C.c_size_t, C.c_uint64, C.c_int, C.c_float
pvp = C.POINTER(C.c_void_p)
pi = C.POINTER(C.c_int)

# name -> (restype, argtypes); every symbol declared in include/atlas_kernels.h
SIGNATURES = {
    # reference ABI
    "atlas_sync": (None, []),
    "atlas_matmul_f32": (None, [vp, vp, vp, ci, ci, ci]),
    "atlas_sgemm_bf16_f32": (None, [vp, vp, vp, ci, ci, ci]),
    "atlas_vec_add_f32": (None, [vp, vp, vp, ci]),
    "atlas_scale_f32": (None, [vp, cf, vp, ci]),
    "atlas_relu_f32": (None, [vp, vp, ci]),
    "atlas_softmax_f32": (None, [vp, vp, ci, ci]),
    "atlas_rmsnorm_f32": (None, [vp, vp, vp, ci, cf]),
    "atlas_rope_apply_f32": (None, [vp, ci, ci, cf]),
    "atlas_silu_mul_f32": (None, [vp, vp, vp, ci]),
    "atlas_vram_copy_f32": (None, [vp, vp, ci]),
    "atlas_adamw_step": (None, [vp, vp, vp, vp, cf, cf, cf, cf, cf, cf, cf, ci]),
    "atlas_qk_norm_inplace": (None, [vp, vp, ci, ci, cf]),
    "atlas_rope_precomputed": (None, [vp, vp, vp, ci, ci, ci, ci]),
    "atlas_kv_cache_write": (None, [vp, vp, vp, vp, ci, ci, ci]),
    "atlas_decode_attention": (None, [vp, vp, vp, vp, ci, ci, ci, ci, cf, ci]),
    "atlas_gpu_argmax": (None, [vp, vp, ci]),
    "atlas_cuda_available": (ci, []),
    "atlas_cuda_device_count": (ci, []),
    "atlas_quantize_int8": (None, [vp, vp, vp, ci, ci]),
    "atlas_dequantize_int8": (None, [vp, vp, vp, ci, ci]),
    "atlas_quantize_int4": (None, [vp, vp, vp, ci]),
    # B200 surface
    "atlasx_last_error": (C.c_char_p, []),
    "atlasx_ctx_create": (ci, [ci, pvp]),
    "atlasx_ctx_destroy": (ci, [vp]),
    "atlasx_ctx_sync": (ci, [vp]),
    "atlasx_ctx_stream": (vp, [vp]),
    "atlasx_ctx_sm_count": (ci, [vp]),
    "atlasx_ctx_set_gemv_impl": (ci, [vp, ci]),
    "atlasx_ctx_poll_device_error": (ci, [vp, pi]),
    "atlasx_malloc": (ci, [vp, sz, pvp]),
    "atlasx_free": (ci, [vp, vp]),
    "atlasx_memset": (ci, [vp, vp, ci, sz]),
    "atlasx_upload": (ci, [vp, vp, vp, sz]),
    "atlasx_download": (ci, [vp, vp, vp, sz]),
    "atlasx_copy_dev": (ci, [vp, vp, vp, sz]),
    "atlasx_fill_normal_f32": (ci, [vp, vp, sz, u64, u64, u64, cf]),
    "atlasx_fill_normal_bf16": (ci, [vp, vp, sz, u64, u64, u64, cf]),
    "atlasx_convert_bf16_to_f32": (ci, [vp, vp, vp, sz]),
    "atlasx_convert_f32_to_bf16": (ci, [vp, vp, vp, sz, ci]),
    "atlasx_quantize_int8": (ci, [vp, vp, ci, ci, vp, vp]),
    "atlasx_dequantize_int8": (ci, [vp, vp, vp, ci, ci, vp]),
    "atlasx_quantize_int4": (ci, [vp, vp, sz, ci, vp, vp]),
    "atlasx_dequantize_int4": (ci, [vp, vp, vp, sz, ci, vp]),
    "atlasx_matrix_upload_f32": (ci, [vp, vp, ci, ci, pvp]),
    "atlasx_matrix_upload_bf16": (ci, [vp, vp, ci, ci, pvp]),
    "atlasx_matrix_upload_int8": (ci, [vp, vp, vp, ci, ci, pvp]),
    "atlasx_matrix_upload_int4": (ci, [vp, vp, vp, ci, ci, ci, ci, pvp]),
    "atlasx_matrix_wrap": (ci, [vp, ci, vp, vp, ci, ci, ci, ci, pvp]),
    "atlasx_matrix_free": (ci, [vp]),
    "atlasx_matrix_info": (ci, [vp, pi, pi, pi]),
    "atlasx_matrix_bytes": (sz, [vp]),
    "atlasx_gemv": (ci, [vp, vp, vp, ci, vp]),
    "atlasx_matrix_sgemm": (ci, [vp, vp, vp, ci, ci, vp]),
    "atlasx_vec_add": (ci, [vp, vp, vp, vp, ci]),
    "atlasx_rmsnorm": (ci, [vp, vp, vp, vp, ci, cf]),
    "atlasx_silu_mul": (ci, [vp, vp, vp, vp, ci]),
    "atlasx_qk_norm_inplace": (ci, [vp, vp, vp, ci, ci, cf]),
    "atlasx_argmax": (ci, [vp, vp, ci, pi]),
    "atlasx_rope_tables_host": (ci, [ci, ci, cf, ci, cf, ci, cf, cf, vp, vp]),
    "atlasx_rope_apply": (ci, [vp, vp, vp, vp, ci, ci, ci, ci]),
    "atlasx_kvcache_create": (ci, [vp, ci, ci, ci, ci, ci, pvp]),
    "atlasx_kvcache_free": (ci, [vp]),
    "atlasx_kvcache_ptrs": (ci, [vp, pvp, pvp, C.POINTER(sz)]),
    "atlasx_kvcache_write": (ci, [vp, vp, vp, vp, vp]),
    "atlasx_decode_attention": (ci, [vp, vp, vp, vp, ci, vp, cf, ci]),
    "atlasx_decode_attention_bytes": (sz, [vp, ci, vp, ci]),
    "atlasx_decode_attention_static": (ci, [vp, ci, vp, vp, ci, ci, ci, ci, vp, vp, ci, vp, cf, ci]),
    "atlasx_model_create": (ci, [vp, C.POINTER(ModelConfigC), vp, pvp]),
    "atlasx_model_free": (ci, [vp]),
    "atlasx_model_set_tensor": (ci, [vp, ci, ci, vp, ci, ci]),
    "atlasx_model_tensor_slice": (ci, [vp, ci, C.POINTER(sz), C.POINTER(sz), C.POINTER(sz), C.POINTER(sz), C.POINTER(sz), C.POINTER(sz), pi]),
    "atlasx_model_set_tensor_slice": (ci, [vp, ci, ci, vp, ci, ci]),
    "atlasx_model_finalize": (ci, [vp]),
    "atlasx_safetensors_open": (ci, [C.c_char_p, pvp]),
    "atlasx_safetensors_close": (ci, [vp]),
    "atlasx_safetensors_count": (ci, [vp]),
    "atlasx_safetensors_find": (ci, [vp, C.c_char_p]),
    "atlasx_safetensors_tensor": (ci, [vp, ci, C.POINTER(C.c_char_p), pi, pi, C.POINTER(sz), C.POINTER(sz)]),
    "atlasx_safetensors_read": (ci, [vp, ci, sz, sz, sz, sz, ci, vp]),
    "atlasx_safetensors_write": (ci, [C.c_char_p, ci, vp, vp, vp, vp, vp]),
    "atlasx_model_load_safetensors": (ci, [vp, vp, ci, C.POINTER(ModelConfigC), vp, pvp, C.POINTER(LoadStatsC)]),
    "atlasx_config_patch_from_json": (ci, [C.c_char_p, C.POINTER(ModelConfigC), vp, pi]),
    "atlasx_model_load_dir": (ci, [vp, C.c_char_p, C.POINTER(ModelConfigC), vp, pvp, C.POINTER(LoadStatsC)]),
    "atlasx_model_reset": (ci, [vp]),
    "atlasx_model_pos": (ci, [vp]),
    "atlasx_model_forward_one": (ci, [vp, C.c_uint32, vp]),
    "atlasx_model_generate_greedy": (ci, [vp, vp, ci, ci, vp, ci, cf, ci, vp, ci, vp, pi]),
    "atlasx_sample_token": (ci, [vp, vp, ci, C.POINTER(SamplingConfigC), ci, vp, ci, vp, ci, C.POINTER(u64), pi, vp]),
    "atlasx_model_generate_sampling": (ci, [vp, vp, ci, ci, C.POINTER(SamplingConfigC), vp, ci, vp, ci, u64, ci, vp, pi]),
    "atlasx_model_decode_timed": (ci, [vp, ci, ci, C.POINTER(cf), vp]),
    "atlasx_model_profile_step": (ci, [vp, ci, vp, vp, vp, pi]),
    "atlasx_model_class_name": (C.c_char_p, [ci]),
    "atlasx_model_step_bytes": (C.c_double, [vp, ci]),
    "atlasx_model_kernel_launches_per_step": (ci, [vp]),
    "atlasx_model_set_options": (ci, [vp, ci, ci]),
    "atlasx_model_set_prefill": (ci, [vp, ci, vp]),
    "atlasx_model_time_classes": (ci, [vp, C.c_uint, ci, vp, vp, vp]),
    "atlasx_model_hidden": (ci, [vp, vp]),
    "atlasx_model_layer_hidden": (ci, [vp, ci, vp]),
    "atlasx_model_set_layer_hook": (ci, [vp, vp, vp]),
    "atlasx_model_set_token_callback": (ci, [vp, vp, vp]),
    "atlasx_model_deposits": (ci, [vp, vp, vp, vp, ci, pi]),
    "atlasx_time_gemv": (ci, [vp, vp, ci, vp, ci, vp, ci, C.POINTER(cf)]),
    "atlasx_time_attention": (ci, [vp, vp, vp, vp, ci, vp, cf, ci, ci, C.POINTER(cf)]),
    "atlasx_comm_unique_id": (ci, [vp]),
    "atlasx_comm_init": (ci, [vp, vp, ci, ci]),
    "atlasx_comm_world": (ci, [vp]),
    "atlasx_comm_selftest_wait_expiry": (ci, [vp, vp, ci]),
    "atlasx_comm_allreduce": (ci, [vp, vp, ci]),
}


def lib():
    """Load the library once.  Raises if it was not built (run `python atlas_b200/build.py`)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise AtlasError("%s is missing: build it with `python atlas_b200/build.py` "
                             "(there is no CPU fallback)" % LIB_PATH)
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(rc):
    if rc != 0:
        raise AtlasError(lib().atlasx_last_error().decode("utf-8", "replace") or ("error %d" % rc))


def cuda_available():
    """cuda_available(), crates/atlas-tensor/src/lib.rs:129-134."""
    return lib().atlas_cuda_available() != 0


def cuda_device_count():
    return lib().atlas_cuda_device_count()
