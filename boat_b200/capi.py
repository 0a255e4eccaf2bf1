"""ctypes bindings of ``libboat_b200.so``: every function declared under ``include/``.

``load()`` returns the library with argument and result types set, so a wrong call fails
in Python instead of corrupting memory.  Names, argument order and meaning are those of
the C headers (which in turn are the reference's).
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

# enum values of include/boat/tensor.h and include/boat_cuda.h
DTYPE_FLOAT64, DTYPE_FLOAT32, DTYPE_FLOAT16 = 0, 1, 2
DTYPE_BFLOAT16 = 11
DEVICE_CPU, DEVICE_CUDA = 0, 1
CUDA_F32, CUDA_BF16, CUDA_F32_TF32 = 0, 1, 2
MMA_FP32, MMA_TF32, MMA_BF16 = 0, 1, 2


class LibraryMissing(RuntimeError):
    pass


class AttentionConfig(C.Structure):
    """boat_attention_config_t (include/boat/layers/attention.h)."""
    _fields_ = [("hidden_size", C.c_size_t), ("num_heads", C.c_size_t), ("head_size", C.c_size_t),
                ("dropout_prob", C.c_float), ("causal_mask", C.c_bool), ("use_bias", C.c_bool),
                ("use_rotary", C.c_bool), ("rotary_theta", C.c_float)]


class LayerNormConfig(C.Structure):
    """boat_layernorm_config_t (include/boat/layers/norm.h)."""
    _fields_ = [("normalized_shape", C.c_size_t), ("eps", C.c_float), ("elementwise_affine", C.c_bool),
                ("use_bias", C.c_bool)]


class MemoryStats(C.Structure):
    """boat_memory_stats_t (include/boat/memory.h)."""
    _fields_ = [("allocated_bytes", C.c_size_t), ("allocated_blocks", C.c_size_t),
                ("peak_allocated_bytes", C.c_size_t), ("freed_bytes", C.c_size_t),
                ("freed_blocks", C.c_size_t)]


def lib_path():
    return os.path.join(_HERE, "libboat_b200.so")


_P, _I, _I64, _SZ, _F, _B, _D = C.c_void_p, C.c_int, C.c_int64, C.c_size_t, C.c_float, C.c_bool, C.c_double
_PI64 = C.POINTER(C.c_int64)
_PP = C.POINTER(C.c_void_p)

_ACCESSORS = ["%s_%s" % (k, p) for k in ("weight", "bias", "grad_weight", "grad_bias") for p in "qkvo"]

# name -> (restype, argtypes)
PROTOTYPES = {
    # include/boat/tensor.h
    "boat_tensor_create": (_P, [_PI64, _SZ, _I, _I]),
    "boat_tensor_create_like": (_P, [_P]),
    "boat_tensor_from_data": (_P, [_PI64, _SZ, _I, _P]),
    "boat_tensor_free": (None, [_P]),
    "boat_tensor_ref": (None, [_P]),
    "boat_tensor_unref": (None, [_P]),
    "boat_tensor_shape": (_PI64, [_P]),
    "boat_tensor_ndim": (_SZ, [_P]),
    "boat_tensor_dtype": (_I, [_P]),
    "boat_tensor_device": (_I, [_P]),
    "boat_tensor_nbytes": (_SZ, [_P]),
    "boat_tensor_nelements": (_SZ, [_P]),
    "boat_tensor_is_contiguous": (_B, [_P]),
    "boat_tensor_data": (_P, [_P]),
    "boat_tensor_const_data": (_P, [_P]),
    "boat_tensor_reshape": (_P, [_P, _PI64, _SZ]),
    "boat_tensor_slice": (_P, [_P, C.POINTER(_SZ), C.POINTER(_SZ), C.POINTER(_SZ)]),
    "boat_tensor_to_device": (_P, [_P, _I]),
    "boat_dtype_size": (_SZ, [_I]),
    "boat_dtype_name": (C.c_char_p, [_I]),
    # include/boat/memory.h
    "boat_memory_allocate": (_P, [_SZ, _I, C.c_char_p, _I]),
    "boat_memory_allocate_zero": (_P, [_SZ, _I, C.c_char_p, _I]),
    "boat_memory_reallocate": (_P, [_P, _SZ, _I, C.c_char_p, _I]),
    "boat_memory_free": (None, [_P]),
    "boat_memory_free_safe": (None, [_PP]),
    "boat_memory_allocate_device": (_P, [_SZ, _I, C.c_char_p, _I]),
    "boat_memory_free_device": (None, [_P, _I]),
    "boat_memory_copy": (None, [_P, _P, _SZ, _I, _I]),
    "boat_memory_set": (None, [_P, _I, _SZ, _I]),
    "boat_memory_get_stats": (MemoryStats, []),
    "boat_memory_reset_stats": (None, []),
    "boat_memory_print_stats": (None, [_P]),
    # include/boat/layers/attention.h
    "boat_attention_create": (_P, [C.POINTER(AttentionConfig)]),
    "boat_attention_free": (None, [_P]),
    "boat_attention_forward": (_P, [_P, _P, _P, _P, _P]),
    "boat_attention_backward": (_B, [_P, _P, _PP, _PP, _PP]),
    "boat_attention_update": (None, [_P, _F]),
    "boat_attention_set_dropout": (None, [_P, _F]),
    "boat_attention_set_causal": (None, [_P, _B]),
    "boat_multihead_attention": (_P, [_P, _SZ, _F, _B, _P]),
    "boat_scaled_dot_product_attention": (_P, [_P, _P, _P, _F, _P, _B, _F]),
    "boat_rotary_position_encoding": (_P, [_P, _SZ, _SZ, _F]),
    "boat_apply_rotary_embedding": (None, [_P, _P, _SZ, _SZ, _F]),
    # include/boat/layers.h
    "boat_attention_layer_create": (_P, [_SZ, _SZ, _F, _B]),
    "boat_attention_layer_free": (None, [_P]),
    "boat_attention_layer_forward": (_P, [_P, _P, _P, _P, _P]),
    "boat_attention_layer_backward": (_P, [_P, _P]),
    "boat_attention_layer_update": (None, [_P, _F]),
    # include/boat/autodiff.h
    "boat_variable_create": (_P, [_P, _B]),
    "boat_variable_create_with_shape": (_P, [_PI64, _SZ, _I, _B]),
    "boat_variable_free": (None, [_P]),
    "boat_variable_data": (_P, [_P]),
    "boat_variable_grad": (_P, [_P]),
    "boat_variable_requires_grad": (_B, [_P]),
    "boat_variable_set_requires_grad": (None, [_P, _B]),
    "boat_variable_zero_grad": (None, [_P]),
    "boat_variable_backward": (None, [_P, _P]),
    "boat_variable_backward_full": (None, [_P]),
    "boat_var_attention": (_P, [_P, _P, _P, _P, _P]),
    "boat_var_add": (_P, [_P, _P]),
    "boat_var_sub": (_P, [_P, _P]),
    "boat_var_mul": (_P, [_P, _P]),
    "boat_var_matmul": (_P, [_P, _P]),
    "boat_var_dense": (_P, [_P, _P]),
    # include/boat/ops.h
    "boat_add": (_P, [_P, _P]),
    "boat_mul": (_P, [_P, _P]),
    "boat_sub": (_P, [_P, _P]),
    "boat_add_": (None, [_P, _P]),
    "boat_sub_": (None, [_P, _P]),
    "boat_mul_scalar": (_P, [_P, _D]),
    "boat_matmul": (_P, [_P, _P]),
    "boat_transpose": (_P, [_P, _I, _I]),
    "boat_gelu": (_P, [_P]),
    # include/boat/layers/norm.h and the dense / norm entries of include/boat/layers.h
    "boat_layernorm_create": (_P, [C.POINTER(LayerNormConfig)]),
    "boat_layernorm_free": (None, [_P]),
    "boat_layernorm_forward": (_P, [_P, _P]),
    "boat_layernorm_backward": (_P, [_P, _P]),
    "boat_layernorm_update": (None, [_P, _F]),
    "boat_layernorm_set_weight": (None, [_P, _P]),
    "boat_layernorm_set_bias": (None, [_P, _P]),
    "boat_dense_layer_create": (_P, [_SZ, _SZ, _B]),
    "boat_dense_layer_free": (None, [_P]),
    "boat_dense_layer_forward": (_P, [_P, _P]),
    "boat_dense_layer_backward": (_P, [_P, _P]),
    "boat_dense_layer_update": (None, [_P, _F]),
    "boat_dense_layer_set_weight": (None, [_P, _P]),
    "boat_dense_layer_set_bias": (None, [_P, _P]),
    "boat_dense_layer_get_weight": (_P, [_P]),
    "boat_dense_layer_get_bias": (_P, [_P]),
    "boat_dense_layer_get_grad_weight": (_P, [_P]),
    "boat_dense_layer_get_grad_bias": (_P, [_P]),
    "boat_norm_layer_create": (_P, [_SZ, _F, _B]),
    "boat_norm_layer_free": (None, [_P]),
    "boat_norm_layer_forward": (_P, [_P, _P]),
    "boat_norm_layer_backward": (_P, [_P, _P]),
    "boat_norm_layer_update": (None, [_P, _F]),
    # include/boat_b200.h
    "boat_gelu_backward": (_P, [_P, _P]),
    "boat_lincomb": (_P, [_P, _F, _P, _F]),
    "boat_layernorm_get_weight": (_P, [_P]),
    "boat_layernorm_get_bias": (_P, [_P]),
    "boat_layernorm_get_grad_weight": (_P, [_P]),
    "boat_layernorm_get_grad_bias": (_P, [_P]),
    "boat_layernorm_to_device": (_I, [_P, _I]),
    "boat_dense_layer_to_device": (_I, [_P, _I]),
    "boat_attention_to_device": (_I, [_P, _I]),
    "boat_attention_set_precision": (_I, [_P, _I]),
    "boat_attention_get_precision": (_I, [_P]),
    "boat_attention_forward_units": (_P, [_P, _P, _P, _P, _I64]),
    "boat_attention_grad_bucket": (_I, [_P, C.POINTER(C.POINTER(C.c_float)), C.POINTER(_SZ)]),
    "boat_attention_allreduce_grads": (_I, [_P]),
    "boat_attention_set_grad_overlap": (_I, [_P, _I]),
    "boat_attention_get_grad_overlap": (_I, [_P]),
    "boat_attention_add_to_optimizer": (_I, [_P, _P]),
    "boat_encoder_block_create": (_P, [_P, _P, _P, _P, _P]),
    "boat_encoder_block_forward": (_P, [_P, _P]),
    "boat_encoder_block_backward": (_P, [_P, _P]),
    "boat_encoder_block_free": (None, [_P]),
    "boat_encoder_block_allreduce_grads": (_I, [_P]),
    "boat_attention_load_safetensors": (_I, [_P, _P, _SZ, C.c_char_p]),
    "boat_attention_load_safetensors_file": (_I, [_P, C.c_char_p, C.c_char_p]),
    # include/boat/optimizers.h
    "boat_sgd_optimizer_create": (_P, [_F, _F]),
    "boat_adam_optimizer_create": (_P, [_F, _F, _F, _F]),
    "boat_optimizer_step": (None, [_P]),
    "boat_optimizer_zero_grad": (None, [_P]),
    "boat_optimizer_free": (None, [_P]),
    "boat_optimizer_add_parameter": (None, [_P, _P, _P]),
    "boat_optimizer_get_learning_rate": (_F, [_P]),
    "boat_optimizer_set_learning_rate": (None, [_P, _F]),
    # include/boat_cuda.h
    "boat_cuda_init": (_I, [_I]),
    "boat_cuda_device_count": (_I, []),
    "boat_cuda_last_error": (C.c_char_p, []),
    "boat_cuda_stream": (_P, []),
    "boat_cuda_set_stream": (_I, [_P]),
    "boat_cuda_sync": (_I, []),
    "boat_cuda_malloc": (_I, [_PP, _SZ]),
    "boat_cuda_free": (_I, [_P]),
    "boat_cuda_memcpy_h2d": (_I, [_P, _P, _SZ]),
    "boat_cuda_memcpy_d2h": (_I, [_P, _P, _SZ]),
    "boat_cuda_memcpy_d2d": (_I, [_P, _P, _SZ]),
    "boat_cuda_copies_after_compute": (_I, []),
    "boat_cuda_upload_async": (_I, [_P, _P, _SZ]),
    "boat_cuda_join_uploads": (_I, []),
    "boat_cuda_download_async": (_I, [_P, _P, _SZ]),
    "boat_cuda_memset": (_I, [_P, _I, _SZ]),
    "boat_cuda_host_alloc": (_P, [_SZ]),
    "boat_cuda_host_free": (_I, [_P]),
    "boat_cuda_host_register": (_I, [_P, _SZ]),
    "boat_cuda_host_unregister": (_I, [_P]),
    "boat_cuda_bytes_in_use": (_SZ, []),
    "boat_cuda_launch_count": (C.c_uint64, []),
    "boat_cuda_profile_enable": (_I, [_I]),
    "boat_cuda_profile_report": (_I, [C.c_char_p, _SZ]),
    "boat_cuda_selftest_wait_timeout": (_I, [C.c_uint64]),
    "boat_cuda_gemm": (_I, [_I, _I, _I, _I64, _I64, _I64, _P, _I64, _P, _I64, _I, _P, _I64, _I, _P]),
    "boat_cuda_attn_fwd": (_I, [_I, _I64, _I64, _I64, _I, _F, _P, _P, _P, _I, _P, _P]),
    "boat_cuda_attn_bwd_scratch_bytes": (_SZ, [_I, _I64, _I64, _I64]),
    "boat_cuda_attn_bwd": (_I, [_I, _I64, _I64, _I64, _I, _F, _P, _P, _P, _P, _P, _P, _I, _P, _P, _P, _P, _SZ]),
    "boat_cuda_attn_bwd_static_capacity": (_SZ, []),
    "boat_cuda_attn_bwd_static": (_I, [_I, _I64, _I64, _I64, _I, _F, _P, _P, _P, _P, _P, _P, _I, _P, _P, _P]),
    "boat_cuda_gemm_set_yielding": (_I, [_I]),
    "boat_cuda_gemm_grouped": (_I, [_I, _I, _I, _I, _I64, _I64, _I64, _P, _I64, _P, _I64, _I, _P, _I64, _I, _P]),
    "boat_cuda_colsum": (_I, [_P, _I, _I64, _I64, _P]),
    "boat_cuda_colsum_multi": (_I, [_P, _I, _I64, _I64, _P, _I]),
    "boat_cuda_convert_multi": (_I, [_P, _I, _P, _P, _I]),
    "boat_cuda_axpy": (_I, [_P, _P, _F, _I64]),
    "boat_cuda_scale": (_I, [_P, _P, _F, _I64]),
    "boat_cuda_add_bias": (_I, [_P, _P, _P, _I64, _I64]),
    "boat_cuda_mul": (_I, [_P, _P, _P, _I64]),
    "boat_cuda_lincomb": (_I, [_P, _P, _F, _P, _F, _I, _I64]),
    "boat_cuda_cast": (_I, [_P, _I, _P, _I, _I64]),
    "boat_cuda_round_tf32": (_I, [_P, _P, _I64]),
    "boat_cuda_transpose": (_I, [_P, _P, _I64, _I64, _I64]),
    "boat_cuda_layernorm_fwd": (_I, [_P, _I, _I64, _I64, _P, _P, _F, _P, _P, _P]),
    "boat_cuda_layernorm_bwd": (_I, [_P, _P, _I, _I64, _I64, _P, _P, _P, _P, _P, _P]),
    "boat_cuda_gelu_fwd": (_I, [_P, _P, _I, _I64]),
    "boat_cuda_gelu_bwd": (_I, [_P, _P, _P, _I, _I64]),
    "boat_cuda_adam_step": (_I, [_I, _P, _P, _P, _P, _P, _F, _F, _F, _F, _F, _F]),
    "boat_cuda_comm_unique_id": (_I, [_P]),
    "boat_cuda_comm_init": (_I, [_I, _I, _P]),
    "boat_cuda_comm_world": (_I, []),
    "boat_cuda_allreduce_sum_f32": (_I, [_P, _I64]),
    "boat_cuda_allreduce_begin": (_I, [_P, _P, _I]),
    "boat_cuda_allreduce_join": (_I, []),
    "boat_cuda_allreduce_pending": (_I, []),
    "boat_cuda_comm_destroy": (_I, []),
}
for _name in _ACCESSORS:
    PROTOTYPES["boat_attention_get_" + _name] = (_P, [_P])


def load():
    """Load ``libboat_b200.so`` (once) and type every entry point.  No fallback: a missing
    library raises ``LibraryMissing`` telling how to build it."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = lib_path()
    if not os.path.exists(path):
        raise LibraryMissing("%s not found - build it with `python -c 'import __graft_entry__ as g; g.build()'` "
                             "or `make -C boat_b200/csrc`" % path)
    lib = C.CDLL(path)
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _LIB = lib
    return lib
