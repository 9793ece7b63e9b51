"""Loads the C-ABI library (include/gonano_cuda.h) through ctypes.

There is no fallback: if the library has not been built the import of any
compute path raises, and if no CUDA device is present every compute call
returns GN_ERR_CUDA, which surfaces here as ``GonanoError``.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "libgonano_cuda.so"

f32p = C.POINTER(C.c_float)
i32p = C.POINTER(C.c_int32)
u64p = C.POINTER(C.c_uint64)
vp = C.c_void_p


class GonanoError(RuntimeError):
    pass


class GnConfig(C.Structure):
    _fields_ = [
        ("sequence_len", C.c_int32), ("vocab_size", C.c_int32), ("n_layer", C.c_int32), ("n_head", C.c_int32),
        ("n_kv_head", C.c_int32), ("embed_dim", C.c_int32), ("rotary_dims", C.c_int32), ("window_pattern", C.c_char * 16),
        ("n_experts", C.c_int32), ("experts_per_token", C.c_int32), ("expert_hidden", C.c_int32), ("shared_hidden", C.c_int32),
        ("moe_clamp", C.c_float), ("moe_scale", C.c_float), ("mla_latent", C.c_int32), ("mla_rotary_dims", C.c_int32),
    ]


class GnOptimizerConfig(C.Structure):
    _fields_ = [("unembedding_lr", C.c_float), ("embedding_lr", C.c_float), ("matrix_lr", C.c_float), ("weight_decay", C.c_float),
                ("scalar_lr", C.c_float), ("lr_mult", C.c_float)]


class GnGenerateOptions(C.Structure):
    _fields_ = [("thinking", C.c_int32), ("thinking_budget", C.c_int32), ("forced", C.c_void_p), ("forced_stride", C.c_int32),
                ("forced_counts", C.c_void_p)]


class GnAttentionParams(C.Structure):
    _fields_ = [
        ("query", vp), ("key", vp), ("value", vp),
        ("query_len", C.c_int32), ("key_len", C.c_int32), ("head_dim", C.c_int32), ("position_offset", C.c_int32),
        ("window", C.c_int32), ("segment_ids", vp),
    ]


# name -> (restype, argtypes); every symbol include/gonano_cuda.h declares.
I, L, F, U32 = C.c_int, C.c_int64, C.c_float, C.c_uint32
SIGNATURES = {
    "gn_last_error": (C.c_char_p, []),
    "gn_version": (C.c_char_p, []),
    "gn_device_count": (I, []),
    "gn_add": (I, [vp, vp, vp, L]), "gn_subtract": (I, [vp, vp, vp, L]), "gn_multiply": (I, [vp, vp, vp, L]),
    "gn_divide": (I, [vp, vp, vp, L]), "gn_scale": (I, [vp, vp, F, L]), "gn_add_scaled": (I, [vp, vp, vp, F, L]),
    "gn_negate": (I, [vp, vp, L]), "gn_abs": (I, [vp, vp, L]), "gn_square": (I, [vp, vp, L]), "gn_relu_squared": (I, [vp, vp, L]),
    "gn_swiglu": (I, [vp, vp, vp, F, L]), "gn_swiglu_backward": (I, [vp, vp, vp, vp, vp, F, L]),
    "gn_exp": (I, [vp, vp, L]), "gn_sigmoid": (I, [vp, vp, L]), "gn_tanh": (I, [vp, vp, L]), "gn_rsqrt": (I, [vp, vp, L]),
    "gn_sum": (I, [vp, L, f32p]), "gn_max": (I, [vp, L, f32p]), "gn_argmax": (I, [vp, L, C.POINTER(C.c_int64)]),
    "gn_matmul": (I, [vp, vp, vp, I, I, I]), "gn_matmul_transposed": (I, [vp, vp, vp, I, I, I]),
    "gn_dot_product": (I, [vp, vp, L, f32p]),
    "gn_indexer_scores": (I, [vp, vp, vp, vp, I, I, I, I]), "gn_indexer_block_max": (I, [vp, vp, I, I, I]),
    "gn_compressor_forward": (I, [vp, vp, vp, vp, I, I, I, I, I, vp, vp]),
    "gn_compressor_backward": (I, [vp, vp, vp, vp, vp, vp, I, I, I, I, I, vp, vp, vp, vp]),
    "gn_compressed_attention_forward": (I, [vp, vp, vp, I, I, I, I, I, I, I, vp, vp]),
    "gn_compressed_attention_forward_at": (I, [vp, vp, vp, I, I, I, I, I, I, I, I, vp, vp]),
    "gn_compressed_attention_backward": (I, [vp, vp, vp, vp, vp, vp, I, I, I, I, I, I, I, vp, vp, vp]),
    "gn_indexer_scores_backward": (I, [vp, vp, vp, vp, I, I, I, I, vp, vp, vp]),
    "gn_indexer_distillation_target": (I, [vp, vp, I, I, I, I, I, I, I, vp]),
    "gn_indexer_distillation_grad": (I, [vp, vp, vp, vp, I, C.c_int64, I, I, I, C.c_float, vp]),
    "gn_attention_windowed_forward": (I, [vp, vp, vp, I, I, I, I, I, I, I, vp, vp]),
    "gn_attention_windowed_backward": (I, [vp, vp, vp, vp, vp, vp, vp, I, I, I, I, I, I, I, vp, vp, vp]),
    "gn_compress_forward": (I, [vp, vp, vp, vp, vp, I, I, I, I, I, I, vp, vp, vp]),
    "gn_compress_backward": (I, [vp, vp, vp, vp, vp, vp, vp, vp, vp, I, I, I, I, I, I, vp, vp, vp, vp, vp]),
    "gn_hierarchical_cap": (I, [I, I]),
    "gn_select_blocks_hierarchical": (I, [vp, I, I, I, I, I, I, I, vp, vp, vp, vp]),
    "gn_select_blocks_within_pool": (I, [vp, I, I, I, I, I, vp, vp, I, vp, vp]),
    "gn_compressed_attention_sparse_backward": (I, [vp, vp, vp, vp, vp, vp, vp, vp, I, I, I, I, I, I, I, vp, vp, vp]),
    "gn_compressed_attention_sparse_forward": (I, [vp, vp, vp, vp, vp, I, I, I, I, I, I, I, vp, vp]),
    "gn_attention_merge": (I, [vp, vp, vp, vp, C.c_int64, I, vp, vp]), "gn_select_blocks": (I, [vp, I, I, I, I, I, vp, vp]),
    "gn_topk_indices": (I, [vp, vp, I, I, I]), "gn_moe_gate_topk": (I, [vp, vp, vp, vp, vp, I, I, I]),
    "gn_grouped_matmul_transposed": (I, [vp, vp, vp, vp, I, I, I]),
    "gn_softmax_last_dim": (I, [vp, vp, L, I]), "gn_rmsnorm_last_dim": (I, [vp, vp, L, I, F]),
    "gn_attention_forward": (I, [C.POINTER(GnAttentionParams), vp, vp]),
    "gn_attention_forward_split": (I, [C.POINTER(GnAttentionParams), I, I, vp, vp, vp]),
    "gn_attention_combine": (I, [vp, vp, vp, I, I, I, vp, vp]),
    "gn_attention_backward": (I, [C.POINTER(GnAttentionParams), vp, vp, vp, vp, vp, vp, vp]),
    "gn_sample_next_token": (I, [vp, I, I, vp, vp, I, U32, F, I, vp]),
    "gn_group_advantage": (I, [vp, I, I, I, vp]),
    "gn_adamw_step": (I, [vp, vp, vp, vp, L, I, F, F, F, F, F]),
    "gn_muon_step": (I, [vp, vp, vp, vp, I, I, F, F, I, F, F]),
    "gn_sinkhorn_step": (I, [vp, vp, vp, I, I, F, F, F, I, F, F]),
    "gn_model_optimizer_init": (I, [vp, C.POINTER(GnOptimizerConfig)]), "gn_model_optimizer_step": (I, [vp]),
    "gn_model_optimizer_step_shard": (I, [vp, I, I]), "gn_model_optimizer_finish": (I, [vp]),
    "gn_pg_loss_backward": (I, [vp, vp, vp, L, I, I, F, F, vp, vp, C.POINTER(C.c_double)]),
    "gn_distillation_loss_backward": (I, [vp, vp, vp, L, I, F, F, vp, vp, C.POINTER(C.c_double), C.POINTER(C.c_int64)]),
    "gn_pg_loss_backward_static": (I, [vp, vp, vp, L, I, I, F, F, vp, vp, vp, vp]),
    "gn_static_loss_max_rows": (I, []),
    "gn_ctx_create": (I, [I, vp, C.POINTER(vp)]), "gn_ctx_destroy": (I, [vp]), "gn_ctx_sync": (I, [vp]),
    "gn_ctx_launch_count": (I, [vp, C.POINTER(C.c_int64)]), "gn_ctx_set_gemm": (I, [vp, I]),
    "gn_ctx_set_option": (I, [vp, C.c_char_p, I]),
    "gn_model_create": (I, [vp, C.POINTER(GnConfig), C.POINTER(vp)]), "gn_model_destroy": (I, [vp]),
    "gn_model_param_count": (I, [vp, C.POINTER(I)]),
    "gn_model_param_info": (I, [vp, I, C.POINTER(C.c_char_p), C.POINTER(I), C.POINTER(I)]),
    "gn_model_upload": (I, [vp, C.c_char_p, vp, L]), "gn_model_download": (I, [vp, C.c_char_p, vp, L]),
    "gn_model_download_grad": (I, [vp, C.c_char_p, vp, L]), "gn_model_upload_grad": (I, [vp, C.c_char_p, vp, L]), "gn_model_zero_grad": (I, [vp]),
    "gn_model_grad_buffer": (I, [vp, C.POINTER(vp), C.POINTER(C.c_int64)]),
    "gn_model_param_buffer": (I, [vp, C.POINTER(vp), C.POINTER(C.c_int64)]),
    "gn_model_checksum": (I, [vp, C.POINTER(C.c_double), C.POINTER(C.c_double)]),
    "gn_model_forward": (I, [vp, vp, I, I, vp]),
    "gn_generate_batch": (I, [vp, vp, I, I, I, I, F, I, vp, vp, vp, vp, C.POINTER(I)]),
    "gn_generate_batch_ex": (I, [vp, vp, I, I, I, I, F, I, vp, C.POINTER(GnGenerateOptions), vp, vp, vp, vp, C.POINTER(I)]),
    "gn_rollout_begin": (I, [vp, vp, I, I, I, I, vp, C.POINTER(GnGenerateOptions)]),
    "gn_rollout_logits": (I, [vp, C.POINTER(vp), C.POINTER(I), C.POINTER(I)]),
    "gn_rollout_sample": (I, [vp, vp, F, I, vp, vp, C.POINTER(I)]),
    "gn_rollout_force": (I, [vp, I, vp, I]), "gn_rollout_forward": (I, [vp, vp]), "gn_rollout_end": (I, [vp, vp, vp, vp]),
    "gn_policy_gradient_step": (I, [vp, vp, vp, vp, I, I, F, I, f32p, vp, vp, vp]),
    "gn_model_kv_info": (I, [vp, C.POINTER(I), C.POINTER(I), C.POINTER(I)]), "gn_model_kv_alloc": (I, [vp, I, I, I]),
    "gn_model_kv_read": (I, [vp, I, I, I, I, I, vp, L]), "gn_model_kv_write": (I, [vp, I, I, I, I, I, vp, L]),
    "gn_model_phase_ms": (I, [vp, C.c_char_p, f32p]),
    "gn_comm_unique_id": (I, [vp]), "gn_ctx_comm_init": (I, [vp, vp, I, I]), "gn_ctx_comm_destroy": (I, [vp]),
    "gn_model_grad_allreduce": (I, [vp]), "gn_ctx_allreduce_max_i64": (I, [vp, C.POINTER(C.c_int64)]),
    "gn_model_optimizer_exchange": (I, [vp]),
    "gn_profile_kernel": (I, [vp, C.c_char_p, C.POINTER(C.c_int64), I, I, f32p]),
}

_lib = None


def load() -> C.CDLL:
    """Returns the loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise GonanoError(f"{LIB_PATH} is missing: build it with `python -m gonano_b200.build` (there is no CPU fallback)")
        lib = C.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(status: int) -> None:
    if status != 0:
        raise GonanoError(f"gonano_cuda status {status}: {load().gn_last_error().decode(errors='replace')}")


def ptr(array):
    """Address of a numpy array or a raw device address (int)."""
    if array is None:
        return None
    if isinstance(array, int):
        return C.c_void_p(array)
    return C.c_void_p(array.ctypes.data)
