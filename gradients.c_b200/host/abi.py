"""ctypes binding of libgd_backend_b200.so: the struct layouts of include/gd_backend_b200.h
(binary-compatible with the reference's src/core/backend.h:21-140,301-325,528-537,579-689)
and typed prototypes for every exported entry point.

Loading fails loudly when the shared library has not been built: there is no Python or CPU
fallback for any entry.
"""
from __future__ import annotations

import ctypes as C
import os

GD_OK = 0
GD_ERR_INVALID_ARGUMENT = -1
GD_ERR_OUT_OF_MEMORY = -2
GD_ERR_BAD_STATE = -5
GD_ERR_UNSUPPORTED = -6
GD_ERR_INTERNAL = -7

STATUS_NAMES = {
    0: "GD_OK", -1: "GD_ERR_INVALID_ARGUMENT", -2: "GD_ERR_OUT_OF_MEMORY", -3: "GD_ERR_FROZEN",
    -4: "GD_ERR_BUSY", -5: "GD_ERR_BAD_STATE", -6: "GD_ERR_UNSUPPORTED", -7: "GD_ERR_INTERNAL",
    -8: "GD_ERR_NOT_IMPLEMENTED", -9: "GD_ERR_IO",
}

# gd_dtype codes (reference include/gradients/tensor.h:49-57)
F16, BF16, F32, I32, U8, U16 = 1, 2, 3, 4, 5, 6
DTYPE_SIZE = {F16: 2, BF16: 2, F32: 4, I32: 4, U8: 1, U16: 2}

P = C.c_void_p
SZ = C.c_size_t
U32 = C.c_uint32
U64 = C.c_uint64
I32_T = C.c_int32
F = C.c_float


class MatrixView(C.Structure):
    _fields_ = [("buffer", P), ("offset", SZ), ("rows", U32), ("cols", U32), ("row_bytes", SZ), ("dtype", U32)]


class BatchedMatrixView(C.Structure):
    _fields_ = [("buffer", P), ("offset", SZ), ("rows", U32), ("cols", U32), ("row_bytes", SZ), ("dtype", U32),
                ("batch_rank", U32), ("batch_count", U32), ("batch_shape", U32 * 6), ("batch_strides", SZ * 6)]


class VectorView(C.Structure):
    _fields_ = [("buffer", P), ("offset", SZ), ("length", U32), ("dtype", U32)]


class TensorView(C.Structure):
    _fields_ = [("buffer", P), ("offset", SZ), ("count", SZ), ("dtype", U32), ("rank", U32),
                ("shape", C.c_int64 * 8), ("strides", C.c_int64 * 8)]


class Fence(C.Structure):
    _fields_ = [("handle", P)]


class AdamwDesc(C.Structure):
    _fields_ = [
        ("param_buffer", P), ("param_offset", SZ), ("master_buffer", P), ("master_offset", SZ),
        ("grad_buffer", P), ("grad_offset", SZ), ("grad_scale_buffer", P), ("grad_scale_offset", SZ),
        ("found_inf_buffer", P), ("found_inf_offset", SZ), ("m_buffer", P), ("m_offset", SZ),
        ("v_buffer", P), ("v_offset", SZ), ("state_f32_buffer", P),
        ("beta1_power_offset", SZ), ("beta2_power_offset", SZ), ("step_scale_offset", SZ),
        ("decay_scale_offset", SZ), ("eps_scaled_offset", SZ), ("state_i32_buffer", P),
        ("param_step_offset", SZ), ("optimizer_step_offset", SZ), ("count", SZ),
        ("param_dtype", U32), ("grad_dtype", U32), ("has_master", U32), ("has_grad_scale", U32),
        ("has_found_inf", U32), ("has_device_state", U32), ("bias_correction", U32),
        ("update_optimizer_step", U32), ("lr", F), ("beta1", F), ("beta2", F), ("eps", F),
        ("weight_decay", F), ("bias_correction1", F), ("bias_correction2", F),
    ]


class AmpStateDesc(C.Structure):
    _fields_ = [("scale_buffer", P), ("scale_offset", SZ), ("flags_buffer", P), ("flags_offset", SZ),
                ("growth_factor", F), ("backoff_factor", F), ("min_scale", F), ("max_scale", F),
                ("growth_interval", U32)]


class AmpUnscaleDesc(C.Structure):
    _fields_ = [("grad_buffer", P), ("grad_offset", SZ), ("count", SZ), ("grad_dtype", U32),
                ("inv_scale_buffer", P), ("inv_scale_offset", SZ), ("found_inf_buffer", P), ("found_inf_offset", SZ)]


class GradNormDesc(C.Structure):
    _fields_ = [("grad_buffer", P), ("grad_offset", SZ), ("count", SZ), ("grad_dtype", U32),
                ("partial_buffer", P), ("partial_offset", SZ), ("partial_count", SZ),
                ("grad_scale_buffer", P), ("grad_scale_offset", SZ),
                ("found_inf_buffer", P), ("found_inf_offset", SZ), ("has_found_inf", U32)]


class EmbeddingArgs(C.Structure):
    _fields_ = [("ids_count", U64), ("vocab", U64), ("dim", U64)]


class RopeArgs(C.Structure):
    _fields_ = [("theta", F), ("n_dims", U32), ("interleaved", U32)]


class RmsNormArgs(C.Structure):
    _fields_ = [("rows", U64), ("cols", U64), ("row_blocks", U64), ("eps", F), ("simdgroups", U32),
                ("wgrad_simdgroups", U32), ("wgrad_row_block", U32), ("reserved0", U32)]


class ConcatArgs(C.Structure):
    _fields_ = [("count", U64), ("inner", U64), ("slice_axis", U64), ("full_axis", U64), ("axis_offset", U64)]


class SdpaVarlenArgs(C.Structure):
    _fields_ = [("scale", F), ("causal", U32), ("sliding_window", U32), ("prefix_len", U32),
                ("max_seqlen", U32), ("use_forward_stats", U32)]


class SdpaDecodeArgs(C.Structure):
    _fields_ = [("scale", F), ("sliding_window", U32), ("prefix_len", U32), ("cache_pos", I32_T)]


class KvCacheAppendArgs(C.Structure):
    _fields_ = [("cache_pos", I32_T)]


GPT_MAX_LAYERS = 64
GPT_MAX_PARAMS = 1 + 10 * GPT_MAX_LAYERS + 3


class GptSpec(C.Structure):
    _fields_ = [("params_buffer", P), ("state_buffer", P), ("scratch_buffer", P), ("scratch_bytes", SZ),
                ("vocab_size", I32_T), ("context_length", I32_T), ("d_model", I32_T), ("n_layers", I32_T), ("n_heads", I32_T),
                ("head_dim", I32_T), ("mlp_hidden", I32_T), ("tied_lm_head", I32_T), ("sdpa_window", I32_T), ("pad_token_id", I32_T),
                ("lm_ce_chunk", I32_T), ("n_params", I32_T), ("dp_world", I32_T), ("dtype", U32),
                ("dropout_p", F), ("logits_softcap", F), ("rms_eps", F), ("rope_theta", F), ("dropout_seed", U64),
                ("adam_beta1", F), ("adam_beta2", F), ("adam_eps", F), ("grad_clip_norm", F),
                ("amp_growth_factor", F), ("amp_backoff_factor", F), ("amp_min_scale", F), ("amp_max_scale", F),
                ("amp_growth_interval", U32),
                ("state_f32_offset", SZ), ("state_i32_offset", SZ), ("partials_offset", SZ), ("clip_scale_offset", SZ),
                ("amp_scale_offset", SZ), ("amp_flags_offset", SZ),
                ("param_offset", SZ * GPT_MAX_PARAMS), ("param_count", SZ * GPT_MAX_PARAMS), ("master_offset", SZ * GPT_MAX_PARAMS),
                ("m_offset", SZ * GPT_MAX_PARAMS), ("v_offset", SZ * GPT_MAX_PARAMS), ("weight_decay", F * GPT_MAX_PARAMS),
                ("global_valid_rows", F)]


class PermuteArgs(C.Structure):
    _fields_ = [("count", U64), ("inner", U64), ("rank", U32), ("active_rank", U32), ("axes", U32 * 8), ("reserved0", U32)]


class GptBatch(C.Structure):
    _fields_ = [("buffer", P), ("input_ids_offset", SZ), ("targets_offset", SZ), ("positions_offset", SZ),
                ("cu_seqlens_offset", SZ), ("n_tokens", C.c_int64), ("n_cu", C.c_int64)]


class GptCompactBatch(C.Structure):
    _fields_ = [("buffer", P), ("tokens_offset", SZ), ("segment_lengths_offset", SZ), ("record_offsets_offset", SZ),
                ("input_ids_offset", SZ), ("targets_offset", SZ), ("positions_offset", SZ), ("cu_seqlens_offset", SZ),
                ("status_offset", SZ), ("n_records", C.c_int64), ("n_segments", C.c_int64), ("context_length", I32_T),
                ("vocab_size", I32_T), ("pad_id", I32_T), ("im_start_id", I32_T), ("im_end_id", I32_T)]


COMPACT_BAD_TOKEN, COMPACT_BAD_LENGTH, COMPACT_BAD_COVER = 1, 2, 4


class GptDecodeState(C.Structure):
    _fields_ = [("cache_buffer", P), ("io_buffer", P), ("k_cache_offset", SZ * GPT_MAX_LAYERS), ("v_cache_offset", SZ * GPT_MAX_LAYERS),
                ("tokens_offset", SZ), ("positions_offset", SZ), ("out_tokens_offset", SZ), ("step_counter_offset", SZ),
                ("batch", I32_T), ("capacity", I32_T), ("max_steps", I32_T)]


TV = C.POINTER(TensorView)
MV = C.POINTER(MatrixView)
BV = C.POINTER(BatchedMatrixView)
VV = C.POINTER(VectorView)

# name -> (restype, argtypes). Every symbol declared in include/gd_backend_b200.h is listed.
_ST = C.c_int
PROTOTYPES = {
    "gd_backend_create_default": (_ST, [C.POINTER(P)]),
    "gd_backend_destroy": (None, [P]),
    "gd_backend_kind_query": (C.c_int, [P]),
    "gd_backend_name": (C.c_char_p, [P]),
    "gd_backend_buffer_create": (_ST, [P, SZ, C.POINTER(P)]),
    "gd_backend_buffer_destroy": (None, [P]),
    "gd_backend_buffer_nbytes": (SZ, [P]),
    "gd_backend_buffer_host_ptr": (P, [P]),
    "gd_backend_buffer_is_host_visible": (C.c_bool, [P]),
    "gd_backend_scope_begin": (_ST, [P]),
    "gd_backend_flush": (_ST, [P]),
    "gd_backend_record_fence": (_ST, [P, C.POINTER(Fence)]),
    "gd_backend_fence_destroy": (None, [C.POINTER(Fence)]),
    "gd_backend_fence_is_complete": (C.c_bool, [C.POINTER(Fence)]),
    "gd_backend_fence_wait": (_ST, [C.POINTER(Fence)]),
    "gd_backend_upload": (_ST, [P, P, SZ, P, SZ]),
    "gd_backend_download": (_ST, [P, P, SZ, P, SZ]),
    "gd_backend_fill": (_ST, [P, P, SZ, SZ, SZ, U32]),
    "gd_backend_rand_uniform": (_ST, [P, P, SZ, SZ, U32, U64, F, F]),
    "gd_backend_matmul": (_ST, [P, MV, MV, MV]),
    "gd_backend_matmul_nt": (_ST, [P, MV, MV, MV]),
    "gd_backend_matmul_tn": (_ST, [P, MV, MV, MV]),
    "gd_backend_batched_matmul": (_ST, [P, BV, BV, BV]),
    "gd_backend_batched_matmul_nt": (_ST, [P, BV, BV, BV]),
    "gd_backend_batched_matmul_tn": (_ST, [P, BV, BV, BV]),
    "gd_backend_linear": (_ST, [P, MV, MV, VV, MV]),
    "gd_backend_reduce_rows": (_ST, [P, MV, VV]),
    "gd_backend_accumulate": (_ST, [P, P, SZ, P, SZ, SZ, U32]),
    "gd_backend_scale": (_ST, [P, P, SZ, P, SZ, SZ, U32, F]),
    "gd_backend_relu": (_ST, [P, TV, TV]),
    "gd_backend_relu_backward": (_ST, [P, TV, TV, TV]),
    "gd_backend_add": (_ST, [P, TV, TV, TV]),
    "gd_backend_mul": (_ST, [P, TV, TV, TV]),
    "gd_backend_sub": (_ST, [P, TV, TV, TV]),
    "gd_backend_sigmoid": (_ST, [P, TV, TV]),
    "gd_backend_sigmoid_backward": (_ST, [P, TV, TV, TV]),
    "gd_backend_tanh": (_ST, [P, TV, TV]),
    "gd_backend_tanh_backward": (_ST, [P, TV, TV, TV]),
    "gd_backend_sigmoid_backward_from_output": (_ST, [P, TV, TV, TV]),
    "gd_backend_tanh_backward_from_output": (_ST, [P, TV, TV, TV]),
    "gd_backend_mul_backward_direct": (_ST, [P, TV, TV, TV, TV, TV]),
    "gd_backend_mul_reduce_suffix": (_ST, [P, TV, TV, TV]),
    "gd_backend_mse_forward": (_ST, [P, TV, TV, TV, U64, F]),
    "gd_backend_mse_backward": (_ST, [P, TV, TV, TV, TV, TV, F]),
    "gd_backend_huber_forward": (_ST, [P, TV, TV, TV, U64, F, F]),
    "gd_backend_huber_backward": (_ST, [P, TV, TV, TV, TV, TV, F, F]),
    "gd_backend_powlu_forward": (_ST, [P, TV, TV, TV, F]),
    "gd_backend_powlu_backward": (_ST, [P, TV, TV, TV, TV, TV, F]),
    "gd_backend_powlu_split_forward": (_ST, [P, TV, TV, F]),
    "gd_backend_powlu_split_backward": (_ST, [P, TV, TV, TV, F]),
    "gd_backend_permute": (_ST, [P, TV, TV, C.POINTER(PermuteArgs)]),
    "gd_backend_dropout_forward": (_ST, [P, TV, TV, TV, F, U64]),
    "gd_backend_dropout_add_forward": (_ST, [P, TV, TV, TV, TV, F, U64]),
    "gd_backend_dropout_backward": (_ST, [P, TV, TV, F, U64]),
    "gd_backend_dropout_backward_mask": (_ST, [P, TV, TV, TV, F]),
    "gd_backend_embedding_forward": (_ST, [P, TV, TV, TV, C.POINTER(EmbeddingArgs)]),
    "gd_backend_embedding_backward": (_ST, [P, TV, TV, TV, TV, C.POINTER(EmbeddingArgs)]),
    "gd_backend_rope": (_ST, [P, TV, TV, TV, C.POINTER(RopeArgs)]),
    "gd_backend_rope_backward": (_ST, [P, TV, TV, TV, C.POINTER(RopeArgs)]),
    "gd_backend_qkv_split_rope_forward": (_ST, [P, TV, TV, TV, TV, TV, U32, U32, C.POINTER(RopeArgs)]),
    "gd_backend_qkv_split_rope_backward": (_ST, [P, TV, TV, TV, TV, TV, U32, U32, C.POINTER(RopeArgs)]),
    "gd_backend_swiglu_forward": (_ST, [P, TV, TV, TV]),
    "gd_backend_swiglu_backward": (_ST, [P, TV, TV, TV, TV, TV]),
    "gd_backend_swiglu_split_forward": (_ST, [P, TV, TV]),
    "gd_backend_swiglu_split_backward": (_ST, [P, TV, TV, TV]),
    "gd_backend_rms_norm_forward": (_ST, [P, TV, TV, TV, C.POINTER(RmsNormArgs)]),
    "gd_backend_rms_norm_forward_stats": (_ST, [P, TV, TV, TV, TV, C.POINTER(RmsNormArgs)]),
    "gd_backend_rms_norm_inv": (_ST, [P, TV, TV, C.POINTER(RmsNormArgs)]),
    "gd_backend_rms_norm_backward": (_ST, [P, TV, TV, TV, TV, C.POINTER(RmsNormArgs)]),
    "gd_backend_rms_norm_backward_stats": (_ST, [P, TV, TV, TV, TV, TV, C.POINTER(RmsNormArgs)]),
    "gd_backend_rms_norm_weight_backward_stats": (_ST, [P, TV, TV, TV, TV, TV, C.POINTER(RmsNormArgs)]),
    "gd_backend_sdpa_varlen": (_ST, [P, TV, TV, TV, TV, TV, TV, C.POINTER(SdpaVarlenArgs)]),
    "gd_backend_sdpa_varlen_backward": (_ST, [P, TV, TV, TV, TV, TV, TV, TV, TV, TV, C.POINTER(SdpaVarlenArgs)]),
    "gd_backend_sdpa_decode": (_ST, [P, TV, TV, TV, TV, TV, C.POINTER(SdpaDecodeArgs)]),
    "gd_backend_sdpa_decode_at": (_ST, [P, TV, TV, TV, TV, C.POINTER(SdpaDecodeArgs)]),
    "gd_backend_sdpa_decode_positions": (_ST, [P, TV, TV, TV, TV, TV, C.POINTER(SdpaDecodeArgs)]),
    "gd_backend_kv_cache_append_at": (_ST, [P, TV, TV, TV, TV, C.POINTER(KvCacheAppendArgs)]),
    "gd_backend_kv_cache_append_positions": (_ST, [P, TV, TV, TV, TV, TV, C.POINTER(KvCacheAppendArgs)]),
    "gd_backend_kv_cache_append_packed": (_ST, [P, TV, TV, TV, TV, TV, TV, C.POINTER(KvCacheAppendArgs)]),
    "gd_backend_cross_entropy_loss": (_ST, [P, TV, TV, TV]),
    "gd_backend_cross_entropy_loss_stats": (_ST, [P, TV, TV, TV, TV, TV]),
    "gd_backend_cross_entropy_backward": (_ST, [P, TV, TV, TV, TV, F]),
    "gd_backend_cross_entropy_backward_stats": (_ST, [P, TV, TV, TV, TV, TV, TV, F]),
    "gd_backend_lm_cross_entropy_online_update": (_ST, [P, TV, TV, TV, TV, TV, TV, U64, U64, F]),
    "gd_backend_lm_cross_entropy_finalize": (_ST, [P, TV, TV, TV, TV, TV, U64, I32_T]),
    "gd_backend_lm_cross_entropy_reduce_normalize": (_ST, [P, TV, TV, TV, TV]),
    "gd_backend_lm_cross_entropy_backward_chunk": (_ST, [P, TV, TV, TV, TV, TV, TV, TV, TV, U64, U64, F, F, I32_T]),
    "gd_backend_amp_begin_step": (_ST, [P, C.POINTER(AmpStateDesc)]),
    "gd_backend_amp_finish_step": (_ST, [P, C.POINTER(AmpStateDesc)]),
    "gd_backend_amp_fill_scale": (_ST, [P, P, SZ, SZ, U32, P, SZ]),
    "gd_backend_amp_scale": (_ST, [P, P, SZ, P, SZ, SZ, U32, P, SZ]),
    "gd_backend_amp_unscale": (_ST, [P, C.POINTER(AmpUnscaleDesc)]),
    "gd_backend_amp_unscale_batch": (_ST, [P, C.POINTER(AmpUnscaleDesc), U32]),
    "gd_backend_grad_clip_scale": (_ST, [P, C.POINTER(GradNormDesc), U32, P, SZ, F, F]),
    "gd_backend_adamw": (_ST, [P, C.POINTER(AdamwDesc)]),
    "gd_backend_adamw_batch": (_ST, [P, C.POINTER(AdamwDesc), U32]),
    "gd_backend_concat_to_full": (_ST, [P, TV, TV, C.POINTER(ConcatArgs)]),
    "gd_backend_concat_from_full": (_ST, [P, TV, TV, C.POINTER(ConcatArgs)]),
    "gd_backend_split_from_full": (_ST, [P, TV, TV, C.POINTER(ConcatArgs)]),
    "gd_backend_split_to_full": (_ST, [P, TV, TV, C.POINTER(ConcatArgs)]),
    # additive entries
    "gdb200_buffer_device_ptr": (P, [P, SZ]),
    "gdb200_stream": (P, [P]),
    "gdb200_device": (C.c_int, [P]),
    "gdb200_launch_count": (U64, [P]),
    "gdb200_last_error": (C.c_char_p, [P]),
    "gdb200_set_gemm_mode": (C.c_int, [P, C.c_int]),
    "gdb200_set_attention_mode": (C.c_int, [P, C.c_int]),
    "gdb200_event_record": (P, [P]),
    "gdb200_event_elapsed_ms": (F, [P, P]),
    "gdb200_event_destroy": (None, [P]),
    "gdb200_flush_l2": (_ST, [P]),
    "gdb200_pinned_alloc": (P, [SZ]),
    "gdb200_pinned_free": (None, [P]),
    "gdb200_upload_async": (_ST, [P, P, SZ, P, SZ]),
    "gdb200_download_async": (_ST, [P, P, SZ, P, SZ]),
    "gdb200_gemm_profile_enable": (None, [P, C.c_int]),
    "gdb200_gemm_profile_read": (_ST, [P, C.POINTER(U64), C.POINTER(C.c_double), C.POINTER(C.c_double), C.POINTER(C.c_double)]),
    "gdb200_matmul_nt_bias": (_ST, [P, MV, MV, VV, MV]),
    "gdb200_matmul_nt_bias_swiglu": (_ST, [P, MV, MV, VV, MV]),
    "gdb200_sdpa_varlen_backward_with_output": (_ST, [P] + [TV] * 11 + [C.POINTER(SdpaVarlenArgs)]),
    "gdb200_sdpa_varlen_backward_with_output_q32": (_ST, [P] + [TV] * 11 + [C.POINTER(SdpaVarlenArgs), C.POINTER(I32_T)]),
    "gdb200_qkv_split_rope_backward_q32": (_ST, [P, TV, TV, TV, TV, TV, U32, U32, C.POINTER(RopeArgs)]),
    "gdb200_embedding_backward_static": (_ST, [P, P, P, P, U64, U64, U64, U32]),
    "gdb200_embedding_backward_static_error": (C.c_char_p, []),
    "gdb200_embedding_backward_static_max_elems": (U64, []),
    "gdb200_gpt_compact_expand": (_ST, [P, C.POINTER(GptCompactBatch)]),
    "gdb200_gpt_train_step": (_ST, [P, C.POINTER(GptSpec), C.POINTER(GptBatch), U64, F, C.POINTER(SZ), C.POINTER(SZ)]),
    "gdb200_gpt_train_step_grad_offsets": (I32_T, [P, C.POINTER(SZ), I32_T]),
    "gdb200_matmul_nt_bias_swiglu_both": (_ST, [P, MV, MV, VV, MV, MV]),
    "gdb200_matmul_nt_swiglu_backward": (_ST, [P, MV, MV, MV, MV]),
    "gdb200_rms_norm_backward_with_weight": (_ST, [P, TV, TV, TV, TV, TV, I32_T, TV, TV, C.POINTER(RmsNormArgs)]),
    "gdb200_rms_norm_backward_with_weight_dropout": (_ST, [P, TV, TV, TV, TV, TV, I32_T, TV, TV, C.POINTER(RmsNormArgs), TV, TV, F, TV]),
    "gdb200_embedding_dropout_rms_norm": (_ST, [P, TV, TV, TV, TV, TV, TV, TV, F, F, U64]),
    "gdb200_lm_cross_entropy_fused_rows": (_ST, [P, TV, TV, TV, TV, TV, TV, F, F, I32_T]),
    "gdb200_matmul_tn_colsum": (_ST, [P, MV, MV, MV, VV]),
    "gdb200_argmax_rows": (_ST, [P, TV, F, TV]),
    "gdb200_gpt_decode_steps": (_ST, [P, C.POINTER(GptSpec), C.POINTER(GptDecodeState), I32_T, I32_T, C.POINTER(SZ)]),
    "gdb200_inject_device_error": (_ST, [P, I32_T]),
    "gdb200_selftest_bounded_wait": (_ST, [P, U32]),
    "gdb200_dp_wait_with": (_ST, [P, P, P, U32, C.POINTER(I32_T)]),
    "gdb200_dp_unique_id": (_ST, [P]),
    "gdb200_dp_init": (_ST, [P, P, C.c_int, C.c_int]),
    "gdb200_dp_all_reduce": (_ST, [P, P, SZ, SZ, U32]),
    "gdb200_dp_join": (_ST, [P]),
    "gdb200_dp_shutdown": (None, [P]),
}

# Exported entries that the Python host never calls (checked for presence only; the tests bind the MiniMax-M3
# entries themselves): helpers the reference's C host uses.
UNBOUND_ENTRIES = [
    "gd_backend_reduce_contiguous", "gd_backend_reduce_axis", "gd_backend_broadcast_axis",
    "gd_backend_broadcast_to", "gd_backend_broadcast_scalar", "gd_backend_reduce_broadcast",
    "gd_backend_minimax_m3_index_topk",
    "gd_backend_minimax_m3_sparse_attention", "gd_backend_minimax_m3_sparse_attention_backward",
]

LIB_NAME = "libgd_backend_b200.so"
_lib = None


def library_path() -> str:
    return os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), LIB_NAME)


def load_library() -> C.CDLL:
    """Load the backend shared library and attach prototypes. Raises if it is not built."""
    global _lib
    if _lib is not None:
        return _lib
    path = library_path()
    if not os.path.exists(path):
        raise RuntimeError(
            f"{path} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
            "(there is no CPU or PyTorch fallback for the gd_backend_* entries)")
    lib = C.CDLL(path, mode=C.RTLD_GLOBAL)
    for name, (restype, argtypes) in PROTOTYPES.items():
        fn = getattr(lib, name)  # AttributeError here means a declared symbol is not exported
        fn.restype = restype
        fn.argtypes = argtypes
    for name in UNBOUND_ENTRIES:
        getattr(lib, name)
    _lib = lib
    return lib


class BackendError(RuntimeError):
    def __init__(self, status: int, what: str, detail: str = ""):
        self.status = status
        name = STATUS_NAMES.get(status, str(status))
        super().__init__(f"{what}: {name}" + (f" ({detail})" if detail else ""))
