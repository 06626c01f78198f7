"""ctypes view of libschedforge_b200.so: the structs and prototypes of
include/schedforge_b200.h.  Loading never needs a GPU; the first compute call does."""
from __future__ import annotations

import ctypes as C
import os

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "libschedforge_b200.so")

SFB_OK, SFB_INVALID_ARGUMENT, SFB_RUNTIME_ERROR, SFB_CUDA_ERROR, SFB_UNSUPPORTED, SFB_DEVICE_TIMEOUT = 0, -1, -2, -3, -4, -5
F32, BF16 = 0, 1
EPI_STORE, EPI_RESIDUAL, EPI_SWIGLU, EPI_ROPE_SPLIT = 0, 1, 2, 3
GEMM_AUTO, GEMM_SIMT, GEMM_TCGEN05 = 0, 1, 2

vp = C.c_void_p
f32p = C.POINTER(C.c_float)
i32p = C.POINTER(C.c_int)


class GemmArgs(C.Structure):
    _fields_ = [("a", vp), ("bt", vp), ("out", vp),
                ("m", C.c_int), ("n", C.c_int), ("k", C.c_int),
                ("epilogue", C.c_int), ("backend", C.c_int), ("out_f32", C.c_int),
                ("residual", vp), ("swiglu_block", C.c_int),
                ("q", vp), ("key", vp), ("value", vp), ("rope_cos", vp), ("rope_sin", vp),
                ("batch", C.c_int), ("seq", C.c_int), ("q_heads", C.c_int), ("kv_heads", C.c_int),
                ("head_dim", C.c_int),
                ("group_offsets", vp), ("groups", C.c_int), ("tile_table", vp),
                ("split_workspace", vp), ("split_workspace_bytes", C.c_size_t), ("bt_tiled", C.c_int),
                ("peer_out", vp * 7), ("peer_count", C.c_int), ("scatter_out", vp * 8), ("scatter_rows", C.c_int),
                ("rope_row_offset", C.c_int), ("bt_scales", vp),
                ("row_ss", vp), ("row_ss_fixed", C.c_int), ("rms_epsilon", C.c_float),
                ("ss_out", vp), ("clear", vp), ("clear_bytes", C.c_size_t),
                ("owner_flags", vp), ("owner_epoch", C.c_uint32), ("owner_rows", C.c_int), ("owner_self", C.c_int),
                ("kv_k_pool", vp), ("kv_v_pool", vp), ("kv_table", vp),
                ("kv_position", C.c_int), ("kv_block_tokens", C.c_int), ("kv_max_blocks", C.c_int),
                ("kv_num_blocks", C.c_int)]


class AttentionArgs(C.Structure):
    _fields_ = [("q", vp), ("key", vp), ("value", vp), ("out", vp)] + \
               [(n, C.c_int) for n in ("batch", "q_heads", "kv_heads", "seq_q", "seq_kv", "head_dim",
                                       "head_dim_value", "causal")] + \
               [("scale", C.c_float), ("token_major", C.c_int), ("dtype", C.c_int), ("backend", C.c_int),
                ("q_head_rows", C.c_int), ("kv_head_rows", C.c_int)]


class DecodeArgs(C.Structure):
    _fields_ = [("q", vp), ("k_pool", vp), ("v_pool", vp), ("block_table", vp), ("context_len", vp),
                ("out", vp), ("partials", vp)] + \
               [(n, C.c_int) for n in ("batch", "q_heads", "kv_heads", "head_dim", "head_dim_value",
                                       "block_tokens", "max_blocks", "num_blocks", "max_context", "splits")] + \
               [("scale", C.c_float), ("dtype", C.c_int), ("uniform_context", C.c_int)]


class DecoderConfig(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("batch", "sequence", "hidden", "intermediate", "query_heads",
                                       "kv_heads", "head_dim")] + \
               [("rms_epsilon", C.c_float), ("rope_theta", C.c_float)] + \
               [(n, C.c_int) for n in ("causal", "ffn_moe", "experts", "top_k", "context_sequence")]


DATA_FIELDS = ("rms1_weight", "query_weight", "key_weight", "value_weight", "output_weight",
               "rms2_weight", "gate_weight", "up_weight", "down_weight", "router_weight",
               "router_bias", "w1", "w3", "w2", "cached_key", "cached_value")


class DecoderData(C.Structure):
    _fields_ = [(n, f32p) for n in DATA_FIELDS]


DATA_BUFFER_FIELDS = ("rms1_weight", "query_weight", "key_weight", "value_weight", "output_weight", "rms2_weight",
                      "gate_weight", "up_weight", "down_weight", "router_weight", "w1", "w3", "w2", "cached_key",
                      "cached_value")


class DecoderDataBuffers(C.Structure):
    _fields_ = [(n, C.POINTER(C.c_float)) for n in DATA_BUFFER_FIELDS]


class CompileOptions(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("dtype", "token_major_attention", "fuse_epilogues",
                                       "gemm_backend", "attention_backend", "page_tokens", "tp_rank",
                                       "tp_size", "seed_block_table", "no_workspace_reuse", "no_pipeline",
                                       "append_new_token", "weight_int8", "kv_capacity", "norm_fusion",
                                       "local_expert_weights", "fixed_order")]


class PlanCost(C.Structure):
    _fields_ = [("measured_milliseconds", C.c_double), ("analytical_score", C.c_double),
                ("workspace_bytes", C.c_size_t), ("materialization_bytes", C.c_size_t), ("measured", C.c_int)]


class PlanCandidate(C.Structure):
    _fields_ = [("options", CompileOptions), ("cost", PlanCost)]


class OptimizationResult(C.Structure):
    _fields_ = [("baseline", PlanCost), ("winner", PlanCost), ("winner_options", CompileOptions),
                ("candidates", C.c_int), ("hardware_measurements", C.c_int), ("speedup", C.c_double)]


class DecoderResult(C.Structure):
    _fields_ = [(n, C.c_double) for n in ("milliseconds", "attention_milliseconds",
                                          "projection_milliseconds", "norm_rope_milliseconds",
                                          "ffn_milliseconds", "residual_milliseconds",
                                          "h2d_milliseconds", "d2h_milliseconds", "tokens_per_second")] + \
               [("kernel_launches", C.c_uint64)]


class DecoderProfile(C.Structure):
    _fields_ = [("name", C.c_char * 64), ("config", DecoderConfig), ("routing", C.c_int),
                ("estimated_flops", C.c_uint64), ("estimated_weight_bytes", C.c_uint64),
                ("estimated_activation_bytes", C.c_uint64)]


MAX_PLAN_CANDIDATES = 17
EVIDENCE_SKIPPED, EVIDENCE_COMPILE_ONLY, EVIDENCE_MEASURED = 0, 1, 2


class DecoderBenchmarkRecord(C.Structure):
    _fields_ = [("profile", DecoderProfile), ("evidence", C.c_int), ("measured", DecoderResult),
                ("max_error", C.c_double), ("plan_cost", PlanCost), ("compile_milliseconds", C.c_double),
                ("llvm_compile_milliseconds", C.c_double), ("memory_planning_milliseconds", C.c_double),
                ("optimizer_speedup", C.c_double), ("optimizer_baseline_milliseconds", C.c_double),
                ("hardware_measurements", C.c_int), ("candidate_count", C.c_int),
                ("candidates", PlanCandidate * MAX_PLAN_CANDIDATES), ("selected_policy", C.c_char * 192),
                ("note", C.c_char * 96)]


class GraphSummary(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("operations", "values", "inputs", "matmuls", "fused_qkv",
                                       "fused_gate_up", "fused_rope")]


class AttentionConfig(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("batch", "query_heads", "kv_heads", "sequence_query",
                                       "sequence_kv", "head_dim", "head_dim_value", "causal")] + \
               [("scale", C.c_float)]


class MoeConfig(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("tokens", "hidden", "intermediate", "experts", "top_k")]


ALLREDUCE_FN = C.CFUNCTYPE(None, vp, vp, C.c_int64, C.c_int, vp)

# Every symbol include/schedforge_b200.h declares (checked by tests/test_abi.py).
EXPORTS = (
    "sfb_last_error sfb_version sfb_launch_count sfb_device_status "
    "sfb_k_rms_norm sfb_k_add sfb_k_swiglu sfb_k_convert sfb_k_gemm_f32 sfb_k_gemm_bf16 sfb_tiled_weight_elems sfb_k_tile_weight_bf16 sfb_k_quantize_weight_int8 sfb_k_dequantize_weight_int8 sfb_gemm_stream_workspace_bytes sfb_k_convert_rows_sumsq sfb_k_row_sumsq "
    "sfb_rope_table sfb_k_rope_split sfb_k_attention_prefill "
    "sfb_attention_decode_workspace sfb_attention_decode_default_splits sfb_k_attention_decode_paged "
    "sfb_k_paged_kv_append sfb_k_paged_kv_gather "
    "sfb_k_moe_route sfb_k_moe_dispatch sfb_moe_dispatch_scratch_bytes sfb_k_moe_dispatch_static sfb_k_moe_combine "
    "sfb_import_stablehlo sfb_import_stablehlo_dump "
    "sfb_decoder_compile sfb_decoder_destroy sfb_decoder_execute sfb_decoder_execute_rows sfb_decoder_upload_input "
    "sfb_decoder_step sfb_decoder_kv_info sfb_decoder_kv_truncate sfb_decoder_kv_release "
    "sfb_decoder_optimize sfb_decoder_row_chunks sfb_decoder_execute_resident sfb_decoder_download_output sfb_decoder_set_allreduce sfb_decoder_peer_bytes sfb_decoder_set_peer_allreduce sfb_k_peer_allreduce_finish sfb_k_peer_reduce_gather sfb_k_peer_wait sfb_k_flag_wait sfb_k_moe_ep_plan sfb_moe_ep_tables sfb_k_moe_ep_send sfb_k_moe_ep_return sfb_decoder_set_peer_collective sfb_peer_alloc sfb_peer_open sfb_peer_close sfb_peer_free "
    "sfb_decoder_dump sfb_decoder_workspace_bytes sfb_decoder_read_tensor sfb_decoder_stream "
    "sfb_attention_execute sfb_attention_decode "
    "sfb_paged_create sfb_paged_destroy sfb_paged_set_free_pages sfb_paged_append sfb_paged_truncate "
    "sfb_paged_release sfb_paged_info sfb_paged_gather sfb_paged_decode "
    "sfb_moe_route_topk sfb_moe_dispatch_tokens sfb_moe_execute sfb_moe_execute_quantized sfb_moe_plan_tasks "
    "sfb_moe_compile sfb_moe_destroy sfb_moe_plan_execute "
    "sfb_make_routing_trace sfb_make_decoder_input sfb_make_decoder_data sfb_decoder_profile_count sfb_decoder_profile_get "
    "sfb_benchmark_decoder_profile sfb_write_decoder_benchmark_csv sfb_write_decoder_plan_candidates_csv "
    "sfb_decoder_compile_milliseconds "
    "sfb_shard_columns sfb_shard_rows"
).split()


class SfbError(RuntimeError):
    """Raised for a non-zero sfb_status; `.status` holds the code."""

    def __init__(self, status, message):
        super().__init__(f"sfb status {status}: {message}")
        self.status = status
        self.message = message


class InvalidArgument(SfbError, ValueError):
    """SFB_INVALID_ARGUMENT — where the reference throws std::invalid_argument."""


_lib = None


def load():
    """Loads the library (building it first when the .so is missing and nvcc exists)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        from . import build
        build.build()
    lib = C.CDLL(LIB_PATH)
    lib.sfb_last_error.restype = C.c_char_p
    lib.sfb_version.restype = C.c_char_p
    lib.sfb_launch_count.restype = C.c_uint64
    lib.sfb_tiled_weight_elems.restype = C.c_int64
    lib.sfb_decoder_compile_milliseconds.restype = C.c_double
    lib.sfb_benchmark_decoder_profile.argtypes = [vp, C.c_char_p, vp, C.c_uint64, C.c_uint64, C.c_int, C.c_int, vp]
    for name in ("sfb_attention_decode_workspace", "sfb_moe_dispatch_scratch_bytes",
                 "sfb_decoder_workspace_bytes", "sfb_gemm_stream_workspace_bytes", "sfb_decoder_peer_bytes"):
        if hasattr(lib, name):
            getattr(lib, name).restype = C.c_size_t
    if hasattr(lib, "sfb_decoder_stream"):
        lib.sfb_decoder_stream.restype = vp
    _lib = lib
    return lib


def check(status):
    if status == SFB_OK:
        return
    message = load().sfb_last_error().decode(errors="replace")
    if status == SFB_INVALID_ARGUMENT:
        raise InvalidArgument(status, message)
    raise SfbError(status, message)
