"""ctypes binding of libgewell_b200.so (the C ABI declared in
include/gewell_b200.h).  There is no CPU fallback: if the CUDA library has
not been built, importing this module raises."""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_char_p, c_float, c_int, c_int32, c_size_t, c_uint32, c_uint64, c_void_p
from pathlib import Path

LIBRARY_PATH = Path(__file__).resolve().parent / "_C" / "libgewell_b200.so"

GW_OK, GW_INVALID_ARGUMENT, GW_CUDA_ERROR, GW_KERNEL_ERROR, GW_UNSUPPORTED = range(5)
TRANSFORM_IDENTITY, TRANSFORM_GELU_TANH_MULTIPLY = 0, 1
QDQ_BF16, QDQ_FP8, QDQ_NVFP4 = 0, 1, 2
STORAGE_BF16, STORAGE_NVFP4_W4A4, STORAGE_FP8_W8A8, STORAGE_ABSENT = 0, 1, 2, 3
POLICY_ALWAYS, POLICY_PREFILL = 0, 1
PHASE_PREFILL, PHASE_DECODE = 0, 1


class Projection(ctypes.Structure):
    """gw_projection (mirrors sm120::Projection, projection.cuh:11-17)."""
    _fields_ = [
        ("storage", c_uint32), ("input", c_uint32), ("output", c_uint32), ("physical_output", c_uint32),
        ("bf16", c_void_p),
        ("nvfp4_data", c_void_p), ("nvfp4_scales", c_void_p),
        ("nvfp4_input_scale", c_float), ("nvfp4_weight_scale", c_float),
        ("fp8_data", c_void_p),
        ("fp8_input_scale", c_float), ("fp8_weight_scale", c_float),
        ("fp8_channel_scales", c_void_p),
    ]


class ArtifactTensorSpec(ctypes.Structure):
    """gw_artifact_tensor_spec: one tensor of a model's artifact inventory."""
    _fields_ = [("layer", c_int32), ("role", c_uint32), ("rank", c_uint32), ("rows", c_uint32), ("columns", c_uint32),
                ("projection", c_uint32)]


class ArtifactEntry(ctypes.Structure):
    """gw_artifact_entry: where a tensor lies in the mapped file."""
    _fields_ = [("offset", c_uint64), ("bytes", c_uint64), ("storage", c_uint32), ("sha256", ctypes.c_uint8 * 32),
                ("data", c_void_p)]


class FfnBlockWeights(ctypes.Structure):
    """gw_ffn_block_weights: one 26B layer's feed-forward weights (device pointers)."""
    _fields_ = [
        ("pre_feedforward_norm", c_void_p), ("router_scale", c_void_p), ("pre_feedforward_norm_2", c_void_p),
        ("post_feedforward_norm_1", c_void_p), ("post_feedforward_norm_2", c_void_p),
        ("post_feedforward_norm", c_void_p), ("layer_scalar", c_void_p),
        ("gate", Projection), ("up", Projection), ("down", Projection),
        ("router_proj", c_void_p), ("router_per_expert_scale", c_void_p), ("experts", c_void_p),
        ("has_bf16", c_int), ("has_fp8", c_int), ("has_nvfp4", c_int),
    ]


class ExpertWeights(ctypes.Structure):
    """gw_expert_weights (mirrors sm120::ExpertWeights, moe.cuh:11-13)."""
    _fields_ = [("gate", Projection), ("up", Projection), ("down", Projection)]


_SIGNATURES = {
    "gw_last_error": (c_char_p, []),
    "gw_abi_version": (c_int, []),
    "gw_nvfp4_scale_storage_bytes": (c_size_t, [c_size_t, c_size_t]),
    "gw_nvfp4_scale_offset": (c_size_t, [c_size_t, c_size_t, c_size_t]),
    "gw_nvfp4_scratch_upper_bound_bytes": (c_size_t, [c_size_t, c_size_t, c_size_t]),
    "gw_fp8_scratch_upper_bound_bytes": (c_size_t, [c_size_t, c_size_t]),
    "gw_nvfp4_dequantize": (c_int, [c_void_p, c_void_p, c_float, c_uint32, c_uint32, c_void_p, c_void_p]),
    "gw_nvfp4_pack_weights": (c_int, [c_void_p, c_uint32, c_uint32, c_float, c_void_p, c_void_p, c_void_p]),
    "gw_nvfp4_quantize_activations": (c_int, [c_void_p, c_uint32, c_uint32, c_float, c_int, c_void_p, c_void_p, c_void_p]),
    "gw_nvfp4_plan_create": (c_int, [c_uint32, c_uint32, c_uint32, POINTER(c_void_p)]),
    "gw_nvfp4_plan_scratch_bytes": (c_size_t, [c_void_p]),
    "gw_nvfp4_plan_run": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_float, c_void_p, c_void_p,
                                  c_size_t, c_void_p, c_int]),
    "gw_nvfp4_plan_destroy": (None, [c_void_p]),
    "gw_nvfp4_linear_static_scratch_limit": (c_size_t, []),
    "gw_nvfp4_linear_static_scratch": (c_int, [c_void_p, c_uint32, c_uint32, c_uint32, c_void_p, c_void_p, c_float,
                                               c_float, c_void_p, c_void_p, c_int]),
    "gw_nvfp4_gemv_w4a16": (c_int, [c_void_p, c_uint32, c_void_p, c_void_p, c_float, c_uint32, c_uint32, c_void_p, c_void_p]),
    "gw_fp8_quantize_activations": (c_int, [c_void_p, c_uint32, c_uint32, c_float, c_int, c_void_p, c_void_p]),
    "gw_fp8_pack_weights": (c_int, [c_void_p, c_uint32, c_uint32, c_float, c_void_p, c_void_p, c_void_p]),
    "gw_fp8_plan_create": (c_int, [c_uint32, c_uint32, c_uint32, c_int, POINTER(c_void_p)]),
    "gw_fp8_plan_scratch_bytes": (c_size_t, [c_void_p]),
    "gw_fp8_plan_run": (c_int, [c_void_p, c_void_p, c_void_p, c_float, c_float, c_void_p, c_void_p, c_void_p,
                                c_size_t, c_void_p, c_int]),
    "gw_fp8_plan_destroy": (None, [c_void_p]),
    "gw_bf16_plan_create": (c_int, [c_uint32, c_uint32, c_uint32, POINTER(c_void_p)]),
    "gw_bf16_plan_scratch_bytes": (c_size_t, [c_void_p]),
    "gw_bf16_plan_run": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "gw_bf16_plan_destroy": (None, [c_void_p]),
    "gw_nvfp4_fp4_activations": (c_int, [c_int, c_int]),
    "gw_bind_projection": (c_int, [c_uint32, c_uint32, c_uint32, c_void_p, c_void_p, c_size_t, POINTER(Projection)]),
    "gw_qkv_projector_create": (c_int, [c_uint32, c_uint32, c_uint32, c_uint32, c_int, POINTER(c_void_p)]),
    "gw_qkv_projector_prepare": (c_int, [c_void_p, c_uint32]),
    "gw_qkv_projector_run": (c_int, [c_void_p] * 8 + [c_int, c_void_p, POINTER(c_int)]),
    "gw_qkv_projector_bytes": (c_size_t, [c_void_p]),
    "gw_qkv_projector_destroy": (None, [c_void_p]),
    "gw_join_nvfp4_pair": (c_int, [c_void_p, c_void_p, c_void_p, c_size_t, c_void_p, POINTER(c_int)]),
    "gw_join_fp8_group": (c_int, [c_void_p, c_uint32, c_void_p, c_void_p, c_size_t, c_void_p, POINTER(c_int)]),
    "gw_rms_norm_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_uint32, c_uint32, c_void_p]),
    "gw_rms_norm_feedforward_bf16": (c_int, [c_void_p] * 7 + [c_uint32, c_uint32, c_void_p]),
    "gw_add_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_uint64, c_void_p]),
    "gw_scale_bf16": (c_int, [c_void_p, c_void_p, c_uint64, c_void_p]),
    "gw_ffn_tail_bf16": (c_int, [c_void_p] * 7 + [c_uint32, c_uint32, c_void_p]),
    "gw_ffn_block_create": (c_int, [c_void_p, c_uint32, c_uint32, c_int, c_uint32, c_void_p, POINTER(c_void_p)]),
    "gw_ffn_block_prepare": (c_int, [c_void_p, c_uint32, c_int]),
    "gw_ffn_block_run": (c_int, [c_void_p, c_void_p, c_void_p]),
    "gw_ffn_block_bytes": (c_size_t, [c_void_p]),
    "gw_ffn_block_destroy": (None, [c_void_p]),
    "gw_ffn_block_buffer": (c_void_p, [c_void_p, c_int]),
    "gw_ffn_block_moe": (c_void_p, [c_void_p]),
    "gw_debug_rsqrt": (c_int, [c_void_p, c_void_p, c_uint32]),
    "gw_rms_norm_reduction_lanes": (c_uint32, [c_uint32, c_uint32]),
    "gw_artifact_open": (c_int, [c_char_p, c_void_p, c_uint32, POINTER(c_void_p)]),
    "gw_artifact_count": (c_uint32, [c_void_p]),
    "gw_artifact_is_mixed": (c_int, [c_void_p]),
    "gw_artifact_file_bytes": (c_uint64, [c_void_p]),
    "gw_artifact_entry_at": (c_int, [c_void_p, c_uint32, c_void_p]),
    "gw_artifact_verify_full": (c_int, [c_void_p]),
    "gw_artifact_close": (None, [c_void_p]),
    "gw_projection_entry_bytes": (c_size_t, [c_uint32, c_uint32, c_uint32]),
    "gw_validate_projection_entry": (c_int, [c_uint32, c_uint32, c_uint32, c_void_p, c_size_t]),
    "gw_projection_workspace_create": (c_int, [POINTER(Projection), c_uint32, c_uint32, c_int, c_void_p, POINTER(c_void_p)]),
    "gw_projection_workspace_prepare": (c_int, [c_void_p, c_uint32, c_int]),
    "gw_projection_workspace_run": (c_int, [c_void_p, POINTER(Projection), c_void_p, c_void_p]),
    "gw_projection_workspace_bytes": (c_size_t, [c_void_p]),
    "gw_projection_workspace_destroy": (None, [c_void_p]),
    "gw_gelu_tanh_multiply_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_uint64, c_void_p]),
    "gw_gelu_tanh_multiply_interleaved_bf16": (c_int, [c_void_p, c_void_p, c_uint32, c_uint32, c_void_p]),
    "gw_mlp_chain_create": (c_int, [c_uint32, c_uint32, c_uint32, c_int, POINTER(c_void_p)]),
    "gw_mlp_chain_prepare": (c_int, [c_void_p, c_uint32]),
    "gw_mlp_chain_run": (c_int, [c_void_p, POINTER(Projection), POINTER(Projection), POINTER(Projection), c_void_p,
                                 c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    "gw_mlp_chain_bytes": (c_size_t, [c_void_p]),
    "gw_mlp_chain_destroy": (None, [c_void_p]),
    "gw_absmax_bf16": (c_int, [c_void_p, c_uint64, c_void_p, c_void_p]),
    "gw_weight_qdq_apply": (c_int, [c_int, c_void_p, c_uint64, c_void_p, c_void_p]),
    "gw_moe_expert_table_create": (c_int, [POINTER(ExpertWeights), c_uint32, POINTER(c_void_p)]),
    "gw_moe_expert_table_destroy": (None, [c_void_p]),
    "gw_moe_create": (c_int, [c_uint32, POINTER(c_void_p)]),
    "gw_moe_create_ex": (c_int, [c_uint32, c_uint32, POINTER(c_void_p)]),
    "gw_moe_expert_table_enable_w4a16": (c_int, [c_void_p, c_void_p]),
    "gw_moe_destroy": (None, [c_void_p]),
    "gw_moe_dispatch": (c_int, [c_void_p, c_void_p, c_void_p, c_uint32, c_void_p]),
    "gw_moe_run": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_uint32, c_int, c_int,
                           c_int, c_int, c_void_p]),
    "gw_moe_selected_experts": (c_void_p, [c_void_p]),
    "gw_moe_routing_weights": (c_void_p, [c_void_p]),
    "gw_moe_offsets": (c_void_p, [c_void_p]),
    "gw_moe_sorted_assignments": (c_void_p, [c_void_p]),
    "gw_moe_inverse": (c_void_p, [c_void_p]),
    "gw_moe_gate_up_capture": (c_void_p, [c_void_p]),
    "gw_moe_activated_capture": (c_void_p, [c_void_p]),
    "gw_moe_down_capture": (c_void_p, [c_void_p]),
    "gw_moe_bytes": (c_size_t, [c_void_p]),
    "gw_moe_routing_bytes": (c_size_t, [c_void_p]),
    "gw_moe_projection_bytes": (c_size_t, [c_void_p]),
    "gw_moe_reduction_bytes": (c_size_t, [c_void_p]),
    "gw_moe_capture": (c_int, [c_void_p, c_int]),
    "gw_moe_stage_timing": (c_int, [c_void_p, c_int]),
    "gw_moe_stage_elapsed_ms": (c_int, [c_void_p, POINTER(c_float)]),
    "gw_moe_run_sorted": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_uint32, c_uint32, c_uint32, c_void_p, c_void_p, c_void_p]),
    "gw_gather_rows_bf16": (c_int, [c_void_p, c_void_p, c_uint32, c_uint32, c_uint32, c_void_p, c_void_p]),
    "gw_moe_combine": (c_int, [c_void_p, c_void_p, c_void_p, c_uint32, c_uint32, c_void_p, c_void_p]),
    "gw_ipc_alloc": (c_int, [c_size_t, POINTER(c_void_p), c_void_p]),
    "gw_ipc_open": (c_int, [c_void_p, POINTER(c_void_p)]),
    "gw_ipc_close": (c_int, [c_void_p]),
    "gw_ipc_free": (c_int, [c_void_p]),
    "gw_moe_ep_dispatch": (c_int, [c_void_p, c_void_p, c_uint32, c_void_p, c_void_p, c_void_p, c_void_p, c_uint32,
                                   c_void_p]),
    "gw_moe_ep_activation_record_bytes": (c_size_t, []),
    "gw_moe_ep_run_gate_up": (c_int, [c_void_p, c_void_p, c_void_p, c_uint32, c_uint32, c_uint32, c_void_p, c_void_p, c_void_p]),
    "gw_moe_ep_finish_at_home": (c_int, [c_void_p, c_uint32, c_void_p, c_void_p, c_void_p, c_uint32, c_void_p, c_void_p, c_void_p]),
    "gw_moe_ep_mailbox_bytes": (c_size_t, []),
    "gw_moe_ep_exchange": (c_int, [c_void_p, c_uint32, c_void_p, c_uint32, c_uint32, c_void_p, c_void_p, c_void_p]),
    "gw_moe_ep_tables": (c_int, [c_void_p, c_void_p, c_uint32, c_uint32, c_void_p, c_void_p, c_void_p, c_void_p,
                                 c_void_p]),
    "gw_moe_ep_run_experts": (c_int, [c_void_p, c_void_p, c_void_p, c_uint32, c_uint32, c_uint32, c_void_p, c_void_p,
                                      c_void_p, c_void_p, c_void_p, c_uint32, c_uint32, c_void_p]),
    "gw_moe_ep_combine": (c_int, [c_void_p, c_uint32, c_void_p, c_void_p, c_void_p, c_uint32, c_void_p, c_void_p]),
    "gw_moe_host_runner_create": (c_int, [c_void_p, c_void_p, c_void_p, c_uint32, c_uint32, POINTER(c_void_p)]),
    "gw_moe_host_runner_destroy": (None, [c_void_p]),
    "gw_moe_host_runner_submit": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_uint32, POINTER(c_uint64)]),
    "gw_moe_host_runner_wait": (c_int, [c_void_p, c_uint64]),
    "gw_moe_host_runner_synchronize": (c_int, [c_void_p]),
    "gw_moe_host_runner_streams": (c_int, [c_void_p, POINTER(c_void_p), POINTER(c_void_p), POINTER(c_void_p)]),
    "gw_moe_host_runner_h2d_bytes": (c_uint64, [c_void_p]),
    "gw_moe_host_runner_d2h_bytes": (c_uint64, [c_void_p]),
    "gw_debug_kernel_error": (c_uint32, []),
    "gw_debug_launch_count": (c_uint64, []),
    "gw_debug_gemm_profile": (c_int, [c_void_p]),
    "gw_debug_rcp_approx": (c_int, [c_void_p, c_void_p, c_uint64, c_void_p]),
    "gw_debug_geglu_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_uint64, c_void_p]),
    "gw_debug_moe_quantized_input": (c_int, [c_void_p, POINTER(c_void_p), POINTER(c_void_p), POINTER(c_uint32),
                                             POINTER(c_uint32)]),
}


class GewellError(RuntimeError):
    """CUDA / kernel failure (the reference throws std::runtime_error)."""


class GewellInvalidArgument(ValueError):
    """Contract violation (the reference throws std::invalid_argument)."""


class GewellUnsupported(NotImplementedError):
    pass


def exported_symbols() -> list[str]:
    return sorted(_SIGNATURES)


def load() -> ctypes.CDLL:
    if not LIBRARY_PATH.exists():
        raise ImportError(
            f"{LIBRARY_PATH} is missing: build it with `python -m gewell_b200.build` "
            "(gewell_b200 has no CPU fallback)")
    lib = ctypes.CDLL(str(LIBRARY_PATH))
    for name, (restype, argtypes) in _SIGNATURES.items():
        fn = getattr(lib, name)          # AttributeError if the symbol is missing
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


def check(lib: ctypes.CDLL, status: int) -> None:
    if status == GW_OK:
        return
    message = lib.gw_last_error().decode("utf-8", "replace")
    if status == GW_INVALID_ARGUMENT:
        raise GewellInvalidArgument(message)
    if status == GW_UNSUPPORTED:
        raise GewellUnsupported(message)
    raise GewellError(message)
