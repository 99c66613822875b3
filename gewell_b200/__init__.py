"""gewell_b200 -- B200 (sm_100a) NVFP4 / FP8 projections and the 26B-A4B MoE
layer behind a C ABI.  The package is a thin host layer over
libgewell_b200.so.  There is no CPU execution path: the first use of any
operator (or of `gewell_b200.lib`) loads the CUDA library and raises
ImportError if it has not been built (`python -m gewell_b200.build`).
"""
from . import _lib
from ._lib import GewellError, GewellInvalidArgument, GewellUnsupported  # noqa: F401

_OPS = (
    "ExpertTable", "Fp8Plan", "Fp8Weight", "MoeWorkspace", "Nvfp4Plan", "Nvfp4Weight", "absmax_bf16",
    "fp8_pack_weights", "fp8_quantize_activations", "gather_rows", "moe_combine", "nvfp4_dequantize",
    "nvfp4_gemv_w4a16", "nvfp4_pack_weights", "nvfp4_quantize_activations", "nvfp4_scale_offset",
    "nvfp4_scale_storage_bytes", "weight_qdq_apply", "kernel_error", "TRANSFORM_IDENTITY",
    "TRANSFORM_GELU_TANH_MULTIPLY", "rcp_approx", "geglu_bf16", "nvfp4_linear_static_scratch", "launch_count", "Bf16Plan", "bind_projection", "ProjectionWorkspace", "MlpChain", "make_projection",
    "rsqrt_device", "rms_norm", "rms_norm_feedforward", "add_bf16", "scale_bf16", "ffn_tail", "FfnBlock", "QkvProjector", "join_nvfp4_pair", "join_fp8_group",
)


def __getattr__(name):
    if name == "lib":
        value = _lib.load()
    elif name == "HostStagedMoe":
        from .host_io import HostStagedMoe as value
    elif name in _OPS:
        from . import ops
        value = getattr(ops, name)
    else:
        raise AttributeError(f"module 'gewell_b200' has no attribute {name!r}")
    globals()[name] = value
    return value
