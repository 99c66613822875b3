"""gewell_b200 -- B200 (sm_100a) NVFP4 / FP8 projections and the 26B-A4B MoE
layer behind a C ABI.  The package is a thin host layer over
libgewell_b200.so; it raises at import time if that library is not built.
There is no CPU execution path.
"""
from . import _lib
from ._lib import GewellError, GewellInvalidArgument, GewellUnsupported  # noqa: F401

lib = _lib.load()

from .ops import (  # noqa: E402,F401
    ExpertTable, Fp8Plan, Fp8Weight, MoeWorkspace, Nvfp4Plan, Nvfp4Weight, absmax_bf16, fp8_pack_weights,
    fp8_quantize_activations, gather_rows, moe_combine, nvfp4_dequantize, nvfp4_gemv_w4a16,
    nvfp4_pack_weights, nvfp4_quantize_activations, nvfp4_scale_offset, nvfp4_scale_storage_bytes,
    weight_qdq_apply, kernel_error,
)
