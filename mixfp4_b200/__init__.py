"""mixfp4_b200: B200-native (sm_100a) block quantizer (E2M1-or-E0M3 per 16 elements, E4M3
block scales) and mixed-format FP4 dequant-linear, behind the Python surface of the
reference package ``project_quant`` (project_quant/__init__.py:1-16).

All compute runs in hand-written CUDA kernels reached through the C ABI declared in
include/mixfp4_b200.h; importing the package does not need a GPU, calling it does.
"""

from .quant import (E0M3_LEVELS, E2M1_LEVELS, SCALE_GROUP_SIZE, CandidateBlocks, GranularityResult, PackedWeight,
                    ScaledCandidate, build_candidates, build_scaled_candidate, dequantize, fake_quantize_activations, quantize_e0m3, quantize_e2m1, packed_nbytes, quant_mixfp4_granularity, quantize_packed, tensor_amax)
from .rotation import TRANSFORM_BANK, TransformSpec, apply_transform, get_transform
from .linear import MixFP4Linear, decode_status, gemm_status, mixfp4_linear, mixfp4_linear_grouped
from .convert import load_packed, named_linears, quantize_model_weights, save_packed

__all__ = [
    "E0M3_LEVELS", "E2M1_LEVELS", "SCALE_GROUP_SIZE", "CandidateBlocks", "GranularityResult", "ScaledCandidate", "build_candidates", "build_scaled_candidate",
    "quantize_e0m3", "quantize_e2m1", "PackedWeight", "dequantize",
    "fake_quantize_activations", "packed_nbytes", "quant_mixfp4_granularity", "quantize_packed", "tensor_amax", "TRANSFORM_BANK",
    "TransformSpec", "apply_transform", "get_transform", "MixFP4Linear", "decode_status", "gemm_status", "mixfp4_linear", "mixfp4_linear_grouped",
    "load_packed", "named_linears", "quantize_model_weights", "save_packed",
]
