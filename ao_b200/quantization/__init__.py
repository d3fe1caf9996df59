from .quant_api import (
    fp6_llm_weight_only,
    int4_weight_only,
    quant_llm_fpx_weight_only,
    quantize,
    quantize_,
)
from .quant_primitives import (
    MappingType,
    ZeroPointDomain,
    choose_qparams_affine,
    dequantize_affine,
    quantize_affine,
)
from .utils import (
    compute_error,
    get_groupwise_affine_qparams,
    groupwise_affine_dequantize_tensor,
    groupwise_affine_dequantize_tensor_from_qparams,
    groupwise_affine_quantize_tensor,
    groupwise_affine_quantize_tensor_from_qparams,
    pack_tinygemm_scales_and_zeros,
    unpack_tinygemm_scales_and_zeros,
)

__all__ = [
    "quantize", "quantize_", "int4_weight_only", "fp6_llm_weight_only",
    "quant_llm_fpx_weight_only", "MappingType", "ZeroPointDomain", "choose_qparams_affine", "quantize_affine",
    "dequantize_affine", "compute_error", "get_groupwise_affine_qparams", "pack_tinygemm_scales_and_zeros",
    "unpack_tinygemm_scales_and_zeros", "groupwise_affine_quantize_tensor_from_qparams",
    "groupwise_affine_dequantize_tensor_from_qparams", "groupwise_affine_quantize_tensor",
    "groupwise_affine_dequantize_tensor",
]
