"""torchao.quantization.utils: re-export of ao_b200.quantization.utils."""
from ao_b200.quantization.utils import *  # noqa: F401,F403
from ao_b200.quantization.utils import (  # noqa: F401
    compute_error,
    get_groupwise_affine_qparams,
    groupwise_affine_dequantize_tensor,
    groupwise_affine_dequantize_tensor_from_qparams,
    groupwise_affine_quantize_tensor,
    groupwise_affine_quantize_tensor_from_qparams,
    pack_tinygemm_scales_and_zeros,
    unpack_tinygemm_scales_and_zeros,
)
