"""torchao.quantization.quant_primitives: re-export of ao_b200.quantization.quant_primitives."""
from ao_b200.quantization.quant_primitives import *  # noqa: F401,F403
from ao_b200.quantization.quant_primitives import (  # noqa: F401
    MappingType,
    ZeroPointDomain,
    choose_qparams_affine,
    dequantize_affine,
    quantize_affine,
)
