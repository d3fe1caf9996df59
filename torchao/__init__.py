"""`torchao` import names for the B200-native implementation in ao_b200: code written against the reference's
weight-only quantized-linear API (torchao/__init__.py, quantization/, dtypes/, ops.py, prototype/quant_llm,
prototype/hqq, utils.py) imports unchanged, e.g.

    from torchao.quantization import quantize, int4_weight_only
    torchao.ops.quant_llm_linear(3, 2, x, w, s, 1)

Only the parts of the package that belong to that path exist here.  Every module is a re-export; the code lives in
ao_b200."""
from ao_b200 import check_status  # noqa: F401

from . import dtypes, ops, quantization, utils  # noqa: F401
from .quantization import quantize  # noqa: F401

__all__ = ["dtypes", "ops", "quantization", "utils", "quantize", "check_status"]
