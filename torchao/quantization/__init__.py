"""torchao.quantization (torchao/quantization/__init__.py): re-export of ao_b200.quantization."""
from ao_b200.quantization import *  # noqa: F401,F403
from ao_b200.quantization import __all__  # noqa: F401

from . import quant_api, quant_primitives, utils  # noqa: F401
