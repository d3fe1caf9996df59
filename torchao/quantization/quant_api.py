"""torchao.quantization.quant_api: re-export of ao_b200.quantization.quant_api."""
from ao_b200.quantization.quant_api import *  # noqa: F401,F403
from ao_b200.quantization.quant_api import (  # noqa: F401
    _get_linear_subclass_inserter,
    _is_linear,
    _replace_with_custom_fn_if_matches_filter,
)
