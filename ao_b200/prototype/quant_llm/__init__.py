from .quant_llm import (
    QuantLlmLinearWeight,
    fp6_llm_weight_only,
    from_scaled_tc_fpx,
    pack_tc_fpx,
    quant_llm_fpx_weight_only,
    to_scaled_tc_fpx,
    unpack_tc_fpx,
)

__all__ = ["QuantLlmLinearWeight", "fp6_llm_weight_only", "quant_llm_fpx_weight_only", "to_scaled_tc_fpx",
           "from_scaled_tc_fpx", "pack_tc_fpx", "unpack_tc_fpx"]

import torch as _torch

if hasattr(_torch.serialization, "add_safe_globals"):   # see ao_b200/dtypes/__init__.py
    _torch.serialization.add_safe_globals([QuantLlmLinearWeight])
