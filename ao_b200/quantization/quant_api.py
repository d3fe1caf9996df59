"""Model-level quantization API — torchao/quantization/quant_api.py:146-191, 255-318, 362-404.

quantize(model, apply_tensor_subclass, filter_fn=None, set_inductor_config=True) walks the modules and swaps
nn.Linear weights for tensor-subclass instances; int4_weight_only / fp6_llm_weight_only
build the conversion functions.  `quantize_` is the spelling of later torchao releases for the same call.
"""
from typing import Callable, Optional

import torch

from .quant_primitives import MappingType, ZeroPointDomain

__all__ = [
    "quantize",
    "quantize_",
    "int4_weight_only",
    "fp6_llm_weight_only",
    "quant_llm_fpx_weight_only",
]


def _replace_with_custom_fn_if_matches_filter(model, replacement_fn, filter_fn, cur_fqn="") -> None:
    """Recursively replaces each module for which filter_fn(module, fqn) holds by replacement_fn(module)
    (torchao/quantization/quant_api.py:146-175)."""
    if filter_fn(model, cur_fqn[:-1]):
        model = replacement_fn(model)
        return model
    for name, child in model.named_children():
        new_child = _replace_with_custom_fn_if_matches_filter(child, replacement_fn, filter_fn, f"{cur_fqn}{name}.")
        if new_child is not child:
            setattr(model, name, new_child)
    return model


def _is_linear(mod, *args):
    """nn.Linear whose weight is not quantized yet (torchao/quantization/quant_api.py:178-191)."""
    from ..dtypes import AffineQuantizedTensor
    from ..prototype.quant_llm import QuantLlmLinearWeight

    return (isinstance(mod, torch.nn.Linear) and hasattr(mod, "weight")
            and not isinstance(mod.weight, AffineQuantizedTensor)
            and not isinstance(mod.weight, QuantLlmLinearWeight))


def _get_linear_subclass_inserter(constructor):
    """torchao/quantization/quant_api.py:255-260"""
    def insert_subclass(lin):
        lin.weight = torch.nn.Parameter(constructor(lin.weight), requires_grad=False)
        return lin

    return insert_subclass


def quantize(model: torch.nn.Module, apply_tensor_subclass: Callable[[torch.Tensor], torch.Tensor],
             filter_fn: Optional[Callable[[torch.nn.Module, str], bool]] = None,
             set_inductor_config: bool = True) -> torch.nn.Module:
    """Converts the weights of the model's linear modules with `apply_tensor_subclass`, in place, and returns
    the model (torchao/quantization/quant_api.py:262-318).

    `set_inductor_config` is accepted for compatibility and has no effect: the kernels here are launched
    directly and nothing goes through a tracing compiler."""
    _replace_with_custom_fn_if_matches_filter(
        model, _get_linear_subclass_inserter(apply_tensor_subclass), _is_linear if filter_fn is None else filter_fn)
    return model


quantize_ = quantize


def int4_weight_only(group_size=128, inner_k_tiles=8):
    """uint4 weight-only asymmetric per-group quantization in the tensor_core_tiled layout
    (torchao/quantization/quant_api.py:362-387); group_size in [256, 128, 64, 32], inner_k_tiles in [8, 4, 2]."""
    def apply_int4_weight_only_quant(weight):
        from ..dtypes import to_affine_quantized

        return to_affine_quantized(weight, MappingType.ASYMMETRIC, (1, group_size), torch.int32, 0, 15, 1e-6,
                                   zero_point_dtype=torch.bfloat16, preserve_zero=False,
                                   zero_point_domain=ZeroPointDomain.FLOAT, extended_layout="tensor_core_tiled",
                                   inner_k_tiles=inner_k_tiles)

    return apply_int4_weight_only_quant


def quant_llm_fpx_weight_only(ebits: int, mbits: int):
    from ..prototype.quant_llm import quant_llm_fpx_weight_only as impl
    return impl(ebits, mbits)


def fp6_llm_weight_only():
    from ..prototype.quant_llm import fp6_llm_weight_only as impl
    return impl()
