from .affine_quantized_tensor import (
    AffineQuantizedTensor,
    PlainAQTLayout,
    TensorCoreTiledAQTLayout,
    to_affine_quantized,
    use_static_linear_outputs,
)

__all__ = ["AffineQuantizedTensor", "PlainAQTLayout", "TensorCoreTiledAQTLayout", "to_affine_quantized",
           "use_static_linear_outputs"]

# torch.load(weights_only=True), the default, only rebuilds classes it has been told about: a state_dict that holds
# quantized weights (torch.save(model.state_dict())) loads without weights_only=False once these are registered
import torch as _torch
from ..quantization.quant_primitives import MappingType as _MappingType, ZeroPointDomain as _ZeroPointDomain

if hasattr(_torch.serialization, "add_safe_globals"):
    _torch.serialization.add_safe_globals([AffineQuantizedTensor, PlainAQTLayout, TensorCoreTiledAQTLayout,
                                           _MappingType, _ZeroPointDomain])
