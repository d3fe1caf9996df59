from .affine_quantized_tensor import (
    AffineQuantizedTensor,
    PlainAQTLayout,
    TensorCoreTiledAQTLayout,
    to_affine_quantized,
)

__all__ = ["AffineQuantizedTensor", "PlainAQTLayout", "TensorCoreTiledAQTLayout", "to_affine_quantized"]
