from .affine_quantized_tensor import (
    AffineQuantizedTensor,
    PlainAQTLayout,
    TensorCoreTiledAQTLayout,
    to_affine_quantized,
    use_static_linear_outputs,
)

__all__ = ["AffineQuantizedTensor", "PlainAQTLayout", "TensorCoreTiledAQTLayout", "to_affine_quantized",
           "use_static_linear_outputs"]
