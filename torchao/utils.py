"""torchao.utils names used on the weight-only quantized-linear path (torchao/utils.py:81-165)."""
from ao_b200.utils import UnwrapTensorSubclass, find_multiple, unwrap_tensor_subclass  # noqa: F401
