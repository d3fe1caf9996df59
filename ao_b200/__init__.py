"""ao_b200: B200-native (sm_100a) weight-only quantized linear behind torchao's Python API."""
from . import _cabi  # noqa: F401

__all__ = []
