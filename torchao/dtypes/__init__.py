"""torchao.dtypes (torchao/dtypes/__init__.py): re-export of ao_b200.dtypes."""
from ao_b200.dtypes import *  # noqa: F401,F403
from ao_b200.dtypes import __all__  # noqa: F401
from ao_b200.dtypes.affine_quantized_tensor import implements, register_layout_cls  # noqa: F401
