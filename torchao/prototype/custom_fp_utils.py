"""torchao.prototype.custom_fp_utils: re-export of ao_b200.prototype.custom_fp_utils."""
from ao_b200.prototype.custom_fp_utils import *  # noqa: F401,F403
from ao_b200.prototype.custom_fp_utils import _f32_to_fpx_unpacked, _fpx_unpacked_to_f32  # noqa: F401
