"""torchao.prototype.hqq: re-export of ao_b200.prototype.hqq."""
from ao_b200.prototype.hqq import *  # noqa: F401,F403
from ao_b200.prototype.hqq import __all__  # noqa: F401
