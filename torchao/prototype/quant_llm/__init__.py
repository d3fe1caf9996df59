"""torchao.prototype.quant_llm: re-export of ao_b200.prototype.quant_llm."""
from ao_b200.prototype.quant_llm import *  # noqa: F401,F403
from ao_b200.prototype.quant_llm import __all__  # noqa: F401
