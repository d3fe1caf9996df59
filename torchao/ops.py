"""torchao.ops of the reference (torchao/ops.py:15-55): the operators go through the PyTorch dispatcher
(torch.ops.torchao.*, registered by ao_b200._torch_ops together with their fake implementations)."""
from torch import Tensor

import torch

import ao_b200._torch_ops  # noqa: F401  (loads the compiled operator library and registers the fake implementations)
from ao_b200.ops import prepack_fp6_weight  # noqa: F401


def quant_llm_linear(EXPONENT: int, MANTISSA: int, _in_feats: Tensor, _weights: Tensor, _scales: Tensor,
                     splitK: int = 1) -> Tensor:
    """Quant-LLM linear layer A @ W.T (torchao/ops.py:15-37): fp16 activations, packed FPx weights, fp16 scales."""
    return torch.ops.torchao.quant_llm_linear.default(EXPONENT, MANTISSA, _in_feats, _weights, _scales, splitK)


def fp6_llm_linear(_in_feats: Tensor, _weights: Tensor, _scales: Tensor, splitK: int = 1) -> Tensor:
    """The e3m2 case under the name of the earlier torchao release."""
    return quant_llm_linear(3, 2, _in_feats, _weights, _scales, splitK)
