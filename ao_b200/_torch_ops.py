"""PyTorch dispatcher registration of the operators (namespace `ao_b200`), the counterpart of the reference's
TORCH_LIBRARY_FRAGMENT(torchao) + fake implementations (torchao/csrc/fp6_llm.cpp:5-8, torchao/ops.py:6-55):

    torch.ops.ao_b200.quant_llm_linear(EXPONENT, MANTISSA, _in_feats, _weights, _scales, splitK) -> Tensor
    torch.ops.ao_b200.weight_int4pack_mm(x, w, qGroupSize, qScaleAndZeros) -> Tensor
    torch.ops.ao_b200.convert_weight_to_int4pack(int_data, innerKTiles) -> Tensor

CUDA implementations call the C ABI through ao_b200.ops; the fake implementations carry the shape / dtype checks, so
the ops trace under FakeTensor / torch.compile / export.  Inference only: no autograd formula, like the reference.
"""
import torch
from torch import Tensor

from . import ops

_lib = torch.library.Library("ao_b200", "DEF")
_lib.define("quant_llm_linear(int EXPONENT, int MANTISSA, Tensor _in_feats, Tensor _weights, Tensor _scales, int splitK) -> Tensor")
_lib.define("weight_int4pack_mm(Tensor x, Tensor w, int qGroupSize, Tensor qScaleAndZeros) -> Tensor")
_lib.define("convert_weight_to_int4pack(Tensor int_data, int innerKTiles) -> Tensor")


def _quant_llm_linear_cuda(EXPONENT, MANTISSA, _in_feats, _weights, _scales, splitK):
    return ops.quant_llm_linear(EXPONENT, MANTISSA, _in_feats, _weights, _scales, splitK)


def _weight_int4pack_mm_cuda(x, w, qGroupSize, qScaleAndZeros):
    return ops.weight_int4pack_mm(x, w, qGroupSize, qScaleAndZeros)


def _convert_weight_to_int4pack_cuda(int_data, innerKTiles):
    return ops.convert_weight_to_int4pack(int_data, innerKTiles)


_lib.impl("quant_llm_linear", _quant_llm_linear_cuda, "CUDA")
_lib.impl("weight_int4pack_mm", _weight_int4pack_mm_cuda, "CUDA")
_lib.impl("convert_weight_to_int4pack", _convert_weight_to_int4pack_cuda, "CUDA")


@torch.library.register_fake("ao_b200::quant_llm_linear")
def _(EXPONENT, MANTISSA, _in_feats, _weights, _scales, splitK=1):
    torch._check(_in_feats.dim() == 2, lambda: f"input should be a 2d tensor, got {_in_feats.dim()}D")
    torch._check(_in_feats.dtype is torch.float16, lambda: f"weight must be FP16, got {_in_feats.dtype}")
    torch._check(_weights.dim() == 2, lambda: f"weight should be a 2d tensor, got {_weights.dim()}D")
    torch._check(_weights.dtype is torch.uint8, lambda: f"weight must be UINT8, got {_weights.dtype}")
    torch._check(_scales.dim() == 1, lambda: f"scale should be a 2d tensor, got {_scales.dim()}D")
    torch._check(_scales.dtype is torch.float16, lambda: f"scale must be FP16, got {_scales.dtype}")
    BS, IC = _in_feats.shape
    OC, _ = _weights.shape
    N_BITS = 1 + EXPONENT + MANTISSA
    torch._check(IC // 8 * N_BITS == _weights.shape[1], lambda: "Dimensions mismatched")
    torch._check(OC == _scales.shape[0], lambda: "Dimensions mismatched")
    return _in_feats.new_empty((BS, OC))


@torch.library.register_fake("ao_b200::weight_int4pack_mm")
def _(x, w, qGroupSize, qScaleAndZeros):
    torch._check(x.dim() == 2, lambda: "x must be a 2D tensor")
    torch._check(x.dtype is torch.bfloat16, lambda: f"expected x to be bf16, got {x.dtype}")
    torch._check(w.dim() == 4 and w.dtype is torch.int32, lambda: "w must be a 4D int32 tensor")
    torch._check(qGroupSize in (32, 64, 128, 256), lambda: f"qGroupSize must be 32, 64, 128, or 256, got {qGroupSize}")
    torch._check(qScaleAndZeros.dim() == 3 and qScaleAndZeros.size(1) == w.size(0) * 8 and qScaleAndZeros.size(2) == 2,
                 lambda: "qScaleAndZeros must be [K/group][N][2]")
    return x.new_empty((x.size(0), w.size(0) * 8))


@torch.library.register_fake("ao_b200::convert_weight_to_int4pack")
def _(int_data, innerKTiles):
    torch._check(int_data.dim() == 2, lambda: "int_data must be 2-D [n][k]")
    torch._check(innerKTiles in (2, 4, 8), lambda: "innerKTiles must be 2, 4, or 8")
    n, k = int_data.shape
    torch._check(n % 8 == 0, lambda: f"expect N to be a multiple of 8, got {n}")
    torch._check(k % (innerKTiles * 16) == 0, lambda: f"expect K to be a multiple of {innerKTiles * 16}, got {k}")
    return int_data.new_empty((n // 8, k // (innerKTiles * 16), 32, innerKTiles // 2), dtype=torch.int32)
