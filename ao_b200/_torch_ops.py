"""PyTorch dispatcher operators of this library, in the reference's own namespace:

    torch.ops.torchao.quant_llm_linear(EXPONENT, MANTISSA, _in_feats, _weights, _scales, splitK) -> Tensor
    torch.ops.torchao._weight_int4pack_mm(x, w, qGroupSize, qScaleAndZeros) -> Tensor
    torch.ops.torchao._convert_weight_to_int4pack(int_data, innerKTiles) -> Tensor

The schemas and CUDA implementations are compiled C++ (ao_b200/csrc/torch/torch_binding.cpp: TORCH_LIBRARY_FRAGMENT /
TORCH_LIBRARY_IMPL, as torchao/csrc/fp6_llm.cpp:5-8 and torchao/csrc/cuda/fp6_llm/fp6_linear.cu:198-200), built by
`python -m ao_b200.build --torch` into ao_b200/lib/torch_ext/ao_b200_torch.so.  The fake (meta) implementations are
registered here in Python with the shape / dtype checks, as the reference does (torchao/ops.py:6-55), so the operators
trace under FakeTensor, torch.compile and export.  Inference only: no autograd formula, like the reference.

Importing this module without the built extension raises: there is no Python fallback for the operators.
"""
import ctypes
import os

import torch

from . import _cabi
from .build import TORCH_EXT_PATH

if not os.path.exists(TORCH_EXT_PATH):
    raise ImportError(f"{TORCH_EXT_PATH} is missing: build it with `python -m ao_b200.build --torch`. "
                      "The torchao:: dispatcher operators have no Python fallback.")
_cabi.lib()                                                   # fails loudly if libao_b200.so has not been built
ctypes.CDLL(_cabi.LIB_PATH, mode=ctypes.RTLD_GLOBAL)          # the extension finds libao_b200.so by its soname
torch.ops.load_library(TORCH_EXT_PATH)


@torch.library.register_fake("torchao::quant_llm_linear")
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


@torch.library.register_fake("torchao::_weight_int4pack_mm")
def _(x, w, qGroupSize, qScaleAndZeros):
    torch._check(x.dim() == 2, lambda: "x must be a 2D tensor")
    torch._check(x.dtype is torch.bfloat16, lambda: f"expected x to be bf16, got {x.dtype}")
    torch._check(w.dim() == 4 and w.dtype is torch.int32, lambda: "w must be a 4D int32 tensor")
    torch._check(qGroupSize in (32, 64, 128, 256), lambda: f"qGroupSize must be 32, 64, 128, or 256, got {qGroupSize}")
    torch._check(qScaleAndZeros.dim() == 3 and qScaleAndZeros.size(1) == w.size(0) * 8 and qScaleAndZeros.size(2) == 2,
                 lambda: "qScaleAndZeros must be [K/group][N][2]")
    return x.new_empty((x.size(0), w.size(0) * 8))


@torch.library.register_fake("torchao::_convert_weight_to_int4pack")
def _(int_data, innerKTiles):
    torch._check(int_data.dim() == 2, lambda: "int_data must be 2-D [n][k]")
    torch._check(innerKTiles in (2, 4, 8), lambda: "innerKTiles must be 2, 4, or 8")
    n, k = int_data.shape
    torch._check(n % 8 == 0, lambda: f"expect N to be a multiple of 8, got {n}")
    torch._check(k % (innerKTiles * 16) == 0, lambda: f"expect K to be a multiple of {innerKTiles * 16}, got {k}")
    return int_data.new_empty((n // 8, k // (innerKTiles * 16), 32, innerKTiles // 2), dtype=torch.int32)
