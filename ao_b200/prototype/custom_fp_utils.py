"""fp32 <-> sub-byte float (ExMy) codec — torchao/prototype/custom_fp_utils.py:27-229 on CUDA kernels.

No inf/nan encodings; round to nearest even; values beyond the largest normal saturate."""
import torch
from torch import Tensor

from .. import _cabi


def _n_ones(n: int) -> int:
    return (1 << n) - 1


EBITS_F32, MBITS_F32 = 8, 23
F32_EXP_BIAS = _n_ones(EBITS_F32 - 1)


def _f32_to_fpx_unpacked(x: Tensor, ebits: int, mbits: int) -> Tensor:
    """fp32 tensor -> uint8 codes, the ExMy bits in the low 1+ebits+mbits bits
    (torchao/prototype/custom_fp_utils.py:27-140)."""
    assert x.dtype == torch.float
    assert 1 + ebits + mbits <= 8
    _cabi.require_cuda(x)
    xc = x.contiguous()
    out = torch.empty(xc.shape, dtype=torch.uint8, device=xc.device)
    if xc.numel():
        with torch.cuda.device(xc.device):
            rc = _cabi.lib().ao_f32_to_fpx_unpacked(_cabi.ptr(xc), xc.numel(), ebits, mbits, _cabi.ptr(out),
                                                    _cabi.stream_ptr(xc.device))
        _cabi.check(rc, "_f32_to_fpx_unpacked")
    return out


def _fpx_unpacked_to_f32(x: Tensor, ebits: int, mbits: int) -> Tensor:
    """uint8 ExMy codes -> fp32 (torchao/prototype/custom_fp_utils.py:145-229)."""
    assert x.dtype == torch.uint8
    assert 1 + ebits + mbits <= 8
    _cabi.require_cuda(x)
    xc = x.contiguous()
    out = torch.empty(xc.shape, dtype=torch.float32, device=xc.device)
    if xc.numel():
        with torch.cuda.device(xc.device):
            rc = _cabi.lib().ao_fpx_unpacked_to_f32(_cabi.ptr(xc), xc.numel(), ebits, mbits, _cabi.ptr(out),
                                                    _cabi.stream_ptr(xc.device))
        _cabi.check(rc, "_fpx_unpacked_to_f32")
    return out
