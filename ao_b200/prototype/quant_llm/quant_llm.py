"""FP6-LLM (e3m2) weight-only path — torchao/prototype/quant_llm/quant_llm.py on CUDA kernels.

Packing, scaling and unpacking keep the reference's names and byte-exact layouts; the per-shape
split-K table of the reference (quant_llm.py:212-345) is not needed because the kernel picks its own
K split, so `splitK` arguments are accepted and ignored.
"""
from typing import Tuple

import torch
from torch import Tensor

from ... import _cabi


def _check_fp6(nbits: int):
    if nbits != 6:
        raise NotImplementedError(f"only 6-bit (e3m2 / e2m3) tensor-core packing is built, got {nbits} bits")


def pack_tc_fpx(tensor: Tensor, nbits: int) -> Tensor:
    """uint8 codes [M][N] -> tensor-core pre-packed uint8 [M][N*nbits/8] (quant_llm.py:60-113)."""
    _check_fp6(nbits)
    from ...ops import prepack_fp6_weight
    return prepack_fp6_weight(tensor)


def unpack_tc_fpx(tensor: Tensor, nbits: int) -> Tensor:
    """Inverse of pack_tc_fpx (quant_llm.py:134-200)."""
    _check_fp6(nbits)
    assert tensor.ndim == 2 and tensor.dtype == torch.uint8
    _cabi.require_cuda(tensor)
    M = tensor.shape[0]
    N = tensor.shape[1] // 3 * 4
    assert (M % 64 == 0) and (N % 64 == 0)
    t = tensor.contiguous()
    out = torch.empty((M, N), dtype=torch.uint8, device=t.device)
    with torch.cuda.device(t.device):
        rc = _cabi.lib().ao_unpack_tc_fp6(_cabi.ptr(t), M, N, _cabi.ptr(out), _cabi.stream_ptr(t.device))
    _cabi.check(rc, "unpack_tc_fpx")
    return out


def to_scaled_tc_fpx(tensor: Tensor, ebits: int, mbits: int) -> Tuple[Tensor, Tensor]:
    """Per-row absmax/max_normal scale (fp32 math, fp16 result), ExMy encode, pre-pack
    (quant_llm.py:116-130).  Built for e3m2."""
    if (ebits, mbits) != (3, 2):
        raise NotImplementedError("to_scaled_tc_fpx is built for fp6 e3m2 only")
    _cabi.require_cuda(tensor)
    assert tensor.ndim == 2
    M, N = tensor.shape
    assert (M % 64 == 0) and (N % 64 == 0)
    t = tensor.contiguous()
    if t.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        t = t.float()
    packed = torch.empty((M, N * 6 // 8), dtype=torch.uint8, device=t.device)
    scale = torch.empty((M,), dtype=torch.float16, device=t.device)
    with torch.cuda.device(t.device):
        rc = _cabi.lib().ao_to_scaled_tc_fp6(_cabi.ptr(t), _cabi.dtype_code(t.dtype), M, N, _cabi.ptr(packed),
                                             _cabi.ptr(scale), _cabi.stream_ptr(t.device))
    _cabi.check(rc, "to_scaled_tc_fpx")
    return packed, scale


def from_scaled_tc_fpx(tensor: Tensor, ebits: int, mbits: int, scale=None) -> Tensor:
    """Unpack, decode to fp32 and apply the per-row scale (quant_llm.py:203-208).  Built for e3m2."""
    if (ebits, mbits) != (3, 2):
        raise NotImplementedError("from_scaled_tc_fpx is built for fp6 e3m2 only")
    assert tensor.ndim == 2 and tensor.dtype == torch.uint8
    _cabi.require_cuda(tensor, scale)
    M = tensor.shape[0]
    N = tensor.shape[1] // 3 * 4
    assert (M % 64 == 0) and (N % 64 == 0)
    t = tensor.contiguous()
    s = None if scale is None else scale.to(torch.float16).contiguous()
    out = torch.empty((M, N), dtype=torch.float32, device=t.device)
    with torch.cuda.device(t.device):
        rc = _cabi.lib().ao_from_scaled_tc_fp6(_cabi.ptr(t), M, N, _cabi.ptr(s), _cabi.ptr(out),
                                               _cabi.stream_ptr(t.device))
    _cabi.check(rc, "from_scaled_tc_fpx")
    return out
