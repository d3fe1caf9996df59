"""choose_qparams_affine / quantize_affine / dequantize_affine on sm_100a kernels.

Same names, arguments, results and errors as torchao/quantization/quant_primitives.py:134-367; the
arithmetic runs in ao_b200/csrc/quant_primitives.cu through the C ABI.  CUDA tensors only.
"""
from enum import Enum
from typing import Dict, Optional, Tuple

import torch

from .. import _cabi

__all__ = [
    "MappingType",
    "ZeroPointDomain",
    "choose_qparams_affine",
    "quantize_affine",
    "dequantize_affine",
]


class MappingType(Enum):
    """torchao/quantization/quant_primitives.py:24-38"""
    SYMMETRIC = 0
    ASYMMETRIC = 1


class ZeroPointDomain(Enum):
    """torchao/quantization/quant_primitives.py:40-47"""
    INT = 0
    FLOAT = 1


_DTYPE_TO_QVALUE_BOUNDS: Dict[torch.dtype, Tuple[int, int]] = {
    torch.uint8: (0, 255),
    torch.int8: (-128, 127),
    torch.int16: (-(2**15), 2**15 - 1),
    torch.int32: (-(2**31), 2**31 - 1),
}
for _bits in range(1, 8):
    _dt = getattr(torch, f"uint{_bits}", None)
    if _dt is not None:
        _DTYPE_TO_QVALUE_BOUNDS[_dt] = (0, 2**_bits - 1)


def _get_and_check_qmin_qmax(dtype, quant_min, quant_max):
    """torchao/quantization/quant_primitives.py:73-93"""
    if dtype not in _DTYPE_TO_QVALUE_BOUNDS:
        raise ValueError(f"Unsupported dtype: {dtype}")
    lo, hi = _DTYPE_TO_QVALUE_BOUNDS[dtype]
    if quant_min is None:
        quant_min = lo
    if quant_max is None:
        quant_max = hi
    assert quant_min >= lo, f"quant_min out of bound for dtype, quant_min_lower_bound: {lo} quant_min: {quant_min}"
    assert quant_max <= hi, f"quant_max out of bound for dtype, quant_max_upper_bound: {hi} quant_max: {quant_max}"
    return quant_min, quant_max


def _get_reduction_params(block_size, input_size):
    """torchao/quantization/quant_primitives.py:95-131 (shape bookkeeping only; host side)."""
    assert len(block_size) == len(input_size)
    shape_for_reduction = []
    reduction_dims = []
    cur_dim = 0
    for i in range(len(block_size)):
        if block_size[i] != input_size[i] and block_size[i] > 1:
            assert input_size[i] % block_size[i] == 0, (
                f"Expecting input size at {i} dimension: {input_size[i]} to be divisible by block_size at {i} "
                f"dimension: {block_size[i]}")
            shape_for_reduction.append(input_size[i] // block_size[i])
            shape_for_reduction.append(block_size[i])
            reduction_dims.append(cur_dim + 1)
            cur_dim += 2
        else:
            shape_for_reduction.append(input_size[i])
            if block_size[i] != 1:
                reduction_dims.append(cur_dim)
            cur_dim += 1
    return shape_for_reduction, reduction_dims


def _qparam_shape(block_size, input_size):
    sfr, rdims = _get_reduction_params(block_size, input_size)
    return [s for d, s in enumerate(sfr) if d not in rdims]


def _check_view(t: torch.Tensor, n: int, what: str):
    # the reference does scale.view(shape_after_reduction); a wrong element count is a RuntimeError there
    if t.numel() != n:
        raise RuntimeError(f"shape '{[n]}' is invalid for input of size {t.numel()} ({what})")


def _storage_dtype(dtype):
    """Sub-byte torch dtypes have no storage of their own here; codes live in uint8."""
    return torch.uint8 if dtype not in _cabi.DTYPE_CODE else dtype


def choose_qparams_affine(
    input: torch.Tensor,
    mapping_type: MappingType,
    block_size: Tuple[int, ...],
    target_dtype: torch.dtype,
    quant_min: Optional[int] = None,
    quant_max: Optional[int] = None,
    eps: Optional[float] = None,
    scale_dtype: Optional[torch.dtype] = None,
    zero_point_dtype: Optional[torch.dtype] = None,
    preserve_zero: bool = True,
    zero_point_domain=ZeroPointDomain.INT,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """torchao/quantization/quant_primitives.py:278-367"""
    quant_min, quant_max = _get_and_check_qmin_qmax(target_dtype, quant_min, quant_max)
    assert mapping_type in [MappingType.SYMMETRIC, MappingType.ASYMMETRIC], f"Unsupported mapping type: {mapping_type}"
    if scale_dtype is None:
        scale_dtype = input.dtype
    if zero_point_dtype is None:
        zero_point_dtype = input.dtype
    assert len(block_size) == input.dim()
    out_shape = _qparam_shape(block_size, input.size())
    if mapping_type == MappingType.SYMMETRIC:
        if not preserve_zero:
            raise ValueError("preserve_zero == False is not supported for symmetric quantization")
        if zero_point_domain != ZeroPointDomain.INT:
            raise ValueError("zero_point_domain != ZeroPointDomain.INT is not supported for symmetric quantization")
    elif not preserve_zero:
        assert zero_point_domain == ZeroPointDomain.FLOAT, "if not preserve_zero, zero_point must be in FLOAT domain"
    _cabi.require_cuda(input)
    x = input.contiguous()
    scale = torch.empty(out_shape, dtype=scale_dtype, device=x.device)
    zero_point = torch.empty(out_shape, dtype=zero_point_dtype, device=x.device)
    if x.numel() == 0:
        return scale, zero_point
    with torch.cuda.device(x.device):
        rc = _cabi.lib().ao_choose_qparams_affine(
            _cabi.ptr(x), _cabi.dtype_code(x.dtype), x.dim(), _cabi.i64_array(x.shape), _cabi.i64_array(block_size),
            mapping_type.value, quant_min, quant_max, 0 if eps is None else 1, 0.0 if eps is None else float(eps),
            _cabi.dtype_code(scale_dtype), _cabi.dtype_code(zero_point_dtype), 1 if preserve_zero else 0,
            zero_point_domain.value, _cabi.ptr(scale), _cabi.ptr(zero_point), _cabi.stream_ptr(x.device))
    _cabi.check(rc, "choose_qparams_affine")
    return scale, zero_point


def quantize_affine(
    input: torch.Tensor,
    block_size: Tuple[int, ...],
    scale: torch.Tensor,
    zero_point: Optional[torch.Tensor],
    output_dtype: torch.dtype,
    quant_min: Optional[int] = None,
    quant_max: Optional[int] = None,
    zero_point_domain: ZeroPointDomain = ZeroPointDomain.INT,
):
    """torchao/quantization/quant_primitives.py:134-206"""
    assert input.dtype in [torch.float32, torch.float16, torch.bfloat16], f"Unsupported input dtype: {input.dtype}"
    quant_min, quant_max = _get_and_check_qmin_qmax(output_dtype, quant_min, quant_max)
    nblocks = 1
    for s in _qparam_shape(block_size, input.size()):
        nblocks *= s
    _check_view(scale, nblocks, "scale")
    if zero_point is not None:
        _check_view(zero_point, nblocks, "zero_point")
    else:
        raise TypeError("quantize_affine needs a zero_point tensor")
    assert zero_point_domain in (ZeroPointDomain.INT, ZeroPointDomain.FLOAT)
    _cabi.require_cuda(input, scale, zero_point)
    x = input.contiguous()
    scale = scale.contiguous()
    zero_point = zero_point.contiguous()
    store_dtype = _storage_dtype(output_dtype)
    out = torch.empty(x.shape, dtype=store_dtype, device=x.device)
    if x.numel() == 0:
        return out
    with torch.cuda.device(x.device):
        rc = _cabi.lib().ao_quantize_affine(
            _cabi.ptr(x), _cabi.dtype_code(x.dtype), x.dim(), _cabi.i64_array(x.shape), _cabi.i64_array(block_size),
            _cabi.ptr(scale), _cabi.dtype_code(scale.dtype), _cabi.ptr(zero_point), _cabi.dtype_code(zero_point.dtype),
            quant_min, quant_max, zero_point_domain.value, _cabi.ptr(out), _cabi.dtype_code(store_dtype),
            _cabi.stream_ptr(x.device))
    _cabi.check(rc, "quantize_affine")
    return out


def dequantize_affine(
    input: torch.Tensor,
    block_size: Tuple[int, ...],
    scale: torch.Tensor,
    zero_point: Optional[torch.Tensor],
    input_dtype: torch.dtype,
    quant_min: Optional[int] = None,
    quant_max: Optional[int] = None,
    zero_point_domain: ZeroPointDomain = ZeroPointDomain.INT,
    *,
    output_dtype: torch.dtype = torch.float32,
):
    """torchao/quantization/quant_primitives.py:208-276"""
    assert input.dtype == _storage_dtype(input_dtype), f"Expected: {input_dtype}, got: {input.dtype}"
    assert output_dtype in [torch.float32, torch.float16, torch.bfloat16], f"Unsupported output dtype: {output_dtype}"
    quant_min, quant_max = _get_and_check_qmin_qmax(input_dtype, quant_min, quant_max)
    nblocks = 1
    for s in _qparam_shape(block_size, input.size()):
        nblocks *= s
    _check_view(scale, nblocks, "scale")
    if zero_point is not None:
        _check_view(zero_point, nblocks, "zero_point")
    assert zero_point_domain in (ZeroPointDomain.INT, ZeroPointDomain.FLOAT), (
        f"Unexpected zero point domain: {zero_point_domain}")
    _cabi.require_cuda(input, scale, zero_point)
    q = input.contiguous()
    scale = scale.contiguous()
    zero_point = None if zero_point is None else zero_point.contiguous()
    out = torch.empty(q.shape, dtype=output_dtype, device=q.device)
    if q.numel() == 0:
        return out
    with torch.cuda.device(q.device):
        rc = _cabi.lib().ao_dequantize_affine(
            _cabi.ptr(q), _cabi.dtype_code(q.dtype), q.dim(), _cabi.i64_array(q.shape), _cabi.i64_array(block_size),
            _cabi.ptr(scale), _cabi.dtype_code(scale.dtype), _cabi.ptr(zero_point),
            _cabi.dtype_code(zero_point.dtype) if zero_point is not None else _cabi.I32, quant_min, quant_max,
            zero_point_domain.value, _cabi.ptr(out), _cabi.dtype_code(output_dtype), _cabi.stream_ptr(q.device))
    _cabi.check(rc, "dequantize_affine")
    return out
