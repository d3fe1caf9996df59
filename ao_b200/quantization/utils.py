"""tinygemm-flavoured group-wise helpers — torchao/quantization/utils.py:50-53, 274-392."""
import torch

from .. import _cabi
from .quant_primitives import (
    MappingType,
    ZeroPointDomain,
    choose_qparams_affine,
    dequantize_affine,
    quantize_affine,
)

__all__ = [
    "compute_error",
    "get_groupwise_affine_qparams",
    "pack_tinygemm_scales_and_zeros",
    "unpack_tinygemm_scales_and_zeros",
    "groupwise_affine_quantize_tensor_from_qparams",
    "groupwise_affine_dequantize_tensor_from_qparams",
    "groupwise_affine_quantize_tensor",
    "groupwise_affine_dequantize_tensor",
]


def compute_error(x, y):
    """SQNR in dB (torchao/quantization/utils.py:50-53)."""
    Ps = torch.linalg.norm(x)
    Pn = torch.linalg.norm(x - y)
    return 20 * torch.log10(Ps / Pn)


def guard_dtype_size(tensor_arg, arg_name, dtype=None, size=None):
    if dtype is not None and tensor_arg.dtype != dtype:
        raise ValueError(f"Expected Tensor argument {arg_name} to have dtype {dtype}, but got {tensor_arg.dtype} instead.")
    if size is not None and tensor_arg.size() != size:
        raise ValueError(f"Expected Tensor argument {arg_name} to have size {size}, but got {tensor_arg.size()} instead.")


def get_groupwise_affine_qparams(w, n_bit=4, groupsize=128, dtype=torch.bfloat16):
    """torchao/quantization/utils.py:274-307"""
    if groupsize > w.shape[-1]:
        groupsize = w.shape[-1]
    assert groupsize > 1
    assert w.shape[-1] % groupsize == 0
    assert w.dim() == 2
    assert n_bit <= 8, f"only n_bit smaller than 8 is supported, got: {n_bit}"
    scale, zero_point = choose_qparams_affine(
        w, MappingType.ASYMMETRIC, (1, groupsize), torch.int32, 0, 2**n_bit - 1, 1e-6, scale_dtype=dtype,
        zero_point_dtype=dtype, preserve_zero=False, zero_point_domain=ZeroPointDomain.FLOAT)
    return scale.to(dtype=dtype).reshape(w.shape[0], -1), zero_point.to(dtype=dtype).reshape(w.shape[0], -1)


def pack_tinygemm_scales_and_zeros(scales, zeros):
    """[N][G] scales and zeros -> [G][N][2] (torchao/quantization/utils.py:310-323)."""
    guard_dtype_size(scales, "scales", dtype=torch.bfloat16, size=zeros.size())
    guard_dtype_size(zeros, "zeros", dtype=torch.bfloat16)
    _cabi.require_cuda(scales, zeros)
    assert scales.dim() == 2
    scales, zeros = scales.contiguous(), zeros.contiguous()
    N, G = scales.shape
    out = torch.empty((G, N, 2), dtype=torch.bfloat16, device=scales.device)
    if out.numel():
        with torch.cuda.device(scales.device):
            rc = _cabi.lib().ao_pack_tinygemm_scales_and_zeros(_cabi.ptr(scales), _cabi.ptr(zeros), N, G, _cabi.ptr(out),
                                                               _cabi.stream_ptr(scales.device))
        _cabi.check(rc, "pack_tinygemm_scales_and_zeros")
    return out


def unpack_tinygemm_scales_and_zeros(scales_and_zeros):
    """[G][N][2] -> ([N][G][1], [N][G][1]) like torch.split(x.transpose(0, 1), 1, 2) in the reference
    (torchao/quantization/utils.py:326-328), as contiguous tensors."""
    assert len(scales_and_zeros.shape) == 3 and scales_and_zeros.shape[2] == 2
    _cabi.require_cuda(scales_and_zeros)
    sz = scales_and_zeros.contiguous()
    G, N, _ = sz.shape
    scale = torch.empty((N, G, 1), dtype=sz.dtype, device=sz.device)
    zero = torch.empty((N, G, 1), dtype=sz.dtype, device=sz.device)
    assert sz.dtype == torch.bfloat16
    if sz.numel():
        with torch.cuda.device(sz.device):
            rc = _cabi.lib().ao_unpack_tinygemm_scales_and_zeros(_cabi.ptr(sz), N, G, _cabi.ptr(scale), _cabi.ptr(zero),
                                                                 _cabi.stream_ptr(sz.device))
        _cabi.check(rc, "unpack_tinygemm_scales_and_zeros")
    return scale, zero


def groupwise_affine_quantize_tensor_from_qparams(w, scales, zeros, n_bit=4, groupsize=128):
    """torchao/quantization/utils.py:331-351"""
    assert groupsize > 1
    if groupsize > w.shape[-1] and scales.shape[-1] == 1:
        groupsize = w.shape[-1]
    assert w.shape[-1] % groupsize == 0
    assert w.dim() == 2
    return quantize_affine(w, (1, groupsize), scales, zeros, torch.int32, 0, 2**n_bit - 1,
                           zero_point_domain=ZeroPointDomain.FLOAT)


def groupwise_affine_dequantize_tensor_from_qparams(w_int4x8, scales, zeros, n_bit=4, groupsize=128):
    """torchao/quantization/utils.py:353-371"""
    assert groupsize > 1
    if groupsize > w_int4x8.shape[-1] and scales.shape[-1] == 1:
        groupsize = w_int4x8.shape[-1]
    assert w_int4x8.shape[-1] % groupsize == 0
    assert w_int4x8.dim() == 2
    return dequantize_affine(w_int4x8, (1, groupsize), scales, zeros, torch.int32, 0, 2**n_bit - 1,
                             zero_point_domain=ZeroPointDomain.FLOAT, output_dtype=scales.dtype)


def groupwise_affine_quantize_tensor(w, n_bit=4, groupsize=128, dtype=torch.bfloat16):
    """torchao/quantization/utils.py:374-380"""
    scales, zeros = get_groupwise_affine_qparams(w, n_bit, groupsize, dtype)
    w_int4x8 = groupwise_affine_quantize_tensor_from_qparams(w, scales, zeros, n_bit, groupsize)
    scales_and_zeros = pack_tinygemm_scales_and_zeros(scales, zeros)
    return w_int4x8, scales_and_zeros


def groupwise_affine_dequantize_tensor(w_int4x8, scales_and_zeros, n_bit=4, groupsize=128):
    """torchao/quantization/utils.py:383-392"""
    scales, zeros = unpack_tinygemm_scales_and_zeros(scales_and_zeros)
    return groupwise_affine_dequantize_tensor_from_qparams(w_int4x8, scales, zeros, n_bit, groupsize)
