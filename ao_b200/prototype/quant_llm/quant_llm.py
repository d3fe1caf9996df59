"""FP6-LLM (e3m2) weight-only path — torchao/prototype/quant_llm/quant_llm.py on CUDA kernels.

Packing, scaling and unpacking keep the reference's names and byte-exact layouts; the per-shape
split-K table of the reference (quant_llm.py:212-345) is not needed because the kernel picks its own
K split, so `splitK` arguments are accepted and ignored.
"""
from typing import Tuple

import torch
from torch import Tensor

from ... import _cabi


_FORMATS = ((3, 2), (2, 3), (2, 2), (3, 1))   # the (ebits, mbits) the reference's linear dispatches


def _check_nbits(nbits: int):
    if nbits not in (5, 6):
        raise NotImplementedError(f"tensor-core packing is built for 5- and 6-bit codes, got {nbits} bits")


def pack_tc_fpx(tensor: Tensor, nbits: int) -> Tensor:
    """uint8 codes [M][N] -> tensor-core pre-packed uint8 [M][N*nbits/8] (quant_llm.py:60-113)."""
    _check_nbits(nbits)
    _cabi.require_cuda(tensor)
    assert tensor.ndim == 2 and tensor.dtype == torch.uint8
    M, N = tensor.shape
    assert (M % 64 == 0) and (N % 64 == 0)
    t = tensor.contiguous()
    out = torch.empty((M, N * nbits // 8), dtype=torch.uint8, device=t.device)
    with torch.cuda.device(t.device):
        rc = _cabi.lib().ao_pack_tc_fpx(_cabi.ptr(t), M, N, nbits, _cabi.ptr(out), _cabi.stream_ptr(t.device))
    _cabi.check(rc, "pack_tc_fpx")
    return out


def unpack_tc_fpx(tensor: Tensor, nbits: int) -> Tensor:
    """Inverse of pack_tc_fpx (quant_llm.py:134-200)."""
    _check_nbits(nbits)
    assert tensor.ndim == 2 and tensor.dtype == torch.uint8
    _cabi.require_cuda(tensor)
    M = tensor.shape[0]
    N = tensor.shape[1] // nbits * 8
    assert (M % 64 == 0) and (N % 64 == 0)
    t = tensor.contiguous()
    out = torch.empty((M, N), dtype=torch.uint8, device=t.device)
    with torch.cuda.device(t.device):
        rc = _cabi.lib().ao_unpack_tc_fpx(_cabi.ptr(t), M, N, nbits, _cabi.ptr(out), _cabi.stream_ptr(t.device))
    _cabi.check(rc, "unpack_tc_fpx")
    return out


def to_scaled_tc_fpx(tensor: Tensor, ebits: int, mbits: int) -> Tuple[Tensor, Tensor]:
    """Per-row absmax/max_normal scale (fp32 math, fp16 result), ExMy encode, pre-pack
    (quant_llm.py:116-130).  Built for e3m2, e2m3, e2m2 and e3m1."""
    if (ebits, mbits) not in _FORMATS:
        raise NotImplementedError(f"to_scaled_tc_fpx: e{ebits}m{mbits} is not built")
    _cabi.require_cuda(tensor)
    assert tensor.ndim == 2
    M, N = tensor.shape
    assert (M % 64 == 0) and (N % 64 == 0)
    t = tensor.contiguous()
    if t.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        t = t.float()
    packed = torch.empty((M, N * (1 + ebits + mbits) // 8), dtype=torch.uint8, device=t.device)
    scale = torch.empty((M,), dtype=torch.float16, device=t.device)
    scratch = torch.empty((M,), dtype=torch.float32, device=t.device)   # fp32 row scales between the two kernels
    with torch.cuda.device(t.device):
        rc = _cabi.lib().ao_to_scaled_tc_fpx(_cabi.ptr(t), _cabi.dtype_code(t.dtype), M, N, ebits, mbits, _cabi.ptr(packed),
                                             _cabi.ptr(scale), _cabi.ptr(scratch), scratch.numel() * 4,
                                             _cabi.stream_ptr(t.device))
    _cabi.check(rc, "to_scaled_tc_fpx")
    return packed, scale


def from_scaled_tc_fpx(tensor: Tensor, ebits: int, mbits: int, scale=None) -> Tensor:
    """Unpack, decode to fp32 and apply the per-row scale (quant_llm.py:203-208)."""
    if (ebits, mbits) not in _FORMATS:
        raise NotImplementedError(f"from_scaled_tc_fpx: e{ebits}m{mbits} is not built")
    assert tensor.ndim == 2 and tensor.dtype == torch.uint8
    _cabi.require_cuda(tensor, scale)
    M = tensor.shape[0]
    N = tensor.shape[1] // (1 + ebits + mbits) * 8
    assert (M % 64 == 0) and (N % 64 == 0)
    t = tensor.contiguous()
    s = None if scale is None else scale.to(torch.float16).contiguous()
    out = torch.empty((M, N), dtype=torch.float32, device=t.device)
    with torch.cuda.device(t.device):
        rc = _cabi.lib().ao_from_scaled_tc_fpx(_cabi.ptr(t), M, N, ebits, mbits, _cabi.ptr(s), _cabi.ptr(out),
                                               _cabi.stream_ptr(t.device))
    _cabi.check(rc, "from_scaled_tc_fpx")
    return out


from torch.utils._python_dispatch import return_and_correct_aliasing  # noqa: E402

from ...dtypes.utils import _ATEN_OP_OR_TORCH_FN_TABLE, _implements  # noqa: E402


class QuantLlmLinearWeight(Tensor):
    """FPx weight of a linear layer: pre-packed codes `fpx_data` (uint8 [out][in*nbits/8]) and one fp16 `scale`
    per output channel (torchao/prototype/quant_llm/quant_llm.py:348-416)."""
    implements = classmethod(_implements)

    @staticmethod
    def __new__(cls, fpx_data: Tensor, scale: Tensor, ebits: int, mbits: int):
        assert fpx_data.ndim == 2
        assert fpx_data.dtype == torch.uint8
        shape = (fpx_data.shape[0], fpx_data.shape[1] // (1 + ebits + mbits) * 8)
        return Tensor._make_wrapper_subclass(cls, shape, device=fpx_data.device, requires_grad=False)

    def __init__(self, fpx_data: Tensor, scale: Tensor, ebits: int, mbits: int):
        self.fpx_data = fpx_data
        self.scale = scale
        self.ebits = ebits
        self.mbits = mbits

    def __tensor_flatten__(self):
        return ["fpx_data", "scale"], [self.ebits, self.mbits]

    @classmethod
    def __tensor_unflatten__(cls, tensor_data_dict, tensor_attributes, outer_size=None, outer_stride=None):
        return cls(tensor_data_dict["fpx_data"], tensor_data_dict["scale"], *tensor_attributes)

    @classmethod
    def from_float(cls, input_float: Tensor, ebits: int, mbits: int):
        fpx_data, scale = to_scaled_tc_fpx(input_float, ebits, mbits)
        return cls(fpx_data, scale, ebits, mbits)

    def dequantize(self, output_dtype=None):
        output_dtype = output_dtype or torch.get_default_dtype()
        return from_scaled_tc_fpx(self.fpx_data, self.ebits, self.mbits, self.scale).to(output_dtype)

    def __repr__(self):
        dtype = f"fp{1 + self.ebits + self.mbits}_e{self.ebits}m{self.mbits}"
        return (f"{self.__class__.__name__}(dtype={dtype}, shape={self.shape}, "
                f"device={self.device}, requires_grad={self.requires_grad})")

    def _apply_fn_to_data(self, fn):
        return self.__class__(fn(self.fpx_data), fn(self.scale), self.ebits, self.mbits)

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        kwargs = {} if kwargs is None else kwargs
        if func in _ATEN_OP_OR_TORCH_FN_TABLE[cls]:
            return _ATEN_OP_OR_TORCH_FN_TABLE[cls][func](*args, **kwargs)
        with torch._C.DisableTorchFunctionSubclass():
            return func(*args, **kwargs)

    @classmethod
    def __torch_dispatch__(cls, func, types, args, kwargs):
        if func in _ATEN_OP_OR_TORCH_FN_TABLE[cls]:
            return _ATEN_OP_OR_TORCH_FN_TABLE[cls][func](func, *args, **kwargs)
        raise NotImplementedError(f"{cls.__name__} dispatch: attempting to run {func}, this is not supported")


@QuantLlmLinearWeight.implements(torch.nn.functional.linear)
def _(*args, **kwargs):
    """quant_llm.py:419-445.  The reference looks splitK up in a per-shape table; the kernel here chooses
    its own K split, so the argument passed on is only a placeholder."""
    from ... import _torch_ops  # noqa: F401  (torch.ops.torchao.quant_llm_linear: the operator a traced graph shows)

    act = args[0]
    weight = args[1]
    bias = args[2] if len(args) >= 3 else None
    assert isinstance(weight, QuantLlmLinearWeight)
    out_dim, in_dim = weight.shape
    act_reshaped = act.reshape(-1, in_dim).half()
    if (bias is not None and type(bias) in (Tensor, torch.nn.Parameter) and bias.dtype is torch.float16 and bias.dim() == 1
            and bias.is_cuda and not torch.compiler.is_compiling()):
        # eager calls: the add happens in the kernel's stores (same bits as the separate add below)
        from ... import ops
        out = ops.quant_llm_linear_bias(weight.ebits, weight.mbits, act_reshaped, weight.fpx_data, weight.scale, bias.detach())
        return out.view(*act.shape[:-1], out_dim).to(act.dtype)
    out = torch.ops.torchao.quant_llm_linear(weight.ebits, weight.mbits, act_reshaped, weight.fpx_data, weight.scale, 1)
    if bias is not None:
        out += bias
    return out.view(*act.shape[:-1], out_dim).to(act.dtype)


@QuantLlmLinearWeight.implements(torch.ops.aten.detach.default)
def _(func, *args, **kwargs):
    return return_and_correct_aliasing(func, args, kwargs, args[0]._apply_fn_to_data(torch.detach))


def quant_llm_fpx_weight_only(ebits: int, mbits: int):
    """Layers whose in_features is not a multiple of 64 or out_features not a multiple of 256 stay as they are
    (quant_llm.py:453-459)."""
    def apply_quant_llm(weight: Tensor) -> Tensor:
        out_dim, in_dim = weight.shape
        if (in_dim % 64 != 0) or (out_dim % 256 != 0):
            return weight
        return QuantLlmLinearWeight.from_float(weight, ebits, mbits)

    return apply_quant_llm


def fp6_llm_weight_only():
    return quant_llm_fpx_weight_only(3, 2)
