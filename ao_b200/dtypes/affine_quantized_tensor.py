"""AffineQuantizedTensor and its layouts — torchao/dtypes/affine_quantized_tensor.py, with the quantize,
pack and linear work done by the sm_100a kernels.

Differences from the reference that are deliberate:
  * a kernel error raises; only "no specialised kernel for this combination" (NotImplementedError) takes the
    reference's dequantize + dense route (affine_quantized_tensor.py:683-690 catches everything);
  * TensorCoreTiledAQTLayout.get_plain unpacks with a kernel (the reference's version cannot run,
    affine_quantized_tensor.py:509-537);
  * the activation is not padded and copied on every call: the linear kernel treats the columns beyond
    the activation's width as zero (affine_quantized_tensor.py:625-627).
"""
from typing import Optional, Tuple

import torch
from torch.utils._python_dispatch import return_and_correct_aliasing

from .. import _cabi, ops
from ..quantization.quant_primitives import (
    MappingType,
    ZeroPointDomain,
    choose_qparams_affine,
    dequantize_affine,
    quantize_affine,
)
from ..quantization.utils import pack_tinygemm_scales_and_zeros, unpack_tinygemm_scales_and_zeros
from ..utils import find_multiple
from .utils import (
    _ATEN_OP_OR_TORCH_FN_TABLE,
    _get_layout_tensor_constructor,
    _implements,
    _register_layout_cls,
)

aten = torch.ops.aten


def _aqt_is_int8(aqt):
    """int8 quantized (the reference's unparenthesised and/or chain, :27-33, made explicit)."""
    return (aqt.layout_tensor.dtype == torch.int8 and (aqt.quant_min is None or aqt.quant_min == -128)
            and (aqt.quant_max is None or aqt.quant_max == 127))


def _aqt_is_uint4(aqt):
    """uint4 quantized, stored in int32 (:42-49)."""
    return (aqt.layout_tensor.dtype == torch.int32 and (aqt.quant_min is None or aqt.quant_min == 0)
            and (aqt.quant_max is None or aqt.quant_max == 15))


class AQTLayout(torch.Tensor):
    """Base class of the layout tensors (:51-82)."""
    extended_layout: Optional[str] = None

    def get_plain(self) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        pass

    @classmethod
    def from_plain(cls, int_data: torch.Tensor, scale: torch.Tensor, zero_point: torch.Tensor):
        pass

    def _get_to_kwargs(self, *args, **kwargs):
        device, dtype, _, memory_format = torch._C._nn._parse_to(*args, **kwargs)
        device = self.device if device is None else device
        dtype = self.dtype if dtype is None else dtype
        memory_format = memory_format if memory_format is not None else torch.preserve_format
        return {"device": device, "dtype": dtype, "memory_format": memory_format}


def _is_int4_weight_only_setting(input_float, mapping_type, block_size, target_dtype, quant_min, quant_max, eps,
                                 scale_dtype, zero_point_dtype, preserve_zero, zero_point_domain):
    """The parameter set of int4_weight_only (quant_api.py:372-385) on a bf16 weight: eligible for the fused
    quantize-and-pack kernel."""
    return (input_float.dim() == 2 and input_float.dtype == torch.bfloat16 and input_float.is_cuda
            and mapping_type == MappingType.ASYMMETRIC and len(block_size) == 2 and block_size[0] == 1
            and block_size[1] in (32, 64, 128, 256) and target_dtype == torch.int32 and quant_min == 0
            and quant_max == 15 and eps == 1e-6 and scale_dtype in (None, torch.bfloat16)
            and zero_point_dtype == torch.bfloat16 and not preserve_zero
            and zero_point_domain == ZeroPointDomain.FLOAT)


class AffineQuantizedTensor(torch.Tensor):
    """quantized = float / scale + zero_point, per block (:84-303).

    fields: layout_tensor, block_size, shape, quant_min, quant_max, zero_point_domain, dtype."""

    @staticmethod
    def __new__(cls, layout_tensor, block_size, shape, quant_min=None, quant_max=None,
                zero_point_domain=ZeroPointDomain.INT, dtype=None, strides=None):
        kwargs = {"device": layout_tensor.device, "layout": layout_tensor.layout, "dtype": dtype,
                  "requires_grad": False}
        if strides is not None:
            kwargs["strides"] = strides
        return torch.Tensor._make_wrapper_subclass(cls, shape, **kwargs)  # type: ignore[attr-defined]

    def __init__(self, layout_tensor, block_size, shape, quant_min=None, quant_max=None,
                 zero_point_domain=ZeroPointDomain.INT, dtype=None, strides=None):
        self.layout_tensor = layout_tensor
        self.block_size = block_size
        self.quant_min = quant_min
        self.quant_max = quant_max
        self.zero_point_domain = zero_point_domain

    def __repr__(self):
        inner = getattr(self.layout_tensor, "packed_weight", getattr(self.layout_tensor, "int_data", None))
        data = self.dequantize() if type(inner) is torch.Tensor else f"<{type(self.layout_tensor).__name__} while tracing>"
        return (f"{self.__class__.__name__}(data={data}, shape={self.shape}, "
                f"device={self.device}, dtype={self.dtype}, requires_grad={self.requires_grad})")

    def dequantize(self, output_dtype=None):
        if output_dtype is None:
            output_dtype = self.dtype
        int_data, scale, zero_point = self.layout_tensor.get_plain()
        block_size = self.block_size
        if tuple(int_data.shape) != tuple(self.shape) and len(block_size) == 2:
            # tiled layout: the codes cover the padded shape
            dq = dequantize_affine(int_data, block_size, scale, zero_point, int_data.dtype, self.quant_min,
                                   self.quant_max, self.zero_point_domain, output_dtype=output_dtype)
            return dq[: self.shape[0], : self.shape[1]]
        return dequantize_affine(int_data, block_size, scale, zero_point, int_data.dtype, self.quant_min,
                                 self.quant_max, self.zero_point_domain, output_dtype=output_dtype)

    def __tensor_flatten__(self):
        return ["layout_tensor"], [self.block_size, self.shape, self.quant_min, self.quant_max,
                                   self.zero_point_domain, self.dtype]

    @classmethod
    def __tensor_unflatten__(cls, tensor_data_dict, tensor_attributes, outer_size, outer_stride):
        layout_tensor = tensor_data_dict["layout_tensor"]
        block_size, shape, quant_min, quant_max, zero_point_domain, dtype = tensor_attributes
        return cls(layout_tensor, block_size, shape if outer_size is None else outer_size, quant_min, quant_max,
                   zero_point_domain, dtype=dtype, strides=outer_stride)

    @classmethod
    def from_float(cls, input_float, mapping_type, block_size, target_dtype, quant_min=None, quant_max=None,
                   eps=None, scale_dtype=None, zero_point_dtype=None, preserve_zero=True,
                   zero_point_domain=ZeroPointDomain.INT, extended_layout="plain", inner_k_tiles=None):
        """:184-229.  With the int4_weight_only setting and the tensor_core_tiled layout the weight is
        quantized and packed by one kernel; otherwise choose_qparams_affine / quantize_affine / from_plain."""
        original_shape = input_float.shape
        if extended_layout == "tensor_core_tiled":
            orig_out_features, orig_in_features = input_float.shape
            in_features = find_multiple(orig_in_features, 1024)
            out_features = find_multiple(orig_out_features, 8)
            input_float = torch.nn.functional.pad(
                input_float, (0, in_features - orig_in_features, 0, out_features - orig_out_features))
            if _is_int4_weight_only_setting(input_float, mapping_type, block_size, target_dtype, quant_min, quant_max,
                                            eps, scale_dtype, zero_point_dtype, preserve_zero, zero_point_domain):
                packed, scale_and_zero = ops.int4_quantize_pack(input_float, block_size[1], inner_k_tiles or 8)
                layout_tensor = TensorCoreTiledAQTLayout(packed, scale_and_zero, False)
                return cls(layout_tensor, block_size, original_shape, quant_min, quant_max, zero_point_domain,
                           dtype=input_float.dtype)

        scale, zero_point = choose_qparams_affine(input_float, mapping_type, block_size, target_dtype, quant_min,
                                                  quant_max, eps, scale_dtype, zero_point_dtype, preserve_zero,
                                                  zero_point_domain)
        int_data = quantize_affine(input_float, block_size, scale, zero_point, target_dtype, quant_min, quant_max,
                                   zero_point_domain)
        layout_cls_ctr = get_layout_tensor_constructor(extended_layout)
        if extended_layout == "tensor_core_tiled":
            layout_tensor = layout_cls_ctr(int_data, scale, zero_point, inner_k_tiles)
        else:
            layout_tensor = layout_cls_ctr(int_data, scale, zero_point)
        return cls(layout_tensor, block_size, original_shape, quant_min, quant_max, zero_point_domain,
                   dtype=input_float.dtype)

    @property
    def extended_layout(self) -> str:
        return self.layout_tensor.extended_layout

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        kwargs = {} if kwargs is None else kwargs
        if func in _ATEN_OP_OR_TORCH_FN_TABLE[cls]:
            return _ATEN_OP_OR_TORCH_FN_TABLE[cls][func](*args, **kwargs)
        with torch._C.DisableTorchFunctionSubclass():
            return func(*args, **kwargs)

    def _get_to_kwargs(self, *args, **kwargs):
        device, dtype, _, memory_format = torch._C._nn._parse_to(*args, **kwargs)
        device = self.device if device is None else device
        dtype = self.dtype if dtype is None else dtype
        memory_format = memory_format if memory_format is not None else torch.preserve_format
        return {"device": device, "dtype": dtype, "memory_format": memory_format}

    def to(self, *args, **kwargs):
        kwargs = self._get_to_kwargs(*args, **kwargs)
        return self.__class__(self.layout_tensor.to(kwargs["device"]), self.block_size, self.shape, self.quant_min,
                              self.quant_max, self.zero_point_domain, dtype=kwargs["dtype"])

    def _apply_fn_to_data(self, fn):
        return self.__class__(fn(self.layout_tensor), self.block_size, self.shape, self.quant_min, self.quant_max,
                              self.zero_point_domain, dtype=self.dtype, strides=self.stride())

    @classmethod
    def __torch_dispatch__(cls, func, types, args, kwargs):
        if func in _ATEN_OP_OR_TORCH_FN_TABLE[cls]:
            return _ATEN_OP_OR_TORCH_FN_TABLE[cls][func](func, *args, **kwargs)
        raise NotImplementedError(f"AffineQuantizedTensor dispatch: attempting to run {func}, this is not supported")


def implements(aten_ops_or_torch_fn):
    return _implements(AffineQuantizedTensor, aten_ops_or_torch_fn)


def register_layout_cls(extended_layout: str):
    return _register_layout_cls(AffineQuantizedTensor, extended_layout)


def get_layout_tensor_constructor(extended_layout: str):
    return _get_layout_tensor_constructor(AffineQuantizedTensor, extended_layout)


@register_layout_cls("plain")
class PlainAQTLayout(AQTLayout):
    """int_data, scale, zero_point stored as they are (:314-408)."""

    def __new__(cls, int_data, scale, zero_point):
        kwargs = {"device": int_data.device, "layout": int_data.layout, "dtype": int_data.dtype,
                  "requires_grad": False}
        return torch.Tensor._make_wrapper_subclass(cls, int_data.shape, **kwargs)  # type: ignore[attr-defined]

    def __init__(self, int_data, scale, zero_point):
        self.int_data = int_data
        self.scale = scale
        self.zero_point = zero_point

    def __tensor_flatten__(self):
        return ["int_data", "scale", "zero_point"], []

    @classmethod
    def __tensor_unflatten__(cls, tensor_data_dict, tensor_attributes, outer_size, outer_stride):
        return cls(tensor_data_dict["int_data"], tensor_data_dict["scale"], tensor_data_dict["zero_point"])

    def to(self, *args, **kwargs):
        kwargs = self._get_to_kwargs(*args, **kwargs)
        return self.__class__(self.int_data.to(kwargs["device"]), self.scale.to(kwargs["device"]),
                              self.zero_point.to(kwargs["device"]))

    def _apply_fn_to_data(self, fn):
        return self.__class__(fn(self.int_data), fn(self.scale), fn(self.zero_point))

    @classmethod
    def __torch_dispatch__(cls, func, types, args, kwargs):
        kwargs = {} if kwargs is None else kwargs
        if func is aten.detach.default:
            return return_and_correct_aliasing(func, args, kwargs, args[0]._apply_fn_to_data(torch.detach))
        if func is aten.t.default:
            tensor = args[0]
            new = tensor.__class__(tensor.int_data.view(tensor.shape[::-1]), tensor.scale, tensor.zero_point)
            return return_and_correct_aliasing(func, args, kwargs, new)
        if func is aten.clone.default:
            return return_and_correct_aliasing(func, args, kwargs, args[0]._apply_fn_to_data(torch.clone))
        raise NotImplementedError(f"PlainAQTLayout dispatch: attempting to run {func}, this is not supported")

    __torch_function__ = torch._C._disabled_torch_function_impl

    def get_plain(self):
        return self.int_data, self.scale, self.zero_point

    @classmethod
    def from_plain(cls, int_data, scale, zero_point):
        return cls(int_data, scale, zero_point)


@register_layout_cls("tensor_core_tiled")
class TensorCoreTiledAQTLayout(AQTLayout):
    """int4 only: codes [n][k] as the 4-d int32 tensor [n/8][k/(inner_k_tiles*16)][32][inner_k_tiles/2], scales and
    zeros interleaved as [k/group][n][2] (:410-537)."""

    def __new__(cls, packed_weight, scale_and_zero, transposed):
        kwargs = {"device": packed_weight.device, "layout": packed_weight.layout, "dtype": packed_weight.dtype,
                  "requires_grad": False}
        return torch.Tensor._make_wrapper_subclass(cls, packed_weight.shape, **kwargs)  # type: ignore[attr-defined]

    def __init__(self, packed_weight, scale_and_zero, transposed):
        self.packed_weight = packed_weight
        self.scale_and_zero = scale_and_zero
        self.transposed = False

    def __tensor_flatten__(self):
        return ["packed_weight", "scale_and_zero"], [self.transposed]

    @classmethod
    def __tensor_unflatten__(cls, tensor_data_dict, tensor_attributes, outer_size, outer_stride):
        transposed, = tensor_attributes
        return cls(tensor_data_dict["packed_weight"], tensor_data_dict["scale_and_zero"], transposed)

    @classmethod
    def from_plain(cls, int_data, scale, zero_point, inner_k_tiles=8):
        packed_weight = ops.convert_weight_to_int4pack(int_data.to(torch.int32), inner_k_tiles or 8)
        scale = scale.reshape(int_data.shape[0], -1)
        zero_point = zero_point.reshape(int_data.shape[0], -1)
        scale_and_zero = pack_tinygemm_scales_and_zeros(scale, zero_point)
        return cls(packed_weight, scale_and_zero, False)

    def to(self, *args, **kwargs):
        kwargs = self._get_to_kwargs(*args, **kwargs)
        device = torch.device(kwargs["device"])
        if device.type != "cuda":
            raise ValueError("TensorCoreTiledAQTLayout is only available for cuda device")
        return self.__class__(self.packed_weight.to(device), self.scale_and_zero.to(device), self.transposed)

    def _apply_fn_to_data(self, fn):
        self.packed_weight = fn(self.packed_weight)
        self.scale_and_zero = fn(self.scale_and_zero)
        return self

    def __repr__(self):
        if type(self.packed_weight) is not torch.Tensor:   # fake / functional tensors while tracing: nothing to unpack
            return (f"TensorCoreTiledAQTLayout(packed_weight={tuple(self.packed_weight.shape)}, "
                    f"scale_and_zero={tuple(self.scale_and_zero.shape)})")
        int_data, scale, zero_point = self.get_plain()
        return f"TensorCoreTiledAQTLayout(int_data={int_data}, scale={scale}, zero_point={zero_point})"

    @classmethod
    def __torch_dispatch__(cls, func, types, args, kwargs):
        kwargs = {} if kwargs is None else kwargs
        if func is aten.detach.default:
            return return_and_correct_aliasing(func, args, kwargs, args[0]._apply_fn_to_data(torch.detach))
        if func is aten.t.default:
            args[0].transposed = not args[0].transposed
            return return_and_correct_aliasing(func, args, kwargs, args[0])
        if func is aten.clone.default:
            t = args[0]
            new = t.__class__(t.packed_weight.clone(), t.scale_and_zero.clone(), t.transposed)
            return return_and_correct_aliasing(func, args, kwargs, new)
        raise NotImplementedError(
            f"TensorCoreTiledAQTLayout dispatch: attempting to run {func}, this is not supported")

    __torch_function__ = torch._C._disabled_torch_function_impl

    def get_plain(self):
        """Exact inverse of from_plain: int32 codes [n][k], scale and zero [n][k/group]."""
        int_data = ops.unpack_int4pack(self.packed_weight)
        scale, zero = unpack_tinygemm_scales_and_zeros(self.scale_and_zero)
        return int_data, scale.reshape(scale.shape[:-1]), zero.reshape(zero.shape[:-1])



class _Int4LinearPlan:
    """Everything F.linear needs for one int4 tensor_core_tiled weight, resolved once: raw pointers, sizes, the C
    entry point.  Calling it is the per-token cost of a decode step, so it touches no tensor-subclass attribute
    (each of those goes through __torch_function__) and does no argument validation beyond what changes per call."""

    __slots__ = ("packed", "sz", "group", "ikt", "N", "K", "n_out", "k_in", "device", "dev_index", "fn", "ws_fn",
                 "p_packed", "p_sz", "ws_cache", "static_out", "fn_bias")

    def __init__(self, w):
        lt = w.layout_tensor
        self.packed, self.sz = lt.packed_weight, lt.scale_and_zero
        self.group = int(w.block_size[1])
        self.ikt = int(self.packed.shape[3]) * 2
        self.N = int(self.packed.shape[0]) * 8
        self.K = int(self.packed.shape[1]) * self.ikt * 16
        shape = torch.Tensor.size(w)
        self.n_out, self.k_in = int(shape[0]), int(shape[1])
        self.device = self.packed.device
        self.dev_index = self.device.index
        lib = _cabi.lib()
        self.fn = lib.ao_int4_tinygemm_linear
        self.fn_bias = lib.ao_int4_tinygemm_linear_bias
        self.ws_fn = lib.ao_int4_tinygemm_linear_workspace_bytes
        self.p_packed = self.packed.data_ptr()
        self.p_sz = self.sz.data_ptr()
        self.ws_cache = {}
        self.static_out = None     # {M: output buffer} once use_static_linear_outputs() has switched it on

    def __call__(self, x, bias):
        k_in = self.k_in
        x2 = x.reshape(-1, k_in)
        if x2.stride(1) != 1 or (x2.stride(0) & 1) or (x2.data_ptr() & 3) or (k_in & 1):
            x2 = torch.nn.functional.pad(x2, (0, k_in & 1)).contiguous()
        M = x2.shape[0]
        if self.static_out is None:
            y = torch.empty((M, self.N), dtype=torch.bfloat16, device=self.device)
        else:
            y = self.static_out.get(M)
            if y is None:
                y = self.static_out[M] = torch.empty((M, self.N), dtype=torch.bfloat16, device=self.device)
        if M:
            stream = torch._C._cuda_getCurrentRawStream(self.dev_index)
            ws = _cabi.workspace_for(self.ws_cache, self.ws_fn, (M, self.N, self.K, self.group, self.ikt), self.device, stream)
            # the bias add rides in the kernels' stores when it can (same bits as the separate add below)
            fuse = (bias is not None and self.n_out == self.N and type(bias) in (torch.Tensor, torch.nn.Parameter)
                    and bias.dtype is torch.bfloat16 and bias.is_contiguous() and bias.device == self.device
                    and bias.numel() == self.N)
            if fuse:
                rc = self.fn_bias(x2.data_ptr(), x2.stride(0), x2.shape[1], self.p_packed, self.p_sz, M, self.N, self.K,
                                  self.group, self.ikt, y.data_ptr(), bias.data_ptr(), ws.data_ptr(), ws.numel(), stream)
                bias = None
            else:
                rc = self.fn(x2.data_ptr(), x2.stride(0), x2.shape[1], self.p_packed, self.p_sz, M, self.N, self.K,
                             self.group, self.ikt, y.data_ptr(), ws.data_ptr(), ws.numel(), stream)
            if rc:
                _cabi.check(rc, "int4 weight-only linear")
        if self.n_out != self.N:
            y = y[:, : self.n_out]
        y = y.reshape(*x.shape[:-1], self.n_out)
        if bias is not None:
            y = y + bias if self.static_out is not None else y.add_(bias)
        return y


def use_static_linear_outputs(module: torch.nn.Module, enabled: bool = True, outputs=None) -> None:
    """Makes every int4 tensor_core_tiled linear of `module` write its result into one buffer per batch size that it
    owns, instead of a fresh tensor per call.  A decode loop then allocates nothing per token, and a caller can read
    the result where it lies (e.g. copy it to the host) without an extra device copy.  The price is the aliasing rule
    of CUDA-graph static outputs: the tensor a call returns is overwritten by the layer's next call with the same
    batch size.

    `outputs` (optional): {submodule name: bf16 [M][out_features] contiguous CUDA tensor} - the caller's own buffers
    for those layers and that batch size, e.g. slices of one staging buffer that leaves the device in a single copy."""
    outputs = outputs or {}
    for name, mod in module.named_modules():
        w = getattr(mod, "weight", None)
        if type(w) is AffineQuantizedTensor and w.extended_layout == "tensor_core_tiled" and w.dtype == torch.bfloat16:
            if "_linear_plan" not in w.__dict__:
                w.__dict__["_linear_plan"] = _Int4LinearPlan(w)
            plan = w.__dict__["_linear_plan"]
            plan.static_out = {} if enabled else None
            buf = outputs.get(name)
            if enabled and buf is not None:
                if not (buf.is_cuda and buf.dtype == torch.bfloat16 and buf.dim() == 2 and buf.is_contiguous()
                        and buf.shape[1] == plan.N and buf.device == plan.device):
                    raise ValueError(f"output buffer of {name!r} must be a contiguous bf16 [M][{plan.N}] tensor on {plan.device}")
                plan.static_out[int(buf.shape[0])] = buf


def _dispatcher_ops():
    """torch.ops.torchao, with the compiled operator library loaded."""
    from .. import _torch_ops  # noqa: F401
    return torch.ops.torchao


def _quantized_linear_op(input_tensor, weight_qtensor, bias):
    """Quantized F.linear (:539-671): the int4 tensor_core_tiled branch runs the sm_100a kernels."""
    if isinstance(weight_qtensor, AffineQuantizedTensor):
        if isinstance(input_tensor, AffineQuantizedTensor):
            input_tensor = input_tensor.dequantize()
        if (_aqt_is_uint4(weight_qtensor) and weight_qtensor.dtype == torch.bfloat16
                and len(weight_qtensor.shape) == 2 and weight_qtensor.zero_point_domain == ZeroPointDomain.FLOAT
                and weight_qtensor.extended_layout == "tensor_core_tiled"):
            assert weight_qtensor.block_size[0] == 1, (
                f"Requires groupwise quantization, got block_size: {weight_qtensor.block_size}")
            assert input_tensor.shape[-1] == weight_qtensor.shape[1], (
                f"need input_tensor shape: {input_tensor.shape} final"
                f"dim to match weight_tensor shape: {weight_qtensor.shape} second dim ")
            packed_weight = weight_qtensor.layout_tensor.packed_weight
            scale_and_zero = weight_qtensor.layout_tensor.scale_and_zero
            orig_act_size = input_tensor.size()
            orig_dtype = input_tensor.dtype
            act_mat = input_tensor.reshape(-1, input_tensor.shape[-1]).to(torch.bfloat16)
            groupsize = weight_qtensor.block_size[1]
            # (plain tensors only: under FakeTensor propagation or tracing there are no addresses to cache)
            if (not torch.compiler.is_compiling() and type(weight_qtensor) is AffineQuantizedTensor
                    and type(packed_weight) is torch.Tensor and type(input_tensor) is torch.Tensor
                    and "_linear_plan" not in weight_qtensor.__dict__):
                weight_qtensor.__dict__["_linear_plan"] = _Int4LinearPlan(weight_qtensor)   # later calls skip the checks
            # through the dispatcher (torchao::_weight_int4pack_mm, the twin of the aten operator the reference calls
            # here, :631), so that a traced graph contains the operator; the kernel reads the activation's missing
            # (padded) columns as zero
            y = _dispatcher_ops()._weight_int4pack_mm(act_mat, packed_weight, groupsize, scale_and_zero)
            orig_out_features = weight_qtensor.shape[-2]
            y = y[:, :orig_out_features]
            y = y.reshape(*orig_act_size[:-1], orig_out_features)
            if bias is not None:
                y += bias
            return y.to(orig_dtype)
    raise NotImplementedError("No specialized dispatch found for quantized linear op")


def _dense_route(func, input_tensor, weight_tensor, *rest):
    """No specialised kernel for this combination: dequantize and run the dense operator."""
    if isinstance(input_tensor, AffineQuantizedTensor):
        input_tensor = input_tensor.dequantize()
    if isinstance(weight_tensor, AffineQuantizedTensor):
        weight_tensor = weight_tensor.dequantize()
    return input_tensor, weight_tensor


@implements(torch.nn.functional.linear)
def functional_linear(*args, **kwargs):
    input_tensor, weight_tensor, bias = args[0], args[1], args[2] if len(args) > 2 else kwargs.get("bias")
    # decode fast path: plain bf16 CUDA activation on an int4 tensor_core_tiled weight whose plan is cached
    plan = None
    if not torch.compiler.is_compiling() and type(weight_tensor) is AffineQuantizedTensor:
        plan = weight_tensor.__dict__.get("_linear_plan")
    if plan is not None and type(input_tensor) is torch.Tensor and input_tensor.dtype is torch.bfloat16 and \
            input_tensor.device == plan.device:
        return plan(input_tensor, bias)
    try:
        return _quantized_linear_op(input_tensor, weight_tensor, bias)
    except NotImplementedError:
        input_tensor, weight_tensor = _dense_route(None, input_tensor, weight_tensor)
        return torch.nn.functional.linear(input_tensor, weight_tensor, bias)


@implements([aten.mm.default, aten.addmm.default])
def aten_mm(func, *args, **kwargs):
    if not args[0].is_floating_point():
        raise NotImplementedError(f"{func} is not implemented for non floating point input")
    if func == aten.addmm.default:
        input_tensor, weight_tensor, bias = args[1], args[2], args[0]
        try:
            return _quantized_linear_op(input_tensor, weight_tensor.t(), bias)
        except NotImplementedError:
            input_tensor, weight_tensor = _dense_route(func, input_tensor, weight_tensor)
            return func(bias, input_tensor, weight_tensor)
    input_tensor, weight_tensor = args[0], args[1]
    try:
        return _quantized_linear_op(input_tensor, weight_tensor.t(), None)
    except NotImplementedError:
        input_tensor, weight_tensor = _dense_route(func, input_tensor, weight_tensor)
        return func(input_tensor, weight_tensor)


@implements([aten.detach.default])
def detach(func, *args, **kwargs):
    return return_and_correct_aliasing(func, args, kwargs, args[0]._apply_fn_to_data(torch.detach))


@implements([aten.clone.default])
def clone(func, *args, **kwargs):
    return return_and_correct_aliasing(func, args, kwargs, args[0]._apply_fn_to_data(torch.clone))


@implements([aten._to_copy.default])
def _to_copy(func, *args, **kwargs):
    return return_and_correct_aliasing(func, args, kwargs,
                                       args[0].to(*args[1:], **kwargs)._apply_fn_to_data(torch.clone))


@implements([aten.t.default])
def t(func, *args, **kwargs):
    block_size = args[0].block_size
    assert len(block_size) == 2
    tensor = args[0]
    new = tensor.__class__(tensor.layout_tensor.t(), (block_size[1], block_size[0]), tensor.shape[::-1],
                           tensor.quant_min, tensor.quant_max, tensor.zero_point_domain, dtype=tensor.dtype,
                           strides=tensor.stride())
    return return_and_correct_aliasing(func, args, kwargs, new)


to_affine_quantized = AffineQuantizedTensor.from_float
