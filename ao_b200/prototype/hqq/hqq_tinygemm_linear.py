"""HQQ -> tinygemm conversion, after HQQLinearTorchWeightOnlyInt4 (torchao/prototype/hqq/hqq_tinygemm_linear.py).

HQQ's own quantiser (hqq.core.quantize, a third-party package) is not part of this library: these functions start from
its outputs (W_q, meta["scale"], meta["zero"]), which is all the reference's class uses of it."""
import torch

from ... import _cabi, ops
from ...quantization.utils import pack_tinygemm_scales_and_zeros


def hqq_quants_to_torch_quants(W_q, scales, zeros, shape, nbits=4, compute_dtype=torch.bfloat16):
    """(W_q - zeros) * scales  ->  (W_q_torch int32 [shape], scales [N][K/g], new_zeros [N][K/g]) with
    W = (W_q_torch - 8) * scales + new_zeros  (hqq_tinygemm_linear.py:173-208).

    W_q: codes, one per element, reshaped here to [groups][group_size]; scales, zeros: one per group."""
    if nbits != 4:
        raise NotImplementedError("only 4-bit HQQ weights")
    _cabi.require_cuda(W_q, scales, zeros)
    groups = scales.numel()
    torch._check(zeros.numel() == groups and W_q.numel() % max(groups, 1) == 0, lambda: "scales / zeros do not match W_q")
    g = W_q.numel() // groups
    wq = W_q.to(torch.uint8).contiguous()
    s = scales.to(compute_dtype).contiguous()
    z = zeros.to(compute_dtype).contiguous()
    q = torch.empty(wq.numel(), dtype=torch.int32, device=wq.device)
    nz = torch.empty(groups, dtype=compute_dtype, device=wq.device)
    with torch.cuda.device(wq.device):
        rc = _cabi.lib().ao_hqq_quants_to_tinygemm(_cabi.ptr(wq), _cabi.ptr(s), _cabi.ptr(z), _cabi.dtype_code(compute_dtype),
                                                   groups, g, _cabi.ptr(q), _cabi.ptr(nz), _cabi.stream_ptr(wq.device))
    _cabi.check(rc, "hqq_quants_to_torch_quants")
    return q.reshape(shape), s.reshape(shape[0], -1), nz.reshape(shape[0], -1)


def hqq_to_tinygemm_weight(W_q, scales, zeros, shape, inner_k_tiles=8):
    """process_hqq_quants (hqq_tinygemm_linear.py:147-171): the tensor_core_tiled weight and its scale_and_zero."""
    q, s, nz = hqq_quants_to_torch_quants(W_q, scales, zeros, shape, compute_dtype=torch.bfloat16)
    return ops.convert_weight_to_int4pack(q, inner_k_tiles), pack_tinygemm_scales_and_zeros(s, nz)
