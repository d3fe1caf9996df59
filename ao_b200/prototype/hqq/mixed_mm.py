"""HQQ-style int4 operand layout — torchao/prototype/hqq/mixed_mm.py:13-33."""
import torch

from ... import _cabi


def pack_2xint4(t):
    """Rows 2r and 2r+1 of an int8/uint8 matrix go to the low / high nibble of row r
    (torchao/prototype/hqq/mixed_mm.py:13-33).  The HQQ path applies it to W_q.T, giving [K/2][N]."""
    assert t.dtype == torch.int8 or t.dtype == torch.uint8
    _cabi.require_cuda(t)
    assert t.dim() == 2 and t.shape[0] % 2 == 0
    tc = t.contiguous()
    R, C = tc.shape
    out = torch.empty((R // 2, C), dtype=t.dtype, device=t.device)
    if out.numel():
        with torch.cuda.device(t.device):
            rc = _cabi.lib().ao_pack_2xint4(_cabi.ptr(tc), R, C, _cabi.ptr(out), _cabi.stream_ptr(t.device))
        _cabi.check(rc, "pack_2xint4")
    return out


def pack_hqq_from_rowmajor(codes):
    """codes uint8 [N][K] -> [K/2][N], i.e. pack_2xint4(codes.T) without materialising the transpose."""
    assert codes.dtype == torch.uint8 and codes.dim() == 2 and codes.shape[1] % 2 == 0
    _cabi.require_cuda(codes)
    c = codes.contiguous()
    N, K = c.shape
    out = torch.empty((K // 2, N), dtype=torch.uint8, device=c.device)
    if out.numel():
        with torch.cuda.device(c.device):
            rc = _cabi.lib().ao_pack_hqq_int4_from_rowmajor(_cabi.ptr(c), N, K, _cabi.ptr(out),
                                                           _cabi.stream_ptr(c.device))
        _cabi.check(rc, "pack_hqq_from_rowmajor")
    return out
