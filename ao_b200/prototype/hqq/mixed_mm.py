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


def mixed_mm(a, b, scales, zeros, group_size, transposed=False, acc_dtype=None, input_precision="ieee",
             fp8_fast_accum=False, kernel_type="compute_bound", BLOCK_M=None, BLOCK_N=None, BLOCK_K=None):
    """Fused int4 dequant GEMM, the reference's triton_mixed_mm (torchao/prototype/hqq/mixed_mm.py:36-173):
    c[M][N] = a[M][K] @ ((unpack(b) - zeros) * scales), fp32 accumulation, c in a's dtype.

    a: bf16 / fp16 [M][K];  b: uint8 [K/2][N] from pack_2xint4;  scales, zeros: [K/group_size][N] in a's dtype
    (any strides: a transposed view of an [N][K/group_size] tensor is accepted, as the reference's tests pass it).
    The tuning arguments of the Triton version (acc_dtype, input_precision, fp8_fast_accum, kernel_type, BLOCK_*)
    are accepted and ignored: the tcgen05 kernel picks its own tiles.  transposed=True is the backward form
    (M x N) x (K x N) -> (M x K): a is [M][N] and the reduction runs along N."""
    _cabi.require_cuda(a, b, scales, zeros)
    assert b.dtype == torch.int8 or b.dtype == torch.uint8, "b must be int8 or uint8"
    assert a.dim() == 2 and b.dim() == 2 and scales.ndim == 2
    if not transposed:
        assert a.shape[1] == b.shape[0] * 2, "incompatible dimensions"
    else:
        assert a.shape[1] == b.shape[1], "transpose requires (M x N) x (K x N), where reduction dim is N"
    assert scales.dtype == a.dtype
    assert scales.shape == zeros.shape
    assert zeros.dtype == a.dtype
    torch._check(a.dtype in (torch.bfloat16, torch.float16), lambda: "mixed_mm: a must be bfloat16 or float16")
    if transposed:
        return _mixed_mm_transposed(a, b, scales, zeros, group_size)
    M, K = a.shape
    N = b.shape[1]
    torch._check(scales.shape == (K // group_size, N),
                 lambda: f"scales must be [K/group_size][N] = {(K // group_size, N)}, got {tuple(scales.shape)}")
    if a.stride(1) != 1 or a.stride(0) % 8 != 0 or a.data_ptr() % 16 != 0:
        a = a.contiguous()
    b = b.contiguous()
    scales = scales.contiguous()
    zeros = zeros.contiguous()
    c = torch.empty((M, N), device=a.device, dtype=a.dtype)
    if M == 0:
        return c
    lib = _cabi.lib()
    nbytes = lib.ao_hqq_int4_linear_workspace_bytes(M, N, K, group_size)
    torch._check(nbytes > 0, lambda: f"mixed_mm: unsupported shape M={M} N={N} K={K} group_size={group_size}")
    with torch.cuda.device(a.device):
        ws = _cabi.workspace(nbytes, a.device)
        rc = lib.ao_hqq_int4_linear(_cabi.ptr(a), _cabi.dtype_code(a.dtype), a.stride(0), _cabi.ptr(b), _cabi.ptr(scales),
                                    _cabi.ptr(zeros), M, N, K, group_size, _cabi.ptr(c), _cabi.ptr(ws), ws.numel(),
                                    _cabi.stream_ptr(a.device))
    _cabi.check(rc, "mixed_mm")
    return c


def _mixed_mm_transposed(a, b, scales, zeros, group_size):
    M, N = a.shape
    K = b.shape[0] * 2
    torch._check(scales.shape == (K // group_size, N),
                 lambda: f"scales must be [K/group_size][N] = {(K // group_size, N)}, got {tuple(scales.shape)}")
    if a.stride(1) != 1 or a.stride(0) % 8 != 0 or a.data_ptr() % 16 != 0:
        a = a.contiguous()
    b, scales, zeros = b.contiguous(), scales.contiguous(), zeros.contiguous()
    c = torch.empty((M, K), device=a.device, dtype=a.dtype)
    if M == 0:
        return c
    lib = _cabi.lib()
    nbytes = lib.ao_hqq_int4_linear_transposed_workspace_bytes(M, N, K, group_size)
    torch._check(nbytes > 0, lambda: f"mixed_mm(transposed): unsupported shape M={M} N={N} K={K} group_size={group_size}")
    with torch.cuda.device(a.device):
        ws = _cabi.workspace(nbytes, a.device)
        rc = lib.ao_hqq_int4_linear_transposed(_cabi.ptr(a), _cabi.dtype_code(a.dtype), a.stride(0), _cabi.ptr(b),
                                               _cabi.ptr(scales), _cabi.ptr(zeros), M, N, K, group_size, _cabi.ptr(c),
                                               _cabi.ptr(ws), ws.numel(), _cabi.stream_ptr(a.device))
    _cabi.check(rc, "mixed_mm(transposed)")
    return c


triton_mixed_mm = mixed_mm  # the reference's name for this operator
