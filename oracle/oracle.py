"""numpy/ctypes front end of the CPU oracle (``oracle.c``).

TEST INFRASTRUCTURE ONLY: this module is the checker for the CUDA kernels and
the timed CPU baseline.  Only the tests, the smoke entry and the benchmark's
CPU-baseline leg may import it; the product package never does.

Floating tensors are passed as float32 numpy arrays whose values are exactly
representable in their logical dtype (one of ``F32``, ``F16``, ``BF16``); the C
side rounds every arithmetic step to the dtype eager PyTorch would give it.
n-d ``block_size`` granularities are canonicalised here to ``[nblocks][block]``
rows exactly as ``_get_reduction_params`` does in the reference
(torchao/quantization/quant_primitives.py:95-131).
"""
import ctypes
import os
import subprocess

import numpy as np

F32, F16, BF16, I32, I64, I8, U8, I16 = range(8)
SYMMETRIC, ASYMMETRIC = 0, 1
ZP_INT, ZP_FLOAT = 0, 1

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "liboracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile oracle.c into oracle/_build/liboracle.so (needs gcc and make)."""
    src = os.path.join(_HERE, "oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "--no-print-directory"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.orc_round_bf16.restype = ctypes.c_float
        _lib.orc_round_bf16.argtypes = [ctypes.c_float]
        _lib.orc_round_f16.restype = ctypes.c_float
        _lib.orc_round_f16.argtypes = [ctypes.c_float]
    return _lib


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def _i64(v):
    return ctypes.c_int64(int(v))


def num_threads() -> int:
    return int(lib().orc_num_threads())


def set_num_threads(n: int) -> int:
    """Sets the thread count of the OpenMP loops (0 or None: every core this process may run on); returns it."""
    import os
    if not n:
        try:
            n = len(os.sched_getaffinity(0))
        except AttributeError:
            n = os.cpu_count() or 1
    lib().orc_set_num_threads(int(n))
    return num_threads()


# ----------------------------------------------------------------------------
# block canonicalisation (quant_primitives.py:95-131)
# ----------------------------------------------------------------------------
def reduction_params(block_size, input_size):
    assert len(block_size) == len(input_size)
    shape_for_reduction, reduction_dims = [], []
    cur = 0
    for b, s in zip(block_size, input_size):
        if b != s and b > 1:
            assert s % b == 0, f"size {s} not divisible by block {b}"
            shape_for_reduction += [s // b, b]
            reduction_dims.append(cur + 1)
            cur += 2
        else:
            shape_for_reduction.append(s)
            if b != 1:
                reduction_dims.append(cur)
            cur += 1
    return shape_for_reduction, reduction_dims


class _Blocks:
    """View of an n-d array as [nblocks][block_elems] rows and back."""

    def __init__(self, shape, block_size):
        self.shape = tuple(shape)
        self.sfr, self.rdims = reduction_params(block_size, shape)
        self.kept = [d for d in range(len(self.sfr)) if d not in self.rdims]
        self.perm = self.kept + self.rdims
        self.kept_shape = [self.sfr[d] for d in self.kept]
        self.nb = int(np.prod(self.kept_shape)) if self.kept_shape else 1
        self.be = int(np.prod([self.sfr[d] for d in self.rdims])) if self.rdims else 1

    def rows(self, x):
        return np.ascontiguousarray(x.reshape(self.sfr).transpose(self.perm).reshape(self.nb, self.be))

    def unrows(self, r):
        permuted_shape = [self.sfr[d] for d in self.perm]
        inv = np.argsort(self.perm)
        return np.ascontiguousarray(r.reshape(permuted_shape).transpose(inv)).reshape(self.shape)


def choose_qparams_affine(x, in_dt, mapping, block_size, qmin, qmax, eps=None, scale_dt=None,
                          zp_dt=None, preserve_zero=True, zp_domain=ZP_INT):
    """Returns (scale, zero_point) as float32 arrays shaped like the reference's outputs."""
    x = np.asarray(x, dtype=np.float32)
    scale_dt = in_dt if scale_dt is None else scale_dt
    zp_dt = in_dt if zp_dt is None else zp_dt
    blk = _Blocks(x.shape, block_size)
    rows = blk.rows(x)
    scale = np.empty(blk.nb, np.float32)
    zp = np.empty(blk.nb, np.float32)
    rc = lib().orc_choose_qparams(_p(rows), _i64(blk.nb), _i64(blk.be), in_dt, mapping, _i64(qmin),
                                  _i64(qmax), 0 if eps is None else 1,
                                  ctypes.c_double(0.0 if eps is None else eps), scale_dt, zp_dt,
                                  1 if preserve_zero else 0, zp_domain, _p(scale), _p(zp))
    if rc == -1:
        raise ValueError("preserve_zero == False is not supported for symmetric quantization")
    if rc == -2:
        raise ValueError("zero_point_domain != ZeroPointDomain.INT is not supported for symmetric quantization")
    if rc == -3:
        raise AssertionError("if not preserve_zero, zero_point must be in FLOAT domain")
    return scale.reshape(blk.kept_shape), zp.reshape(blk.kept_shape)


def quantize_affine(x, in_dt, block_size, scale, scale_dt, zp, zp_dt, qmin, qmax, zp_domain=ZP_INT):
    x = np.asarray(x, dtype=np.float32)
    blk = _Blocks(x.shape, block_size)
    rows = blk.rows(x)
    s = np.ascontiguousarray(np.asarray(scale, np.float32).reshape(blk.nb))
    z = np.ascontiguousarray(np.asarray(zp, np.float32).reshape(blk.nb))
    out = np.empty((blk.nb, blk.be), np.int32)
    lib().orc_quantize(_p(rows), _i64(blk.nb), _i64(blk.be), in_dt, _p(s), scale_dt, _p(z), zp_dt,
                       _i64(qmin), _i64(qmax), zp_domain, _p(out))
    return blk.unrows(out)


def dequantize_affine(q, block_size, scale, scale_dt, zp, zp_dt, qmin, qmax, zp_domain=ZP_INT,
                      out_dt=F32):
    q = np.asarray(q, dtype=np.int32)
    blk = _Blocks(q.shape, block_size)
    rows = blk.rows(q)
    s = np.ascontiguousarray(np.asarray(scale, np.float32).reshape(blk.nb))
    z = None if zp is None else np.ascontiguousarray(np.asarray(zp, np.float32).reshape(blk.nb))
    out = np.empty((blk.nb, blk.be), np.float32)
    lib().orc_dequantize(_p(rows), _i64(blk.nb), _i64(blk.be), _p(s), scale_dt,
                         None if z is None else _p(z), zp_dt, _i64(qmin), _i64(qmax), zp_domain,
                         out_dt, _p(out))
    return blk.unrows(out)


# ----------------------------------------------------------------------------
# packers
# ----------------------------------------------------------------------------
def pack_tinygemm_scales_and_zeros(scale_bits, zero_bits):
    """scale_bits / zero_bits: uint16 (bf16 bit patterns) [N][G] -> uint16 [G][N][2]."""
    s = np.ascontiguousarray(scale_bits, np.uint16)
    z = np.ascontiguousarray(zero_bits, np.uint16)
    N, G = s.shape
    out = np.empty((G, N, 2), np.uint16)
    lib().orc_pack_scales_and_zeros(_p(s), _p(z), _i64(N), _i64(G), _p(out))
    return out


def pack_tinygemm(codes, inner_k_tiles=8):
    codes = np.ascontiguousarray(codes, np.int32)
    N, K = codes.shape
    out = np.empty((N // 8, K // (inner_k_tiles * 16), 32, inner_k_tiles // 2), np.int32)
    rc = lib().orc_pack_tinygemm(_p(codes), _i64(N), _i64(K), int(inner_k_tiles), _p(out))
    if rc:
        raise ValueError(f"pack_tinygemm: bad shape/inner_k_tiles (rc={rc})")
    return out


def unpack_tinygemm(packed):
    packed = np.ascontiguousarray(packed, np.int32)
    NT, KO, _, half = packed.shape
    ikt = half * 2
    N, K = NT * 8, KO * ikt * 16
    out = np.empty((N, K), np.int32)
    rc = lib().orc_unpack_tinygemm(_p(packed), _i64(N), _i64(K), int(ikt), _p(out))
    if rc:
        raise ValueError(f"unpack_tinygemm: rc={rc}")
    return out


def pack_2xint4(t):
    t = np.ascontiguousarray(t, np.uint8)
    R, C = t.shape
    out = np.empty((R // 2, C), np.uint8)
    lib().orc_pack_2xint4(_p(t), _i64(R), _i64(C), _p(out))
    return out


# ----------------------------------------------------------------------------
# fp6 / fpx
# ----------------------------------------------------------------------------
def f32_to_fpx_unpacked(x, ebits, mbits):
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty(x.shape, np.uint8)
    lib().orc_f32_to_fpx(_p(x), _i64(x.size), int(ebits), int(mbits), _p(out))
    return out


def fpx_unpacked_to_f32(c, ebits, mbits):
    c = np.ascontiguousarray(c, np.uint8)
    out = np.empty(c.shape, np.float32)
    lib().orc_fpx_to_f32(_p(c), _i64(c.size), int(ebits), int(mbits), _p(out))
    return out


def pack_tc_fp6(codes):
    codes = np.ascontiguousarray(codes, np.uint8)
    M, N = codes.shape
    out = np.empty(M * N * 3 // 4, np.uint8)
    rc = lib().orc_pack_tc_fp6(_p(codes), _i64(M), _i64(N), _p(out))
    if rc:
        raise AssertionError("pack_tc_fp6 needs M % 64 == 0 and N % 64 == 0")
    return out.reshape(M, -1)


def unpack_tc_fp6(packed):
    packed = np.ascontiguousarray(packed, np.uint8)
    M = packed.shape[0]
    N = packed.shape[1] // 3 * 4
    out = np.empty((M, N), np.uint8)
    rc = lib().orc_unpack_tc_fp6(_p(packed), _i64(M), _i64(N), _p(out))
    if rc:
        raise AssertionError("unpack_tc_fp6 needs M % 64 == 0 and N % 64 == 0")
    return out


def to_scaled_tc_fp6(w_f32, ebits=3, mbits=2, return_codes=False):
    """-> (packed uint8 [M][N*6/8], scale fp16 bits uint16 [M]) (+ codes [M][N])."""
    w = np.ascontiguousarray(w_f32, np.float32)
    M, N = w.shape
    packed = np.empty(M * N * 3 // 4, np.uint8)
    scale = np.empty(M, np.uint16)
    codes = np.empty((M, N), np.uint8)
    rc = lib().orc_to_scaled_tc_fp6(_p(w), _i64(M), _i64(N), int(ebits), int(mbits), _p(packed),
                                    _p(scale), _p(codes))
    if rc:
        raise AssertionError("to_scaled_tc_fp6: bad shape or format")
    if return_codes:
        return packed.reshape(M, -1), scale, codes
    return packed.reshape(M, -1), scale


def from_scaled_tc_fp6(packed, scale_bits=None, ebits=3, mbits=2):
    packed = np.ascontiguousarray(packed, np.uint8)
    M = packed.shape[0]
    N = packed.shape[1] // 3 * 4
    out = np.empty((M, N), np.float32)
    s = None if scale_bits is None else np.ascontiguousarray(scale_bits, np.uint16)
    rc = lib().orc_from_scaled_tc_fp6(_p(packed), _i64(M), _i64(N), int(ebits), int(mbits),
                                      None if s is None else _p(s), _p(out))
    if rc:
        raise AssertionError("from_scaled_tc_fp6: bad shape")
    return out


# ----------------------------------------------------------------------------
# generic tensor-core pre-packing for any bit width (numpy restatement of
# torchao/prototype/quant_llm/quant_llm.py:15-86): the code's bits are split into 1-, 2- and 4-bit planes
# (highest bits first); every plane is laid out so that word t of each 128-byte piece is warp lane t's data
# ----------------------------------------------------------------------------
_BIT_ORDER = {
    1: [1, 5, 9, 13, 17, 21, 25, 29, 3, 7, 11, 15, 19, 23, 27, 31, 0, 4, 8, 12, 16, 20, 24, 28, 2, 6, 10, 14, 18, 22, 26, 30],
    2: [1, 5, 9, 13, 3, 7, 11, 15, 0, 4, 8, 12, 2, 6, 10, 14],
    4: [1, 5, 3, 7, 0, 4, 2, 6],
}


def _pack_bits(x, n_bits):
    """8 // n_bits consecutive elements of the last axis -> one byte, first element in the highest bits."""
    per = 8 // n_bits
    out = np.zeros(x.shape[:-1] + (x.shape[-1] // per,), np.uint8)
    for i in range(per):
        out |= (x[..., i::per].astype(np.uint8) << (8 - (i + 1) * n_bits)).astype(np.uint8)
    return out


def _unpack_bits(x, n_bits):
    per = 8 // n_bits
    parts = [(x >> (8 - (i + 1) * n_bits)) & ((1 << n_bits) - 1) for i in range(per)]
    return np.stack(parts, axis=-1).reshape(x.shape[:-1] + (x.shape[-1] * per,))


def _bit_interleave(x, n_bits, undo=False):
    x = x.reshape(-1, 4)[:, ::-1]                       # bytes of a 32-bit word, most significant first
    x = _unpack_bits(x, n_bits).reshape(-1, 4 * (8 // n_bits))
    order = _BIT_ORDER[n_bits]
    if undo:
        order = [order.index(i) for i in range(len(order))]
    x = _pack_bits(x[:, order], n_bits)
    return x.reshape(-1, 4)[:, ::-1].reshape(-1)


def pack_tc_fpx(codes, nbits):
    """codes uint8 [M][N] (one nbits-wide code per byte) -> uint8 [M][N * nbits / 8]."""
    t = np.ascontiguousarray(codes, np.uint8)
    M, N = t.shape
    assert M % 64 == 0 and N % 64 == 0
    t = t.reshape(M // 64, 4, 2, 8, N // 16, 2, 8).transpose(0, 4, 1, 5, 2, 3, 6).reshape(-1, 32, 2)
    t = t.transpose(1, 0, 2).reshape(-1)
    used, planes = 0, []
    for y in (1, 2, 4):
        if nbits & y:
            plane = (t >> (nbits - used - y)) & ((1 << y) - 1)
            plane = _pack_bits(plane, y)
            plane = plane.reshape(32, -1, 4).transpose(1, 0, 2)[:, :, ::-1].reshape(-1)
            planes.append(_bit_interleave(np.ascontiguousarray(plane), y))
            used += y
    return np.concatenate(planes).reshape(M, -1)


def unpack_tc_fpx(packed, nbits):
    """Inverse of pack_tc_fpx."""
    p = np.ascontiguousarray(packed, np.uint8)
    M = p.shape[0]
    size = p.size
    N = p.shape[1] // nbits * 8
    flat = p.reshape(-1)
    offset, used = 0, 0
    total = None
    for y in (1, 2, 4):
        if nbits & y:
            n = size * y // nbits
            plane = _bit_interleave(flat[offset:offset + n], y, undo=True)
            plane = plane.reshape(-1, 32, 4)[:, :, ::-1].transpose(1, 0, 2).reshape(-1)
            vals = _unpack_bits(np.ascontiguousarray(plane), y).astype(np.uint8) << (nbits - used - y)
            total = vals if total is None else (total | vals)
            offset += n
            used += y
    t = total.reshape(32, -1, 2).transpose(1, 0, 2).reshape(M // 64, N // 16, 4, 2, 2, 8, 8)
    return np.ascontiguousarray(t.transpose(0, 2, 4, 5, 1, 3, 6)).reshape(M, N)


def to_scaled_tc_fpx(w_f32, ebits, mbits):
    """to_scaled_tc_fpx for any ExMy the generic packer takes (quant_llm.py:116-130): per-row scale =
    max(absmax, 1e-12) / max_normal in fp32, codes of w / scale, pre-packed.  -> (packed, fp16 scale bits)."""
    w = np.ascontiguousarray(w_f32, np.float32)
    bias = (1 << (ebits - 1)) - 1
    max_normal = np.float32(2.0 ** (((1 << ebits) - 1) - bias) * (((1 << (mbits + 1)) - 1) / (1 << mbits)))
    amax = np.maximum(np.abs(w).max(axis=1), np.float32(1e-12)).astype(np.float32)
    scale = (amax / max_normal).astype(np.float32)
    codes = f32_to_fpx_unpacked((w / scale[:, None]).astype(np.float32), ebits, mbits)
    return pack_tc_fpx(codes, 1 + ebits + mbits), scale.astype(np.float16).view(np.uint16)


def from_scaled_tc_fpx(packed, scale_bits, ebits, mbits):
    codes = unpack_tc_fpx(packed, 1 + ebits + mbits)
    v = fpx_unpacked_to_f32(codes, ebits, mbits)
    if scale_bits is not None:
        v = v * f16_bits_to_f32(np.asarray(scale_bits, np.uint16))[:, None]
    return v.astype(np.float32)


def hqq_quants_to_torch_quants(wq, scale_bits, zero_bits, dt):
    """torchao/prototype/hqq/hqq_tinygemm_linear.py:173-208 for 4 bits: wq uint8 [groups][g], scale / zero bit
    patterns [groups] of dtype dt (BF16 or F16) -> (int32 codes [groups][g], new_zero bit patterns [groups]);
    every operation rounded to dt."""
    if dt == BF16:
        to_f, rnd = bf16_bits_to_f32, lambda v: bf16_bits_to_f32(f32_to_bf16_bits(v))
        to_bits = f32_to_bf16_bits
    else:
        to_f, rnd = f16_bits_to_f32, lambda v: np.asarray(v, np.float32).astype(np.float16).astype(np.float32)
        to_bits = lambda v: np.asarray(v, np.float32).astype(np.float16).view(np.uint16)
    s = to_f(np.asarray(scale_bits).reshape(-1, 1)).astype(np.float32)
    z = to_f(np.asarray(zero_bits).reshape(-1, 1)).astype(np.float32)
    w = np.asarray(wq, np.float32)
    s8 = rnd(s * np.float32(8))
    nz = rnd(s8 - rnd(z * s))
    min_val = rnd(nz - s8)
    wr = rnd(rnd(w - z) * s)
    t = rnd(rnd(wr - min_val) / s)
    q = np.clip(np.rint(t), 0, 15).astype(np.int32)
    return q, to_bits(nz.reshape(-1))


# ----------------------------------------------------------------------------
# GEMM oracles
# ----------------------------------------------------------------------------
def linear_f32(x, w):
    """y = x @ w.T with float32 operands, double accumulation -> float32 [M][N]."""
    x = np.ascontiguousarray(x, np.float32)
    w = np.ascontiguousarray(w, np.float32)
    M, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K
    y = np.empty((M, N), np.float32)
    lib().orc_linear_f32(_p(x), _p(w), _i64(M), _i64(N), _i64(K), _p(y))
    return y


def int4_linear_dequant_then_matmul(x, codes_u8, scale, zero, group_size, wbuf=None):
    """The reference's CPU route for an int4 AffineQuantizedTensor: dequantise the whole
    weight to bf16, then a dense matmul.  All floats are bf16 values carried in float32."""
    x = np.ascontiguousarray(x, np.float32)
    codes_u8 = np.ascontiguousarray(codes_u8, np.uint8)
    scale = np.ascontiguousarray(scale, np.float32)
    zero = np.ascontiguousarray(zero, np.float32)
    M, K = x.shape
    N = codes_u8.shape[0]
    if wbuf is None:
        wbuf = np.empty((N, K), np.float32)
    y = np.empty((M, N), np.float32)
    lib().orc_int4_linear_dequant_then_matmul(_p(x), _p(codes_u8), _p(scale), _p(zero), _i64(M),
                                              _i64(N), _i64(K), _i64(group_size), _p(wbuf), _p(y))
    return y


# ----------------------------------------------------------------------------
# bf16 / fp16 bit helpers (numpy has no bf16)
# ----------------------------------------------------------------------------
def bf16_bits_to_f32(bits):
    return (np.asarray(bits, np.uint16).astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(x):
    """Exact for values already representable in bf16; rounds to nearest even otherwise."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    r = u + 0x7FFF + ((u >> 16) & 1)
    return (r >> 16).astype(np.uint16)


def f16_bits_to_f32(bits):
    return np.asarray(bits, np.uint16).view(np.float16).astype(np.float32)
