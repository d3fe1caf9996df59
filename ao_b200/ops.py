"""Operator layer: thin wrappers that allocate outputs with torch and call the C ABI.

Covers the operators the reference reaches through the PyTorch dispatcher on this path:
  * aten::_convert_weight_to_int4pack / aten::_weight_int4pack_mm (PyTorch's tinygemm ops, called at
    torchao/dtypes/affine_quantized_tensor.py:461, 631) -> convert_weight_to_int4pack, weight_int4pack_mm
  * torchao::quant_llm_linear (torchao/ops.py:15-55) -> quant_llm_linear / fp6_llm_linear
  * the fp6 pre-packer (torchao/prototype/quant_llm/quant_llm.py:90-130) -> prepack_fp6_weight
CUDA tensors only; errors surface as exceptions, never as a silent dense fallback.
"""
import torch
from torch import Tensor

from . import _cabi


def _stream(t):
    return _cabi.stream_ptr(t.device)


# ---------------------------------------------------------------------------------------------
# int4 tensor_core_tiled ("tinygemm") operators
# ---------------------------------------------------------------------------------------------
def convert_weight_to_int4pack(int_data: Tensor, inner_k_tiles: int = 8) -> Tensor:
    """int32 codes [N][K] (values 0..15) -> int32 [N/8][K/(inner_k_tiles*16)][32][inner_k_tiles/2]."""
    _cabi.require_cuda(int_data)
    torch._check(int_data.dim() == 2, lambda: "int_data must be 2-D [n][k]")
    torch._check(inner_k_tiles in (2, 4, 8), lambda: "innerKTiles must be 2, 4, or 8")
    codes = int_data.to(torch.int32).contiguous()
    N, K = codes.shape
    torch._check(N % 8 == 0, lambda: f"expect N to be a multiple of 8, got {N}")
    torch._check(K % (inner_k_tiles * 16) == 0, lambda: f"expect K to be a multiple of {inner_k_tiles * 16}, got {K}")
    out = torch.empty((N // 8, K // (inner_k_tiles * 16), 32, inner_k_tiles // 2), dtype=torch.int32,
                      device=codes.device)
    with torch.cuda.device(codes.device):
        rc = _cabi.lib().ao_pack_tinygemm_int4(_cabi.ptr(codes), N, K, inner_k_tiles, _cabi.ptr(out), _stream(codes))
    _cabi.check(rc, "convert_weight_to_int4pack")
    return out


def unpack_int4pack(packed: Tensor) -> Tensor:
    """Inverse of convert_weight_to_int4pack: int32 codes [N][K]."""
    _cabi.require_cuda(packed)
    torch._check(packed.dim() == 4 and packed.shape[2] == 32 and packed.dtype == torch.int32,
                 lambda: "expected an int32 [N/8][K/(ikt*16)][32][ikt/2] tensor")
    packed = packed.contiguous()
    ikt = packed.shape[3] * 2
    N, K = packed.shape[0] * 8, packed.shape[1] * ikt * 16
    out = torch.empty((N, K), dtype=torch.int32, device=packed.device)
    with torch.cuda.device(packed.device):
        rc = _cabi.lib().ao_unpack_tinygemm_int4(_cabi.ptr(packed), N, K, ikt, _cabi.ptr(out), _stream(packed))
    _cabi.check(rc, "unpack_int4pack")
    return out


def weight_int4pack_mm(x: Tensor, packed: Tensor, group_size: int, scale_and_zero: Tensor, x_cols=None, *,
                       out: Tensor = None, workspace: Tensor = None, decode_kernel: bool = False) -> Tensor:
    """y[M][N] = x[M][K] @ dequant(W)^T for a tensor_core_tiled weight; bf16 in, bf16 out.

    x may have fewer columns than the (padded) weight: the missing ones count as zero.
    `out` (bf16 [M][N], contiguous) and `workspace` (uint8, zero-filled once, see int4_workspace_bytes) let a
    caller that replays the call in a CUDA graph keep every buffer it touches fixed.
    `decode_kernel=True` (M <= 16) runs the decode GEMV whatever the batch size, i.e. the kernel the peer-memory
    exchange path uses (weight_int4pack_mm_gather): its results then match that path bit for bit; by default batches
    of 5 rows and more (2 and more on long reductions) go to the tcgen05 kernel, whose fp32 sums are taken in another
    order."""
    _cabi.require_cuda(x, packed, scale_and_zero)
    torch._check(x.dim() == 2 and x.dtype == torch.bfloat16, lambda: "x must be a 2-D bfloat16 tensor")
    torch._check(packed.dim() == 4 and packed.dtype == torch.int32 and packed.shape[2] == 32,
                 lambda: "packed weight must be int32 [N/8][K/(ikt*16)][32][ikt/2]")
    torch._check(scale_and_zero.dim() == 3 and scale_and_zero.shape[2] == 2 and scale_and_zero.dtype == torch.bfloat16,
                 lambda: "scale_and_zero must be bfloat16 [K/group][N][2]")
    ikt = packed.shape[3] * 2
    N, K = packed.shape[0] * 8, packed.shape[1] * ikt * 16
    M = x.shape[0]
    torch._check(x.shape[1] <= K, lambda: f"x has {x.shape[1]} columns, the weight only {K}")
    torch._check(scale_and_zero.shape[0] == K // group_size and scale_and_zero.shape[1] == N,
                 lambda: f"scale_and_zero shape {tuple(scale_and_zero.shape)} does not match K/group={K // group_size}, N={N}")
    if x.stride(1) != 1 or x.stride(0) % 2 != 0 or x.data_ptr() % 4 != 0 or x.shape[1] % 2 != 0:
        x = torch.nn.functional.pad(x, (0, x.shape[1] % 2)).contiguous()
    packed = packed.contiguous()
    scale_and_zero = scale_and_zero.contiguous()
    if out is None:
        y = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    else:
        torch._check(out.shape == (M, N) and out.dtype == torch.bfloat16 and out.is_contiguous() and out.device == x.device,
                     lambda: "out must be a contiguous bfloat16 [M][N] tensor on x's device")
        y = out
    if M == 0:
        return y
    lib = _cabi.lib()
    torch._check(not decode_kernel or M <= 16, lambda: f"the decode kernel takes at most 16 rows, got {M}")
    ws_fn, fn = ((lib.ao_int4_gemv_workspace_bytes, lib.ao_int4_gemv) if decode_kernel else
                 (lib.ao_int4_tinygemm_linear_workspace_bytes, lib.ao_int4_tinygemm_linear))
    nbytes = ws_fn(M, N, K, group_size, ikt)
    torch._check(nbytes > 0, lambda: f"unsupported int4 linear shape M={M} N={N} K={K} group={group_size}")
    with torch.cuda.device(x.device):
        if workspace is None:
            ws = _cabi.workspace(nbytes, x.device)
        else:
            torch._check(workspace.dtype == torch.uint8 and workspace.numel() >= nbytes and workspace.device == x.device,
                         lambda: f"workspace must be a uint8 tensor of at least {nbytes} bytes on x's device")
            ws = workspace
        rc = fn(_cabi.ptr(x), x.stride(0), x.shape[1], _cabi.ptr(packed), _cabi.ptr(scale_and_zero), M, N, K, group_size,
                ikt, _cabi.ptr(y), _cabi.ptr(ws), ws.numel(), _stream(x))
    _cabi.check(rc, "weight_int4pack_mm")
    return y


def gather_slot_bytes(world: int, M: int, N: int) -> int:
    """Payload bytes one call site of weight_int4pack_mm_gather needs (counters, output [world][M][N], landing area)."""
    from .comm import PeerExchange
    return PeerExchange.site_bytes(world, M, N)


def weight_int4pack_mm_gather(x: Tensor, packed: Tensor, group_size: int, scale_and_zero: Tensor, exchange,
                              slot_offset_bytes: int = 0, workspace: Tensor = None, wait: bool = True, site=None) -> Tensor:
    """Row-sharded weight_int4pack_mm with the output exchange fused into the kernel's epilogue.

    Uses the call site at `slot_offset_bytes` of the exchange's payload (ao_b200.comm.PeerExchange; gather_slot_bytes
    bytes), or `site` (PeerExchange.reserve).  Every CTA of the GEMV stores its rows into all peers' landing areas as
    it finishes; with wait=True a small second kernel collects the peers' rows, and the returned view
    [world][M][N_local] is complete when that kernel completes.  With wait=False only this rank's own block is
    written: call gather_wait(exchange, [sites]) later in the stream, before the same site is used again.  The view
    is overwritten by the next call of the site.  Every rank must make the same calls in the same order; M <= 8."""
    _cabi.require_cuda(x, packed, scale_and_zero)
    torch._check(x.dim() == 2 and x.dtype == torch.bfloat16 and x.stride(1) == 1, lambda: "x must be 2-D bfloat16")
    ikt = packed.shape[3] * 2
    N, K = packed.shape[0] * 8, packed.shape[1] * ikt * 16
    M = x.shape[0]
    world, rank = exchange.world, exchange.rank
    st = site if site is not None else exchange.site(slot_offset_bytes, M, N)
    torch._check(st.M == M and st.N == N, lambda: "call site was reserved for a different shape")
    lib = _cabi.lib()
    nbytes = lib.ao_int4_gemv_workspace_bytes(M, N, K, group_size, ikt)
    torch._check(nbytes > 0, lambda: f"unsupported shape M={M} N={N} K={K} group={group_size}")
    fn = lib.ao_int4_gemv_gather if wait else lib.ao_int4_gemv_push
    with torch.cuda.device(x.device):
        ws = _cabi.workspace(nbytes, x.device) if workspace is None else workspace
        rc = fn(_cabi.ptr(x), x.stride(0), x.shape[1], _cabi.ptr(packed), _cabi.ptr(scale_and_zero), M, N, K, group_size, ikt,
                world, rank, st.peer_landing, st.y_ptr, st.state, _cabi.ptr(ws), ws.numel(), _stream(x))
    _cabi.check(rc, "weight_int4pack_mm_gather")
    return st.y


def gather_exchange(exchange, sites, push: bool = True, workspace: Tensor = None) -> None:
    """All-gather of the given call sites (at most 8 layers) in one small kernel.  push=True: every rank's own block
    site.y[rank] (written there by weight_int4pack_mm(..., out=site.y[rank])) is sent to all peers first; push=False:
    the rows were already sent by weight_int4pack_mm_gather(..., wait=False).  When the kernel completes, every
    site's gathered output site.y [world][M][N] is complete on this GPU."""
    import ctypes
    n, world = len(sites), exchange.world
    torch._check(1 <= n <= 8, lambda: "gather_exchange takes 1 to 8 call sites")
    landing = (ctypes.c_void_p * (n * world))(*[p for s in sites for p in s.peer_landing])
    arr = ctypes.c_void_p * n
    ys = arr(*[s.y_ptr for s in sites])
    states = arr(*[s.state for s in sites])
    Ms, Ns = _cabi.i64_array([s.M for s in sites]), _cabi.i64_array([s.N for s in sites])
    dev = exchange.device
    with torch.cuda.device(dev):
        ws = _cabi.workspace(256, dev) if workspace is None else workspace
        rc = _cabi.lib().ao_gather_exchange(n, landing, ys, states, Ms, Ns, world, exchange.rank, 1 if push else 0,
                                            _cabi.ptr(ws), _cabi.stream_ptr(dev))
    _cabi.check(rc, "gather_exchange")


def gather_wait(exchange, sites, workspace: Tensor = None) -> None:
    """The receiving half alone, for call sites whose rows were pushed by the GEMV epilogue (wait=False)."""
    gather_exchange(exchange, sites, push=False, workspace=workspace)


def int4_workspace_bytes(M: int, N: int, K: int, group_size: int, inner_k_tiles: int = 8) -> int:
    """Bytes of zero-initialised scratch weight_int4pack_mm needs for this shape (0: unsupported shape)."""
    return int(_cabi.lib().ao_int4_tinygemm_linear_workspace_bytes(M, N, K, group_size, inner_k_tiles))


def int4_quantize_pack(weight: Tensor, group_size: int, inner_k_tiles: int = 8):
    """bf16 W [N][K] -> (tensor_core_tiled int32 weight, scale_and_zero bf16 [K/g][N][2]) in one pass."""
    _cabi.require_cuda(weight)
    torch._check(weight.dim() == 2 and weight.dtype == torch.bfloat16, lambda: "weight must be 2-D bfloat16")
    w = weight.contiguous()
    N, K = w.shape
    packed = torch.empty((N // 8, K // (inner_k_tiles * 16), 32, inner_k_tiles // 2), dtype=torch.int32, device=w.device)
    sz = torch.empty((K // group_size, N, 2), dtype=torch.bfloat16, device=w.device)
    with torch.cuda.device(w.device):
        rc = _cabi.lib().ao_int4_quantize_pack_tinygemm(_cabi.ptr(w), N, K, group_size, inner_k_tiles, _cabi.ptr(packed),
                                                        _cabi.ptr(sz), _stream(w))
    _cabi.check(rc, "int4_quantize_pack")
    return packed, sz


def int4_groupwise_quantize(weight: Tensor, group_size: int, want_codes=torch.int32):
    """bf16 W [N][K] -> (scale bf16 [N][K/g], zero bf16 [N][K/g], codes [N][K] int32 or uint8)."""
    _cabi.require_cuda(weight)
    torch._check(weight.dim() == 2 and weight.dtype == torch.bfloat16, lambda: "weight must be 2-D bfloat16")
    w = weight.contiguous()
    N, K = w.shape
    scale = torch.empty((N, K // group_size), dtype=torch.bfloat16, device=w.device)
    zero = torch.empty_like(scale)
    codes = torch.empty((N, K), dtype=want_codes, device=w.device)
    i32 = _cabi.ptr(codes) if want_codes == torch.int32 else None
    u8 = _cabi.ptr(codes) if want_codes == torch.uint8 else None
    with torch.cuda.device(w.device):
        rc = _cabi.lib().ao_int4_groupwise_quantize(_cabi.ptr(w), N, K, group_size, _cabi.ptr(scale), _cabi.ptr(zero),
                                                    i32, u8, _stream(w))
    _cabi.check(rc, "int4_groupwise_quantize")
    return scale, zero, codes


# ---------------------------------------------------------------------------------------------
# fp6 (e3m2) operators
# ---------------------------------------------------------------------------------------------
def prepack_fp6_weight(codes: Tensor) -> Tensor:
    """One e3m2 code per byte, uint8 [N][K] -> tensor-core pre-packed uint8 [N][K*6/8]
    (pack_tc_fpx(codes, 6), torchao/prototype/quant_llm/quant_llm.py:90-113)."""
    _cabi.require_cuda(codes)
    assert codes.ndim == 2 and codes.dtype == torch.uint8
    M, N = codes.shape
    assert (M % 64 == 0) and (N % 64 == 0)
    codes = codes.contiguous()
    out = torch.empty((M, N * 6 // 8), dtype=torch.uint8, device=codes.device)
    with torch.cuda.device(codes.device):
        rc = _cabi.lib().ao_pack_tc_fp6(_cabi.ptr(codes), M, N, _cabi.ptr(out), _stream(codes))
    _cabi.check(rc, "prepack_fp6_weight")
    return out


def quant_llm_linear(EXPONENT: int, MANTISSA: int, _in_feats: Tensor, _weights: Tensor, _scales: Tensor,
                     splitK: int = 1) -> Tensor:
    """Quant-LLM linear layer A @ W.T (torchao/ops.py:15-55).  _in_feats fp16 [BS][IC], _weights packed FPx uint8
    [OC][IC/8*nbits], _scales fp16 [OC] -> fp16 [BS][OC].  Formats: e3m2, e2m3 (fp6), e2m2, e3m1 (fp5); `splitK` is accepted and ignored (the
    kernel chooses its own K split)."""
    return _quant_llm_linear(EXPONENT, MANTISSA, _in_feats, _weights, _scales, None)


def quant_llm_linear_bias(EXPONENT: int, MANTISSA: int, _in_feats: Tensor, _weights: Tensor, _scales: Tensor,
                          bias: Tensor) -> Tensor:
    """quant_llm_linear followed by `out += bias` (the linear dispatch of QuantLlmLinearWeight,
    torchao/prototype/quant_llm/quant_llm.py:433-445) in one kernel: the add happens in the kernel's stores, on the
    fp16-rounded product, so the bits are those of the separate add.  bias fp16 [OC]."""
    torch._check(bias.dim() == 1 and bias.dtype is torch.float16 and bias.shape[0] == _weights.shape[0],
                 lambda: f"bias must be FP16 [OC], got {bias.dtype} {tuple(bias.shape)}")
    return _quant_llm_linear(EXPONENT, MANTISSA, _in_feats, _weights, _scales, bias)


def _quant_llm_linear(EXPONENT, MANTISSA, _in_feats, _weights, _scales, bias):
    torch._check(_in_feats.dim() == 2, lambda: f"input should be a 2d tensor, got {_in_feats.dim()}D")
    torch._check(_in_feats.dtype is torch.float16, lambda: f"weight must be FP16, got {_in_feats.dtype}")
    torch._check(_weights.dim() == 2, lambda: f"weight should be a 2d tensor, got {_weights.dim()}D")
    torch._check(_weights.dtype is torch.uint8, lambda: f"weight must be UINT8, got {_weights.dtype}")
    torch._check(_scales.dim() == 1, lambda: f"scale should be a 2d tensor, got {_scales.dim()}D")
    torch._check(_scales.dtype is torch.float16, lambda: f"scale must be FP16, got {_scales.dtype}")
    BS, IC = _in_feats.shape
    OC, _ = _weights.shape
    N_BITS = 1 + EXPONENT + MANTISSA
    torch._check(IC // 8 * N_BITS == _weights.shape[1], lambda: "Dimensions mismatched")
    torch._check(OC == _scales.shape[0], lambda: "Dimensions mismatched")
    torch._check((EXPONENT, MANTISSA) in ((3, 2), (2, 3), (2, 2), (3, 1)),
                 lambda: f"FP{1 + EXPONENT + MANTISSA} E{EXPONENT}M{MANTISSA} is not supported.")   # fp6_linear.cu:193
    torch._check(IC % 64 == 0, lambda: f"Expect IC to be a multiple of 64, got {IC}")
    torch._check(OC % 64 == 0, lambda: f"Expect OC to be a multiple of 64, got {OC}")
    _cabi.require_cuda(_in_feats, _weights, _scales)
    x = _in_feats if (_in_feats.stride(1) == 1 and _in_feats.stride(0) % 2 == 0 and _in_feats.data_ptr() % 4 == 0) \
        else _in_feats.contiguous()
    w = _weights.contiguous()
    s = _scales.contiguous()
    y = torch.empty((BS, OC), dtype=torch.float16, device=x.device)
    if BS == 0:
        return y
    lib = _cabi.lib()
    nbytes = lib.ao_fp6_linear_workspace_bytes(BS, OC, IC)
    torch._check(nbytes > 0, lambda: f"unsupported fp6 linear shape BS={BS} OC={OC} IC={IC}")
    with torch.cuda.device(x.device):
        ws = _cabi.workspace(nbytes, x.device)
        if bias is None:
            rc = lib.ao_fpx_linear(EXPONENT, MANTISSA, _cabi.ptr(x), x.stride(0), _cabi.ptr(w), _cabi.ptr(s), BS, OC, IC,
                                   _cabi.ptr(y), _cabi.ptr(ws), ws.numel(), _stream(x))
        else:
            _cabi.require_cuda(bias)
            b = bias.contiguous()
            rc = lib.ao_fpx_linear_bias(EXPONENT, MANTISSA, _cabi.ptr(x), x.stride(0), _cabi.ptr(w), _cabi.ptr(s), _cabi.ptr(b),
                                        BS, OC, IC, _cabi.ptr(y), _cabi.ptr(ws), ws.numel(), _stream(x))
    _cabi.check(rc, "quant_llm_linear")
    return y


def fp6_llm_linear(_in_feats: Tensor, _weights: Tensor, _scales: Tensor, splitK: int = 1) -> Tensor:
    """The e3m2 case under the name of the earlier torchao release."""
    return quant_llm_linear(3, 2, _in_feats, _weights, _scales, splitK)
