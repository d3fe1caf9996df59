"""GPU parity at the benchmark configurations' own shapes.

Every test quantises a seeded synthetic weight with the CPU oracle (oracle/: the restatement of the reference's
choose_qparams_affine / quantize_affine / dequantize_affine and fp6 codec, pinned to the reference by the golden
fixtures), checks that the kernels produce the same codes / packed bytes / scales BIT FOR BIT, and then holds the
linear kernels to
    max|y - y_ref| <= 1e-2 * max|y_ref|,   y_ref = x.float() @ dequant_fp32(W_q).T
with the dequantised fp32 weight taken from the oracle.  The dense fp32 product itself is numpy's (BLAS) for the
batched shapes and the oracle's double-accumulating loop for M <= 16.

  config 1  int4 plain layout, 4096 x 4096, group 64, M = 1 (the reference's CPU-runnable case)
  config 2  Llama-3-8B decode layer set, tensor_core_tiled, groups 64 and 128, M in {1, 4, 8, 16}
  config 3  FP6 e3m2, Llama-2-7B shapes, M in {1, 16, 64, 128}
  config 4  HQQ-layout int4, 8192 x 8192, group 64, M in {64, 256, 1024, 4096}
  config 5  Llama-3-70B layers, group 128, M in {1, 32, 256}: the whole layer and a 1/8 row shard
"""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests import gpu_util as tu

pytestmark = pytest.mark.gpu
TOL = 1e-2


def rel_err(y, ref):
    return float(np.max(np.abs(y - ref)) / max(np.max(np.abs(ref)), 1e-30))


def ref_linear(x_f32, wd):
    """fp32 dequant-matmul oracle output: exact-ish loop for decode batches, BLAS for the batched shapes."""
    if x_f32.shape[0] <= 16:
        return orc.linear_f32(x_f32, wd)
    return np.ascontiguousarray(x_f32, np.float32) @ np.ascontiguousarray(wd, np.float32).T


def int4_oracle(w_bf16, group):
    wf = w_bf16.float().numpy()
    s, z = orc.choose_qparams_affine(wf, orc.BF16, orc.ASYMMETRIC, [1, group], 0, 15, 1e-6, orc.BF16, orc.BF16, False,
                                     orc.ZP_FLOAT)
    q = orc.quantize_affine(wf, orc.BF16, [1, group], s, orc.BF16, z, orc.BF16, 0, 15, orc.ZP_FLOAT)
    wd = orc.dequantize_affine(q, [1, group], s, orc.BF16, z, orc.BF16, 0, 15, orc.ZP_FLOAT, orc.F32)
    return s, z, q, wd


def make_x(M, K, seed, dtype=torch.bfloat16):
    return torch.randn(M, K, generator=torch.Generator().manual_seed(seed)).to(dtype)


# ---------------------------------------------------------------------------------------------------------------
# config 1
# ---------------------------------------------------------------------------------------------------------------
def test_config1_int4_plain_4096x4096_g64_m1():
    from ao_b200.dtypes import to_affine_quantized
    from ao_b200.quantization import MappingType, ZeroPointDomain
    N = K = 4096
    w = tu.make_weight((N, K), seed=1234, outliers=False)
    x = make_x(1, K, 1234)
    s, z, q, wd = int4_oracle(w, 64)
    aqt = to_affine_quantized(w.cuda(), MappingType.ASYMMETRIC, (1, 64), torch.int32, 0, 15, 1e-6,
                              zero_point_dtype=torch.bfloat16, preserve_zero=False,
                              zero_point_domain=ZeroPointDomain.FLOAT)
    int_data, scale, zero = aqt.layout_tensor.get_plain()
    assert np.array_equal(tu.bits(int_data), q)
    assert np.array_equal(tu.bits(scale), orc.f32_to_bf16_bits(s))
    assert np.array_equal(tu.bits(zero), orc.f32_to_bf16_bits(z))
    y = torch.nn.functional.linear(x.cuda(), aqt)
    assert y.shape == (1, N) and y.dtype == torch.bfloat16
    assert rel_err(tu.f32(y), ref_linear(x.float().numpy(), wd)) <= TOL


# ---------------------------------------------------------------------------------------------------------------
# config 2
# ---------------------------------------------------------------------------------------------------------------
LLAMA3_8B = {"qkv": (6144, 4096), "o": (4096, 4096), "gate_up": (28672, 4096), "down": (4096, 14336)}


@pytest.mark.parametrize("group", [64, 128])
@pytest.mark.parametrize("layer", list(LLAMA3_8B))
def test_config2_llama3_8b_decode_layer(layer, group):
    from ao_b200 import _cabi, ops
    N, K = LLAMA3_8B[layer]
    w = tu.make_weight((N, K), seed=N + K + group)   # 0.1 % of the entries x20
    s, z, q, wd = int4_oracle(w, group)
    packed, sz = ops.int4_quantize_pack(w.cuda(), group, 8)
    assert np.array_equal(tu.bits(packed), orc.pack_tinygemm(q, 8))
    assert np.array_equal(tu.bits(sz), orc.pack_tinygemm_scales_and_zeros(orc.f32_to_bf16_bits(s), orc.f32_to_bf16_bits(z)))
    for M in (1, 4, 8, 16):
        x = make_x(M, K, M)
        y = ops.weight_int4pack_mm(x.cuda(), packed, group, sz)
        assert rel_err(tu.f32(y), ref_linear(x.float().numpy(), wd)) <= TOL, f"M={M}"
    assert _cabi.workspace_status("cuda") == 0


# ---------------------------------------------------------------------------------------------------------------
# config 3
# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("shape", [(4096, 4096), (11008, 4096), (4096, 11008), (12288, 4096)], ids=lambda s: f"{s[0]}x{s[1]}")
def test_config3_fp6_llama2_7b_layer(shape):
    from ao_b200 import _cabi, ops
    from ao_b200.prototype.quant_llm.quant_llm import to_scaled_tc_fpx
    N, K = shape
    w = tu.make_weight((N, K), seed=N + K, dtype=torch.float16, outliers=False)
    packed_ref, scale_ref = orc.to_scaled_tc_fp6(w.float().numpy())
    wd = orc.from_scaled_tc_fp6(packed_ref, scale_ref)
    packed, scale = to_scaled_tc_fpx(w.cuda(), 3, 2)
    assert np.array_equal(tu.bits(packed), packed_ref) and np.array_equal(tu.bits(scale), scale_ref)
    for M in (1, 16, 64, 128):
        x = make_x(M, K, M, torch.float16)
        y = ops.quant_llm_linear(3, 2, x.cuda(), packed, scale, 1)
        assert y.shape == (M, N) and y.dtype == torch.float16
        y_ref = ref_linear(x.float().numpy(), wd)
        assert rel_err(tu.f32(y), y_ref) <= TOL, f"M={M}"
        # the reference's own bar (test/test_ops.py:47-62): mean |err| / mean |y| < 1e-3
        assert float(np.mean(np.abs(tu.f32(y) - y_ref)) / np.mean(np.abs(y_ref))) < 1e-3, f"M={M}"
    assert _cabi.workspace_status("cuda") == 0


# ---------------------------------------------------------------------------------------------------------------
# config 4
# ---------------------------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def hqq_8192():
    """8192 x 8192, group 64: codes / scale / zero from the oracle, zero converted to HQQ's convention
    (q - z_hqq) * s with z_hqq = 8 - z / s rounded to bf16, and the fp32 weight that convention dequantises to."""
    from ao_b200 import ops
    from ao_b200.prototype.hqq import pack_hqq_from_rowmajor
    N = K = 8192
    g = 64
    w = tu.make_weight((N, K), seed=4, outliers=False)
    s, z, q, _ = int4_oracle(w, g)
    s_d, z_d, codes = ops.int4_groupwise_quantize(w.cuda(), g, want_codes=torch.uint8)
    assert np.array_equal(tu.bits(codes), q.astype(np.uint8))
    assert np.array_equal(tu.bits(s_d), orc.f32_to_bf16_bits(s)) and np.array_equal(tu.bits(z_d), orc.f32_to_bf16_bits(z))
    z_hqq = (8.0 - z_d.float() / s_d.float()).to(torch.bfloat16)
    zf = z_hqq.float().cpu().numpy()
    wd = (q.astype(np.float32).reshape(N, K // g, g) - zf[:, :, None]) * s[:, :, None]
    return dict(N=N, K=K, g=g, packed=pack_hqq_from_rowmajor(codes), sT=s_d.T.contiguous(),
                zT=z_hqq.T.contiguous(), wd=np.ascontiguousarray(wd.reshape(N, K), np.float32))


@pytest.mark.parametrize("M", [64, 256, 1024, 4096])
def test_config4_hqq_int4_8192x8192_g64(hqq_8192, M):
    from ao_b200 import _cabi
    from ao_b200.prototype.hqq import mixed_mm
    h = hqq_8192
    x = make_x(M, h["K"], M)
    y = mixed_mm(x.cuda(), h["packed"], h["sT"], h["zT"], h["g"])
    assert y.shape == (M, h["N"]) and y.dtype == torch.bfloat16
    assert rel_err(tu.f32(y), ref_linear(x.float().numpy(), h["wd"])) <= TOL
    assert _cabi.workspace_status("cuda") == 0


# ---------------------------------------------------------------------------------------------------------------
# config 5
# ---------------------------------------------------------------------------------------------------------------
LLAMA3_70B = {"qkv": (10240, 8192), "o": (8192, 8192), "gate_up": (57344, 8192), "down": (8192, 28672)}


@pytest.mark.parametrize("layer", list(LLAMA3_70B))
def test_config5_llama3_70b_layer_whole_and_one_eighth_shard(layer):
    """Group 128.  The whole layer on one GPU and rank 3's shard of an 8-way row split (rows [3N/8, 4N/8)),
    quantised on the device from the shard alone: the shard's packed bytes, scales and outputs must be exactly the
    corresponding slice of the whole layer's, because quantisation groups run along K."""
    from ao_b200 import _cabi, ops
    from ao_b200.sharding import row_shard_bounds
    N, K = LLAMA3_70B[layer]
    g = 128
    w = tu.make_weight((N, K), seed=N + K, outliers=False)
    s, z, q, wd = int4_oracle(w, g)
    wc = w.cuda()
    packed, sz = ops.int4_quantize_pack(wc, g, 8)
    assert np.array_equal(tu.bits(packed), orc.pack_tinygemm(q, 8))
    lo, hi = row_shard_bounds(N, 8, 3, 8)
    packed_s, sz_s = ops.int4_quantize_pack(wc[lo:hi].contiguous(), g, 8)
    assert torch.equal(packed_s, packed[lo // 8: hi // 8]) and torch.equal(sz_s, sz[:, lo:hi])
    del wc
    for M in (1, 32, 256):
        x = make_x(M, K, M)
        y_ref = ref_linear(x.float().numpy(), wd)
        y = ops.weight_int4pack_mm(x.cuda(), packed, g, sz)
        assert rel_err(tu.f32(y), y_ref) <= TOL, f"whole layer, M={M}"
        y_s = ops.weight_int4pack_mm(x.cuda(), packed_s, g, sz_s)
        assert rel_err(tu.f32(y_s), y_ref[:, lo:hi]) <= TOL, f"shard, M={M}"
    assert _cabi.workspace_status("cuda") == 0
