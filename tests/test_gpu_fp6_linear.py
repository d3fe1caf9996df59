"""GPU parity of the FP6 (e3m2) linear: outputs within max|y - y_ref| <= 1e-2 * max|y_ref| of the fp32
dequant-matmul oracle x.float() @ from_scaled_tc_fpx(w).T, and under the reference's own mean-relative-error bar."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests import golden_util as gu
from tests import gpu_util as tu

pytestmark = pytest.mark.gpu
MAN = gu.manifest()
TOL = 1e-2


def rel_err(y, ref):
    return float(np.max(np.abs(y - ref)) / max(np.max(np.abs(ref)), 1e-30))


@pytest.mark.parametrize("case", MAN["fp6_linear"], ids=lambda c: c["name"])
def test_fp6_linear_vs_reference_fixture(case):
    from ao_b200 import _cabi, ops
    A = gu.load("linear.npz")
    n = case["name"]
    packed = tu.to_torch(A[f"{n}/packed"], "u8")
    scale = tu.to_torch(A[f"{n}/scale"], "f16")
    for M in case["Ms"]:
        x = tu.to_torch(A[f"{n}/x_m{M}"], "f16")
        y = ops.quant_llm_linear(3, 2, x, packed, scale, 1)
        assert y.shape == (M, case["N"]) and y.dtype == torch.float16
        assert rel_err(tu.f32(y), A[f"{n}/y_m{M}"]) <= TOL, f"M={M}"
    assert _cabi.workspace_status("cuda") == 0


@pytest.mark.parametrize("shape", [(256, 512), (1088, 1024), (4096, 4096), (4096, 11008)], ids=str)
def test_fp6_gemv_vs_oracle(shape):
    from ao_b200 import _cabi, ops
    from ao_b200.prototype.quant_llm.quant_llm import to_scaled_tc_fpx
    N, K = shape
    w = tu.make_weight((N, K), seed=N + K, dtype=torch.float16, outliers=False)
    packed_ref, scale_ref = orc.to_scaled_tc_fp6(w.float().numpy())
    wd = orc.from_scaled_tc_fp6(packed_ref, scale_ref)
    packed, scale = to_scaled_tc_fpx(w.cuda(), 3, 2)
    assert np.array_equal(tu.bits(packed), packed_ref) and np.array_equal(tu.bits(scale), scale_ref)
    g = torch.Generator().manual_seed(N)
    for M in (1, 2, 3, 5, 8, 9, 16):
        x = torch.randn(M, K, generator=g).half()
        y_ref = orc.linear_f32(x.float().numpy(), wd)
        y = ops.fp6_llm_linear(x.cuda(), packed, scale)
        assert rel_err(tu.f32(y), y_ref) <= TOL, f"M={M}"
        assert torch.equal(y, ops.fp6_llm_linear(x.cuda(), packed, scale)), "two runs must give identical bits"
    assert _cabi.workspace_status("cuda") == 0


@pytest.mark.parametrize("BS,OC,IC", [(1, 2048, 4096), (2, 8192, 8192), (64, 256, 512)])
def test_random_bytes_like_the_reference_op_test(BS, OC, IC):
    """Every byte random, scale and activation in [0.5, 1.5): the reference's test/test_ops.py:24-62 checks
    mean |err| / mean |y| < 1e-3 against fp16_act @ from_scaled_tc_fpx(w).half().T."""
    from ao_b200 import ops
    from ao_b200.prototype.quant_llm.quant_llm import from_scaled_tc_fpx
    g = torch.Generator().manual_seed(BS + OC)
    w = torch.randint(256, (OC, IC // 8 * 6), dtype=torch.uint8, generator=g).cuda()
    scale = (torch.rand(OC, generator=g).half() + 0.5).cuda()
    act = (torch.rand(BS, IC, generator=g).half() + 0.5).cuda()
    out = ops.quant_llm_linear(3, 2, act, w, scale, 5)
    ref = act.float() @ from_scaled_tc_fpx(w, 3, 2, scale).T
    err = (out.float() - ref).abs().mean() / ref.abs().mean()
    assert float(err) < 1e-3


def test_quant_llm_weight_subclass_linear():
    from ao_b200.prototype.quant_llm import QuantLlmLinearWeight, fp6_llm_weight_only
    from ao_b200.quantization import quantize
    torch.manual_seed(0)
    lin = torch.nn.Linear(512, 256, bias=True, device="cuda", dtype=torch.float16)
    ref_w = lin.weight.detach().clone()
    skip = torch.nn.Linear(100, 256, device="cuda", dtype=torch.float16)  # in_features % 64 != 0: left as is
    m = torch.nn.Sequential(lin)
    quantize(m, fp6_llm_weight_only())
    assert isinstance(m[0].weight, QuantLlmLinearWeight)
    assert fp6_llm_weight_only()(skip.weight) is skip.weight
    x = torch.randn(2, 3, 512, device="cuda", dtype=torch.float16)
    y = m(x).detach()
    assert y.shape == (2, 3, 256) and y.dtype == torch.float16
    ref = torch.nn.functional.linear(x.float(), m[0].weight.detach().dequantize(torch.float32), lin.bias.detach().float())
    assert float((y.float() - ref).abs().max() / ref.abs().max()) <= TOL
    # fp6 keeps ~2 mantissa bits: the quantized layer stays close to the original one
    y0 = torch.nn.functional.linear(x, ref_w, lin.bias.detach())
    assert float(20 * torch.log10(y0.float().norm() / (y0.float() - y.float()).norm())) > 15


def test_bad_arguments_raise():
    from ao_b200 import ops
    w = torch.zeros(256, 384, dtype=torch.uint8, device="cuda")
    s = torch.ones(256, dtype=torch.float16, device="cuda")
    x = torch.zeros(1, 512, dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError, match="weight must be FP16"):
        ops.quant_llm_linear(3, 2, x.float(), w, s, 1)
    with pytest.raises(RuntimeError, match="Dimensions mismatched"):
        ops.quant_llm_linear(3, 2, x, w[:, :100], s, 1)
    with pytest.raises(RuntimeError, match="is not supported"):
        ops.quant_llm_linear(2, 1, x, torch.zeros(256, 256, dtype=torch.uint8, device="cuda"), s, 1)


@pytest.mark.parametrize("N,K", [(256, 512), (1024, 4096), (4096, 1024)])
def test_fp6_prefill_vs_oracle(N, K):
    """M > 16 runs the tcgen05 kernel."""
    from ao_b200 import _cabi, ops
    from ao_b200.prototype.quant_llm.quant_llm import to_scaled_tc_fpx
    w = tu.make_weight((N, K), seed=N + 3 * K, dtype=torch.float16, outliers=False)
    packed_ref, scale_ref = orc.to_scaled_tc_fp6(w.float().numpy())
    wd = orc.from_scaled_tc_fp6(packed_ref, scale_ref)
    packed, scale = to_scaled_tc_fpx(w.cuda(), 3, 2)
    g = torch.Generator().manual_seed(K)
    for M in (17, 64, 100, 128, 256, 300):
        x = torch.randn(M, K, generator=g).half()
        y_ref = orc.linear_f32(x.float().numpy(), wd)
        y = ops.fp6_llm_linear(x.cuda(), packed, scale)
        assert y.shape == (M, N) and y.dtype == torch.float16
        assert rel_err(tu.f32(y), y_ref) <= TOL, f"M={M}"
        assert torch.equal(y, ops.fp6_llm_linear(x.cuda(), packed, scale))
    assert _cabi.workspace_status("cuda") == 0


def test_fp6_prefill_two_row_tiles_per_block():
    """1024 x 4736 (37 row tiles of 128, the last one half full: N % 128 = 0 is not required, N % 64 is): 128-column
    token tiles with two row tiles per thread block; the last block's second row tile lies beyond N."""
    from ao_b200 import _cabi, ops
    from ao_b200.prototype.quant_llm.quant_llm import to_scaled_tc_fpx
    N, K, M = 4672, 512, 1024
    w = tu.make_weight((N, K), seed=N + K, dtype=torch.float16, outliers=False)
    packed_ref, scale_ref = orc.to_scaled_tc_fp6(w.float().numpy())
    wd = orc.from_scaled_tc_fp6(packed_ref, scale_ref)
    packed, scale = to_scaled_tc_fpx(w.cuda(), 3, 2)
    x = torch.randn(M, K, generator=torch.Generator().manual_seed(1)).half()
    y = ops.fp6_llm_linear(x.cuda(), packed, scale)
    y_ref = np.ascontiguousarray(x.float().numpy()) @ wd.T
    assert rel_err(tu.f32(y), y_ref) <= TOL
    assert torch.equal(y, ops.fp6_llm_linear(x.cuda(), packed, scale))
    assert _cabi.workspace_status("cuda") == 0


def test_e2m3_codec_bit_exact_vs_reference_fixture():
    from ao_b200.prototype.quant_llm.quant_llm import from_scaled_tc_fpx, to_scaled_tc_fpx
    A = gu.load("e2m3.npz")
    for name, dt in (("scaled_e2m3_f16", "f16"), ("scaled_e2m3_f32", "f32")):
        w = tu.to_torch(A[f"{name}/w"], dt)
        packed, scale = to_scaled_tc_fpx(w, 2, 3)
        assert np.array_equal(tu.bits(packed), A[f"{name}/packed"])
        assert np.array_equal(tu.bits(scale), A[f"{name}/scale"])
        assert np.array_equal(tu.f32(from_scaled_tc_fpx(packed, 2, 3, scale)), A[f"{name}/dequant_f32"])


def test_e2m3_linear_vs_reference_fixture_and_oracle():
    from ao_b200 import _cabi, ops
    from ao_b200.prototype.quant_llm import quant_llm_fpx_weight_only
    A = gu.load("e2m3.npz")
    packed = tu.to_torch(A["e2m3_lin/packed"], "u8")
    scale = tu.to_torch(A["e2m3_lin/scale"], "f16")
    for M in (1, 16, 64):
        x = tu.to_torch(A[f"e2m3_lin/x_m{M}"], "f16")
        y = ops.quant_llm_linear(2, 3, x, packed, scale, 1)
        assert rel_err(tu.f32(y), A[f"e2m3_lin/y_m{M}"]) <= TOL, f"M={M}"
    # larger shapes against the oracle, decode and prefill kernels
    N, K = 1024, 4096
    w = tu.make_weight((N, K), seed=77, dtype=torch.float16, outliers=False)
    packed_ref, scale_ref = orc.to_scaled_tc_fp6(w.float().numpy(), 2, 3)
    wd = orc.from_scaled_tc_fp6(packed_ref, scale_ref, 2, 3)
    lin = torch.nn.Linear(K, N, bias=False, device="cuda", dtype=torch.float16)
    with torch.no_grad():
        lin.weight.copy_(w)
    from ao_b200.quantization import quantize
    quantize(lin, quant_llm_fpx_weight_only(2, 3))
    assert np.array_equal(tu.bits(lin.weight.fpx_data), packed_ref)
    g = torch.Generator().manual_seed(5)
    for M in (1, 3, 8, 17, 100, 256):
        x = torch.randn(M, K, generator=g).half()
        y = lin(x.cuda()).detach()
        assert rel_err(tu.f32(y), orc.linear_f32(x.float().numpy(), wd)) <= TOL, f"M={M}"
    assert _cabi.workspace_status("cuda") == 0
    with pytest.raises(RuntimeError, match="is not supported"):
        ops.quant_llm_linear(2, 1, x.cuda(), torch.zeros(N, K // 8 * 4, dtype=torch.uint8, device="cuda"),
                             torch.ones(N, dtype=torch.float16, device="cuda"), 1)


def test_generic_packer_5_and_6_bits_bit_exact():
    from ao_b200.prototype.quant_llm.quant_llm import pack_tc_fpx, unpack_tc_fpx
    A = gu.load("fp5.npz")
    for key, nbits in (("pack5", 5), ("pack6", 6)):
        codes = torch.from_numpy(A[f"{key}/codes"]).cuda()
        packed = pack_tc_fpx(codes, nbits)
        assert np.array_equal(packed.cpu().numpy(), A[f"{key}/packed"])
        assert torch.equal(unpack_tc_fpx(packed, nbits), codes)


@pytest.mark.parametrize("fmt", [(2, 2), (3, 1)], ids=["e2m2", "e3m1"])
def test_fp5_formats_codec_and_linear(fmt):
    from ao_b200 import _cabi, ops
    from ao_b200.prototype.quant_llm import quant_llm_fpx_weight_only
    from ao_b200.prototype.quant_llm.quant_llm import from_scaled_tc_fpx, to_scaled_tc_fpx
    from ao_b200.quantization import quantize
    e, m = fmt
    name = f"e{e}m{m}"
    A = gu.load("fp5.npz")
    w = tu.to_torch(A[f"{name}/w"], "f16")
    packed, scale = to_scaled_tc_fpx(w, e, m)
    assert np.array_equal(tu.bits(packed), A[f"{name}/packed"])
    assert np.array_equal(tu.bits(scale), A[f"{name}/scale"])
    assert np.array_equal(tu.f32(from_scaled_tc_fpx(packed, e, m, scale)), A[f"{name}/dequant_f32"])
    packed = tu.to_torch(A[f"{name}_lin/packed"], "u8")
    scale = tu.to_torch(A[f"{name}_lin/scale"], "f16")
    for M in (1, 16, 64):
        x = tu.to_torch(A[f"{name}_lin/x_m{M}"], "f16")
        y = ops.quant_llm_linear(e, m, x, packed, scale, 1)
        assert rel_err(tu.f32(y), A[f"{name}_lin/y_m{M}"]) <= TOL, f"M={M}"
    # larger shapes against the oracle, decode and prefill kernels, through the weight subclass
    N, K = 1024, 4096
    w = tu.make_weight((N, K), seed=91 + e, dtype=torch.float16, outliers=False)
    packed_ref, scale_ref = orc.to_scaled_tc_fpx(w.float().numpy(), e, m)
    wd = orc.from_scaled_tc_fpx(packed_ref, scale_ref, e, m)
    lin = torch.nn.Linear(K, N, bias=False, device="cuda", dtype=torch.float16)
    with torch.no_grad():
        lin.weight.copy_(w)
    quantize(lin, quant_llm_fpx_weight_only(e, m))
    assert np.array_equal(tu.bits(lin.weight.fpx_data), packed_ref)
    g = torch.Generator().manual_seed(6)
    for M in (1, 4, 8, 17, 100, 256):
        x = torch.randn(M, K, generator=g).half()
        y = lin(x.cuda()).detach()
        assert rel_err(tu.f32(y), orc.linear_f32(x.float().numpy(), wd)) <= TOL, f"M={M}"
    assert _cabi.workspace_status("cuda") == 0
