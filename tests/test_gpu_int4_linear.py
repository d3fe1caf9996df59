"""GPU parity of the int4 tensor_core_tiled linear (decode GEMV): outputs within
max|y - y_ref| <= 1e-2 * max|y_ref| of the fp32 dequant-matmul oracle."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests import golden_util as gu
from tests import gpu_util as tu

pytestmark = pytest.mark.gpu
MAN = gu.manifest()
TOL = 1e-2  # max-abs error relative to max|y_ref| (the bar stated for GEMM outputs)


def rel_err(y, ref):
    return float(np.max(np.abs(y - ref)) / max(np.max(np.abs(ref)), 1e-30))


def quantize_oracle(w_bf16, group):
    wf = w_bf16.float().numpy()
    s, z = orc.choose_qparams_affine(wf, orc.BF16, orc.ASYMMETRIC, [1, group], 0, 15, 1e-6, orc.BF16, orc.BF16, False,
                                     orc.ZP_FLOAT)
    q = orc.quantize_affine(wf, orc.BF16, [1, group], s, orc.BF16, z, orc.BF16, 0, 15, orc.ZP_FLOAT)
    wd = orc.dequantize_affine(q, [1, group], s, orc.BF16, z, orc.BF16, 0, 15, orc.ZP_FLOAT, orc.F32)
    return s, z, q, wd


def device_operands(s, z, q, ikt):
    from ao_b200 import ops
    from ao_b200.quantization import utils as ut
    packed = ops.convert_weight_to_int4pack(torch.from_numpy(q).cuda(), ikt)
    sz = ut.pack_tinygemm_scales_and_zeros(tu.bf16_from_f32(s), tu.bf16_from_f32(z))
    return packed, sz


@pytest.mark.parametrize("case", MAN["linear"], ids=lambda c: c["name"])
def test_int4_linear_vs_reference_fixture(case):
    from ao_b200 import _cabi, ops
    A = gu.load("linear.npz")
    n, g = case["name"], case["group"]
    q = A[f"{n}/q"].astype(np.int32)
    packed = ops.convert_weight_to_int4pack(torch.from_numpy(q).cuda(), 8)
    sz = tu.to_torch(A[f"{n}/scale_and_zero"], "bf16")
    for M in case["Ms"]:
        x = tu.to_torch(A[f"{n}/x_m{M}"], "bf16")
        y = ops.weight_int4pack_mm(x, packed, g, sz)
        assert y.shape == (M, case["N"]) and y.dtype == torch.bfloat16
        assert rel_err(tu.f32(y), A[f"{n}/y_m{M}"]) <= TOL
        assert _cabi.workspace_status(x.device) == 0


@pytest.mark.parametrize("group", [32, 64, 128, 256])
@pytest.mark.parametrize("ikt", [8, 4, 2])
def test_int4_gemv_vs_oracle_all_batch_sizes(group, ikt):
    from ao_b200 import _cabi, ops
    N, K = 328, 2048  # N = 41 tiles: an odd tile count exercises the half-empty last row pair
    w = tu.make_weight((N, K), seed=group + ikt)
    s, z, q, wd = quantize_oracle(w, group)
    packed, sz = device_operands(s, z, q, ikt)
    g = torch.Generator().manual_seed(group)
    for M in (1, 2, 3, 4, 5, 8, 9, 13, 16):
        x = torch.randn(M, K, generator=g).bfloat16()
        y_ref = orc.linear_f32(x.float().numpy(), wd)
        y = ops.weight_int4pack_mm(x.cuda(), packed, group, sz)
        assert rel_err(tu.f32(y), y_ref) <= TOL, f"M={M}"
        y2 = ops.weight_int4pack_mm(x.cuda(), packed, group, sz)
        assert torch.equal(y, y2), "two runs must give identical bits"
    assert _cabi.workspace_status("cuda") == 0


@pytest.mark.parametrize("shape", [(4096, 4096), (6144, 4096), (4096, 14336)], ids=str)
@pytest.mark.parametrize("group", [64, 128])
def test_llama3_8b_decode_layers_vs_oracle(shape, group):
    """Llama-3-8B decode layers at full size (the oracle needs a few seconds each)."""
    from ao_b200 import _cabi, ops
    N, K = shape
    w = tu.make_weight((N, K), seed=N + K + group)
    s, z, q, wd = quantize_oracle(w, group)
    packed, sz = ops.int4_quantize_pack(w.cuda(), group, 8)
    assert np.array_equal(tu.bits(packed), orc.pack_tinygemm(q, 8))
    g = torch.Generator().manual_seed(1)
    for M in (1, 4, 8, 16):
        x = torch.randn(M, K, generator=g).bfloat16()
        y_ref = orc.linear_f32(x.float().numpy(), wd)
        y = ops.weight_int4pack_mm(x.cuda(), packed, group, sz)
        assert rel_err(tu.f32(y), y_ref) <= TOL, f"M={M}"
    assert _cabi.workspace_status("cuda") == 0


def test_gate_up_full_size_properties():
    """28672 x 4096 (gate_up): linearity in x and agreement with dequantize_affine + matmul on the GPU."""
    from ao_b200 import ops
    from ao_b200.quantization import quant_primitives as qp
    g = torch.Generator(device="cuda").manual_seed(5)
    w = (torch.randn(28672, 4096, generator=g, device="cuda") * 0.02).bfloat16()
    packed, sz = ops.int4_quantize_pack(w, 64, 8)
    s, z, q = ops.int4_groupwise_quantize(w, 64, torch.int32)
    wd = qp.dequantize_affine(q, (1, 64), s, z, torch.int32, 0, 15, qp.ZeroPointDomain.FLOAT, output_dtype=torch.float32)
    x = torch.randn(8, 4096, generator=g, device="cuda").bfloat16()
    y = ops.weight_int4pack_mm(x, packed, 64, sz).float()
    y_ref = x.float() @ wd.T
    assert float((y - y_ref).abs().max() / y_ref.abs().max()) <= TOL
    # rows of a batch are independent: row i of the M=8 result equals the M=1 result on that row
    y1 = ops.weight_int4pack_mm(x[3:4].contiguous(), packed, 64, sz).float()
    assert float((y1 - y[3:4]).abs().max()) <= 2 ** -7 * float(y_ref.abs().max())
    # x = 0 gives exactly 0; scaling x by 2 scales y by 2 exactly (powers of two commute with rounding)
    assert float(ops.weight_int4pack_mm(torch.zeros_like(x), packed, 64, sz).abs().max()) == 0.0
    y2 = ops.weight_int4pack_mm(x * 2, packed, 64, sz).float()
    assert torch.equal(y2, y * 2)


def test_narrow_activation_is_zero_extended():
    """x with fewer columns than the padded weight (the reference pads the activation every call)."""
    from ao_b200 import ops
    N, K, Kx = 64, 1024, 1000
    w = tu.make_weight((N, K), seed=9)
    s, z, q, wd = quantize_oracle(w, 64)
    packed, sz = device_operands(s, z, q, 8)
    x = torch.randn(3, Kx, generator=torch.Generator().manual_seed(2)).bfloat16()
    xp = torch.nn.functional.pad(x, (0, K - Kx))
    y_ref = orc.linear_f32(xp.float().numpy(), wd)
    y = ops.weight_int4pack_mm(x.cuda(), packed, 64, sz)
    assert rel_err(tu.f32(y), y_ref) <= TOL


def test_matches_installed_pytorch_tinygemm():
    """Same packed operands through torch's own aten::_weight_int4pack_mm (the kernel to beat)."""
    from ao_b200 import ops
    N, K, g = 512, 4096, 128
    w = tu.make_weight((N, K), seed=21)
    packed, sz = ops.int4_quantize_pack(w.cuda(), g, 8)
    x = torch.randn(4, K, generator=torch.Generator().manual_seed(3)).bfloat16().cuda()
    try:
        y_t = torch.ops.aten._weight_int4pack_mm(x, packed, g, sz)
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"installed torch operator unavailable: {e}")
    y = ops.weight_int4pack_mm(x, packed, g, sz)
    ref = y_t.float()
    assert float((y.float() - ref).abs().max() / ref.abs().max()) <= 2e-2  # tinygemm itself rounds weights to bf16


def test_bad_arguments_raise():
    from ao_b200 import ops
    packed = torch.zeros(8, 8, 32, 4, dtype=torch.int32, device="cuda")
    sz = torch.zeros(16, 64, 2, dtype=torch.bfloat16, device="cuda")
    x = torch.zeros(1, 1024, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError):
        ops.weight_int4pack_mm(x.float(), packed, 64, sz)
    with pytest.raises(RuntimeError):
        ops.weight_int4pack_mm(x, packed, 64, sz[:8])
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        ops.weight_int4pack_mm(x.cpu(), packed, 64, sz)


def test_k_slab_kernels_share_one_workspace_over_many_launches():
    """The decode kernels with K slabs (int4 at M = 8 on K = 14336, fp6 on a small N) and the split-K tcgen05 kernel
    use the same workspace one after the other; the launch number that tags the slab partial sums advances with
    every launch.  Results must keep the bits of the first launch and the status word must stay clean."""
    from ao_b200 import _cabi, ops
    from ao_b200.prototype.quant_llm.quant_llm import to_scaled_tc_fpx
    g = torch.Generator(device="cuda").manual_seed(11)
    w = (torch.randn(1024, 14336, generator=g, device="cuda") * 0.02).bfloat16()
    packed, sz = ops.int4_quantize_pack(w, 64, 8)
    x8 = torch.randn(8, 14336, generator=g, device="cuda").bfloat16()
    x64 = torch.randn(64, 14336, generator=g, device="cuda").bfloat16()
    assert _cabi.lib().ao_int4_gemv_workspace_bytes(8, 1024, 14336, 64, 8) > 256 + 4 * 16384, "expected a K-slab plan"
    w6 = (torch.randn(1024, 4096, generator=g, device="cuda") * 0.02).half()
    p6, s6 = to_scaled_tc_fpx(w6, 3, 2)
    x6 = torch.randn(1, 4096, generator=g, device="cuda").half()
    first = None
    for it in range(40):
        ys = (ops.weight_int4pack_mm(x8, packed, 64, sz), ops.quant_llm_linear(3, 2, x6, p6, s6, 1),
              ops.weight_int4pack_mm(x64, packed, 64, sz), ops.weight_int4pack_mm(x8[:4].contiguous(), packed, 64, sz))
        if first is None:
            first = [y.clone() for y in ys]
            wd = ops.int4_groupwise_quantize(w, 64, torch.int32)
            from ao_b200.quantization import quant_primitives as qp
            wdq = qp.dequantize_affine(wd[2], (1, 64), wd[0], wd[1], torch.int32, 0, 15, qp.ZeroPointDomain.FLOAT,
                                       output_dtype=torch.float32)
            ref = x8.float() @ wdq.T
            assert float((ys[0].float() - ref).abs().max() / ref.abs().max()) <= TOL
        else:
            for y, f in zip(ys, first):
                assert torch.equal(y, f), f"launch {it}"
    assert _cabi.workspace_status("cuda") == 0
