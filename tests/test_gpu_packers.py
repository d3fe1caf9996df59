"""GPU parity of the packers and the fp6 codec: packed bytes are compared bit for bit with the
reference's recorded outputs (tests/golden) and with the CPU oracle."""
import os

import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests import golden_util as gu
from tests import gpu_util as tu

pytestmark = pytest.mark.gpu
MAN = gu.manifest()


@pytest.mark.parametrize("ikt", [2, 4, 8])
def test_tinygemm_pack_unpack_vs_oracle(ikt):
    from ao_b200 import ops
    rng = np.random.default_rng(ikt)
    codes = rng.integers(0, 16, size=(136, 1024), dtype=np.int32)
    packed = ops.convert_weight_to_int4pack(torch.from_numpy(codes).cuda(), ikt)
    assert np.array_equal(tu.bits(packed), orc.pack_tinygemm(codes, ikt))
    assert np.array_equal(tu.bits(ops.unpack_int4pack(packed)), codes)


def test_tinygemm_pack_matches_pytorch_operator_fixture():
    """tests/golden/tinygemm.npz holds what aten::_convert_weight_to_int4pack of the pinned torch build
    produced on a B200 (see tests/golden/make_tinygemm_golden.py)."""
    from ao_b200 import ops
    path = os.path.join(gu.GOLDEN, "tinygemm.npz")
    if not os.path.exists(path):
        pytest.skip("tinygemm.npz fixture not generated yet")
    A = gu.load("tinygemm.npz")
    codes = torch.from_numpy(A["codes"]).cuda()
    for ikt in (2, 4, 8):
        assert np.array_equal(tu.bits(ops.convert_weight_to_int4pack(codes, ikt)), A[f"packed_ikt{ikt}"])


def test_tinygemm_pack_matches_installed_pytorch_operator():
    """Live cross-check against the installed torch's operator (two codes per byte, even k high)."""
    from ao_b200 import ops
    rng = np.random.default_rng(11)
    codes = torch.from_numpy(rng.integers(0, 16, size=(64, 2048), dtype=np.int32)).cuda()
    u8 = (codes[:, ::2] << 4 | codes[:, 1::2]).to(torch.uint8).contiguous()
    try:
        ref = torch.ops.aten._convert_weight_to_int4pack(u8, 8)
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"installed torch operator unavailable: {e}")
    assert torch.equal(ops.convert_weight_to_int4pack(codes, 8), ref)


def test_scales_and_zeros_interleave():
    from ao_b200.quantization import utils as ut
    for case in MAN["linear"]:
        A = gu.load("linear.npz")
        n = case["name"]
        s = tu.to_torch(A[f"{n}/scale"], "bf16")
        z = tu.to_torch(A[f"{n}/zero"], "bf16")
        sz = ut.pack_tinygemm_scales_and_zeros(s, z)
        assert np.array_equal(tu.bits(sz), A[f"{n}/scale_and_zero"])
        s2, z2 = ut.unpack_tinygemm_scales_and_zeros(sz)
        assert torch.equal(s2.squeeze(-1), s) and torch.equal(z2.squeeze(-1), z)
    with pytest.raises(ValueError, match="to have dtype"):
        ut.pack_tinygemm_scales_and_zeros(s.float(), z)


def test_hqq_row_pair_packing():
    from ao_b200.prototype.hqq.mixed_mm import pack_2xint4, pack_hqq_from_rowmajor
    A = gu.load("linear.npz")
    for case in MAN["linear"]:
        n = case["name"]
        q = tu.to_torch(A[f"{n}/q"], "u8")
        assert np.array_equal(tu.bits(pack_2xint4(q.T.contiguous())), A[f"{n}/hqq_packed"])
        assert np.array_equal(tu.bits(pack_hqq_from_rowmajor(q)), A[f"{n}/hqq_packed"])
    t = torch.arange(16, dtype=torch.uint8, device="cuda").reshape(4, 4)
    # the docstring example of the reference (mixed_mm.py:13-33)
    assert pack_2xint4(t).cpu().tolist() == [[0 | 4 << 4, 1 | 5 << 4, 2 | 6 << 4, 3 | 7 << 4],
                                             [8 | 12 << 4, 9 | 13 << 4, 10 | 14 << 4, 11 | 15 << 4]]


@pytest.mark.parametrize("fmt", [(3, 2), (2, 3), (2, 2), (3, 1)])
def test_fpx_codec_bit_exact(fmt):
    from ao_b200.prototype.custom_fp_utils import _f32_to_fpx_unpacked, _fpx_unpacked_to_f32
    e, m = fmt
    A = gu.load("fp6.npz")
    k = f"codec_e{e}m{m}"
    vals = _fpx_unpacked_to_f32(tu.to_torch(A[f"{k}/codes"], "u8"), e, m)
    assert np.array_equal(tu.bits(vals).view(np.uint32), A[f"{k}/values"].view(np.uint32))
    assert np.array_equal(tu.bits(_f32_to_fpx_unpacked(vals, e, m)), A[f"{k}/reencoded"])
    assert np.array_equal(tu.bits(_f32_to_fpx_unpacked(tu.to_torch(A[f"{k}/x"], "f32"), e, m)), A[f"{k}/x_codes"])


def test_e3m2_rounding_known_answers():
    from ao_b200.prototype.custom_fp_utils import _f32_to_fpx_unpacked
    x = torch.tensor([29.0, 26.0, 0.1251, 0.0314, 0.03], device="cuda")
    assert _f32_to_fpx_unpacked(x, 3, 2).cpu().tolist() == [0b011111, 0b011110, 0b000010, 0b000001, 0b000000]
    assert _f32_to_fpx_unpacked(-x, 3, 2).cpu().tolist() == [0b111111, 0b111110, 0b100010, 0b100001, 0b100000]


def test_fp6_pack_unpack_bit_exact():
    from ao_b200.prototype.quant_llm.quant_llm import pack_tc_fpx, unpack_tc_fpx
    A = gu.load("fp6.npz")
    x = tu.to_torch(A["pack_fp6/bytes_in"], "u8")
    packed = pack_tc_fpx(x, 6)
    assert np.array_equal(tu.bits(packed), A["pack_fp6/packed"])
    assert np.array_equal(tu.bits(unpack_tc_fpx(packed, 6)), A["pack_fp6/unpacked"])
    rng = np.random.default_rng(5)
    big = rng.integers(0, 64, size=(512, 1088), dtype=np.uint8)
    p = pack_tc_fpx(torch.from_numpy(big).cuda(), 6)
    assert np.array_equal(tu.bits(p), orc.pack_tc_fp6(big))
    assert np.array_equal(tu.bits(unpack_tc_fpx(p, 6)), big)


@pytest.mark.parametrize("case", MAN["fp6"], ids=lambda c: c["name"])
def test_to_scaled_tc_fpx_bit_exact(case):
    from ao_b200.prototype.quant_llm.quant_llm import from_scaled_tc_fpx, to_scaled_tc_fpx
    A = gu.load("fp6.npz")
    n = case["name"]
    dt = "f16" if n.endswith("f16") else "f32"
    w = tu.to_torch(A[f"{n}/w"], dt)
    packed, scale = to_scaled_tc_fpx(w, 3, 2)
    assert packed.dtype == torch.uint8 and scale.dtype == torch.float16
    assert np.array_equal(tu.bits(packed), A[f"{n}/packed"])
    assert np.array_equal(tu.bits(scale), A[f"{n}/scale"])
    assert np.array_equal(tu.bits(from_scaled_tc_fpx(packed, 3, 2, scale)).view(np.uint32),
                          A[f"{n}/dequant_f32"].view(np.uint32))
    assert np.array_equal(tu.bits(from_scaled_tc_fpx(packed, 3, 2)).view(np.uint32),
                          A[f"{n}/dequant_noscale_f32"].view(np.uint32))


def test_to_scaled_tc_fpx_llama_shape_vs_oracle():
    from ao_b200.prototype.quant_llm.quant_llm import to_scaled_tc_fpx
    w = tu.make_weight((1024, 4096), seed=77, dtype=torch.float16, outliers=False)
    packed, scale = to_scaled_tc_fpx(w.cuda(), 3, 2)
    p_ref, s_ref = orc.to_scaled_tc_fp6(w.float().numpy())
    assert np.array_equal(tu.bits(packed), p_ref)
    assert np.array_equal(tu.bits(scale), s_ref)
    z_packed, z_scale = to_scaled_tc_fpx(torch.zeros(64, 64, device="cuda"), 3, 2)
    A = gu.load("fp6.npz")
    assert np.array_equal(tu.bits(z_packed), A["scaled_fp6_zero/packed"])
    assert np.array_equal(tu.bits(z_scale), A["scaled_fp6_zero/scale"])
