"""Pins the CPU oracle (oracle/oracle.c) against outputs of the reference implementation.

The fixtures under tests/golden/ were produced by tests/golden/make_golden.py, which imports
the reference's own modules; every comparison here is bit-exact."""
import numpy as np
import pytest

from oracle import oracle as orc
from tests import golden_util as gu

MAN = gu.manifest()


@pytest.mark.parametrize("case", MAN["primitives"], ids=lambda c: c["name"])
def test_primitives_match_reference(case):
    A = gu.load("primitives.npz")
    n = case["name"]
    in_dt = case["in_dt"]
    x = gu.as_f32(A[f"{n}/x"], in_dt)
    mapping = orc.SYMMETRIC if case["mapping"] == "sym" else orc.ASYMMETRIC
    dom = orc.ZP_FLOAT if case["zp_domain"] == "float" else orc.ZP_INT
    sdt = case["scale_dtype_out"]
    zdt = case["zp_dtype_out"]
    tq = {"i8": (-128, 127), "u8": (0, 255), "i32": (-2**31, 2**31 - 1)}[case["target"]]
    qmin = tq[0] if case["qmin"] is None else case["qmin"]
    qmax = tq[1] if case["qmax"] is None else case["qmax"]
    s, z = orc.choose_qparams_affine(x, gu.DT_CODE[in_dt], mapping, case["block"], qmin, qmax, case["eps"],
                                     gu.DT_CODE[sdt], gu.DT_CODE[zdt], case["preserve_zero"], dom)
    s_ref = gu.as_f32(A[f"{n}/scale"], sdt)
    z_ref = gu.as_f32(A[f"{n}/zp"], zdt)
    assert s.shape == s_ref.shape and z.shape == z_ref.shape
    assert np.array_equal(s.view(np.uint32), s_ref.view(np.uint32)), "scale differs from reference"
    assert np.array_equal(z.view(np.uint32), z_ref.view(np.uint32)), "zero_point differs from reference"
    q = orc.quantize_affine(x, gu.DT_CODE[in_dt], case["block"], s_ref, gu.DT_CODE[sdt], z_ref, gu.DT_CODE[zdt],
                            qmin, qmax, dom)
    assert np.array_equal(q, A[f"{n}/q"].astype(np.int32)), "codes differ from reference"
    for d in case["deq"]:
        dq = orc.dequantize_affine(q, case["block"], s_ref, gu.DT_CODE[sdt], z_ref, gu.DT_CODE[zdt], qmin, qmax,
                                   dom, gu.DT_CODE[d])
        ref = gu.as_f32(A[f"{n}/deq_{d}"], d)
        assert np.array_equal(dq.view(np.uint32), ref.view(np.uint32)), f"dequant {d} differs"


def test_quantize_dequantize_from_given_qparams():
    """Random (also negative) scales/zeros, as the reference tests do against the legacy formulas."""
    A = gu.load("primitives.npz")
    x, s, z = A["from_qparams/x"], A["from_qparams/scale"], A["from_qparams/zero"]
    q = orc.quantize_affine(x, orc.F32, [1, 128], s, orc.F32, z, orc.F32, 0, 15, orc.ZP_FLOAT)
    assert np.array_equal(q, A["from_qparams/q"])
    sb = gu.as_f32(A["from_qparams/scale_bf16"], "bf16")
    zb = gu.as_f32(A["from_qparams/zero_bf16"], "bf16")
    dq = orc.dequantize_affine(A["from_qparams/q_in"], [1, 128], sb, orc.BF16, zb, orc.BF16, 0, 15,
                               orc.ZP_FLOAT, orc.BF16)
    assert np.array_equal(orc.f32_to_bf16_bits(dq), A["from_qparams/deq_bf16"])
    s2, z2 = orc.choose_qparams_affine(x, orc.F32, orc.ASYMMETRIC, [1, 128], 0, 15, 1e-6, orc.BF16, orc.BF16,
                                       False, orc.ZP_FLOAT)
    assert np.array_equal(orc.f32_to_bf16_bits(s2), A["from_qparams/legacy_scale_bf16"])
    assert np.array_equal(orc.f32_to_bf16_bits(z2), A["from_qparams/legacy_zero_bf16"])


def test_error_cases_match_reference():
    x = np.zeros((4, 8), np.float32)
    with pytest.raises(ValueError, match="preserve_zero == False is not supported for symmetric"):
        orc.choose_qparams_affine(x, orc.F32, orc.SYMMETRIC, [1, 8], 0, 15, 1e-6, orc.BF16, orc.BF16, False)
    with pytest.raises(ValueError, match="ZeroPointDomain.INT is not supported for symmetric"):
        orc.choose_qparams_affine(x, orc.F32, orc.SYMMETRIC, [1, 8], 0, 15, 1e-6, orc.BF16, orc.BF16, True,
                                  orc.ZP_FLOAT)
    # all-zero per-tensor input: scale == eps of the input dtype (test_quant_primitives.py:385-392)
    s, _ = orc.choose_qparams_affine(np.zeros((10, 10), np.float32), orc.F32, orc.ASYMMETRIC, [10, 10], -128, 127)
    assert s.reshape(-1)[0] == np.float32(np.finfo(np.float32).eps)


@pytest.mark.parametrize("fmt", [(3, 2), (2, 3), (2, 2), (3, 1)])
def test_fpx_codec_matches_reference(fmt):
    e, m = fmt
    A = gu.load("fp6.npz")
    k = f"codec_e{e}m{m}"
    assert np.array_equal(orc.fpx_unpacked_to_f32(A[f"{k}/codes"], e, m).view(np.uint32),
                          A[f"{k}/values"].view(np.uint32))
    assert np.array_equal(orc.f32_to_fpx_unpacked(A[f"{k}/values"], e, m), A[f"{k}/reencoded"])
    assert np.array_equal(orc.f32_to_fpx_unpacked(A[f"{k}/x"], e, m), A[f"{k}/x_codes"])


def test_e3m2_rounding_known_answers():
    """test/prototype/mx_formats/test_custom_cast.py:398-413 of the reference."""
    A = gu.load("fp6.npz")
    x = A["e3m2_rounding/x"]
    assert orc.f32_to_fpx_unpacked(x, 3, 2).tolist() == [0b011111, 0b011110, 0b000010, 0b000001, 0b000000]
    assert np.array_equal(orc.f32_to_fpx_unpacked(x, 3, 2), A["e3m2_rounding/enc"])
    assert np.array_equal(orc.f32_to_fpx_unpacked(-x, 3, 2), A["e3m2_rounding/enc_neg"])


def test_fp6_pack_matches_reference():
    A = gu.load("fp6.npz")
    packed = orc.pack_tc_fp6(A["pack_fp6/bytes_in"] & 0x3F)
    # the reference packs the low 6 bits of each byte; upper bits of random bytes are dropped
    assert np.array_equal(packed, A["pack_fp6/packed"])
    assert np.array_equal(orc.unpack_tc_fp6(A["pack_fp6/packed"]), A["pack_fp6/unpacked"])


@pytest.mark.parametrize("case", MAN["fp6"], ids=lambda c: c["name"])
def test_to_scaled_tc_fp6_matches_reference(case):
    A = gu.load("fp6.npz")
    n = case["name"]
    dt = "f16" if n.endswith("f16") else "f32"
    w = gu.as_f32(A[f"{n}/w"], dt)
    packed, scale = orc.to_scaled_tc_fp6(w)
    assert np.array_equal(packed, A[f"{n}/packed"])
    assert np.array_equal(scale, A[f"{n}/scale"])
    assert np.array_equal(orc.from_scaled_tc_fp6(packed, scale).view(np.uint32), A[f"{n}/dequant_f32"].view(np.uint32))
    assert np.array_equal(orc.from_scaled_tc_fp6(packed).view(np.uint32),
                          A[f"{n}/dequant_noscale_f32"].view(np.uint32))


def test_to_scaled_tc_fp6_zero_weight():
    A = gu.load("fp6.npz")
    packed, scale = orc.to_scaled_tc_fp6(np.zeros((64, 64), np.float32))
    assert np.array_equal(packed, A["scaled_fp6_zero/packed"])
    assert np.array_equal(scale, A["scaled_fp6_zero/scale"])


@pytest.mark.parametrize("case", MAN["linear"], ids=lambda c: c["name"])
def test_int4_linear_oracle(case):
    A = gu.load("linear.npz")
    n, g = case["name"], case["group"]
    w = gu.as_f32(A[f"{n}/w"], "bf16")
    s, z = orc.choose_qparams_affine(w, orc.BF16, orc.ASYMMETRIC, [1, g], 0, 15, 1e-6, orc.BF16, orc.BF16, False,
                                     orc.ZP_FLOAT)
    assert np.array_equal(orc.f32_to_bf16_bits(s), A[f"{n}/scale"])
    assert np.array_equal(orc.f32_to_bf16_bits(z), A[f"{n}/zero"])
    q = orc.quantize_affine(w, orc.BF16, [1, g], s, orc.BF16, z, orc.BF16, 0, 15, orc.ZP_FLOAT)
    assert np.array_equal(q.astype(np.uint8), A[f"{n}/q"])
    sz = orc.pack_tinygemm_scales_and_zeros(A[f"{n}/scale"], A[f"{n}/zero"])
    assert np.array_equal(sz, A[f"{n}/scale_and_zero"])
    assert np.array_equal(orc.pack_2xint4(np.ascontiguousarray(A[f"{n}/q"].T)), A[f"{n}/hqq_packed"])
    wd = orc.dequantize_affine(q, [1, g], s, orc.BF16, z, orc.BF16, 0, 15, orc.ZP_FLOAT, orc.F32)
    for M in case["Ms"]:
        x = gu.as_f32(A[f"{n}/x_m{M}"], "bf16")
        y = orc.linear_f32(x, wd)
        ref = A[f"{n}/y_m{M}"]
        # accumulation order differs from the BLAS the reference used; values agree to fp32 noise
        assert np.max(np.abs(y - ref)) <= 2e-5 * max(1.0, np.max(np.abs(ref)))
        # the timed CPU route (dequantise to bf16 as the reference does, then matmul): rounding every
        # weight to bf16 costs more than the 1e-2 GEMM bar on outlier groups, so only a sanity bound
        yb = orc.int4_linear_dequant_then_matmul(x, A[f"{n}/q"], s, z, g)
        assert np.max(np.abs(yb - ref)) <= 5e-2 * np.max(np.abs(ref))


@pytest.mark.parametrize("case", MAN["fp6_linear"], ids=lambda c: c["name"])
def test_fp6_linear_oracle(case):
    A = gu.load("linear.npz")
    n = case["name"]
    w = gu.as_f32(A[f"{n}/w"], "f16")
    packed, scale = orc.to_scaled_tc_fp6(w)
    assert np.array_equal(packed, A[f"{n}/packed"]) and np.array_equal(scale, A[f"{n}/scale"])
    wd = orc.from_scaled_tc_fp6(packed, scale)
    for M in case["Ms"]:
        x = gu.as_f32(A[f"{n}/x_m{M}"], "f16")
        y = orc.linear_f32(x, wd)
        ref = A[f"{n}/y_m{M}"]
        assert np.max(np.abs(y - ref)) <= 2e-5 * max(1.0, np.max(np.abs(ref)))


def test_tinygemm_pack_roundtrip():
    rng = np.random.default_rng(0)
    for ikt in (2, 4, 8):
        codes = rng.integers(0, 16, size=(16, 256), dtype=np.int32)
        p = orc.pack_tinygemm(codes, ikt)
        assert p.shape == (2, 256 // (ikt * 16), 32, ikt // 2)
        assert np.array_equal(orc.unpack_tinygemm(p), codes)


@pytest.mark.parametrize("key", ["bf16_g64", "bf16_g128", "f16_g64", "f16_g128"])
def test_hqq_quants_to_torch_quants_matches_reference_expressions(key):
    A = gu.load("hqq_convert.npz")
    dt = orc.BF16 if key.startswith("bf16") else orc.F16
    q, nz = orc.hqq_quants_to_torch_quants(A[f"{key}/W_q"], A[f"{key}/scales"], A[f"{key}/zeros"], dt)
    assert np.array_equal(q.reshape(A[f"{key}/q"].shape), A[f"{key}/q"])
    assert np.array_equal(nz.reshape(A[f"{key}/new_zeros"].shape), A[f"{key}/new_zeros"])


@pytest.mark.parametrize("name", ["scaled_e2m3_f16", "scaled_e2m3_f32"])
def test_e2m3_to_scaled_and_from_scaled_match_reference(name):
    A = gu.load("e2m3.npz")
    w = A[f"{name}/w"]
    wf = orc.f16_bits_to_f32(w) if w.dtype == np.uint16 else w.astype(np.float32)
    packed, scale = orc.to_scaled_tc_fp6(wf, 2, 3)
    assert np.array_equal(packed, A[f"{name}/packed"])
    assert np.array_equal(scale, A[f"{name}/scale"])
    assert np.array_equal(orc.from_scaled_tc_fp6(packed, scale, 2, 3), A[f"{name}/dequant_f32"])


def test_generic_tc_packer_matches_reference_for_5_and_6_bits():
    A = gu.load("fp5.npz")
    for key, nbits in (("pack5", 5), ("pack6", 6)):
        packed = orc.pack_tc_fpx(A[f"{key}/codes"], nbits)
        assert np.array_equal(packed, A[f"{key}/packed"])
        assert np.array_equal(orc.unpack_tc_fpx(packed, nbits), A[f"{key}/codes"])
    assert np.array_equal(orc.pack_tc_fpx(A["pack6/codes"], 6), orc.pack_tc_fp6(A["pack6/codes"]))


@pytest.mark.parametrize("fmt", [(2, 2), (3, 1)], ids=["e2m2", "e3m1"])
def test_fp5_to_scaled_and_from_scaled_match_reference(fmt):
    A = gu.load("fp5.npz")
    e, m = fmt
    name = f"e{e}m{m}"
    packed, scale = orc.to_scaled_tc_fpx(orc.f16_bits_to_f32(A[f"{name}/w"]), e, m)
    assert np.array_equal(packed, A[f"{name}/packed"])
    assert np.array_equal(scale, A[f"{name}/scale"])
    assert np.array_equal(orc.from_scaled_tc_fpx(packed, scale, e, m), A[f"{name}/dequant_f32"])
