"""GPU parity of the affine quantization primitives: bit-exact against the reference's recorded
outputs (tests/golden) and against the CPU oracle on larger seeded inputs."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests import golden_util as gu
from tests import gpu_util as tu

pytestmark = pytest.mark.gpu
MAN = gu.manifest()


def _mods():
    from ao_b200.quantization import quant_primitives as qp
    return qp


@pytest.mark.parametrize("case", MAN["primitives"], ids=lambda c: c["name"])
def test_primitives_bit_exact_vs_reference(case):
    qp = _mods()
    A = gu.load("primitives.npz")
    n = case["name"]
    x = tu.to_torch(A[f"{n}/x"], case["in_dt"])
    mapping = qp.MappingType.SYMMETRIC if case["mapping"] == "sym" else qp.MappingType.ASYMMETRIC
    dom = qp.ZeroPointDomain.FLOAT if case["zp_domain"] == "float" else qp.ZeroPointDomain.INT
    sdt = None if case["scale_dt"] is None else tu.TORCH_DT[case["scale_dt"]]
    zdt = None if case["zp_dt"] is None else tu.TORCH_DT[case["zp_dt"]]
    target = tu.TORCH_DT[case["target"]]
    s, z = qp.choose_qparams_affine(x, mapping, tuple(case["block"]), target, case["qmin"], case["qmax"], case["eps"],
                                    scale_dtype=sdt, zero_point_dtype=zdt, preserve_zero=case["preserve_zero"],
                                    zero_point_domain=dom)
    assert str(s.dtype) == "torch." + case["scale_dtype_out"] and str(z.dtype) == "torch." + case["zp_dtype_out"]
    assert tuple(s.shape) == A[f"{n}/scale"].shape
    assert np.array_equal(tu.bits(s), A[f"{n}/scale"]), "scale"
    assert np.array_equal(tu.bits(z), A[f"{n}/zp"]), "zero_point"
    q = qp.quantize_affine(x, tuple(case["block"]), s, z, target, case["qmin"], case["qmax"], dom)
    assert q.dtype == target
    assert np.array_equal(tu.bits(q), A[f"{n}/q"]), "codes"
    for d in case["deq"]:
        dq = qp.dequantize_affine(q, tuple(case["block"]), s, z, target, case["qmin"], case["qmax"], dom,
                                  output_dtype=tu.TORCH_DT[d])
        assert np.array_equal(tu.bits(dq), A[f"{n}/deq_{d}"]), f"dequant {d}"


def test_quantize_dequantize_from_given_qparams():
    from ao_b200.quantization import utils as ut
    A = gu.load("primitives.npz")
    x = tu.to_torch(A["from_qparams/x"], "f32")
    s = tu.to_torch(A["from_qparams/scale"], "f32")
    z = tu.to_torch(A["from_qparams/zero"], "f32")
    q = ut.groupwise_affine_quantize_tensor_from_qparams(x, s, z, 4, 128)
    assert np.array_equal(tu.bits(q), A["from_qparams/q"])
    qi = tu.to_torch(A["from_qparams/q_in"], "i32")
    sb = tu.to_torch(A["from_qparams/scale_bf16"], "bf16")
    zb = tu.to_torch(A["from_qparams/zero_bf16"], "bf16")
    dq = ut.groupwise_affine_dequantize_tensor_from_qparams(qi, sb, zb, 4, 128)
    assert np.array_equal(tu.bits(dq), A["from_qparams/deq_bf16"])
    s2, z2 = ut.get_groupwise_affine_qparams(x, 4, 128, torch.bfloat16)
    assert np.array_equal(tu.bits(s2), A["from_qparams/legacy_scale_bf16"])
    assert np.array_equal(tu.bits(z2), A["from_qparams/legacy_zero_bf16"])


@pytest.mark.parametrize("group", [32, 64, 128, 256])
def test_int4_fast_path_vs_oracle(group):
    """The fused int4 kernels against the oracle on a 512 x 4096 weight with outliers."""
    from ao_b200 import ops
    qp = _mods()
    w = tu.make_weight((512, 4096), seed=100 + group)
    wf = w.float().numpy()
    s_ref, z_ref = orc.choose_qparams_affine(wf, orc.BF16, orc.ASYMMETRIC, [1, group], 0, 15, 1e-6, orc.BF16, orc.BF16,
                                             False, orc.ZP_FLOAT)
    q_ref = orc.quantize_affine(wf, orc.BF16, [1, group], s_ref, orc.BF16, z_ref, orc.BF16, 0, 15, orc.ZP_FLOAT)
    wc = w.cuda()
    s, z, q = ops.int4_groupwise_quantize(wc, group, torch.int32)
    assert np.array_equal(tu.bits(s), orc.f32_to_bf16_bits(s_ref))
    assert np.array_equal(tu.bits(z), orc.f32_to_bf16_bits(z_ref))
    assert np.array_equal(tu.bits(q), q_ref)
    _, _, q8 = ops.int4_groupwise_quantize(wc, group, torch.uint8)
    assert np.array_equal(tu.bits(q8), q_ref.astype(np.uint8))
    # general kernels give the same bits as the fast path
    s2, z2 = qp.choose_qparams_affine(wc, qp.MappingType.ASYMMETRIC, (1, group), torch.int32, 0, 15, 1e-6,
                                      zero_point_dtype=torch.bfloat16, preserve_zero=False,
                                      zero_point_domain=qp.ZeroPointDomain.FLOAT)
    assert torch.equal(s2, s) and torch.equal(z2, z)
    q2 = qp.quantize_affine(wc, (1, group), s, z, torch.int32, 0, 15, qp.ZeroPointDomain.FLOAT)
    assert torch.equal(q2, q)
    for ikt in (8, 4, 2):
        packed, sz = ops.int4_quantize_pack(wc, group, ikt)
        assert np.array_equal(tu.bits(packed), orc.pack_tinygemm(q_ref, ikt))
        assert np.array_equal(tu.bits(sz), orc.pack_tinygemm_scales_and_zeros(orc.f32_to_bf16_bits(s_ref),
                                                                             orc.f32_to_bf16_bits(z_ref)))
    dq = qp.dequantize_affine(q, (1, group), s, z, torch.int32, 0, 15, qp.ZeroPointDomain.FLOAT,
                              output_dtype=torch.bfloat16)
    dq_ref = orc.dequantize_affine(q_ref, [1, group], s_ref, orc.BF16, z_ref, orc.BF16, 0, 15, orc.ZP_FLOAT, orc.BF16)
    assert np.array_equal(tu.bits(dq), orc.f32_to_bf16_bits(dq_ref))


def test_full_size_properties_llama3_gate_up():
    """28672 x 4096, g=64: too large for the scalar oracle in a test, so size-independent properties:
    idempotence, fused == unfused, codes in range, reconstruction error bounded by half a step."""
    from ao_b200 import ops
    qp = _mods()
    g = torch.Generator(device="cuda").manual_seed(3)
    w = (torch.randn(28672, 4096, generator=g, device="cuda") * 0.02).bfloat16()
    s, z, q = ops.int4_groupwise_quantize(w, 64, torch.int32)
    s1, z1, q1 = ops.int4_groupwise_quantize(w, 64, torch.int32)
    assert torch.equal(s, s1) and torch.equal(z, z1) and torch.equal(q, q1)
    assert int(q.min()) >= 0 and int(q.max()) <= 15
    packed, sz = ops.int4_quantize_pack(w, 64, 8)
    assert torch.equal(packed, ops.convert_weight_to_int4pack(q, 8))
    assert torch.equal(ops.unpack_int4pack(packed), q)
    assert torch.equal(sz[..., 0].t().contiguous(), s) and torch.equal(sz[..., 1].t().contiguous(), z)
    dq = qp.dequantize_affine(q, (1, 64), s, z, torch.int32, 0, 15, qp.ZeroPointDomain.FLOAT, output_dtype=torch.float32)
    err = (dq - w.float()).abs().view(28672, 64, 64).amax(-1)
    # half a quantization step, plus what the bf16 rounding of scale / zero / recomputed minimum can add
    # (the recomputed minimum differs from the true one in a few percent of the groups, which clamps)
    bound = s.float() * 1.5 + 1e-6
    assert bool((err <= bound).all())
    assert float((err <= s.float() * 0.75).float().mean()) > 0.9
    # re-quantizing the dequantized weight with the same qparams returns the same codes
    q_again = qp.quantize_affine(dq.bfloat16(), (1, 64), s, z, torch.int32, 0, 15, qp.ZeroPointDomain.FLOAT)
    assert (q_again != q).float().mean().item() < 1e-3


def test_empty_and_degenerate_inputs():
    qp = _mods()
    x = torch.zeros(0, 64, device="cuda", dtype=torch.bfloat16)
    s, z = qp.choose_qparams_affine(x, qp.MappingType.ASYMMETRIC, (1, 64), torch.int32, 0, 15, 1e-6,
                                    zero_point_dtype=torch.bfloat16, preserve_zero=False,
                                    zero_point_domain=qp.ZeroPointDomain.FLOAT)
    assert s.shape == (0,) and z.shape == (0,)
    # all-zero tensor, per-tensor: scale == eps of the dtype (test_quant_primitives.py:385-392 of the reference)
    s, z = qp.choose_qparams_affine(torch.zeros(10, 10, device="cuda"), qp.MappingType.ASYMMETRIC, (10, 10), torch.int8)
    assert float(s) == float(torch.finfo(torch.float32).eps)


@pytest.mark.parametrize("cfg", [
    # (dtype, mapping, block, target, qmin, qmax, domain, preserve_zero)
    ("bf16", "asym", (1, 64), "int32", 0, 15, "float", False),      # int4 weight-only setting, general entry points
    ("bf16", "asym", (1, 32), "uint8", 0, 255, "int", True),
    ("f16", "asym", (1, 128), "int32", 0, 15, "float", False),
    ("f32", "sym", (1, 256), "int8", -128, 127, "int", True),
    ("bf16", "sym", (1, 2048), "int8", -128, 127, "int", True),     # per row: one warp per block
    ("f32", "asym", (1, 24), "int32", 0, 15, "float", False),       # 3 vectors per block: warp-per-block kernel
], ids=lambda c: "-".join(map(str, c)))
def test_vectorised_primitives_vs_oracle_large(cfg):
    """The 128-bit-load variants of choose / quantize / dequantize (contiguous blocks) on 1.5 M elements."""
    qp = _mods()
    dt, mapping, block, target, qmin, qmax, dom, pz = cfg
    odt = {"bf16": orc.BF16, "f16": orc.F16, "f32": orc.F32}[dt]
    tdt = tu.TORCH_DT[dt]
    cols = 2048 if 2048 % block[1] == 0 else block[1] * 64
    g = torch.Generator().manual_seed(sum(block) + qmax)
    x = (torch.randn(768, cols, generator=g) * 0.05).to(tdt)
    xf = x.float().numpy()
    m = orc.SYMMETRIC if mapping == "sym" else orc.ASYMMETRIC
    d = orc.ZP_FLOAT if dom == "float" else orc.ZP_INT
    zdt_o = odt if dom == "float" else orc.I32
    s_ref, z_ref = orc.choose_qparams_affine(xf, odt, m, list(block), qmin, qmax, None, odt, zdt_o, pz, d)
    q_ref = orc.quantize_affine(xf, odt, list(block), s_ref, odt, z_ref, zdt_o, qmin, qmax, d)
    dq_ref = orc.dequantize_affine(q_ref, list(block), s_ref, odt, z_ref, zdt_o, qmin, qmax, d, odt)
    M = qp.MappingType.SYMMETRIC if mapping == "sym" else qp.MappingType.ASYMMETRIC
    D = qp.ZeroPointDomain.FLOAT if dom == "float" else qp.ZeroPointDomain.INT
    zdt_t = tdt if dom == "float" else torch.int32
    s, z = qp.choose_qparams_affine(x.cuda(), M, block, tu.TORCH_DT[target], qmin, qmax, None, scale_dtype=tdt,
                                    zero_point_dtype=zdt_t, preserve_zero=pz, zero_point_domain=D)

    def same(t, ref, ref_dt):
        if ref_dt == orc.BF16:
            return np.array_equal(tu.bits(t), orc.f32_to_bf16_bits(ref).reshape(tu.bits(t).shape))
        if ref_dt == orc.F16:
            return np.array_equal(tu.bits(t), np.asarray(ref, np.float32).astype(np.float16).view(np.uint16).reshape(tu.bits(t).shape))
        return np.array_equal(tu.bits(t).reshape(-1), np.asarray(ref).reshape(-1).astype(tu.bits(t).dtype))

    assert same(s, s_ref, odt), "scale"
    assert same(z, z_ref, zdt_o if dom == "float" else orc.I32), "zero point"
    q = qp.quantize_affine(x.cuda(), block, s, z, tu.TORCH_DT[target], qmin, qmax, D)
    assert np.array_equal(tu.bits(q).astype(np.int64), np.asarray(q_ref).astype(np.int64)), "codes"
    dq = qp.dequantize_affine(q, block, s, z, q.dtype, qmin, qmax, D, output_dtype=tdt)
    assert same(dq, dq_ref, odt), "dequantized"
