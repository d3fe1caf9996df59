"""GPU tests of the user-facing API: quantize(m, int4_weight_only(..)), AffineQuantizedTensor and its layouts,
modelled on test/quantization/test_quant_api.py and test/integration/test_integration.py of the reference."""
import copy

import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests import gpu_util as tu

pytestmark = pytest.mark.gpu


def _sqnr(x, y):
    x, y = x.detach().float(), y.detach().float()
    return float(20 * torch.log10(torch.linalg.norm(x) / torch.linalg.norm(x - y)))


@pytest.mark.parametrize("group_size", [32, 64, 128, 256])
@pytest.mark.parametrize("inner_k_tiles", [8, 4, 2])
def test_quantize_int4_weight_only_linear(group_size, inner_k_tiles):
    from ao_b200.dtypes import AffineQuantizedTensor, TensorCoreTiledAQTLayout
    from ao_b200.quantization import int4_weight_only, quantize
    torch.manual_seed(0)
    m = torch.nn.Sequential(torch.nn.Linear(1024, 1024, bias=False), torch.nn.Linear(1024, 512, bias=True))
    m = m.to(device="cuda", dtype=torch.bfloat16)
    ref = copy.deepcopy(m)
    out = quantize(m, int4_weight_only(group_size=group_size, inner_k_tiles=inner_k_tiles))
    assert out is m
    for lin in m:
        assert isinstance(lin.weight, AffineQuantizedTensor)
        assert isinstance(lin.weight.layout_tensor, TensorCoreTiledAQTLayout)
        assert lin.weight.shape == lin.weight.dequantize().shape
    x = torch.randn(2, 1024, device="cuda", dtype=torch.bfloat16)
    y, y_ref = m(x), ref(x)
    assert y.dtype == torch.bfloat16 and y.shape == y_ref.shape
    assert _sqnr(y_ref, y) >= 10  # test_integration.py:735-763
    # quantizing twice does not touch already quantized weights
    w0 = m[0].weight
    quantize(m, int4_weight_only(group_size=group_size))
    assert m[0].weight is w0


def test_int4_aqt_matches_oracle_bit_for_bit():
    from ao_b200.dtypes import to_affine_quantized
    from ao_b200.quantization import MappingType, ZeroPointDomain
    w = tu.make_weight((256, 2048), seed=4)
    aqt = to_affine_quantized(w.cuda(), MappingType.ASYMMETRIC, (1, 64), torch.int32, 0, 15, 1e-6,
                              zero_point_dtype=torch.bfloat16, preserve_zero=False,
                              zero_point_domain=ZeroPointDomain.FLOAT, extended_layout="tensor_core_tiled",
                              inner_k_tiles=8)
    wf = w.float().numpy()
    s, z = orc.choose_qparams_affine(wf, orc.BF16, orc.ASYMMETRIC, [1, 64], 0, 15, 1e-6, orc.BF16, orc.BF16, False,
                                     orc.ZP_FLOAT)
    q = orc.quantize_affine(wf, orc.BF16, [1, 64], s, orc.BF16, z, orc.BF16, 0, 15, orc.ZP_FLOAT)
    int_data, scale, zero = aqt.layout_tensor.get_plain()
    assert np.array_equal(tu.bits(int_data), q)
    assert np.array_equal(tu.bits(scale), orc.f32_to_bf16_bits(s))
    assert np.array_equal(tu.bits(zero), orc.f32_to_bf16_bits(z))
    assert np.array_equal(tu.bits(aqt.layout_tensor.packed_weight), orc.pack_tinygemm(q, 8))
    dq = orc.dequantize_affine(q, [1, 64], s, orc.BF16, z, orc.BF16, 0, 15, orc.ZP_FLOAT, orc.BF16)
    assert np.array_equal(tu.bits(aqt.dequantize()), orc.f32_to_bf16_bits(dq))
    # the fused constructor and the step-by-step route (plain -> from_plain) agree
    plain = to_affine_quantized(w.cuda(), MappingType.ASYMMETRIC, (1, 64), torch.int32, 0, 15, 1e-6,
                                zero_point_dtype=torch.bfloat16, preserve_zero=False,
                                zero_point_domain=ZeroPointDomain.FLOAT)
    assert torch.equal(plain.layout_tensor.int_data, int_data)
    assert _sqnr(w.cuda(), aqt.dequantize()) >= 15  # test_integration.py:631-658


def test_plain_layout_linear_takes_dequantize_route():
    """Config "runs on CPU today" of the reference: x @ dequantize_affine(W_q).T, here on the GPU."""
    from ao_b200.dtypes import to_affine_quantized
    from ao_b200.quantization import MappingType, ZeroPointDomain
    w = tu.make_weight((4096, 4096), seed=1234, outliers=False)
    x = torch.randn(1, 4096, generator=torch.Generator().manual_seed(1234)).bfloat16()
    aqt = to_affine_quantized(w.cuda(), MappingType.ASYMMETRIC, (1, 64), torch.int32, 0, 15, 1e-6,
                              zero_point_dtype=torch.bfloat16, preserve_zero=False,
                              zero_point_domain=ZeroPointDomain.FLOAT)
    y = torch.nn.functional.linear(x.cuda(), aqt)
    y_ref = x.cuda().float() @ aqt.dequantize(torch.float32).T
    assert float((y.float() - y_ref).abs().max() / y_ref.abs().max()) <= 2e-2


def test_odd_shapes_are_padded_like_the_reference():
    from ao_b200.quantization import int4_weight_only, quantize
    torch.manual_seed(1)
    lin = torch.nn.Linear(1000, 260, bias=True, device="cuda", dtype=torch.bfloat16)
    ref = copy.deepcopy(lin)
    quantize(lin, int4_weight_only(group_size=32))
    assert tuple(lin.weight.shape) == (260, 1000)
    assert tuple(lin.weight.layout_tensor.packed_weight.shape) == (264 // 8, 1024 // 128, 32, 4)
    x = torch.randn(3, 5, 1000, device="cuda", dtype=torch.bfloat16)
    y = lin(x)
    assert y.shape == (3, 5, 260)
    assert _sqnr(ref(x), y) >= 10


def test_state_dict_roundtrip_and_flatten():
    from ao_b200.dtypes import AffineQuantizedTensor
    from ao_b200.quantization import int4_weight_only, quantize
    torch.manual_seed(2)
    m = torch.nn.Sequential(torch.nn.Linear(1024, 256, bias=False)).to(device="cuda", dtype=torch.bfloat16)
    quantize(m, int4_weight_only(group_size=128))
    x = torch.randn(4, 1024, device="cuda", dtype=torch.bfloat16)
    y = m(x)
    w = m[0].weight
    names, attrs = w.__tensor_flatten__()
    assert names == ["layout_tensor"]
    inner_names, inner_attrs = w.layout_tensor.__tensor_flatten__()
    assert inner_names == ["packed_weight", "scale_and_zero"]
    layout2 = type(w.layout_tensor).__tensor_unflatten__(
        {n: getattr(w.layout_tensor, n).clone() for n in inner_names}, inner_attrs, None, None)
    w2 = AffineQuantizedTensor.__tensor_unflatten__({"layout_tensor": layout2}, attrs, None, None)
    m2 = torch.nn.Sequential(torch.nn.Linear(1024, 256, bias=False)).to(device="cuda", dtype=torch.bfloat16)
    m2[0].weight = torch.nn.Parameter(w2, requires_grad=False)
    assert torch.equal(m2(x), y)
    sd = m.state_dict()
    assert isinstance(sd["0.weight"], AffineQuantizedTensor)


def test_bias_is_fused_with_the_bits_of_the_separate_add():
    """F.linear with a bias on an int4 tensor_core_tiled weight: the kernels add the bias in their stores, and the
    result has the bits of `y = linear(x, w); y += bias` (affine_quantized_tensor.py:638-640) for the decode kernel,
    the tcgen05 kernel and the 16-row block route."""
    from ao_b200 import ops
    from ao_b200.quantization import int4_weight_only, quantize
    torch.manual_seed(5)
    lin = torch.nn.Linear(2048, 512, bias=True, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        lin.bias.mul_(3.0)
    quantize(lin, int4_weight_only(group_size=64))
    lt = lin.weight.layout_tensor
    for M in (1, 5, 8, 16, 64, 300):
        x = torch.randn(M, 2048, device="cuda", dtype=torch.bfloat16)
        lin(x)                                   # first call builds the plan
        y = lin(x)                               # fast path: fused bias
        ref = ops.weight_int4pack_mm(x, lt.packed_weight, 64, lt.scale_and_zero)
        ref += lin.bias
        assert torch.equal(y, ref), f"M={M}"


def test_fp6_bias_is_fused_with_the_bits_of_the_separate_add():
    """F.linear with an fp16 bias on a QuantLlmLinearWeight: one kernel, and the bits of
    `out = quant_llm_linear(...); out += bias` (quant_llm.py:433-445) on the decode kernel (with and without K slabs),
    the tcgen05 kernel and the 16-row block route; for every FPx format."""
    from ao_b200 import ops
    from ao_b200.prototype.quant_llm import quant_llm_fpx_weight_only
    from ao_b200.quantization import quantize
    torch.manual_seed(6)
    for ebits, mbits in ((3, 2), (2, 3), (2, 2), (3, 1)):
        lin = torch.nn.Linear(1024, 512, bias=True, device="cuda", dtype=torch.float16)
        with torch.no_grad():
            lin.bias.mul_(3.0)
        quantize(lin, quant_llm_fpx_weight_only(ebits, mbits))
        w = lin.weight
        for M in (1, 5, 8, 16, 64, 300):
            x = torch.randn(M, 1024, device="cuda", dtype=torch.float16)
            y = lin(x)
            ref = ops.quant_llm_linear(ebits, mbits, x, w.fpx_data, w.scale)
            ref += lin.bias
            assert y.dtype == torch.float16 and torch.equal(y, ref), f"e{ebits}m{mbits} M={M}"
        with pytest.raises(RuntimeError):
            ops.quant_llm_linear_bias(ebits, mbits, x, w.fpx_data, w.scale, lin.bias.float())


def test_filter_fn_and_transpose():
    from ao_b200.dtypes import AffineQuantizedTensor
    from ao_b200.quantization import int4_weight_only, quantize
    m = torch.nn.Sequential(torch.nn.Linear(1024, 64), torch.nn.Linear(64, 1024)).to(device="cuda", dtype=torch.bfloat16)
    quantize(m, int4_weight_only(group_size=32), filter_fn=lambda mod, fqn: isinstance(mod, torch.nn.Linear) and fqn == "0")
    assert isinstance(m[0].weight, AffineQuantizedTensor) and not isinstance(m[1].weight, AffineQuantizedTensor)
    wt = m[0].weight.t()
    assert wt.shape == (1024, 64)  # test/dtypes/test_affine_quantized.py:12-26


def test_clone_makes_independent_storage():
    from ao_b200.quantization import int4_weight_only, quantize
    lin = torch.nn.Linear(1024, 64, bias=False, device="cuda", dtype=torch.bfloat16)
    quantize(lin, int4_weight_only(group_size=64))
    w = lin.weight
    c = w.clone()
    assert c.layout_tensor.packed_weight.data_ptr() != w.layout_tensor.packed_weight.data_ptr()
    assert torch.equal(c.layout_tensor.packed_weight, w.layout_tensor.packed_weight)
    x = torch.randn(2, 1024, device="cuda", dtype=torch.bfloat16)
    assert torch.equal(torch.nn.functional.linear(x, c), lin(x))


def test_dispatcher_ops_opcheck():
    """torch.ops.torchao.*: the four checks the reference runs on its operator (test/test_ops.py:24-45) - schema,
    autograd registration, fake tensor, AOT dispatch with dynamic shapes - and equality with the direct calls."""
    import torchao  # noqa: F401
    from ao_b200 import ops
    from torch.library import opcheck
    utils = ["test_schema", "test_autograd_registration", "test_faketensor", "test_aot_dispatch_dynamic"]
    w = torch.randint(256, (256, 512 // 8 * 6), dtype=torch.uint8, device="cuda")
    s = torch.rand(256, dtype=torch.float16, device="cuda") + 0.5
    x = torch.rand(5, 512, dtype=torch.float16, device="cuda") + 0.5
    opcheck(torch.ops.torchao.quant_llm_linear, (3, 2, x, w, s, 1), test_utils=utils)
    assert torch.equal(torch.ops.torchao.quant_llm_linear(3, 2, x, w, s, 1), ops.quant_llm_linear(3, 2, x, w, s, 1))
    assert torch.equal(torchao.ops.quant_llm_linear(3, 2, x, w, s, 1), ops.quant_llm_linear(3, 2, x, w, s, 1))
    codes = torch.randint(0, 16, (64, 1024), dtype=torch.int32, device="cuda")
    opcheck(torch.ops.torchao._convert_weight_to_int4pack, (codes, 8), test_utils=utils)
    packed = torch.ops.torchao._convert_weight_to_int4pack(codes, 8)
    assert torch.equal(packed, ops.convert_weight_to_int4pack(codes, 8))
    sz = torch.rand(1024 // 64, 64, 2, device="cuda").bfloat16()
    xb = torch.randn(3, 1024, device="cuda").bfloat16()
    opcheck(torch.ops.torchao._weight_int4pack_mm, (xb, packed, 64, sz), test_utils=utils)
    assert torch.equal(torch.ops.torchao._weight_int4pack_mm(xb, packed, 64, sz), ops.weight_int4pack_mm(xb, packed, 64, sz))
    with pytest.raises(RuntimeError, match="is not supported"):
        torch.ops.torchao.quant_llm_linear(2, 1, x, torch.zeros(256, 256, dtype=torch.uint8, device="cuda"), s, 1)
