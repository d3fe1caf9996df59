"""The dispatcher ops (ao_b200/_torch_ops.py) without a GPU: schemas exist, fake implementations give the right
shapes and raise the reference's messages (torchao/ops.py:40-55, test/test_ops.py:24-45)."""
import pytest
import torch
from torch._subclasses.fake_tensor import FakeTensorMode

import ao_b200._torch_ops  # noqa: F401  (loads the compiled operator library, registers the fake implementations)


def test_torchao_import_names_resolve():
    """The reference's import names work unchanged (torchao/__init__.py, quantization/__init__.py, ops.py)."""
    import torchao
    from torchao.dtypes import AffineQuantizedTensor, to_affine_quantized  # noqa: F401
    from torchao.prototype.quant_llm import QuantLlmLinearWeight, fp6_llm_weight_only  # noqa: F401
    from torchao.quantization import int4_weight_only, quantize  # noqa: F401
    from torchao.quantization.quant_primitives import choose_qparams_affine, dequantize_affine, quantize_affine  # noqa: F401
    from torchao.utils import unwrap_tensor_subclass  # noqa: F401
    import ao_b200.quantization
    assert quantize is ao_b200.quantization.quantize
    assert callable(torchao.ops.quant_llm_linear) and callable(torchao.ops.prepack_fp6_weight)


def test_schemas_registered():
    assert str(torch.ops.torchao.quant_llm_linear.default._schema).startswith("torchao::quant_llm_linear(int EXPONENT")
    assert "qGroupSize" in str(torch.ops.torchao._weight_int4pack_mm.default._schema)
    assert "innerKTiles" in str(torch.ops.torchao._convert_weight_to_int4pack.default._schema)


def test_fake_implementations_shapes():
    with FakeTensorMode():
        x = torch.empty(5, 512, dtype=torch.float16, device="cuda")
        w = torch.empty(256, 512 // 8 * 6, dtype=torch.uint8, device="cuda")
        s = torch.empty(256, dtype=torch.float16, device="cuda")
        y = torch.ops.torchao.quant_llm_linear(3, 2, x, w, s, 1)
        assert y.shape == (5, 256) and y.dtype == torch.float16 and y.device.type == "cuda"
        codes = torch.empty(64, 1024, dtype=torch.int32, device="cuda")
        packed = torch.ops.torchao._convert_weight_to_int4pack(codes, 8)
        assert packed.shape == (8, 8, 32, 4) and packed.dtype == torch.int32
        xb = torch.empty(3, 1024, dtype=torch.bfloat16, device="cuda")
        sz = torch.empty(1024 // 64, 64, 2, dtype=torch.bfloat16, device="cuda")
        out = torch.ops.torchao._weight_int4pack_mm(xb, packed, 64, sz)
        assert out.shape == (3, 64) and out.dtype == torch.bfloat16


def test_fake_implementations_raise_like_the_reference():
    with FakeTensorMode():
        x = torch.empty(5, 512, dtype=torch.float16, device="cuda")
        w = torch.empty(256, 384, dtype=torch.uint8, device="cuda")
        s = torch.empty(256, dtype=torch.float16, device="cuda")
        with pytest.raises(RuntimeError, match="input should be a 2d tensor"):
            torch.ops.torchao.quant_llm_linear(3, 2, x.reshape(-1), w, s, 1)
        with pytest.raises(RuntimeError, match="weight must be FP16"):
            torch.ops.torchao.quant_llm_linear(3, 2, x.float(), w, s, 1)
        with pytest.raises(RuntimeError, match="Dimensions mismatched"):
            torch.ops.torchao.quant_llm_linear(3, 2, x, w[:, :100], s, 1)
        with pytest.raises(RuntimeError, match="Dimensions mismatched"):
            torch.ops.torchao.quant_llm_linear(3, 2, x, w, s[:10], 1)
        with pytest.raises(RuntimeError, match="innerKTiles must be 2, 4, or 8"):
            torch.ops.torchao._convert_weight_to_int4pack(torch.empty(64, 1024, dtype=torch.int32, device="cuda"), 3)
