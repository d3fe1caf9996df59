"""The dispatcher ops (ao_b200/_torch_ops.py) without a GPU: schemas exist, fake implementations give the right
shapes and raise the reference's messages (torchao/ops.py:40-55, test/test_ops.py:24-45)."""
import pytest
import torch
from torch._subclasses.fake_tensor import FakeTensorMode

import ao_b200._torch_ops  # noqa: F401  (registers the ops)


def test_schemas_registered():
    assert str(torch.ops.ao_b200.quant_llm_linear.default._schema).startswith("ao_b200::quant_llm_linear(int EXPONENT")
    assert "qGroupSize" in str(torch.ops.ao_b200.weight_int4pack_mm.default._schema)
    assert "innerKTiles" in str(torch.ops.ao_b200.convert_weight_to_int4pack.default._schema)


def test_fake_implementations_shapes():
    with FakeTensorMode():
        x = torch.empty(5, 512, dtype=torch.float16, device="cuda")
        w = torch.empty(256, 512 // 8 * 6, dtype=torch.uint8, device="cuda")
        s = torch.empty(256, dtype=torch.float16, device="cuda")
        y = torch.ops.ao_b200.quant_llm_linear(3, 2, x, w, s, 1)
        assert y.shape == (5, 256) and y.dtype == torch.float16 and y.device.type == "cuda"
        codes = torch.empty(64, 1024, dtype=torch.int32, device="cuda")
        packed = torch.ops.ao_b200.convert_weight_to_int4pack(codes, 8)
        assert packed.shape == (8, 8, 32, 4) and packed.dtype == torch.int32
        xb = torch.empty(3, 1024, dtype=torch.bfloat16, device="cuda")
        sz = torch.empty(1024 // 64, 64, 2, dtype=torch.bfloat16, device="cuda")
        out = torch.ops.ao_b200.weight_int4pack_mm(xb, packed, 64, sz)
        assert out.shape == (3, 64) and out.dtype == torch.bfloat16


def test_fake_implementations_raise_like_the_reference():
    with FakeTensorMode():
        x = torch.empty(5, 512, dtype=torch.float16, device="cuda")
        w = torch.empty(256, 384, dtype=torch.uint8, device="cuda")
        s = torch.empty(256, dtype=torch.float16, device="cuda")
        with pytest.raises(RuntimeError, match="input should be a 2d tensor"):
            torch.ops.ao_b200.quant_llm_linear(3, 2, x.reshape(-1), w, s, 1)
        with pytest.raises(RuntimeError, match="weight must be FP16"):
            torch.ops.ao_b200.quant_llm_linear(3, 2, x.float(), w, s, 1)
        with pytest.raises(RuntimeError, match="Dimensions mismatched"):
            torch.ops.ao_b200.quant_llm_linear(3, 2, x, w[:, :100], s, 1)
        with pytest.raises(RuntimeError, match="Dimensions mismatched"):
            torch.ops.ao_b200.quant_llm_linear(3, 2, x, w, s[:10], 1)
        with pytest.raises(RuntimeError, match="innerKTiles must be 2, 4, or 8"):
            torch.ops.ao_b200.convert_weight_to_int4pack(torch.empty(64, 1024, dtype=torch.int32, device="cuda"), 3)
