"""Checkpoint round trips of quantized models, after test/quantization/test_quant_api.py:192-218 (state_dict of an
unwrapped model saved, loaded and copied into a freshly quantized model) and :605-620 (state_dict that holds the tensor
subclasses themselves, loaded with assign=True), for the int4 tensor_core_tiled AffineQuantizedTensor and for
QuantLlmLinearWeight (fp6).  Outputs before and after must be bit-identical."""
import copy
import io

import pytest
import torch

pytestmark = pytest.mark.gpu


class ToyLinearModel(torch.nn.Module):
    def __init__(self, m=1024, n=512, k=256, dtype=torch.bfloat16):
        super().__init__()
        self.linear1 = torch.nn.Linear(m, n, bias=False).to(dtype)
        self.linear2 = torch.nn.Linear(n, k, bias=True).to(dtype)

    def forward(self, x):
        return self.linear2(self.linear1(x))


def _save_load(state_dict):
    f = io.BytesIO()
    torch.save(state_dict, f)
    f.seek(0)
    return torch.load(f)          # the default weights_only=True: the subclasses are registered as safe globals


def _apis():
    from ao_b200.prototype.quant_llm import fp6_llm_weight_only
    from ao_b200.quantization import int4_weight_only
    return {"int4_tiled": (int4_weight_only(group_size=64), torch.bfloat16),
            "fp6": (fp6_llm_weight_only(), torch.float16)}


@pytest.mark.parametrize("kind", ["int4_tiled", "fp6"])
def test_state_dict_of_subclasses_save_load_assign(kind):
    """test_quant_api.py:605-620: save the quantized model's state_dict, load it into an unquantized copy with
    assign=True."""
    from ao_b200.quantization import quantize
    api, dtype = _apis()[kind]
    torch.manual_seed(0)
    m = ToyLinearModel(dtype=dtype).eval().cuda()
    m_copy = copy.deepcopy(m)
    x = torch.randn(3, 1024, device="cuda", dtype=dtype)
    quantize(m, api)
    ref = m(x)
    state_dict = _save_load(m.state_dict())
    assert type(state_dict["linear1.weight"]) is type(m.linear1.weight)
    m_copy.load_state_dict(state_dict, assign=True)
    assert type(m_copy.linear1.weight) is type(m.linear1.weight)
    assert torch.equal(m_copy(x), ref)


@pytest.mark.parametrize("kind", ["int4_tiled", "fp6"])
def test_state_dict_into_meta_model_assign(kind):
    """The usual way to load a quantized checkpoint: build the model on the meta device, assign the loaded tensors."""
    from ao_b200.quantization import quantize
    api, dtype = _apis()[kind]
    torch.manual_seed(1)
    m = ToyLinearModel(dtype=dtype).eval().cuda()
    x = torch.randn(2, 5, 1024, device="cuda", dtype=dtype)
    quantize(m, api)
    ref = m(x)
    state_dict = _save_load(m.state_dict())
    with torch.device("meta"):
        m2 = ToyLinearModel(dtype=dtype).eval()
    m2.load_state_dict(state_dict, assign=True)
    assert m2.linear1.weight.device.type == "cuda" and m2.linear2.bias.device.type == "cuda"
    assert torch.equal(m2(x), ref)


@pytest.mark.parametrize("kind", ["int4_tiled", "fp6"])
def test_unwrapped_state_dict_save_load(kind):
    """test_quant_api.py:192-218: quantize + unwrap_tensor_subclass, save the (plain-tensor) state_dict, load it into
    a second model prepared the same way."""
    from ao_b200.quantization import quantize
    from ao_b200.utils import unwrap_tensor_subclass
    api, dtype = _apis()[kind]

    def prepare(model):
        quantize(model, api)
        unwrap_tensor_subclass(model)
        return model

    torch.manual_seed(2)
    m = prepare(ToyLinearModel(dtype=dtype).eval().cuda())
    x = torch.randn(4, 1024, device="cuda", dtype=dtype)
    ref = m(x)
    sd = m.state_dict()
    assert all(type(v) is torch.Tensor for v in sd.values()), {k: type(v) for k, v in sd.items()}
    state_dict = _save_load(sd)
    torch.manual_seed(3)                                    # different weights until the checkpoint is loaded
    m2 = prepare(ToyLinearModel(dtype=dtype).eval().cuda())
    assert not torch.equal(m2(x), ref)
    m2.load_state_dict(state_dict)
    assert torch.equal(m2(x), ref)
