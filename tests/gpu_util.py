"""torch <-> numpy plumbing for the GPU parity tests (bf16 / fp16 travel as uint16 bit patterns)."""
import numpy as np
import torch

from oracle import oracle as orc

TORCH_DT = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16, "i32": torch.int32,
            "i64": torch.int64, "i8": torch.int8, "u8": torch.uint8,
            "float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16,
            "int32": torch.int32, "int64": torch.int64, "int8": torch.int8, "uint8": torch.uint8}


def to_torch(arr, dt, device="cuda"):
    """Fixture array -> torch tensor of dtype dt on device."""
    tdt = TORCH_DT[dt]
    if tdt in (torch.bfloat16, torch.float16):
        return torch.from_numpy(np.ascontiguousarray(arr).view(np.int16)).view(tdt).to(device)
    return torch.from_numpy(np.ascontiguousarray(arr)).to(tdt).to(device)


def bits(t):
    """torch tensor -> numpy array in the fixture representation."""
    t = t.detach().cpu().contiguous()
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.numpy()


def f32(t):
    """torch tensor -> float32 numpy values."""
    return t.detach().float().cpu().numpy()


def bf16_from_f32(values, device="cuda"):
    """float32 numpy values (exact in bf16) -> bf16 tensor."""
    return to_torch(orc.f32_to_bf16_bits(values), "bf16", device)


def make_weight(shape, seed, dtype=torch.bfloat16, outliers=True):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(*shape, generator=g) * 0.02
    if outliers:
        mask = torch.rand(*shape, generator=g) < 0.001
        w = torch.where(mask, w * 20, w)
    return w.to(dtype)
