"""Loading of the golden fixtures (tests/golden/*.npz) and dtype plumbing shared by the tests."""
import json
import os

import numpy as np

from oracle import oracle as orc

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
DT_CODE = {"f32": orc.F32, "f16": orc.F16, "bf16": orc.BF16, "i32": orc.I32, "i64": orc.I64,
           "i8": orc.I8, "u8": orc.U8, "float32": orc.F32, "float16": orc.F16, "bfloat16": orc.BF16,
           "int32": orc.I32, "int64": orc.I64, "int8": orc.I8, "uint8": orc.U8}
_cache = {}


def manifest():
    with open(os.path.join(GOLDEN, "manifest.json")) as f:
        return json.load(f)


def load(fname):
    if fname not in _cache:
        with np.load(os.path.join(GOLDEN, fname)) as z:
            _cache[fname] = {k: z[k] for k in z.files}
    return _cache[fname]


def as_f32(arr, dt):
    """Fixture array (uint16 bit patterns for bf16 / fp16) -> float32 values."""
    if dt in ("bf16", "bfloat16"):
        return orc.bf16_bits_to_f32(arr)
    if dt in ("f16", "float16"):
        return orc.f16_bits_to_f32(arr)
    return np.asarray(arr).astype(np.float32)


def bits_of(values_f32, dt):
    """float32 values that are exact in dt -> the stored representation used by the fixtures."""
    if dt in ("bf16", "bfloat16"):
        return orc.f32_to_bf16_bits(values_f32)
    if dt in ("f16", "float16"):
        return np.asarray(values_f32, np.float32).astype(np.float16).view(np.uint16)
    return values_f32
