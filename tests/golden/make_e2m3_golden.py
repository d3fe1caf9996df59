"""Golden vectors for the second 6-bit format the reference's linear dispatches, fp6 e2m3
(torchao/csrc/cuda/fp6_llm/fp6_linear.cu:181-182): to_scaled_tc_fpx / from_scaled_tc_fpx of the reference
(torchao/prototype/quant_llm/quant_llm.py:116-130, 203-208) and the fp32 dequant-matmul.
Run once:  python make_e2m3_golden.py /path/to/reference
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from make_golden import load_reference, make_weight, store  # noqa: E402


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: python " + sys.argv[0] + " <path of a torchao 0.3.1 source tree>")
    ref = sys.argv[1]
    ql = load_reference(ref)["quant_llm"]
    arrays = {}
    for name, shape, dt, seed in [("scaled_e2m3_f16", (128, 192), torch.float16, 62), ("scaled_e2m3_f32", (64, 128), torch.float32, 63)]:
        w = make_weight(shape, dt, seed, outliers=False)
        packed, scale = ql.to_scaled_tc_fpx(w, 2, 3)
        arrays[f"{name}/w"] = store(w)
        arrays[f"{name}/packed"] = store(packed)
        arrays[f"{name}/scale"] = store(scale)
        arrays[f"{name}/dequant_f32"] = store(ql.from_scaled_tc_fpx(packed, 2, 3, scale))
    N, K = 256, 512
    w = make_weight((N, K), torch.float16, 71, outliers=False)
    packed, scale = ql.to_scaled_tc_fpx(w, 2, 3)
    wd = ql.from_scaled_tc_fpx(packed, 2, 3, scale)
    arrays["e2m3_lin/w"] = store(w)
    arrays["e2m3_lin/packed"] = store(packed)
    arrays["e2m3_lin/scale"] = store(scale)
    g = torch.Generator().manual_seed(171)
    for M in (1, 16, 64):
        x = torch.randn(M, K, generator=g).half()
        arrays[f"e2m3_lin/x_m{M}"] = store(x)
        arrays[f"e2m3_lin/y_m{M}"] = store(x.float() @ wd.T)
    np.savez_compressed(os.path.join(HERE, "e2m3.npz"), **arrays)
    print("e2m3.npz", len(arrays), "arrays")


if __name__ == "__main__":
    main()
