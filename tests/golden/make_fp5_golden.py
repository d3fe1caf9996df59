"""Golden vectors for the 5-bit formats of the reference's linear (e2m2, e3m1): generic pre-packing
_pack_tc_fpx / _unpack_tc_fpx on random codes, to_scaled_tc_fpx / from_scaled_tc_fpx, and the fp32 dequant-matmul
(torchao/prototype/quant_llm/quant_llm.py:60-86, 116-130, 134-208).  Run once:  python make_fp5_golden.py /path/to/reference"""
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
    g = torch.Generator().manual_seed(5)
    codes = torch.randint(0, 32, (128, 192), dtype=torch.uint8, generator=g)
    arrays["pack5/codes"] = store(codes)
    arrays["pack5/packed"] = store(ql._pack_tc_fpx(codes, 5))
    assert torch.equal(ql._unpack_tc_fpx(ql._pack_tc_fpx(codes, 5), 5), codes)
    codes6 = torch.randint(0, 64, (64, 128), dtype=torch.uint8, generator=g)
    arrays["pack6/codes"] = store(codes6)
    arrays["pack6/packed"] = store(ql._pack_tc_fpx(codes6, 6))
    for e, m in ((2, 2), (3, 1)):
        name = f"e{e}m{m}"
        w = make_weight((128, 192), torch.float16, 80 + e, outliers=False)
        packed, scale = ql.to_scaled_tc_fpx(w, e, m)
        arrays[f"{name}/w"] = store(w)
        arrays[f"{name}/packed"] = store(packed)
        arrays[f"{name}/scale"] = store(scale)
        arrays[f"{name}/dequant_f32"] = store(ql.from_scaled_tc_fpx(packed, e, m, scale))
        N, K = 256, 512
        w = make_weight((N, K), torch.float16, 90 + e, outliers=False)
        packed, scale = ql.to_scaled_tc_fpx(w, e, m)
        wd = ql.from_scaled_tc_fpx(packed, e, m, scale)
        arrays[f"{name}_lin/w"] = store(w)
        arrays[f"{name}_lin/packed"] = store(packed)
        arrays[f"{name}_lin/scale"] = store(scale)
        gx = torch.Generator().manual_seed(190 + e)
        for M in (1, 16, 64):
            x = torch.randn(M, K, generator=gx).half()
            arrays[f"{name}_lin/x_m{M}"] = store(x)
            arrays[f"{name}_lin/y_m{M}"] = store(x.float() @ wd.T)
    np.savez_compressed(os.path.join(HERE, "fp5.npz"), **arrays)
    print("fp5.npz", len(arrays), "arrays")


if __name__ == "__main__":
    main()
