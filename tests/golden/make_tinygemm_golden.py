"""Pins the tensor_core_tiled weight layout with PyTorch's own tinygemm operators.

The layout is defined by aten::_convert_weight_to_int4pack (PyTorch ATen, not part of the
reference checkout).  This script runs on a machine WITH a CUDA GPU:

    python tests/golden/make_tinygemm_golden.py [out_dir]

and writes tinygemm.npz: seeded int4 codes, the packed tensors the installed torch produces for
inner_k_tiles 2/4/8, and the codes recovered by pushing an identity matrix through
aten::_weight_int4pack_mm (scale 1, zero 0), which checks the layout's meaning independently of
any packing code here.  The installed torch takes two codes per byte ([n][k/2] uint8, even k in
the high nibble); the reference revision passed one code per int32 — same output layout.
"""
import os
import sys

import numpy as np
import torch


def main():
    out_dir = sys.argv[1] if len(sys.argv) > 1 else os.path.dirname(os.path.abspath(__file__))
    rng = np.random.default_rng(20240607)
    N, K = 64, 1024
    codes = rng.integers(0, 16, size=(N, K), dtype=np.int32)
    ct = torch.from_numpy(codes).cuda()
    arrays = {"codes": codes, "torch_version": np.array(torch.__version__)}
    orders = {}
    for name, u8 in (("even_k_high_nibble", (ct[:, ::2] << 4 | ct[:, 1::2]).to(torch.uint8)),
                     ("even_k_low_nibble", (ct[:, 1::2] << 4 | ct[:, ::2]).to(torch.uint8))):
        try:
            packed = torch.ops.aten._convert_weight_to_int4pack(u8.contiguous(), 8)
        except Exception as e:  # noqa: BLE001
            orders[name] = f"failed: {e}"
            continue
        # identity through the matmul: y[k][n] = (q[n][k] - 8) * 1 + 0
        sz = torch.zeros(K // 32, N, 2, dtype=torch.bfloat16, device="cuda")
        sz[..., 0] = 1
        eye = torch.eye(K, dtype=torch.bfloat16, device="cuda")
        y = torch.ops.aten._weight_int4pack_mm(eye, packed, 32, sz)
        rec = (y.float().t() + 8).round().to(torch.int32)
        orders[name] = bool(torch.equal(rec, ct))
        if orders[name]:
            arrays["input_order"] = np.array(name)
            for ikt in (2, 4, 8):
                arrays[f"packed_ikt{ikt}"] = torch.ops.aten._convert_weight_to_int4pack(u8.contiguous(), ikt).cpu().numpy()
            arrays["recovered_codes"] = rec.cpu().numpy()
    print("nibble orders that reproduce the codes through _weight_int4pack_mm:", orders)
    # the reference-era signature (int32 [n][k]) for the record
    try:
        p_old = torch.ops.aten._convert_weight_to_int4pack(ct, 8)
        arrays["packed_ikt8_int32_input"] = p_old.cpu().numpy()
        print("int32 [n][k] input accepted")
    except Exception as e:  # noqa: BLE001
        print("int32 [n][k] input rejected:", str(e)[:120])
    # a numeric golden for the matmul itself on a small problem
    g = torch.Generator().manual_seed(7)
    x = torch.randn(4, K, generator=g).bfloat16().cuda()
    scale = (torch.rand(N, K // 64, generator=g) * 0.02 + 0.001).bfloat16()
    zero = (torch.randn(N, K // 64, generator=g) * 0.01).bfloat16()
    sz = torch.stack([scale, zero], 2).transpose(0, 1).contiguous().cuda()
    if "packed_ikt8" in arrays:
        y = torch.ops.aten._weight_int4pack_mm(x, torch.from_numpy(arrays["packed_ikt8"]).cuda(), 64, sz)
        arrays["mm_x"] = x.cpu().view(torch.int16).numpy().view(np.uint16)
        arrays["mm_scale"] = scale.view(torch.int16).numpy().view(np.uint16)
        arrays["mm_zero"] = zero.view(torch.int16).numpy().view(np.uint16)
        arrays["mm_y"] = y.cpu().view(torch.int16).numpy().view(np.uint16)
    os.makedirs(out_dir, exist_ok=True)
    np.savez_compressed(os.path.join(out_dir, "tinygemm.npz"), **arrays)
    print("wrote", os.path.join(out_dir, "tinygemm.npz"))


if __name__ == "__main__":
    main()
