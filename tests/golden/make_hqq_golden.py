"""Golden vectors for hqq_quants_to_torch_quants (torchao/prototype/hqq/hqq_tinygemm_linear.py:173-208).

The reference's module imports the third-party `hqq` package at its top and cannot be imported here; the method body
is a short sequence of torch tensor expressions, evaluated below with the CPU build of torch in the same order and
dtypes, so that every intermediate is rounded exactly as in the reference.  Run once:  python make_hqq_golden.py
"""
import os

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def reference_expressions(W_q, scales, zeros, shape, nbits, compute_dtype):
    W_q = W_q.to(dtype=compute_dtype)
    scales = scales.to(dtype=compute_dtype)
    zeros = zeros.to(dtype=compute_dtype)
    max_int, min_int, dump = 2 ** nbits - 1, 0, 2 ** (nbits - 1)
    new_zeros = (scales * dump) - zeros * scales
    min_val = new_zeros - scales * dump
    W_r = (W_q - zeros) * scales
    W_q = W_r.sub(min_val).div(scales).round().clamp_(min_int, max_int).to(torch.int32).reshape(shape).contiguous()
    return W_q, scales.contiguous().reshape(shape[0], -1), new_zeros.contiguous().reshape(shape[0], -1)


def bits(t):
    return t.view(torch.int16).numpy().view(np.uint16) if t.dtype in (torch.bfloat16, torch.float16) else t.numpy()


def main():
    out = {}
    gen = torch.Generator().manual_seed(1234)
    for name, dt in (("bf16", torch.bfloat16), ("f16", torch.float16)):
        for g in (64, 128):
            N, K = 48, 512
            W_q = torch.randint(0, 16, (N * K // g, g), dtype=torch.uint8, generator=gen)
            scales = (torch.rand(N * K // g, 1, generator=gen) * 0.02 + 1e-3).to(dt)
            zeros = (torch.rand(N * K // g, 1, generator=gen) * 15).to(dt)
            q, s, nz = reference_expressions(W_q, scales, zeros, (N, K), 4, dt)
            key = f"{name}_g{g}"
            out[f"{key}/W_q"] = W_q.numpy()
            out[f"{key}/scales"] = bits(scales)
            out[f"{key}/zeros"] = bits(zeros)
            out[f"{key}/q"] = q.numpy()
            out[f"{key}/new_zeros"] = bits(nz)
    np.savez_compressed(os.path.join(HERE, "hqq_convert.npz"), **out)
    print("wrote hqq_convert.npz with", len(out), "arrays")


if __name__ == "__main__":
    main()
