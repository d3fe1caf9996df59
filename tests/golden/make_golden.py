"""Generates the golden fixtures in this directory from the REFERENCE implementation.

Run once, in a container that has the reference checkout (it is not available
where the GPU tests run):

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's own hot-path modules (torchao 0.3.1) on CPU and
records their outputs on seeded inputs:

  primitives.npz   choose_qparams_affine / quantize_affine / dequantize_affine for the int4
                   fast path and the other granularities / domains, plus the legacy tinygemm
                   formulas the reference's tests compare against
                   (test/quantization/test_quant_primitives.py:50-127, 451-504)
  fp6.npz          _f32_to_fpx_unpacked / _fpx_unpacked_to_f32 on all 64 codes, the rounding
                   known answers (test/prototype/mx_formats/test_custom_cast.py:398-413),
                   _pack_tc_fp6 == _pack_tc_fpx(.., 6) on random bytes
                   (test/prototype/test_quant_llm.py:28-33), to_scaled_tc_fpx / from_scaled_tc_fpx
  linear.npz       fp32 dequant-matmul outputs (x @ dequantize_affine(W_q).T and
                   x @ from_scaled_tc_fpx(w).T) on small seeded problems, pack_2xint4,
                   pack_tinygemm_scales_and_zeros
  manifest.json    parameters of every case

`import torchao` fails under recent torch (an unrelated autoquant import), so the needed
modules are loaded through stub parent packages.
"""
import importlib
import json
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference(ref):
    def stub(name, path):
        m = types.ModuleType(name)
        m.__path__ = [path]
        sys.modules[name] = m

    stub("torchao", f"{ref}/torchao")
    stub("torchao.quantization", f"{ref}/torchao/quantization")
    stub("torchao.prototype", f"{ref}/torchao/prototype")
    stub("torchao.prototype.quant_llm", f"{ref}/torchao/prototype/quant_llm")
    stub("torchao.prototype.hqq", f"{ref}/torchao/prototype/hqq")
    stub("torchao.dtypes", f"{ref}/torchao/dtypes")
    lib = torch.library.Library("torchao", "FRAGMENT")
    lib.define("quant_llm_linear(int EXPONENT, int MANTISSA, Tensor _in_feats, Tensor _weights, "
               "Tensor _scales, int splitK) -> Tensor")
    mods = {}
    for name in ["torchao.quantization.quant_primitives", "torchao.quantization.utils",
                 "torchao.prototype.custom_fp_utils", "torchao.prototype.quant_llm.quant_llm"]:
        mods[name.split(".")[-1]] = importlib.import_module(name)
    mods["_lib"] = lib
    return mods


DT = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16, "i32": torch.int32,
      "i64": torch.int64, "i8": torch.int8, "u8": torch.uint8}


def store(t):
    """bf16 / fp16 tensors are stored as their uint16 bit patterns."""
    t = t.detach().contiguous()
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.numpy()


def make_weight(shape, dtype, seed, outliers=True):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(*shape, generator=g) * 0.02
    if outliers:
        mask = torch.rand(*shape, generator=g) < 0.001
        w = torch.where(mask, w * 20, w)
    return w.to(dtype)


def primitives(mods, arrays, manifest):
    qp = mods["quant_primitives"]
    MT, ZD = qp.MappingType, qp.ZeroPointDomain
    cases = [
        # the int4 weight-only fast path (quant_api.py:372-385)
        dict(name="int4_g64_bf16", in_dt="bf16", shape=[64, 512], block=[1, 64], mapping="asym",
             target="i32", qmin=0, qmax=15, eps=1e-6, scale_dt=None, zp_dt="bf16", preserve_zero=False,
             zp_domain="float", deq=["bf16", "f32"], seed=1),
        dict(name="int4_g128_bf16", in_dt="bf16", shape=[48, 1024], block=[1, 128], mapping="asym",
             target="i32", qmin=0, qmax=15, eps=1e-6, scale_dt=None, zp_dt="bf16", preserve_zero=False,
             zp_domain="float", deq=["bf16", "f32"], seed=2),
        dict(name="int4_g32_bf16", in_dt="bf16", shape=[16, 256], block=[1, 32], mapping="asym",
             target="i32", qmin=0, qmax=15, eps=1e-6, scale_dt=None, zp_dt="bf16", preserve_zero=False,
             zp_domain="float", deq=["bf16"], seed=3),
        dict(name="int4_g256_bf16", in_dt="bf16", shape=[16, 1024], block=[1, 256], mapping="asym",
             target="i32", qmin=0, qmax=15, eps=1e-6, scale_dt=None, zp_dt="bf16", preserve_zero=False,
             zp_domain="float", deq=["bf16"], seed=4),
        dict(name="int4_g64_f16", in_dt="f16", shape=[32, 256], block=[1, 64], mapping="asym",
             target="i32", qmin=0, qmax=15, eps=1e-6, scale_dt=None, zp_dt="bf16", preserve_zero=False,
             zp_domain="float", deq=["f16", "f32"], seed=5),
        dict(name="int4_g64_f32", in_dt="f32", shape=[32, 256], block=[1, 64], mapping="asym",
             target="i32", qmin=0, qmax=15, eps=1e-6, scale_dt=None, zp_dt="bf16", preserve_zero=False,
             zp_domain="float", deq=["f32", "bf16"], seed=6),
        # legacy tinygemm helper setting: fp32 input, bf16 scale/zero (test_quant_primitives.py:451-480)
        dict(name="tinygemm_qparams_f32_in", in_dt="f32", shape=[10, 256], block=[1, 128], mapping="asym",
             target="i8", qmin=0, qmax=15, eps=1e-6, scale_dt="bf16", zp_dt="bf16", preserve_zero=False,
             zp_domain="float", deq=["bf16"], seed=7, randn_unit=True),
        # all-zero group exercises the eps clamp
        dict(name="int4_g64_zero_rows", in_dt="bf16", shape=[8, 128], block=[1, 64], mapping="asym",
             target="i32", qmin=0, qmax=15, eps=1e-6, scale_dt=None, zp_dt="bf16", preserve_zero=False,
             zp_domain="float", deq=["bf16"], seed=8, zero_rows=True),
        # other granularities / domains (test_quant_primitives.py:165-371)
        dict(name="int8_sym_per_channel_f32", in_dt="f32", shape=[10, 10], block=[1, 10], mapping="sym",
             target="i8", qmin=None, qmax=None, eps=None, scale_dt="f32", zp_dt="i64", preserve_zero=True,
             zp_domain="int", deq=["f32"], seed=9, randn_unit=True),
        dict(name="int8_sym_per_channel_bf16", in_dt="bf16", shape=[24, 96], block=[1, 96], mapping="sym",
             target="i8", qmin=-127, qmax=127, eps=None, scale_dt=None, zp_dt="i64", preserve_zero=True,
             zp_domain="int", deq=["bf16", "f32"], seed=10, randn_unit=True),
        dict(name="int8_asym_per_tensor_f32", in_dt="f32", shape=[10, 10], block=[10, 10], mapping="asym",
             target="i8", qmin=None, qmax=None, eps=None, scale_dt="f32", zp_dt="i32", preserve_zero=True,
             zp_domain="int", deq=["f32"], seed=11, randn_unit=True),
        dict(name="uint8_asym_per_token_f16", in_dt="f16", shape=[3, 5, 32], block=[1, 1, 32], mapping="asym",
             target="u8", qmin=None, qmax=None, eps=None, scale_dt="f32", zp_dt="i32", preserve_zero=True,
             zp_domain="int", deq=["f16", "f32"], seed=12, randn_unit=True),
        dict(name="int8_sym_group_axis0_f32", in_dt="f32", shape=[64, 12], block=[16, 1], mapping="sym",
             target="i8", qmin=-8, qmax=7, eps=1e-5, scale_dt="f32", zp_dt="i32", preserve_zero=True,
             zp_domain="int", deq=["f32"], seed=13, randn_unit=True),
        dict(name="int8_asym_4d_blocks_bf16", in_dt="bf16", shape=[3, 4, 10, 8], block=[3, 2, 5, 1], mapping="asym",
             target="i8", qmin=None, qmax=None, eps=None, scale_dt="f32", zp_dt="f32", preserve_zero=True,
             zp_domain="int", deq=["bf16"], seed=14, randn_unit=True),
        dict(name="int4_group_int_domain_bf16", in_dt="bf16", shape=[32, 128], block=[1, 32], mapping="asym",
             target="i32", qmin=0, qmax=15, eps=1e-6, scale_dt=None, zp_dt="i32", preserve_zero=True,
             zp_domain="int", deq=["bf16", "f32"], seed=15),
    ]
    for c in cases:
        dt = DT[c["in_dt"]]
        if c.get("randn_unit"):
            g = torch.Generator().manual_seed(c["seed"])
            x = torch.randn(*c["shape"], generator=g).to(dt)
        else:
            x = make_weight(c["shape"], dt, c["seed"])
        if c.get("zero_rows"):
            x[::2] = 0
        mapping = MT.SYMMETRIC if c["mapping"] == "sym" else MT.ASYMMETRIC
        dom = ZD.FLOAT if c["zp_domain"] == "float" else ZD.INT
        sdt = None if c["scale_dt"] is None else DT[c["scale_dt"]]
        zdt = None if c["zp_dt"] is None else DT[c["zp_dt"]]
        s, z = qp.choose_qparams_affine(x, mapping, tuple(c["block"]), DT[c["target"]], c["qmin"], c["qmax"],
                                        c["eps"], scale_dtype=sdt, zero_point_dtype=zdt,
                                        preserve_zero=c["preserve_zero"], zero_point_domain=dom)
        q = qp.quantize_affine(x, tuple(c["block"]), s, z, DT[c["target"]], c["qmin"], c["qmax"], dom)
        n = c["name"]
        arrays[f"{n}/x"] = store(x)
        arrays[f"{n}/scale"] = store(s)
        arrays[f"{n}/zp"] = store(z)
        arrays[f"{n}/q"] = store(q)
        c["scale_dtype_out"] = str(s.dtype).replace("torch.", "")
        c["zp_dtype_out"] = str(z.dtype).replace("torch.", "")
        for d in c["deq"]:
            dq = qp.dequantize_affine(q, tuple(c["block"]), s, z, DT[c["target"]], c["qmin"], c["qmax"], dom,
                                      output_dtype=DT[d])
            arrays[f"{n}/deq_{d}"] = store(dq)
        manifest["primitives"].append(c)

    # quantize/dequantize with externally supplied (random, possibly negative) qparams, as
    # test_quant_primitives.py:482-504 does against the legacy formulas.
    ut = mods["utils"]
    g = torch.Generator().manual_seed(21)
    inp = torch.randn(10, 256, generator=g)
    sc = torch.randn(10, 2, generator=g)
    ze = torch.randn(10, 2, generator=g)
    arrays["from_qparams/x"] = store(inp)
    arrays["from_qparams/scale"] = store(sc)
    arrays["from_qparams/zero"] = store(ze)
    arrays["from_qparams/q"] = store(ut.groupwise_affine_quantize_tensor_from_qparams(inp, sc, ze, 4, 128))
    qi = torch.randint(0, 15, (10, 256), dtype=torch.int32, generator=g)
    scb, zeb = sc.bfloat16(), ze.bfloat16()
    arrays["from_qparams/q_in"] = store(qi)
    arrays["from_qparams/scale_bf16"] = store(scb)
    arrays["from_qparams/zero_bf16"] = store(zeb)
    arrays["from_qparams/deq_bf16"] = store(ut.groupwise_affine_dequantize_tensor_from_qparams(qi, scb, zeb, 4, 128))
    # legacy formula of the reference's own test file (test_quant_primitives.py:50-69), restated
    to_quant = inp.reshape(-1, 128)
    mx, mn = to_quant.amax(1, keepdim=True), to_quant.amin(1, keepdim=True)
    scales = (mx - mn).clamp(min=1e-6) / 15
    zeros = mn + scales * 8
    arrays["from_qparams/legacy_scale_bf16"] = store(scales.bfloat16().reshape(10, -1))
    arrays["from_qparams/legacy_zero_bf16"] = store(zeros.bfloat16().reshape(10, -1))
    s2, z2 = ut.get_groupwise_affine_qparams(inp, 4, 128, torch.bfloat16)
    assert torch.equal(s2, scales.bfloat16().reshape(10, -1)) and torch.equal(z2, zeros.bfloat16().reshape(10, -1))


def fp6(mods, arrays, manifest):
    cf = mods["custom_fp_utils"]
    ql = mods["quant_llm"]
    for (e, m) in [(3, 2), (2, 3), (2, 2), (3, 1)]:
        nb = 1 + e + m
        codes = torch.arange(2 ** nb, dtype=torch.uint8)
        vals = cf._fpx_unpacked_to_f32(codes, e, m)
        back = cf._f32_to_fpx_unpacked(vals, e, m)
        arrays[f"codec_e{e}m{m}/codes"] = store(codes)
        arrays[f"codec_e{e}m{m}/values"] = store(vals)
        arrays[f"codec_e{e}m{m}/reencoded"] = store(back)
        g = torch.Generator().manual_seed(100 + nb * 10 + e)
        x = torch.cat([torch.randn(4096, generator=g) * 4, torch.randn(2048, generator=g) * 0.05,
                       torch.randn(1024, generator=g) * 40,
                       # exact ties between neighbouring codes and values next to them
                       ((vals[:-1] + vals[1:]) / 2), torch.tensor([0.0, -0.0, 1e-30, -1e-30, 1e30, -1e30])])
        arrays[f"codec_e{e}m{m}/x"] = store(x)
        arrays[f"codec_e{e}m{m}/x_codes"] = store(cf._f32_to_fpx_unpacked(x, e, m))
    kat = torch.tensor([29.0, 26.0, 0.1251, 0.0314, 0.03])
    arrays["e3m2_rounding/x"] = store(kat)
    arrays["e3m2_rounding/enc"] = store(cf._f32_to_fpx_unpacked(kat, 3, 2))
    arrays["e3m2_rounding/enc_neg"] = store(cf._f32_to_fpx_unpacked(-kat, 3, 2))
    assert arrays["e3m2_rounding/enc"].tolist() == [0b011111, 0b011110, 0b000010, 0b000001, 0]

    g = torch.Generator().manual_seed(31)
    xb = torch.randint(256, size=(256, 64), dtype=torch.uint8, generator=g)
    fast, generic = ql._pack_tc_fp6(xb), ql._pack_tc_fpx(xb, 6)
    assert torch.equal(fast, generic)
    arrays["pack_fp6/bytes_in"] = store(xb)
    arrays["pack_fp6/packed"] = store(fast)
    arrays["pack_fp6/unpacked"] = store(ql._unpack_tc_fp6(fast))

    for name, shape, dt, seed in [("scaled_fp6_f16", (128, 192), torch.float16, 32),
                                  ("scaled_fp6_f32", (64, 128), torch.float32, 33)]:
        w = make_weight(shape, dt, seed, outliers=False)
        packed, scale = ql.to_scaled_tc_fpx(w, 3, 2)
        arrays[f"{name}/w"] = store(w)
        arrays[f"{name}/packed"] = store(packed)
        arrays[f"{name}/scale"] = store(scale)
        arrays[f"{name}/dequant_f32"] = store(ql.from_scaled_tc_fpx(packed, 3, 2, scale))
        arrays[f"{name}/dequant_noscale_f32"] = store(ql.from_scaled_tc_fpx(packed, 3, 2))
        manifest["fp6"].append(dict(name=name, shape=list(shape)))
    w0 = torch.zeros(64, 64)
    packed, scale = ql.to_scaled_tc_fpx(w0, 3, 2)
    arrays["scaled_fp6_zero/packed"] = store(packed)
    arrays["scaled_fp6_zero/scale"] = store(scale)


def linear(mods, arrays, manifest):
    qp = mods["quant_primitives"]
    ut = mods["utils"]
    ql = mods["quant_llm"]
    MT, ZD = qp.MappingType, qp.ZeroPointDomain
    for name, N, K, gs, Ms, seed in [("int4_lin_g64", 64, 1024, 64, [1, 4, 16], 41),
                                     ("int4_lin_g128", 48, 2048, 128, [1, 8], 42),
                                     ("int4_lin_g32_m64", 128, 1024, 32, [64], 43)]:
        w = make_weight((N, K), torch.bfloat16, seed)
        s, z = qp.choose_qparams_affine(w, MT.ASYMMETRIC, (1, gs), torch.int32, 0, 15, 1e-6,
                                        zero_point_dtype=torch.bfloat16, preserve_zero=False,
                                        zero_point_domain=ZD.FLOAT)
        q = qp.quantize_affine(w, (1, gs), s, z, torch.int32, 0, 15, ZD.FLOAT)
        wd = qp.dequantize_affine(q, (1, gs), s, z, torch.int32, 0, 15, ZD.FLOAT, output_dtype=torch.float32)
        arrays[f"{name}/w"] = store(w)
        arrays[f"{name}/scale"] = store(s)
        arrays[f"{name}/zero"] = store(z)
        arrays[f"{name}/q"] = store(q.to(torch.uint8))
        arrays[f"{name}/scale_and_zero"] = store(ut.pack_tinygemm_scales_and_zeros(s, z))
        # transposed-rows nibble packing of the HQQ path (mixed_mm.py:13-33 applied to W_q.T)
        t = q.to(torch.uint8).T.contiguous()
        t = t.reshape(t.shape[0] // 2, 2, t.shape[1]).permute(1, 0, 2)
        arrays[f"{name}/hqq_packed"] = store((t[0] & 0xF) | (t[1] << 4))
        g = torch.Generator().manual_seed(seed + 100)
        for M in Ms:
            x = torch.randn(M, K, generator=g).bfloat16()
            arrays[f"{name}/x_m{M}"] = store(x)
            arrays[f"{name}/y_m{M}"] = store(x.float() @ wd.T)
        manifest["linear"].append(dict(name=name, N=N, K=K, group=gs, Ms=Ms))
    for name, N, K, Ms, seed in [("fp6_lin", 256, 512, [1, 16, 64], 51)]:
        w = make_weight((N, K), torch.float16, seed, outliers=False)
        packed, scale = ql.to_scaled_tc_fpx(w, 3, 2)
        wd = ql.from_scaled_tc_fpx(packed, 3, 2, scale)
        arrays[f"{name}/w"] = store(w)
        arrays[f"{name}/packed"] = store(packed)
        arrays[f"{name}/scale"] = store(scale)
        g = torch.Generator().manual_seed(seed + 100)
        for M in Ms:
            x = torch.randn(M, K, generator=g).half()
            arrays[f"{name}/x_m{M}"] = store(x)
            arrays[f"{name}/y_m{M}"] = store(x.float() @ wd.T)
        manifest["fp6_linear"].append(dict(name=name, N=N, K=K, Ms=Ms))


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: python " + sys.argv[0] + " <path of a torchao 0.3.1 source tree>")
    ref = sys.argv[1]
    mods = load_reference(ref)
    manifest = {"reference": "torchao 0.3.1", "torch": torch.__version__, "primitives": [], "fp6": [],
                "linear": [], "fp6_linear": []}
    for fname, fn in [("primitives.npz", primitives), ("fp6.npz", fp6), ("linear.npz", linear)]:
        arrays = {}
        fn(mods, arrays, manifest)
        np.savez_compressed(os.path.join(HERE, fname), **arrays)
        print(fname, len(arrays), "arrays", os.path.getsize(os.path.join(HERE, fname)) // 1024, "KiB")
    with open(os.path.join(HERE, "manifest.json"), "w") as f:
        json.dump(manifest, f, indent=1)


if __name__ == "__main__":
    main()
