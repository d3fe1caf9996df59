"""GPU parity of the HQQ-layout fused int4 GEMM (mixed_mm / triton_mixed_mm), after test/hqq/test_triton_mm.py of the
reference: c = a @ ((W_q - zeros) * scales).T with W_q packed by pack_2xint4(W_q.T).  The HQQ quantiser itself is a
third-party package; as in the reference's dependency-free variant the codes are synthetic, and a second case takes
scales / zeros from choose_qparams_affine converted to HQQ's convention (z_hqq = 8 - z / s)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _reference(x, W_q, scales, zeros, g):
    """fp32 dequant-matmul: scales / zeros [N][K/g]."""
    N, K = W_q.shape
    s = scales.float().repeat_interleave(g, dim=1)
    z = zeros.float().repeat_interleave(g, dim=1)
    return x.float() @ ((W_q.float() - z) * s).T


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "fp16"])
@pytest.mark.parametrize("group_size", [32, 64, 128, 256])
@pytest.mark.parametrize("shape", [(16, 128, 256), (16, 4096, 4096), (100, 1024, 2048), (300, 512, 1024), (1, 256, 512)],
                         ids=lambda s: "x".join(map(str, s)))
def test_mixed_mm_synthetic_codes(shape, group_size, dtype):
    from ao_b200 import _cabi
    from ao_b200.prototype.hqq import pack_2xint4, triton_mixed_mm
    M, N, K = shape
    g = torch.Generator(device="cuda").manual_seed(M + N + K + group_size)
    W_q = torch.randint(0, 16, (N, K), dtype=torch.uint8, device="cuda", generator=g)
    scales = (torch.rand(N, K // group_size, device="cuda", generator=g) * 0.01 + 0.002).to(dtype)
    zeros = (torch.rand(N, K // group_size, device="cuda", generator=g) * 15).to(dtype)
    x = torch.randn(M, K, device="cuda", generator=g).to(dtype)
    packed_w = pack_2xint4(W_q.T)
    assert packed_w.shape == (K // 2, N)
    out = triton_mixed_mm(x, packed_w, scales.T, zeros.T, transposed=False, group_size=group_size, fp8_fast_accum=False,
                          kernel_type="compute_bound")
    assert out.shape == (M, N) and out.dtype == dtype
    ref = _reference(x, W_q, scales, zeros, group_size)
    err = float((out.float() - ref).abs().max() / ref.abs().max())
    assert err <= 1e-2, err
    out2 = triton_mixed_mm(x, packed_w, scales.T, zeros.T, group_size=group_size)
    assert torch.equal(out, out2), "two runs must give identical bits"
    assert _cabi.workspace_status("cuda") == 0


@pytest.mark.parametrize("M", [64, 256, 1024])
def test_mixed_mm_hqq_style_quantized_weight(M):
    """Config 'HQQ-style int4 asymmetric with float zero point, axis=1, group 64' at a reduced size."""
    from ao_b200 import ops
    from ao_b200.prototype.hqq import mixed_mm, pack_hqq_from_rowmajor
    from tests import gpu_util as tu
    N, K, g = 2048, 2048, 64
    w = tu.make_weight((N, K), seed=11, outliers=False).cuda()
    s, z, codes = ops.int4_groupwise_quantize(w, g, want_codes=torch.uint8)
    z_hqq = (8.0 - z.float() / s.float()).to(torch.bfloat16)
    x = torch.randn(M, K, generator=torch.Generator().manual_seed(M)).bfloat16().cuda()
    out = mixed_mm(x, pack_hqq_from_rowmajor(codes), s.T, z_hqq.T, g)
    ref = _reference(x, codes, s, z_hqq, g)
    assert float((out.float() - ref).abs().max() / ref.abs().max()) <= 1e-2
    # and it still is the original layer to within int4 quantization noise
    y0 = x.float() @ w.float().T
    assert float(20 * torch.log10(y0.norm() / (y0 - out.float()).norm())) >= 15


def test_mixed_mm_argument_checks():
    from ao_b200.prototype.hqq import mixed_mm
    a = torch.zeros(4, 256, dtype=torch.bfloat16, device="cuda")
    b = torch.zeros(128, 128, dtype=torch.uint8, device="cuda")
    s = torch.zeros(4, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(AssertionError, match="incompatible dimensions"):
        mixed_mm(a[:, :128], b, s, s, 64)
    with pytest.raises(AssertionError):
        mixed_mm(a, b, s.half(), s.half(), 64)
    with pytest.raises(AssertionError, match="transpose requires"):
        mixed_mm(a[:, :100], b, s, s, 64, transposed=True)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "fp16"])
@pytest.mark.parametrize("group_size", [32, 64, 128, 256])
@pytest.mark.parametrize("shape", [(16, 128, 256), (16, 4096, 4096), (100, 1024, 2048), (300, 512, 1024)],
                         ids=lambda s: "x".join(map(str, s)))
def test_mixed_mm_transposed(shape, group_size, dtype):
    """transposed=True: (M x N) x (K x N) -> (M x K), reduction along N (test/hqq/test_triton_mm.py:115-127)."""
    from ao_b200.prototype.hqq import pack_2xint4, triton_mixed_mm
    M, N, K = shape
    g = torch.Generator(device="cuda").manual_seed(M + N + K + group_size)
    W_q = torch.randint(0, 16, (N, K), dtype=torch.uint8, device="cuda", generator=g)
    scales = (torch.rand(N, K // group_size, device="cuda", generator=g) * 0.01 + 0.002).to(dtype)
    zeros = (torch.rand(N, K // group_size, device="cuda", generator=g) * 15).to(dtype)
    x = torch.randn(M, N, device="cuda", generator=g).to(dtype)
    out = triton_mixed_mm(x, pack_2xint4(W_q.T), scales.T, zeros.T, transposed=True, group_size=group_size)
    assert out.shape == (M, K) and out.dtype == dtype
    s = scales.float().repeat_interleave(group_size, dim=1)
    z = zeros.float().repeat_interleave(group_size, dim=1)
    ref = x.float() @ ((W_q.float() - z) * s)
    assert float((out.float() - ref).abs().max() / ref.abs().max()) <= 1e-2


@pytest.mark.parametrize("key", ["bf16_g64", "bf16_g128", "f16_g64", "f16_g128"])
def test_hqq_quants_to_torch_quants_bit_exact(key):
    from ao_b200.prototype.hqq import hqq_quants_to_torch_quants
    from tests import golden_util as gu
    from tests import gpu_util as tu
    A = gu.load("hqq_convert.npz")
    dt = "bf16" if key.startswith("bf16") else "f16"
    tdt = torch.bfloat16 if dt == "bf16" else torch.float16
    W_q = torch.from_numpy(A[f"{key}/W_q"]).cuda()
    scales, zeros = tu.to_torch(A[f"{key}/scales"], dt), tu.to_torch(A[f"{key}/zeros"], dt)
    shape = tuple(A[f"{key}/q"].shape)
    q, s, nz = hqq_quants_to_torch_quants(W_q, scales, zeros, shape, compute_dtype=tdt)
    assert q.dtype == torch.int32 and tuple(q.shape) == shape
    assert np.array_equal(q.cpu().numpy(), A[f"{key}/q"])
    assert np.array_equal(tu.bits(nz), A[f"{key}/new_zeros"])
    assert np.array_equal(tu.bits(s).reshape(-1), A[f"{key}/scales"].reshape(-1))


def test_hqq_weight_through_both_int4_linears():
    """The same HQQ-convention weight through mixed_mm (HQQ layout) and, converted, through the tinygemm linear."""
    from ao_b200 import ops
    from ao_b200.prototype.hqq import hqq_to_tinygemm_weight, mixed_mm, pack_2xint4
    N, K, g, M = 512, 1024, 64, 48
    gen = torch.Generator(device="cuda").manual_seed(3)
    W_q = torch.randint(0, 16, (N, K), dtype=torch.uint8, device="cuda", generator=gen)
    scales = (torch.rand(N, K // g, device="cuda", generator=gen) * 0.01 + 0.002).bfloat16()
    zeros = (torch.rand(N, K // g, device="cuda", generator=gen) * 15).bfloat16()
    x = torch.randn(M, K, device="cuda", generator=gen).bfloat16()
    ref = _reference(x, W_q, scales, zeros, g)
    y_hqq = mixed_mm(x, pack_2xint4(W_q.T), scales.T, zeros.T, g)
    packed, sz = hqq_to_tinygemm_weight(W_q.reshape(-1, g), scales.reshape(-1, 1), zeros.reshape(-1, 1), (N, K))
    y_tg = ops.weight_int4pack_mm(x, packed, g, sz)
    for y in (y_hqq, y_tg):
        assert float((y.float() - ref).abs().max() / ref.abs().max()) <= 2e-2
