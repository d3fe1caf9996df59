"""GPU parity of the prefill-shaped int4 linear (tcgen05 kernel, M > 16): max|y - y_ref| <= 1e-2 * max|y_ref| against
the fp32 dequant-matmul oracle  x.float() @ dequantize_affine(W_q, fp32).T."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests import gpu_util as tu

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _quantized(N, K, g, seed):
    from ao_b200 import ops
    w = tu.make_weight((N, K), seed=seed)
    wf = w.float().numpy()
    s, z = orc.choose_qparams_affine(wf, orc.BF16, orc.ASYMMETRIC, [1, g], 0, 15, 1e-6, orc.BF16, orc.BF16, False,
                                     orc.ZP_FLOAT)
    q = orc.quantize_affine(wf, orc.BF16, [1, g], s, orc.BF16, z, orc.BF16, 0, 15, orc.ZP_FLOAT)
    wd = orc.dequantize_affine(q, [1, g], s, orc.BF16, z, orc.BF16, 0, 15, orc.ZP_FLOAT, orc.F32)
    packed, sz = ops.int4_quantize_pack(w.cuda(), g, 8)
    assert np.array_equal(tu.bits(packed), orc.pack_tinygemm(q, 8))
    return packed, sz, wd


def _check(y, y_ref, what):
    err = float(np.max(np.abs(tu.f32(y) - y_ref)) / np.max(np.abs(y_ref)))
    assert err <= TOL, f"{what}: rel err {err}"


@pytest.mark.parametrize("g", [32, 64, 128, 256])
@pytest.mark.parametrize("N,K", [(256, 512), (1024, 2048), (4096, 4096)])
def test_prefill_vs_oracle(N, K, g):
    from ao_b200 import _cabi, ops
    packed, sz, wd = _quantized(N, K, g, seed=N + K + g)
    gen = torch.Generator().manual_seed(g)
    for M in (17, 32, 33, 64, 100, 128, 129, 256, 300):
        x = torch.randn(M, K, generator=gen).bfloat16()
        y = ops.weight_int4pack_mm(x.cuda(), packed, g, sz)
        assert y.shape == (M, N)
        _check(y, orc.linear_f32(x.float().numpy(), wd), f"M={M}")
        assert torch.equal(y, ops.weight_int4pack_mm(x.cuda(), packed, g, sz)), "two runs must give identical bits"
    assert _cabi.workspace_status("cuda") == 0


@pytest.mark.parametrize("g", [32, 64, 128, 256])
@pytest.mark.parametrize("M", [1700, 2048, 2304])
def test_prefill_two_token_tiles_per_block(M, g):
    """With many token tiles each thread block multiplies one dequantised weight stage into two token tiles (two
    accumulators in tensor memory).  With 9472 weight rows that form is the one chosen at these M (it needs fewer
    waves of blocks); M = 1700 leaves the last block one ragged tile and one tile entirely past the end, M = 2304
    an odd number of token tiles."""
    from ao_b200 import _cabi, ops
    N, K = 9472, 512
    packed, sz, wd = _quantized(N, K, g, seed=M + g)
    x = torch.randn(M, K, generator=torch.Generator().manual_seed(M)).bfloat16()
    y = ops.weight_int4pack_mm(x.cuda(), packed, g, sz)
    assert y.shape == (M, N)
    _check(y, np.ascontiguousarray(x.float().numpy()) @ wd.T, f"M={M}")
    y256 = torch.cat([ops.weight_int4pack_mm(x[i:i + 256].cuda(), packed, g, sz) for i in range(0, M, 256)])
    _check(y256, tu.f32(y), "256 rows at a time (one token tile per block) against the two-tile form")
    assert torch.equal(y, ops.weight_int4pack_mm(x.cuda(), packed, g, sz)), "two runs must give identical bits"
    assert _cabi.workspace_status("cuda") == 0


@pytest.mark.parametrize("g", [32, 128])
@pytest.mark.parametrize("M,N,K", [(1024, 4736, 512), (200, 19072, 256)], ids=["1024x4736x512", "200x19072x256"])
def test_prefill_two_row_tiles_per_block(M, N, K, g):
    """128-column token tiles on layers with many row tiles run with two row tiles (256 weight rows) per thread block
    against one activation stage.  Both shapes have an odd number of row tiles (37, 149): the last block's second row
    tile lies entirely beyond N."""
    from ao_b200 import _cabi, ops
    packed, sz, wd = _quantized(N, K, g, seed=M + N + g)
    x = torch.randn(M, K, generator=torch.Generator().manual_seed(N)).bfloat16()
    y = ops.weight_int4pack_mm(x.cuda(), packed, g, sz)
    assert y.shape == (M, N)
    _check(y, np.ascontiguousarray(x.float().numpy()) @ wd.T, f"M={M}")
    # the same rows in batches of 64 (one row tile per block, 64-column tiles): within tolerance of each other
    y64 = torch.cat([ops.weight_int4pack_mm(x[i:i + 64].cuda(), packed, g, sz) for i in range(0, M, 64)])
    _check(y64, tu.f32(y), "64 rows at a time")
    assert torch.equal(y, ops.weight_int4pack_mm(x.cuda(), packed, g, sz)), "two runs must give identical bits"
    assert _cabi.workspace_status("cuda") == 0


@pytest.mark.parametrize("g", [32, 64, 128])
@pytest.mark.parametrize("K", [128, 384])
def test_prefill_single_and_odd_iteration_counts(K, g):
    """K = 128 is one iteration of the tcgen05 kernels (only one of the two issuing warps has work, only one accumulator
    is written), K = 384 an odd number of them."""
    from ao_b200 import _cabi, ops
    N = 384
    packed, sz, wd = _quantized(N, K, g, seed=K + g)
    gen = torch.Generator().manual_seed(K)
    for M in (5, 17, 64, 100, 200, 600):
        x = torch.randn(M, K, generator=gen).bfloat16()
        y = ops.weight_int4pack_mm(x.cuda(), packed, g, sz)
        _check(y, np.ascontiguousarray(x.float().numpy()) @ wd.T, f"M={M}")
        assert torch.equal(y, ops.weight_int4pack_mm(x.cuda(), packed, g, sz)), "two runs must give identical bits"
    assert _cabi.workspace_status("cuda") == 0


def test_prefill_matches_decode_kernel_rows():
    """The same activation rows through the decode kernel (16 at a time) and through the prefill kernel."""
    from ao_b200 import ops
    N, K, g = 2048, 4096, 64
    packed, sz, wd = _quantized(N, K, g, seed=5)
    x = torch.randn(64, K, generator=torch.Generator().manual_seed(5)).bfloat16().cuda()
    y = ops.weight_int4pack_mm(x, packed, g, sz)
    y16 = torch.cat([ops.weight_int4pack_mm(x[i:i + 16], packed, g, sz) for i in range(0, 64, 16)])
    ref = orc.linear_f32(tu.f32(x), wd)
    _check(y, ref, "prefill")
    _check(y16, ref, "decode")
    assert float((y.float() - y16.float()).abs().max() / y16.float().abs().max()) <= TOL


def test_prefill_narrow_and_strided_activation():
    """x narrower than the padded K (missing columns count as zero) and with a row stride larger than its width."""
    from ao_b200 import ops
    N, K, g = 512, 1024, 128
    packed, sz, wd = _quantized(N, K, g, seed=9)
    big = torch.randn(48, 1536, generator=torch.Generator().manual_seed(9)).bfloat16().cuda()
    x = big[:, :1000]
    y = ops.weight_int4pack_mm(x, packed, g, sz)
    xp = np.zeros((48, K), np.float32)
    xp[:, :1000] = tu.f32(x)
    _check(y, orc.linear_f32(xp, wd), "narrow x")


def test_prefill_through_quantized_module_large_batch():
    from ao_b200.quantization import int4_weight_only, quantize
    torch.manual_seed(0)
    lin = torch.nn.Linear(4096, 1024, bias=True, device="cuda", dtype=torch.bfloat16)
    w0, b0 = lin.weight.detach().clone(), lin.bias.detach().clone()
    quantize(lin, int4_weight_only(group_size=64))
    x = torch.randn(4, 512, 4096, device="cuda", dtype=torch.bfloat16)
    y = lin(x)
    assert y.shape == (4, 512, 1024)
    y = y.detach()
    ref = torch.nn.functional.linear(x.float(), lin.weight.detach().dequantize(torch.float32), b0.float())
    assert float((y.float() - ref).abs().max() / ref.abs().max()) <= TOL
    y0 = torch.nn.functional.linear(x, w0, b0)
    assert float(20 * torch.log10(y0.float().norm() / (y0.float() - y.float()).norm())) >= 10
