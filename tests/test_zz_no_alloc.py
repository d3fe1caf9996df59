"""The workspace-free int4 GEMV entry point (scratch in a device array inside the library), called through the C ABI
and compared with the regular entry point on the same inputs, two calls in a row."""
import ctypes

import pytest
import torch

from tests import gpu_util as tu

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _setup(N, K, g, M, seed):
    from ao_b200 import ops
    w = tu.make_weight((N, K), seed=seed).cuda()
    packed, sz = ops.int4_quantize_pack(w, g, 8)
    x = torch.randn(M, K, generator=torch.Generator().manual_seed(seed + 1)).bfloat16().cuda()
    return packed, sz, x


def _static(lib, x, packed, sz, M, N, K, g):
    from ao_b200 import _cabi
    y = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    rc = lib.ao_int4_gemv_static_scratch(_cabi.ptr(x), x.stride(0), K, _cabi.ptr(packed), _cabi.ptr(sz), M, N, K, g, 8,
                                         _cabi.ptr(y), _cabi.stream_ptr())
    return rc, y


@pytest.mark.parametrize("N,K,g,M", [(4096, 4096, 64, 1), (1024, 14336, 128, 4), (2048, 4096, 64, 16)])
def test_static_scratch_matches_regular_entry_point(N, K, g, M):
    from ao_b200 import _cabi, ops
    lib = _cabi.lib()
    packed, sz, x = _setup(N, K, g, M, seed=N + K + M)
    need = lib.ao_int4_gemv_workspace_bytes(M, N, K, g, 8)
    assert 0 < need <= lib.ao_int4_gemv_static_scratch_max_bytes()
    # the regular entry point of the same kernel, with a caller-owned workspace
    ws = torch.zeros(need, dtype=torch.uint8, device="cuda")
    y_ref = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    rc = lib.ao_int4_gemv(_cabi.ptr(x), x.stride(0), K, _cabi.ptr(packed), _cabi.ptr(sz), M, N, K, g, 8, _cabi.ptr(y_ref),
                          _cabi.ptr(ws), ws.numel(), _cabi.stream_ptr())
    assert rc == 0
    for _ in range(2):  # the second call finds the first call's contents in the shared array
        rc, y = _static(lib, x, packed, sz, M, N, K, g)
        assert rc == 0, lib.ao_status_string(rc)
        torch.cuda.synchronize()
        err = float((y.float() - y_ref.float()).abs().max() / y_ref.float().abs().max())
        assert err <= TOL
        assert torch.equal(y, y_ref)  # same kernel, same order of additions


def _regular(lib, x, packed, sz, M, N, K, g):
    """The regular entry point on a fresh, zero-filled, caller-owned workspace."""
    from ao_b200 import _cabi
    need = lib.ao_int4_gemv_workspace_bytes(M, N, K, g, 8)
    ws = torch.zeros(need, dtype=torch.uint8, device="cuda")
    y = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    rc = lib.ao_int4_gemv(_cabi.ptr(x), x.stride(0), K, _cabi.ptr(packed), _cabi.ptr(sz), M, N, K, g, 8, _cabi.ptr(y),
                          _cabi.ptr(ws), ws.numel(), _cabi.stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    assert int(ws[:4].view(torch.int32).item()) == 0
    return y


def test_static_scratch_k_slab_calls_with_changing_inputs():
    """Shapes whose K range is cut into slabs leave partial sums in the shared array.  Consecutive calls with
    DIFFERENT activations, and with a second slab shape in between, must never pick up an earlier call's partial
    sums: every result has to equal the regular entry point's bit for bit."""
    from ao_b200 import _cabi
    lib = _cabi.lib()
    A = dict(N=2048, K=4096, g=64, M=16)
    B = dict(N=1024, K=14336, g=64, M=8)
    ops_a = _setup(A["N"], A["K"], A["g"], A["M"], seed=11)
    ops_b = _setup(B["N"], B["K"], B["g"], B["M"], seed=12)
    for shp in (A, B):   # both shapes really take the slab path (their workspace holds slab slots)
        assert lib.ao_int4_gemv_workspace_bytes(shp["M"], shp["N"], shp["K"], shp["g"], 8) > 256 + 16384 * 4
    gen = torch.Generator().manual_seed(77)
    for it in range(4):
        for shp, (packed, sz, _) in ((A, ops_a), (B, ops_b)):
            M, N, K, g = shp["M"], shp["N"], shp["K"], shp["g"]
            x = (torch.randn(M, K, generator=gen) * (1 + it)).bfloat16().cuda()
            rc, y = _static(lib, x, packed, sz, M, N, K, g)
            assert rc == 0, lib.ao_status_string(rc)
            torch.cuda.synchronize()
            y_ref = _regular(lib, x, packed, sz, M, N, K, g)
            assert torch.equal(y, y_ref), f"call {it} of shape {N}x{K}: static-scratch result differs"


def test_static_scratch_rejects_oversized_requests():
    from ao_b200 import _cabi
    lib = _cabi.lib()
    M, N, K, g = 16, 28672, 4096, 64
    assert lib.ao_int4_gemv_workspace_bytes(M, N, K, g, 8) > lib.ao_int4_gemv_static_scratch_max_bytes()
    dummy = torch.zeros(16, dtype=torch.int32, device="cuda")
    rc = lib.ao_int4_gemv_static_scratch(_cabi.ptr(dummy), K, K, _cabi.ptr(dummy), _cabi.ptr(dummy), M, N, K, g, 8,
                                         _cabi.ptr(dummy), _cabi.stream_ptr())
    assert rc == 7  # AO_ERR_WORKSPACE
    assert b"workspace" in lib.ao_status_string(rc).lower()
