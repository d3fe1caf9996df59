"""CPU-side checks of the boundary: the C-ABI library loads and exports every declared symbol, and
host-side argument logic behaves like the reference (no kernels run here)."""
import ctypes
import os

import pytest
import torch

from ao_b200 import _cabi


def test_library_exports_every_declared_symbol():
    from ao_b200 import build
    path = build.build()
    assert os.path.exists(path)
    handle = ctypes.CDLL(path)
    declared = _cabi.declared_symbols()
    assert len(declared) >= 20
    for name in declared:
        assert hasattr(handle, name), f"{name} declared in include/ao_b200.h but not exported"
        assert name in _cabi.PROTOTYPES, f"{name} has no ctypes prototype"
    assert set(_cabi.PROTOTYPES) == set(declared)


def test_status_strings_and_version():
    lib = _cabi.lib()
    assert lib.ao_abi_version() >= 1
    assert lib.ao_status_string(0) == b"ok"
    assert b"workspace" in lib.ao_status_string(7)


def test_workspace_query_is_host_only():
    lib = _cabi.lib()
    # decode shapes of the Llama-3-8B layer set
    for (n, k) in [(6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336)]:
        for m in (1, 4, 8, 16):
            for g in (64, 128):
                assert lib.ao_int4_tinygemm_linear_workspace_bytes(m, n, k, g, 8) > 0
    assert lib.ao_int4_tinygemm_linear_workspace_bytes(1, 4096, 4100, 64, 8) == 0  # K not a multiple of 128


def test_cpu_tensors_are_refused():
    from ao_b200.quantization.quant_primitives import MappingType, choose_qparams_affine
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        choose_qparams_affine(torch.randn(4, 8), MappingType.ASYMMETRIC, (1, 8), torch.int8)


def test_reference_error_behaviour_on_host():
    from ao_b200.quantization.quant_primitives import (MappingType, ZeroPointDomain, choose_qparams_affine,
                                                       quantize_affine, _get_reduction_params)
    x = torch.randn(10, 256)
    with pytest.raises(ValueError, match="preserve_zero == False is not supported for symmetric quantization"):
        choose_qparams_affine(x, MappingType.SYMMETRIC, (1, 128), torch.int8, 0, 15, 1e-6, torch.bfloat16,
                              torch.bfloat16, preserve_zero=False)
    with pytest.raises(ValueError, match="Unsupported dtype"):
        choose_qparams_affine(x, MappingType.ASYMMETRIC, (1, 128), torch.float64)
    with pytest.raises(AssertionError, match="Unsupported input dtype:"):
        quantize_affine(x.to(torch.int32), (10, 256), torch.ones(1), torch.zeros(1), torch.int8)
    with pytest.raises(RuntimeError, match="is invalid for input of size 1"):
        quantize_affine(x, (1, 1), torch.ones(1), torch.zeros(1), torch.int8)
    # the docstring example of the reference
    assert _get_reduction_params((3, 3, 2, 10), (3, 3, 10, 10)) == ([3, 3, 5, 2, 10], [0, 1, 3, 4])


def test_reciprocal_multiply_matches_division_for_bf16_operands():
    """The int4 fast path computes round_bf16(r / s) as round_bf16(r * (1 / s)) (r, s bf16 values, fp32 arithmetic).
    Exhaustive over every pair of bf16 significands and a spread of exponents: both give the same bf16 value."""
    import numpy as np

    def rbf16(v):
        u = np.asarray(v, np.float32).view(np.uint32)
        r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint32) << 16
        return r.view(np.float32)

    sig = (128 + np.arange(128, dtype=np.float32)) / 128.0          # 1.0 .. 1.9921875 in steps of 2^-7
    r_sig, s_sig = np.meshgrid(sig, sig, indexing="ij")
    for er in (-20, -3, 0, 5):
        for es in (-19, -8, 0, 2):
            r = np.ldexp(r_sig, er).astype(np.float32)
            s = np.ldexp(s_sig, es).astype(np.float32)
            exact = rbf16(r / s)
            fast = rbf16(r * (np.float32(1.0) / s))
            assert np.array_equal(exact, fast), (er, es)


def test_linear_plans_exist_for_a_sweep_of_shapes():
    """The workspace queries run the same host-side planning as the launches (tile sizes, K slabs over waves of CTAs):
    every supported shape of a sweep over batch sizes, rows and reductions gets a plan with a sane workspace size."""
    lib = _cabi.lib()
    for M in (1, 2, 4, 5, 8, 9, 16, 17, 32, 33, 64, 65, 128, 129, 200, 256, 257, 300, 512, 1000, 1024, 1536, 1700, 4096, 20000):
        for N in (128, 256, 384, 1024, 4096, 4736, 6144, 10240, 28672, 57344):
            for K in (128, 256, 384, 2048, 4096, 8192, 14336, 28672):
                for g in (32, 128):
                    nbytes = lib.ao_int4_tinygemm_linear_workspace_bytes(M, N, K, g, 8)
                    assert 0 < nbytes < (1 << 32), (M, N, K, g, nbytes)
                assert 0 < lib.ao_hqq_int4_linear_workspace_bytes(M, N, K, 64) < (1 << 32), (M, N, K)
                assert 0 < lib.ao_fp6_linear_workspace_bytes(M, N, K) < (1 << 32), (M, N, K)
