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
