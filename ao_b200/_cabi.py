"""ctypes binding of the C-ABI library (include/ao_b200.h, built by ao_b200/build.py).

This is the only place Python touches the kernels: torch supplies device memory
(``tensor.data_ptr()``) and the current stream, everything else goes through the
``extern "C"`` entry points.  There is no CPU fallback: a missing library or a
non-CUDA tensor raises.
"""
import ctypes
import os
import re

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("AO_B200_LIB") or os.path.join(_HERE, "lib", "libao_b200.so")
HEADER_PATH = os.path.join(os.path.dirname(_HERE), "include", "ao_b200.h")

AO_OK = 0
F32, F16, BF16, I32, I64, I8, U8, I16 = range(8)
MAP_SYMMETRIC, MAP_ASYMMETRIC = 0, 1
ZP_INT, ZP_FLOAT = 0, 1

DTYPE_CODE = {
    torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16, torch.int32: I32,
    torch.int64: I64, torch.int8: I8, torch.uint8: U8, torch.int16: I16,
}

_lib = None

_c = ctypes
_ptr, _i64, _int, _size, _dbl = _c.c_void_p, _c.c_int64, _c.c_int, _c.c_size_t, _c.c_double
_i64p = _c.POINTER(_c.c_int64)

# name -> (restype, argtypes); must list every function include/ao_b200.h declares
PROTOTYPES = {
    "ao_status_string": (_c.c_char_p, [_int]),
    "ao_abi_version": (_int, []),
    "ao_choose_qparams_affine": (_int, [_ptr, _int, _int, _i64p, _i64p, _int, _i64, _i64, _int, _dbl, _int, _int,
                                        _int, _int, _ptr, _ptr, _ptr]),
    "ao_quantize_affine": (_int, [_ptr, _int, _int, _i64p, _i64p, _ptr, _int, _ptr, _int, _i64, _i64, _int, _ptr,
                                  _int, _ptr]),
    "ao_dequantize_affine": (_int, [_ptr, _int, _int, _i64p, _i64p, _ptr, _int, _ptr, _int, _i64, _i64, _int, _ptr,
                                    _int, _ptr]),
    "ao_int4_groupwise_quantize": (_int, [_ptr, _i64, _i64, _int, _ptr, _ptr, _ptr, _ptr, _ptr]),
    "ao_int4_quantize_pack_tinygemm": (_int, [_ptr, _i64, _i64, _int, _int, _ptr, _ptr, _ptr]),
    "ao_pack_tinygemm_int4": (_int, [_ptr, _i64, _i64, _int, _ptr, _ptr]),
    "ao_unpack_tinygemm_int4": (_int, [_ptr, _i64, _i64, _int, _ptr, _ptr]),
    "ao_pack_tinygemm_scales_and_zeros": (_int, [_ptr, _ptr, _i64, _i64, _ptr, _ptr]),
    "ao_unpack_tinygemm_scales_and_zeros": (_int, [_ptr, _i64, _i64, _ptr, _ptr, _ptr]),
    "ao_pack_2xint4": (_int, [_ptr, _i64, _i64, _ptr, _ptr]),
    "ao_pack_hqq_int4_from_rowmajor": (_int, [_ptr, _i64, _i64, _ptr, _ptr]),
    "ao_f32_to_fpx_unpacked": (_int, [_ptr, _i64, _int, _int, _ptr, _ptr]),
    "ao_fpx_unpacked_to_f32": (_int, [_ptr, _i64, _int, _int, _ptr, _ptr]),
    "ao_pack_tc_fp6": (_int, [_ptr, _i64, _i64, _ptr, _ptr]),
    "ao_unpack_tc_fp6": (_int, [_ptr, _i64, _i64, _ptr, _ptr]),
    "ao_to_scaled_tc_fp6": (_int, [_ptr, _int, _i64, _i64, _ptr, _ptr, _ptr]),
    "ao_from_scaled_tc_fp6": (_int, [_ptr, _i64, _i64, _ptr, _ptr, _ptr]),
    "ao_pack_tc_fpx": (_int, [_ptr, _i64, _i64, _int, _ptr, _ptr]),
    "ao_unpack_tc_fpx": (_int, [_ptr, _i64, _i64, _int, _ptr, _ptr]),
    "ao_to_scaled_tc_fpx": (_int, [_ptr, _int, _i64, _i64, _int, _int, _ptr, _ptr, _ptr, _size, _ptr]),
    "ao_from_scaled_tc_fpx": (_int, [_ptr, _i64, _i64, _int, _int, _ptr, _ptr, _ptr]),
    "ao_fpx_linear": (_int, [_int, _int, _ptr, _i64, _ptr, _ptr, _i64, _i64, _i64, _ptr, _ptr, _size, _ptr]),
    "ao_fpx_linear_bias": (_int, [_int, _int, _ptr, _i64, _ptr, _ptr, _ptr, _i64, _i64, _i64, _ptr, _ptr, _size, _ptr]),
    "ao_int4_tinygemm_linear_workspace_bytes": (_size, [_i64, _i64, _i64, _int, _int]),
    "ao_int4_tinygemm_linear": (_int, [_ptr, _i64, _i64, _ptr, _ptr, _i64, _i64, _i64, _int, _int, _ptr, _ptr,
                                       _size, _ptr]),
    "ao_int4_tinygemm_linear_bias": (_int, [_ptr, _i64, _i64, _ptr, _ptr, _i64, _i64, _i64, _int, _int, _ptr, _ptr, _ptr,
                                            _size, _ptr]),
    "ao_int4_gemv_bias": (_int, [_ptr, _i64, _i64, _ptr, _ptr, _i64, _i64, _i64, _int, _int, _ptr, _ptr, _ptr, _size, _ptr]),
    "ao_int4_gemv_workspace_bytes": (_size, [_i64, _i64, _i64, _int, _int]),
    "ao_int4_gemv_static_scratch_max_bytes": (_size, []),
    "ao_int4_gemv_static_scratch": (_int, [_ptr, _i64, _i64, _ptr, _ptr, _i64, _i64, _i64, _int, _int, _ptr, _ptr]),
    "ao_int4_gemv_gather": (_int, [_ptr, _i64, _i64, _ptr, _ptr, _i64, _i64, _i64, _int, _int, _int, _int,
                                   _c.POINTER(_ptr), _ptr, _ptr, _ptr, _size, _ptr]),
    "ao_int4_gemv_push": (_int, [_ptr, _i64, _i64, _ptr, _ptr, _i64, _i64, _i64, _int, _int, _int, _int,
                                 _c.POINTER(_ptr), _ptr, _ptr, _ptr, _size, _ptr]),
    "ao_gather_exchange": (_int, [_int, _c.POINTER(_ptr), _c.POINTER(_ptr), _c.POINTER(_ptr), _i64p, _i64p, _int, _int,
                                  _int, _ptr, _ptr]),
    "ao_comm_export": (_int, [_ptr, _ptr, _i64p]),
    "ao_comm_import": (_int, [_ptr, _c.POINTER(_ptr)]),
    "ao_comm_close": (_int, [_ptr]),
    "ao_hqq_int4_linear_transposed_workspace_bytes": (_size, [_i64, _i64, _i64, _int]),
    "ao_hqq_int4_linear_transposed": (_int, [_ptr, _int, _i64, _ptr, _ptr, _ptr, _i64, _i64, _i64, _int, _ptr, _ptr, _size,
                                             _ptr]),
    "ao_hqq_quants_to_tinygemm": (_int, [_ptr, _ptr, _ptr, _int, _i64, _int, _ptr, _ptr, _ptr]),
    "ao_hqq_int4_linear_workspace_bytes": (_size, [_i64, _i64, _i64, _int]),
    "ao_hqq_int4_linear": (_int, [_ptr, _int, _i64, _ptr, _ptr, _ptr, _i64, _i64, _i64, _int, _ptr, _ptr, _size, _ptr]),
    "ao_fp6_linear_workspace_bytes": (_size, [_i64, _i64, _i64]),
    "ao_fp6_linear": (_int, [_ptr, _i64, _ptr, _ptr, _i64, _i64, _i64, _ptr, _ptr, _size, _ptr]),
    "ao_fp6_gemv_workspace_bytes": (_size, [_i64, _i64, _i64]),
    "ao_fp6_gemv": (_int, [_ptr, _i64, _ptr, _ptr, _i64, _i64, _i64, _ptr, _ptr, _size, _ptr]),
    "ao_int4_gemv": (_int, [_ptr, _i64, _i64, _ptr, _ptr, _i64, _i64, _i64, _int, _int, _ptr, _ptr, _size, _ptr]),
}


def declared_symbols():
    """Function names declared in include/ao_b200.h (parsed from the header text)."""
    with open(HEADER_PATH) as f:
        text = f.read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ao_[a-z0-9_]+)\s*\(", text)))


def lib():
    """The loaded C-ABI library.  Raises if it has not been built (python -m ao_b200.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m ao_b200.build` (nvcc, sm_100a). "
                "ao_b200 has no CPU or PyTorch fallback.")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


class AoError(RuntimeError):
    def __init__(self, status, what):
        self.status = status
        msg = lib().ao_status_string(status).decode()
        super().__init__(f"{what}: {msg} (status {status})")


def check(status, what):
    if status != AO_OK:
        raise AoError(status, what)


def require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("ao_b200 runs on CUDA tensors only (sm_100a); there is no CPU fallback — got a "
                               f"{t.device} tensor")


def dtype_code(dtype):
    try:
        return DTYPE_CODE[dtype]
    except KeyError:
        raise ValueError(f"Unsupported dtype: {dtype}") from None


def ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def stream_ptr(device=None):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def i64_array(values):
    values = [int(v) for v in values]
    return (ctypes.c_int64 * len(values))(*values)


# ----------------------------------------------------------------------------------------------
# workspaces: zero-filled once, then kept ready by the kernels; one per (device, stream)
# ----------------------------------------------------------------------------------------------
_workspaces = {}


def workspace(nbytes, device):
    """A zero-initialised scratch buffer of at least nbytes for the current stream of `device`.

    While a CUDA graph is being captured the capture stream has no buffer yet; allocating one there would put its
    zero fill into the graph.  The buffer of a warm-up call on this device (any stream) is used instead when it is
    large enough: replays of the graph then must not overlap with eager calls that use the same buffer."""
    device = torch.device(device)
    index = device.index if device.index is not None else torch.cuda.current_device()
    key = (index, torch.cuda.current_stream(device).cuda_stream)
    buf = _workspaces.get(key)
    if buf is not None and buf.numel() >= nbytes:
        return buf
    if torch.cuda.is_current_stream_capturing():
        for (idx, _), other in _workspaces.items():
            if idx == index and other.numel() >= nbytes:
                return other
    size = max(int(nbytes), 1 << 20)
    buf = torch.zeros(size, dtype=torch.uint8, device=device)
    _workspaces[key] = buf
    return buf


def workspace_for(cache, query_fn, shape_args, device, raw_stream):
    """Hot-path variant of workspace(): `cache` (a dict owned by the caller) maps (raw stream, shape) to the buffer."""
    key = (raw_stream,) + shape_args
    buf = cache.get(key)
    if buf is None:
        nbytes = query_fn(*shape_args)
        if nbytes <= 0:
            raise RuntimeError(f"unsupported linear shape {shape_args}")
        buf = workspace(nbytes, device)
        cache[key] = buf
    return buf


def workspace_status(device):
    """Status word the kernels leave in the workspace of the current stream (syncs)."""
    device = torch.device(device)
    key = (device.index if device.index is not None else torch.cuda.current_device(),
           torch.cuda.current_stream(device).cuda_stream)
    buf = _workspaces.get(key)
    if buf is None:
        return AO_OK
    return int(buf[:4].view(torch.int32).item())
