// Shared device/host helpers for the ao_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/ao_b200.h"

#if defined(__CUDA_ARCH__) && (__CUDA_ARCH__ < 1000)
#error "ao_b200 kernels are written for sm_100a only"
#endif

namespace ao {

constexpr int kNumSMs = 148;  // B200: 2 dies x 74 SMs

inline cudaStream_t as_stream(ao_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

inline int launch_status() { return cudaGetLastError() == cudaSuccess ? AO_OK : AO_ERR_LAUNCH; }

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

__host__ __device__ inline bool is_float_dtype(int dt) { return dt == AO_F32 || dt == AO_F16 || dt == AO_BF16; }

// ---------------------------------------------------------------------------------------------
// Rounding to a logical dtype while carrying the value in fp32.  Eager PyTorch evaluates every
// half-precision elementwise op as "compute in fp32, round the result to the output dtype"; the
// kernels reproduce that step by step, with the non-contracting __f*_rn intrinsics, so that codes,
// scales and zero points come out bit-identical.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ float round_f16(float v) { return __half2float(__float2half_rn(v)); }

__device__ __forceinline__ float round_to(int dt, float v) {
    if (dt == AO_BF16) return round_bf16(v);
    if (dt == AO_F16) return round_f16(v);
    return v;
}

__host__ __device__ __forceinline__ int promote_dtype(int a, int b) { return a == b ? a : AO_F32; }

// loads / stores of one element of a runtime dtype, value carried as fp32 (integers exactly
// representable for the magnitudes that occur: zero points and codes)
__device__ __forceinline__ float load_as_f32(const void* p, int dt, int64_t i) {
    switch (dt) {
        case AO_F32: return static_cast<const float*>(p)[i];
        case AO_F16: return __half2float(static_cast<const __half*>(p)[i]);
        case AO_BF16: return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
        case AO_I32: return static_cast<float>(static_cast<const int32_t*>(p)[i]);
        case AO_I64: return static_cast<float>(static_cast<const int64_t*>(p)[i]);
        case AO_I8: return static_cast<float>(static_cast<const int8_t*>(p)[i]);
        case AO_U8: return static_cast<float>(static_cast<const uint8_t*>(p)[i]);
        case AO_I16: return static_cast<float>(static_cast<const int16_t*>(p)[i]);
    }
    return 0.f;
}

__device__ __forceinline__ int32_t load_as_i32(const void* p, int dt, int64_t i) {
    switch (dt) {
        case AO_I32: return static_cast<const int32_t*>(p)[i];
        case AO_I64: return static_cast<int32_t>(static_cast<const int64_t*>(p)[i]);
        case AO_I8: return static_cast<const int8_t*>(p)[i];
        case AO_U8: return static_cast<const uint8_t*>(p)[i];
        case AO_I16: return static_cast<const int16_t*>(p)[i];
        default: return static_cast<int32_t>(load_as_f32(p, dt, i));  // float zero point -> .to(int32)
    }
}

// v is already rounded to dt (floats) or integral (ints)
__device__ __forceinline__ void store_from_f32(void* p, int dt, int64_t i, float v) {
    switch (dt) {
        case AO_F32: static_cast<float*>(p)[i] = v; break;
        case AO_F16: static_cast<__half*>(p)[i] = __float2half_rn(v); break;
        case AO_BF16: static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v); break;
        case AO_I32: static_cast<int32_t*>(p)[i] = static_cast<int32_t>(v); break;
        case AO_I64: static_cast<int64_t*>(p)[i] = static_cast<int64_t>(v); break;
        case AO_I8: static_cast<int8_t*>(p)[i] = static_cast<int8_t>(static_cast<int32_t>(v)); break;
        case AO_U8: static_cast<uint8_t*>(p)[i] = static_cast<uint8_t>(static_cast<int32_t>(v)); break;
        case AO_I16: static_cast<int16_t*>(p)[i] = static_cast<int16_t>(static_cast<int32_t>(v)); break;
    }
}

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t bits16) { return __uint_as_float(bits16 << 16); }

__device__ __forceinline__ float warp_min(float v, int width) {
    for (int o = width >> 1; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_max(float v, int width) {
    for (int o = width >> 1; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

}  // namespace ao
