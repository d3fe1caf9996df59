// FPx (ExMy, no inf/nan, saturating, round-to-nearest-even) codec and the FP6 tensor-core
// pre-packed weight layout.
//
// Packed layout (torchao/prototype/quant_llm/quant_llm.py:90-106), for codes [M][N], F = N/16:
// the code at row = a*64 + b*32 + c*16 + (1-d)*8 + e, col = f*16 + g*8 + h contributes
//   its top 2 bits to byte  ((((a*F + f)*2 + b)*8 + e)*8 + h)*2 + d           of the 2-bit plane,
//                            at bit position 6 - 2*(2c + g);
//   its low 4 bits to byte  (((((a*F + f)*2 + b)*2 + c)*8 + e)*8 + h)*2 + d   of the 4-bit plane,
//                            high nibble for g = 0, low nibble for g = 1.
// The 2-bit plane (M*N/4 bytes) is followed by the 4-bit plane (M*N/2 bytes).
#include "common.cuh"

namespace ao {

// custom_fp_utils.py:27-140
__device__ __forceinline__ uint32_t f32_to_fpx_bits(float xf, int ebits, int mbits) {
    const int exp_bias = (1 << (ebits - 1)) - 1;
    const uint32_t max_int = (1u << (ebits + mbits)) - 1;
    const uint32_t sign_mask = 1u << (ebits + mbits);
    const uint32_t magic_adder = (1u << (23 - mbits - 1)) - 1;
    // largest normal: all exponent and mantissa bits set
    const float max_normal = __uint_as_float(static_cast<uint32_t>(((1 << ebits) - 1) - exp_bias + 127) << 23) *
                             (static_cast<float>((1 << (mbits + 1)) - 1) / static_cast<float>(1 << mbits));
    const float min_normal = __uint_as_float(static_cast<uint32_t>(1 - exp_bias + 127) << 23);
    const uint32_t denorm_mask_int = static_cast<uint32_t>((127 - exp_bias) + (23 - mbits) + 1) << 23;
    uint32_t xb = __float_as_uint(xf);
    const uint32_t sign = xb & 0x80000000u;
    xb ^= sign;
    const float x = __uint_as_float(xb);
    uint32_t res;
    if (x >= max_normal) {
        res = max_int;
    } else if (x < min_normal) {
        res = (__float_as_uint(__fadd_rn(x, __uint_as_float(denorm_mask_int))) - denorm_mask_int) & 0xffu;
    } else {
        uint32_t nx = xb;
        const uint32_t mant_odd = (nx >> (23 - mbits)) & 1u;
        nx += (static_cast<uint32_t>(exp_bias - 127) << 23) + magic_adder;
        nx += mant_odd;
        res = (nx >> (23 - mbits)) & 0xffu;
    }
    return res | ((sign >> (31 - mbits - ebits)) & sign_mask);
}

// custom_fp_utils.py:145-229
__device__ __forceinline__ float fpx_bits_to_f32(uint32_t c, int ebits, int mbits) {
    const uint32_t sign_mask = 1u << (ebits + mbits);
    const int exp_bias = (1 << (ebits - 1)) - 1;
    const uint32_t sign = c & sign_mask;
    const uint32_t pos = (c ^ sign) & (sign_mask - 1);
    const uint32_t e = pos >> mbits, m = pos & ((1u << mbits) - 1);
    uint32_t res;
    if (pos == 0) {
        res = 0;
    } else if (e == 0) {
        // subnormal: m * 2^(1 - bias - mbits), exact in fp32
        res = __float_as_uint(static_cast<float>(m) * __uint_as_float(static_cast<uint32_t>(1 - exp_bias - mbits + 127) << 23));
    } else {
        res = ((e - exp_bias + 127) << 23) | (m << (23 - mbits));
    }
    return __uint_as_float(res | (sign << (31 - (ebits + mbits))));
}

__global__ void __launch_bounds__(256) f32_to_fpx_kernel(const float* __restrict__ x, int64_t n, int ebits, int mbits,
                                                         uint8_t* __restrict__ out) {
    const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += step)
        out[i] = static_cast<uint8_t>(f32_to_fpx_bits(x[i], ebits, mbits));
}

__global__ void __launch_bounds__(256) fpx_to_f32_kernel(const uint8_t* __restrict__ c, int64_t n, int ebits, int mbits,
                                                         float* __restrict__ out) {
    const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += step)
        out[i] = fpx_bits_to_f32(c[i], ebits, mbits);
}

constexpr int kFT = 8;              // 16-column groups per tile
constexpr int kTileCols = kFT * 16; // 128 columns
constexpr int kTilePad = 4;

// 1-bit plane of the 5-bit formats: 128 bytes per (a, f); word t (row d = t / 4 of every 8-row group, column pair
// cp = t % 4) holds the top bit of row b * 16 + c * 8 + d, column g * 8 + 2 cp + hb at bit
// hb * 16 + (1 - c) * 8 + (3 - b) * 2 + (1 - g).
__device__ __forceinline__ void emit_top_bit_plane(const uint8_t (*codes)[kTileCols + kTilePad], int64_t a, int64_t F,
                                                   int64_t f0, int nf, uint8_t* __restrict__ plane1) {
    uint32_t* p1 = reinterpret_cast<uint32_t*>(plane1 + (a * F + f0) * 128);
    for (int wi = threadIdx.x; wi < nf * 32; wi += blockDim.x) {
        const int t = wi % 32, f = wi / 32, d = t >> 2, cp = t & 3;
        uint32_t word = 0;
#pragma unroll
        for (int bit = 0; bit < 32; ++bit) {
            const int hb = bit >> 4, c = 1 - ((bit >> 3) & 1), b = 3 - ((bit >> 1) & 3), g = 1 - (bit & 1);
            const uint32_t v = codes[b * 16 + c * 8 + d][f * 16 + g * 8 + 2 * cp + hb];
            word |= ((v >> 4) & 1u) << bit;
        }
        p1[wi] = word;
    }
}

// Writes the packed bytes of the tile (a, f0 .. f0+nf) from the codes staged in shared memory: 6-bit codes as a
// 2-bit and a 4-bit plane, 5-bit codes as a 1-bit and a 4-bit plane (plane_hi: the first plane).
__device__ __forceinline__ void emit_fp6_tile(const uint8_t (*codes)[kTileCols + kTilePad], int64_t a, int64_t F,
                                              int64_t f0, int nf, uint8_t* __restrict__ plane2,
                                              uint8_t* __restrict__ plane4, int nbits = 6) {
    if (nbits == 5) {
        emit_top_bit_plane(codes, a, F, f0, nf, plane2);
    } else {
    // 2-bit plane: 256 bytes per f, written as 32-bit words (4 consecutive bytes: d = 0,1 of h, h+1)
    uint32_t* p2 = reinterpret_cast<uint32_t*>(plane2 + (a * F + f0) * 256);
    for (int wi = threadIdx.x; wi < nf * 64; wi += blockDim.x) {
        uint32_t word = 0;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int j = (wi % 64) * 4 + k, f = wi / 64;
            const int d = j & 1, h = (j >> 1) & 7, e = (j >> 4) & 7, b = j >> 7;
            uint32_t byte = 0;
#pragma unroll
            for (int cg = 0; cg < 4; ++cg) {
                const int c = cg >> 1, g = cg & 1;
                const uint32_t v = codes[b * 32 + c * 16 + (1 - d) * 8 + e][f * 16 + g * 8 + h];
                byte |= ((v >> 4) & 3u) << (6 - 2 * cg);
            }
            word |= byte << (8 * k);
        }
        p2[wi] = word;
    }
    }
    uint32_t* p4 = reinterpret_cast<uint32_t*>(plane4 + (a * F + f0) * 512);
    for (int wi = threadIdx.x; wi < nf * 128; wi += blockDim.x) {
        uint32_t word = 0;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int j = (wi % 128) * 4 + k, f = wi / 128;
            const int d = j & 1, h = (j >> 1) & 7, e = (j >> 4) & 7, c = (j >> 7) & 1, b = j >> 8;
            const uint8_t* r = codes[b * 32 + c * 16 + (1 - d) * 8 + e];
            const uint32_t byte = ((r[f * 16 + h] & 15u) << 4) | (r[f * 16 + 8 + h] & 15u);
            word |= byte << (8 * k);
        }
        p4[wi] = word;
    }
}

// grid (ceil(F / kFT), M / 64)
__global__ void __launch_bounds__(256) pack_tc_fp6_kernel(const uint8_t* __restrict__ codes_in, int64_t M, int64_t N,
                                                          uint8_t* __restrict__ out, int nbits) {
    __shared__ __align__(16) uint8_t codes[64][kTileCols + kTilePad];
    const int64_t a = blockIdx.y, F = N / 16, f0 = static_cast<int64_t>(blockIdx.x) * kFT;
    const int nf = static_cast<int>(min(static_cast<int64_t>(kFT), F - f0));
    const int cols = nf * 16;
    for (int i = threadIdx.x; i < 64 * (cols / 4); i += blockDim.x) {
        const int r = i / (cols / 4), c4 = (i % (cols / 4)) * 4;
        *reinterpret_cast<uint32_t*>(&codes[r][c4]) =
            *reinterpret_cast<const uint32_t*>(codes_in + (a * 64 + r) * N + f0 * 16 + c4);
    }
    __syncthreads();
    emit_fp6_tile(codes, a, F, f0, nf, out, out + M * N * (nbits - 4) / 8, nbits);
}

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// One CTA per 64 rows: pass 1 finds each row's absmax (scale = max(absmax, 1e-12) / max_normal in
// fp32, quant_llm.py:126-127), pass 2 encodes w / scale and packs tile by tile.
template <typename T>
__global__ void __launch_bounds__(512) to_scaled_tc_fp6_kernel(const T* __restrict__ w, int64_t M, int64_t N, int ebits,
                                                               int mbits, float max_normal, uint8_t* __restrict__ packed,
                                                               __half* __restrict__ scale_out) {
    __shared__ __align__(16) uint8_t codes[64][kTileCols + kTilePad];
    __shared__ float s_scale[64];
    const int64_t a = blockIdx.x, F = N / 16;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int r = warp; r < 64; r += nwarps) {
        const T* row = w + (a * 64 + r) * N;
        float amax = 0.f;
        for (int64_t c = lane; c < N; c += 32) amax = fmaxf(amax, fabsf(to_f32<T>(row[c])));
        amax = warp_max(amax, 32);
        if (lane == 0) {
            const float s = __fdiv_rn(fmaxf(amax, 1e-12f), max_normal);
            s_scale[r] = s;
            scale_out[a * 64 + r] = __float2half_rn(s);
        }
    }
    __syncthreads();
    for (int64_t f0 = 0; f0 < F; f0 += kFT) {
        const int nf = static_cast<int>(min(static_cast<int64_t>(kFT), F - f0));
        const int cols = nf * 16;
        for (int i = threadIdx.x; i < 64 * cols; i += blockDim.x) {
            const int r = i / cols, c = i % cols;
            const float v = __fdiv_rn(to_f32<T>(w[(a * 64 + r) * N + f0 * 16 + c]), s_scale[r]);
            codes[r][c] = static_cast<uint8_t>(f32_to_fpx_bits(v, ebits, mbits));
        }
        __syncthreads();
        emit_fp6_tile(codes, a, F, f0, nf, packed, packed + M * N * (ebits + mbits - 3) / 8, 1 + ebits + mbits);
        __syncthreads();
    }
}

// to_scaled_tc_fpx in two kernels: per-row absmax -> scale (one warp per row, vector loads; scale =
// max(absmax, 1e-12) / max_normal in fp32, quant_llm.py:126-127), then encode w / scale and pack, one CTA per
// 64 rows x 128 columns.
template <typename T>
__global__ void __launch_bounds__(256) row_scale_kernel(const T* __restrict__ w, int64_t M, int64_t N, float max_normal,
                                                        float* __restrict__ scale_f32, __half* __restrict__ scale_out) {
    const int lane = threadIdx.x & 31;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= M) return;
    const T* r = w + row * N;
    float amax = 0.f;
    // N is a multiple of 64 and rows start 16-byte aligned: 8 (16-bit) or 4 (fp32) elements per load
    constexpr int V = 16 / sizeof(T);
    for (int64_t c = static_cast<int64_t>(lane) * V; c < N; c += 32 * V) {
        const uint4 q = __ldg(reinterpret_cast<const uint4*>(r + c));
        const T* e = reinterpret_cast<const T*>(&q);
#pragma unroll
        for (int k = 0; k < V; ++k) amax = fmaxf(amax, fabsf(to_f32<T>(e[k])));
    }
    amax = warp_max(amax, 32);
    if (lane == 0) {
        const float s = __fdiv_rn(fmaxf(amax, 1e-12f), max_normal);
        scale_f32[row] = s;
        scale_out[row] = __float2half_rn(s);
    }
}

// grid (ceil(F / kFT), M / 64)
template <typename T>
__global__ void __launch_bounds__(256) encode_pack_tc_fp6_kernel(const T* __restrict__ w, int64_t M, int64_t N, int ebits,
                                                                 int mbits, const float* __restrict__ scale_f32,
                                                                 uint8_t* __restrict__ packed) {
    __shared__ __align__(16) uint8_t codes[64][kTileCols + kTilePad];
    const int64_t a = blockIdx.y, F = N / 16, f0 = static_cast<int64_t>(blockIdx.x) * kFT;
    const int nf = static_cast<int>(min(static_cast<int64_t>(kFT), F - f0));
    const int cols = nf * 16;
    for (int i = threadIdx.x; i < 64 * (cols / 4); i += blockDim.x) {
        const int r = i / (cols / 4), c4 = (i % (cols / 4)) * 4;
        const float s = scale_f32[a * 64 + r];
        const T* src = w + (a * 64 + r) * N + f0 * 16 + c4;
        uint32_t word = 0;
#pragma unroll
        for (int k = 0; k < 4; ++k)
            word |= f32_to_fpx_bits(__fdiv_rn(to_f32<T>(src[k]), s), ebits, mbits) << (8 * k);
        *reinterpret_cast<uint32_t*>(&codes[r][c4]) = word;
    }
    __syncthreads();
    emit_fp6_tile(codes, a, F, f0, nf, packed, packed + M * N * (ebits + mbits - 3) / 8, 1 + ebits + mbits);
}

__device__ __forceinline__ uint32_t fp6_code_at(const uint8_t* __restrict__ plane2, const uint8_t* __restrict__ plane4,
                                                int64_t F, int64_t row, int64_t col, int nbits = 6) {
    if (nbits == 5) {
        // top bit from the 1-bit plane (see emit_top_bit_plane), low four bits from the 4-bit plane
        const int64_t a5 = row >> 6, f5 = col >> 4;
        const int r5 = static_cast<int>(row & 63), b5 = r5 >> 4, c5 = (r5 >> 3) & 1, d5 = r5 & 7;
        const int g5 = static_cast<int>((col >> 3) & 1), cp5 = static_cast<int>((col & 7) >> 1), hb5 = static_cast<int>(col & 1);
        const int bit = hb5 * 16 + (1 - c5) * 8 + (3 - b5) * 2 + (1 - g5);
        const int64_t byte = ((a5 * F + f5) * 32 + d5 * 4 + cp5) * 4 + (bit >> 3);
        const uint32_t top = (plane2[byte] >> (bit & 7)) & 1u;
        return (top << 4) | (fp6_code_at(plane2, plane4, F, row, col, 6) & 15u);
    }
    const int64_t a = row >> 6;
    const int r = static_cast<int>(row & 63);
    const int b = r >> 5, c = (r >> 4) & 1, d = 1 - ((r >> 3) & 1), e = r & 7;
    const int64_t f = col >> 4;
    const int g = static_cast<int>((col >> 3) & 1), h = static_cast<int>(col & 7);
    const int64_t b2 = ((((a * F + f) * 2 + b) * 8 + e) * 8 + h) * 2 + d;
    const int64_t b4 = (((((a * F + f) * 2 + b) * 2 + c) * 8 + e) * 8 + h) * 2 + d;
    const uint32_t hi = (plane2[b2] >> (6 - 2 * (2 * c + g))) & 3u;
    const uint32_t lo = (plane4[b4] >> (4 - 4 * g)) & 15u;
    return (hi << 4) | lo;
}

__global__ void __launch_bounds__(256) unpack_tc_fp6_kernel(const uint8_t* __restrict__ packed, int64_t M, int64_t N,
                                                            uint8_t* __restrict__ codes_out, int nbits) {
    const int64_t total = M * N, F = N / 16;
    const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += step)
        codes_out[i] = static_cast<uint8_t>(fp6_code_at(packed, packed + total * (nbits - 4) / 8, F, i / N, i % N, nbits));
}

__global__ void __launch_bounds__(256) from_scaled_tc_fp6_kernel(const uint8_t* __restrict__ packed, int64_t M, int64_t N,
                                                                 int ebits, int mbits, const __half* __restrict__ scale,
                                                                 float* __restrict__ out) {
    const int64_t total = M * N, F = N / 16;
    const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += step) {
        const int64_t row = i / N;
        float v = fpx_bits_to_f32(fp6_code_at(packed, packed + total * (ebits + mbits - 3) / 8, F, row, i % N, 1 + ebits + mbits), ebits, mbits);
        if (scale) v = __fmul_rn(v, __half2float(scale[row]));
        out[i] = v;
    }
}

static int grid_1d(int64_t items) {
    int64_t g = (items + 255) / 256;
    const int64_t cap = static_cast<int64_t>(kNumSMs) * 16;
    return static_cast<int>(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace ao

using namespace ao;

static int check_fpx(int ebits, int mbits) {
    if (ebits < 1 || mbits < 0 || 1 + ebits + mbits > 8) return AO_ERR_ARG;
    return AO_OK;
}

extern "C" int ao_f32_to_fpx_unpacked(const float* x, int64_t n, int ebits, int mbits, uint8_t* out,
                                      ao_stream_t stream) {
    int rc = check_fpx(ebits, mbits);
    if (rc) return rc;
    if (n < 0) return AO_ERR_SHAPE;
    if (n == 0) return AO_OK;
    f32_to_fpx_kernel<<<grid_1d(n), 256, 0, as_stream(stream)>>>(x, n, ebits, mbits, out);
    return launch_status();
}

extern "C" int ao_fpx_unpacked_to_f32(const uint8_t* codes, int64_t n, int ebits, int mbits, float* out,
                                      ao_stream_t stream) {
    int rc = check_fpx(ebits, mbits);
    if (rc) return rc;
    if (n < 0) return AO_ERR_SHAPE;
    if (n == 0) return AO_OK;
    fpx_to_f32_kernel<<<grid_1d(n), 256, 0, as_stream(stream)>>>(codes, n, ebits, mbits, out);
    return launch_status();
}

static int check_tc_shape(int64_t M, int64_t N) {
    if (M < 64 || N < 64 || M % 64 != 0 || N % 64 != 0 || M / 64 > 65535) return AO_ERR_SHAPE;
    return AO_OK;
}

extern "C" int ao_pack_tc_fpx(const uint8_t* codes, int64_t M, int64_t N, int nbits, uint8_t* packed_out,
                              ao_stream_t stream) {
    if (nbits != 5 && nbits != 6) return AO_ERR_UNSUPPORTED;
    int rc = check_tc_shape(M, N);
    if (rc) return rc;
    if (!aligned(codes, 4) || !aligned(packed_out, 4)) return AO_ERR_ALIGN;
    dim3 grid(static_cast<unsigned>((N / 16 + kFT - 1) / kFT), static_cast<unsigned>(M / 64));
    pack_tc_fp6_kernel<<<grid, 256, 0, as_stream(stream)>>>(codes, M, N, packed_out, nbits);
    return launch_status();
}

extern "C" int ao_unpack_tc_fpx(const uint8_t* packed, int64_t M, int64_t N, int nbits, uint8_t* codes_out,
                                ao_stream_t stream) {
    if (nbits != 5 && nbits != 6) return AO_ERR_UNSUPPORTED;
    int rc = check_tc_shape(M, N);
    if (rc) return rc;
    unpack_tc_fp6_kernel<<<grid_1d(M * N), 256, 0, as_stream(stream)>>>(packed, M, N, codes_out, nbits);
    return launch_status();
}

extern "C" int ao_pack_tc_fp6(const uint8_t* codes, int64_t M, int64_t N, uint8_t* packed_out, ao_stream_t stream) {
    return ao_pack_tc_fpx(codes, M, N, 6, packed_out, stream);
}

extern "C" int ao_unpack_tc_fp6(const uint8_t* packed, int64_t M, int64_t N, uint8_t* codes_out, ao_stream_t stream) {
    return ao_unpack_tc_fpx(packed, M, N, 6, codes_out, stream);
}

// largest finite value of a sign-magnitude ExMy format without inf / nan (custom_fp_utils.py:62-66)
static float fpx_max_normal(int ebits, int mbits) {
    const int exp_bias = (1 << (ebits - 1)) - 1;
    return ldexpf(1.0f, ((1 << ebits) - 1) - exp_bias) * (static_cast<float>((1 << (mbits + 1)) - 1) / static_cast<float>(1 << mbits));
}

extern "C" int ao_to_scaled_tc_fpx(const void* w, int w_dtype, int64_t M, int64_t N, int ebits, int mbits,
                                   uint8_t* packed_out, void* scale_f16_out, void* workspace, size_t workspace_bytes,
                                   ao_stream_t stream) {
    if (ebits < 1 || mbits < 0 || (ebits + mbits != 5 && ebits + mbits != 4)) return AO_ERR_UNSUPPORTED;   // 5 or 6 bits
    int rc = check_tc_shape(M, N);
    if (rc) return rc;
    if (!aligned(packed_out, 4)) return AO_ERR_ALIGN;
    cudaStream_t st = as_stream(stream);
    auto* so = static_cast<__half*>(scale_f16_out);
    const float mx = fpx_max_normal(ebits, mbits);
    if (workspace != nullptr && workspace_bytes >= static_cast<size_t>(M) * 4 && aligned(workspace, 4) && aligned(w, 16)) {
        // two kernels: row scales (fp32 copies in the workspace), then encode + pack with one CTA per 64 x 128 tile
        auto* sf = static_cast<float*>(workspace);
        const unsigned g1 = static_cast<unsigned>((M + 7) / 8);
        dim3 g2(static_cast<unsigned>((N / 16 + kFT - 1) / kFT), static_cast<unsigned>(M / 64));
        switch (w_dtype) {
            case AO_F32:
                row_scale_kernel<float><<<g1, 256, 0, st>>>(static_cast<const float*>(w), M, N, mx, sf, so);
                encode_pack_tc_fp6_kernel<float><<<g2, 256, 0, st>>>(static_cast<const float*>(w), M, N, ebits, mbits, sf, packed_out);
                break;
            case AO_F16:
                row_scale_kernel<__half><<<g1, 256, 0, st>>>(static_cast<const __half*>(w), M, N, mx, sf, so);
                encode_pack_tc_fp6_kernel<__half><<<g2, 256, 0, st>>>(static_cast<const __half*>(w), M, N, ebits, mbits, sf, packed_out);
                break;
            case AO_BF16:
                row_scale_kernel<__nv_bfloat16><<<g1, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(w), M, N, mx, sf, so);
                encode_pack_tc_fp6_kernel<__nv_bfloat16><<<g2, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(w), M, N, ebits, mbits, sf, packed_out);
                break;
            default: return AO_ERR_DTYPE;
        }
        return launch_status();
    }
    // no workspace: one CTA per 64 rows does both passes
    const unsigned grid = static_cast<unsigned>(M / 64);
    switch (w_dtype) {
        case AO_F32: to_scaled_tc_fp6_kernel<float><<<grid, 512, 0, st>>>(static_cast<const float*>(w), M, N, ebits, mbits, mx, packed_out, so); break;
        case AO_F16: to_scaled_tc_fp6_kernel<__half><<<grid, 512, 0, st>>>(static_cast<const __half*>(w), M, N, ebits, mbits, mx, packed_out, so); break;
        case AO_BF16: to_scaled_tc_fp6_kernel<__nv_bfloat16><<<grid, 512, 0, st>>>(static_cast<const __nv_bfloat16*>(w), M, N, ebits, mbits, mx, packed_out, so); break;
        default: return AO_ERR_DTYPE;
    }
    return launch_status();
}

extern "C" int ao_from_scaled_tc_fpx(const uint8_t* packed, int64_t M, int64_t N, int ebits, int mbits,
                                     const void* scale_f16, float* out, ao_stream_t stream) {
    if (ebits < 1 || mbits < 0 || (ebits + mbits != 5 && ebits + mbits != 4)) return AO_ERR_UNSUPPORTED;
    int rc = check_tc_shape(M, N);
    if (rc) return rc;
    from_scaled_tc_fp6_kernel<<<grid_1d(M * N), 256, 0, as_stream(stream)>>>(packed, M, N, ebits, mbits,
                                                                             static_cast<const __half*>(scale_f16), out);
    return launch_status();
}

extern "C" int ao_to_scaled_tc_fp6(const void* w, int w_dtype, int64_t M, int64_t N, uint8_t* packed_out,
                                   void* scale_f16_out, ao_stream_t stream) {
    return ao_to_scaled_tc_fpx(w, w_dtype, M, N, 3, 2, packed_out, scale_f16_out, nullptr, 0, stream);
}

extern "C" int ao_from_scaled_tc_fp6(const uint8_t* packed, int64_t M, int64_t N, const void* scale_f16, float* out,
                                     ao_stream_t stream) {
    return ao_from_scaled_tc_fpx(packed, M, N, 3, 2, scale_f16, out, stream);
}
