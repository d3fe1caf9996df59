// int4 weight layouts: the tensor_core_tiled ("tinygemm") layout, its scale/zero interleave, and the
// HQQ row-pair nibble layout.
//
// tensor_core_tiled: int32 [N/8][K/(ikt*16)][32][ikt/2].  Word (nt, ko, t, j) belongs to warp lane t
// (row n = nt*8 + t/4, c = t%4) and holds, lsb first, the codes at
//   A[2c], A[2c+8], B[2c], B[2c+8], A[2c+1], A[2c+9], B[2c+1], B[2c+9]
// where A and B are the 16-wide k tiles number (ko*ikt + 2j) and (ko*ikt + 2j + 1).  That is the B
// operand of an m16n8k16 MMA for lane t, two k tiles per word, which is what
// aten::_convert_weight_to_int4pack produces (called at torchao/dtypes/affine_quantized_tensor.py:461).
#include "common.cuh"

namespace ao {

__global__ void __launch_bounds__(256) pack_tinygemm_kernel(const int32_t* __restrict__ codes, int64_t N, int64_t K,
                                                            int ikt, int32_t* __restrict__ out) {
    const int half = ikt / 2;
    const int64_t KO = K / (ikt * 16);
    const int64_t n_words = (N / 8) * KO * 32 * half;
    const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t wi = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; wi < n_words; wi += step) {
        const int j = static_cast<int>(wi % half);
        const int t = static_cast<int>((wi / half) % 32);
        const int64_t ko = (wi / (half * 32)) % KO;
        const int64_t nt = wi / (static_cast<int64_t>(half) * 32 * KO);
        const int64_t n = nt * 8 + (t >> 2);
        const int c = t & 3;
        const int32_t* r = codes + n * K + (ko * ikt + 2 * j) * 16 + 2 * c;
        // two 8-byte loads per k tile: (2c, 2c+1) and (2c+8, 2c+9)
        const int2 a0 = *reinterpret_cast<const int2*>(r);
        const int2 a1 = *reinterpret_cast<const int2*>(r + 8);
        const int2 b0 = *reinterpret_cast<const int2*>(r + 16);
        const int2 b1 = *reinterpret_cast<const int2*>(r + 24);
        const uint32_t word = (a0.x & 15) | ((a1.x & 15) << 4) | ((b0.x & 15) << 8) | ((b1.x & 15) << 12) |
                              ((a0.y & 15) << 16) | ((a1.y & 15) << 20) | ((b0.y & 15) << 24) |
                              (static_cast<uint32_t>(b1.y & 15) << 28);
        out[wi] = static_cast<int32_t>(word);
    }
}

__global__ void __launch_bounds__(256) unpack_tinygemm_kernel(const int32_t* __restrict__ packed, int64_t N, int64_t K,
                                                              int ikt, int32_t* __restrict__ codes) {
    const int half = ikt / 2;
    const int64_t KO = K / (ikt * 16);
    const int64_t n_words = (N / 8) * KO * 32 * half;
    const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t wi = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; wi < n_words; wi += step) {
        const int j = static_cast<int>(wi % half);
        const int t = static_cast<int>((wi / half) % 32);
        const int64_t ko = (wi / (half * 32)) % KO;
        const int64_t nt = wi / (static_cast<int64_t>(half) * 32 * KO);
        const int64_t n = nt * 8 + (t >> 2);
        const int c = t & 3;
        int32_t* r = codes + n * K + (ko * ikt + 2 * j) * 16 + 2 * c;
        const uint32_t w = static_cast<uint32_t>(packed[wi]);
        *reinterpret_cast<int2*>(r) = make_int2(w & 15, (w >> 16) & 15);
        *reinterpret_cast<int2*>(r + 8) = make_int2((w >> 4) & 15, (w >> 20) & 15);
        *reinterpret_cast<int2*>(r + 16) = make_int2((w >> 8) & 15, (w >> 24) & 15);
        *reinterpret_cast<int2*>(r + 24) = make_int2((w >> 12) & 15, (w >> 28) & 15);
    }
}

// [N][G] x2 -> [G][N][2]; tiles of 32x32 through shared memory so both sides stay coalesced
__global__ void __launch_bounds__(256) pack_scales_zeros_kernel(const uint16_t* __restrict__ scale,
                                                                const uint16_t* __restrict__ zero, int64_t N, int64_t G,
                                                                uint32_t* __restrict__ out) {
    __shared__ uint32_t tile[32][33];
    const int64_t n0 = static_cast<int64_t>(blockIdx.y) * 32, g0 = static_cast<int64_t>(blockIdx.x) * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    for (int r = ty; r < 32; r += 8) {
        const int64_t n = n0 + r, g = g0 + tx;
        if (n < N && g < G) tile[r][tx] = scale[n * G + g] | (static_cast<uint32_t>(zero[n * G + g]) << 16);
    }
    __syncthreads();
    for (int r = ty; r < 32; r += 8) {
        const int64_t g = g0 + r, n = n0 + tx;
        if (n < N && g < G) out[g * N + n] = tile[tx][r];
    }
}

__global__ void __launch_bounds__(256) unpack_scales_zeros_kernel(const uint32_t* __restrict__ sz, int64_t N, int64_t G,
                                                                  uint16_t* __restrict__ scale,
                                                                  uint16_t* __restrict__ zero) {
    __shared__ uint32_t tile[32][33];
    const int64_t n0 = static_cast<int64_t>(blockIdx.y) * 32, g0 = static_cast<int64_t>(blockIdx.x) * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    for (int r = ty; r < 32; r += 8) {
        const int64_t g = g0 + r, n = n0 + tx;
        if (n < N && g < G) tile[r][tx] = sz[g * N + n];
    }
    __syncthreads();
    for (int r = ty; r < 32; r += 8) {
        const int64_t n = n0 + r, g = g0 + tx;
        if (n < N && g < G) {
            const uint32_t v = tile[tx][r];
            if (scale) scale[n * G + g] = static_cast<uint16_t>(v & 0xffff);
            if (zero) zero[n * G + g] = static_cast<uint16_t>(v >> 16);
        }
    }
}

// rows 2r / 2r+1 -> low / high nibble
__global__ void __launch_bounds__(256) pack_2xint4_kernel(const uint8_t* __restrict__ t, int64_t R2, int64_t C,
                                                          uint8_t* __restrict__ out) {
    const int64_t total = R2 * C;
    const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += step) {
        const int64_t r = i / C, c = i % C;
        out[i] = static_cast<uint8_t>((t[(2 * r) * C + c] & 0xF) | (t[(2 * r + 1) * C + c] << 4));
    }
}

// codes [N][K] -> out [K/2][N]: out[r][n] = codes[n][2r] | codes[n][2r+1] << 4.  64(k) x 32(n) tiles.
__global__ void __launch_bounds__(256) pack_hqq_from_rowmajor_kernel(const uint8_t* __restrict__ codes, int64_t N,
                                                                     int64_t K, uint8_t* __restrict__ out) {
    __shared__ uint8_t tile[32][64 + 4];
    const int64_t n0 = static_cast<int64_t>(blockIdx.y) * 32, k0 = static_cast<int64_t>(blockIdx.x) * 64;
    for (int i = threadIdx.x; i < 32 * 64; i += blockDim.x) {
        const int r = i / 64, c = i % 64;
        if (n0 + r < N && k0 + c < K) tile[r][c] = codes[(n0 + r) * K + k0 + c];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 32 * 32; i += blockDim.x) {
        const int kr = i / 32, n = i % 32;
        if (n0 + n < N && k0 + 2 * kr + 1 < K)
            out[(k0 / 2 + kr) * N + n0 + n] = static_cast<uint8_t>((tile[n][2 * kr] & 0xF) | (tile[n][2 * kr + 1] << 4));
    }
}

static int grid_1d(int64_t items) {
    int64_t g = (items + 255) / 256;
    const int64_t cap = static_cast<int64_t>(kNumSMs) * 16;
    return static_cast<int>(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace ao

using namespace ao;

static int check_tiled_shape(int64_t N, int64_t K, int ikt) {
    if (!(ikt == 2 || ikt == 4 || ikt == 8)) return AO_ERR_ARG;
    if (N < 8 || N % 8 != 0 || K < ikt * 16 || K % (ikt * 16) != 0) return AO_ERR_SHAPE;
    return AO_OK;
}

extern "C" int ao_pack_tinygemm_int4(const int32_t* codes, int64_t N, int64_t K, int inner_k_tiles,
                                     int32_t* packed_out, ao_stream_t stream) {
    int rc = check_tiled_shape(N, K, inner_k_tiles);
    if (rc) return rc;
    if (!aligned(codes, 8)) return AO_ERR_ALIGN;
    pack_tinygemm_kernel<<<grid_1d(N * K / 8), 256, 0, as_stream(stream)>>>(codes, N, K, inner_k_tiles, packed_out);
    return launch_status();
}

extern "C" int ao_unpack_tinygemm_int4(const int32_t* packed, int64_t N, int64_t K, int inner_k_tiles,
                                       int32_t* codes_out, ao_stream_t stream) {
    int rc = check_tiled_shape(N, K, inner_k_tiles);
    if (rc) return rc;
    if (!aligned(codes_out, 8)) return AO_ERR_ALIGN;
    unpack_tinygemm_kernel<<<grid_1d(N * K / 8), 256, 0, as_stream(stream)>>>(packed, N, K, inner_k_tiles, codes_out);
    return launch_status();
}

extern "C" int ao_pack_tinygemm_scales_and_zeros(const void* scale, const void* zero, int64_t N, int64_t G,
                                                 void* scale_and_zero_out, ao_stream_t stream) {
    if (N < 1 || G < 1 || (N + 31) / 32 > 65535) return AO_ERR_SHAPE;
    if (!aligned(scale_and_zero_out, 4)) return AO_ERR_ALIGN;
    dim3 grid(static_cast<unsigned>((G + 31) / 32), static_cast<unsigned>((N + 31) / 32));
    pack_scales_zeros_kernel<<<grid, 256, 0, as_stream(stream)>>>(static_cast<const uint16_t*>(scale),
                                                                   static_cast<const uint16_t*>(zero), N, G,
                                                                   static_cast<uint32_t*>(scale_and_zero_out));
    return launch_status();
}

extern "C" int ao_unpack_tinygemm_scales_and_zeros(const void* scale_and_zero, int64_t N, int64_t G, void* scale_out,
                                                   void* zero_out, ao_stream_t stream) {
    if (N < 1 || G < 1 || (N + 31) / 32 > 65535) return AO_ERR_SHAPE;
    if (!aligned(scale_and_zero, 4)) return AO_ERR_ALIGN;
    dim3 grid(static_cast<unsigned>((G + 31) / 32), static_cast<unsigned>((N + 31) / 32));
    unpack_scales_zeros_kernel<<<grid, 256, 0, as_stream(stream)>>>(static_cast<const uint32_t*>(scale_and_zero), N, G,
                                                                     static_cast<uint16_t*>(scale_out),
                                                                     static_cast<uint16_t*>(zero_out));
    return launch_status();
}

extern "C" int ao_pack_2xint4(const uint8_t* t, int64_t R, int64_t C, uint8_t* out, ao_stream_t stream) {
    if (R < 2 || R % 2 != 0 || C < 1) return AO_ERR_SHAPE;
    pack_2xint4_kernel<<<grid_1d(R / 2 * C), 256, 0, as_stream(stream)>>>(t, R / 2, C, out);
    return launch_status();
}

// hqq_quants_to_torch_quants (torchao/prototype/hqq/hqq_tinygemm_linear.py:173-208): HQQ's (W_q, scale, zero) with
// W = (W_q - zero) * scale  ->  the tinygemm convention W = (q - 8) * scale + new_zero, every operation rounded to the
// compute dtype as the reference's tensor expressions do.
__global__ void hqq_to_tinygemm_kernel(const uint8_t* __restrict__ wq, const void* __restrict__ scales,
                                       const void* __restrict__ zeros, int dt, int64_t groups, int g,
                                       int32_t* __restrict__ q_out, void* __restrict__ new_zeros) {
    const int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (idx >= groups * g) return;
    const int64_t gi = idx / g;
    const float s = load_as_f32(scales, dt, gi), z = load_as_f32(zeros, dt, gi);
    const float s8 = round_to(dt, __fmul_rn(s, 8.f));
    const float nz = round_to(dt, __fsub_rn(s8, round_to(dt, __fmul_rn(z, s))));
    const float min_val = round_to(dt, __fsub_rn(nz, s8));
    const float w = static_cast<float>(wq[idx]);
    const float wr = round_to(dt, __fmul_rn(round_to(dt, __fsub_rn(w, z)), s));
    float t = round_to(dt, __fsub_rn(wr, min_val));
    t = round_to(dt, __fdiv_rn(t, s));
    t = rintf(t);
    t = fminf(fmaxf(t, 0.f), 15.f);
    q_out[idx] = static_cast<int32_t>(t);
    if (idx % g == 0) store_from_f32(new_zeros, dt, gi, nz);
}

extern "C" int ao_hqq_quants_to_tinygemm(const uint8_t* wq, const void* scales, const void* zeros, int dtype,
                                         int64_t groups, int group_size, int32_t* q_out, void* new_zeros_out,
                                         ao_stream_t stream) {
    if (groups < 0 || group_size < 1) return AO_ERR_SHAPE;
    if (dtype != AO_BF16 && dtype != AO_F16 && dtype != AO_F32) return AO_ERR_DTYPE;
    if (groups == 0) return AO_OK;
    const int64_t n = groups * group_size;
    if ((n + 255) / 256 > 2147483647LL) return AO_ERR_SHAPE;
    hqq_to_tinygemm_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, as_stream(stream)>>>(
        wq, scales, zeros, dtype, groups, group_size, q_out, new_zeros_out);
    return launch_status();
}

extern "C" int ao_pack_hqq_int4_from_rowmajor(const uint8_t* codes, int64_t N, int64_t K, uint8_t* out,
                                              ao_stream_t stream) {
    if (N < 1 || K < 2 || K % 2 != 0 || (N + 31) / 32 > 65535) return AO_ERR_SHAPE;
    dim3 grid(static_cast<unsigned>((K + 63) / 64), static_cast<unsigned>((N + 31) / 32));
    pack_hqq_from_rowmajor_kernel<<<grid, 256, 0, as_stream(stream)>>>(codes, N, K, out);
    return launch_status();
}
