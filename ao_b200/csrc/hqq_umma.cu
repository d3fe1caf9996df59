// Fused int4 dequant GEMM on the HQQ weight layout (torchao/prototype/hqq/mixed_mm.py:36-173, kernel
// torchao/prototype/hqq/kernels.py:162-387):  c[M][N] = a[M][K] @ ((q - zeros) * scales)[K][N]
//   b       uint8 [K/2][N]: row r holds k = 2r in the low nibble and k = 2r + 1 in the high nibble (pack_2xint4)
//   scales, zeros  [K/g][N] in the activation dtype (bf16 or fp16), one per group of g along K
// The pipeline is umma_linear.cuh.  The packed bytes run along N, so the dequantised operand tile is MN-major:
// a thread takes 8 bytes (8 consecutive n of one k pair), reorders the bytes with one prmt so that a masked
// shift yields (n, n+1) pairs, turns codes into 16-bit floats with one logic op per pair, applies
// (q - z) * s as q * s - z * s with two fp16x2/bf16x2 FMAs and stores one 16-byte chunk per k.
#include "umma_linear_ts.cuh"

namespace ao {
namespace umma {

template <bool BF16>
__device__ __forceinline__ uint32_t fma2(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    if constexpr (BF16)
        asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    else
        asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// TRANSPOSED: the backward form c[M][K] = a[M][N] @ W[N][K] (reduction along N): the CTA's 128 output rows are k
// values, the packed bytes run along the reduction dimension, and the operand tile is K-major again.
template <int GSHIFT, bool BF16, bool TRANSPOSED = false>
struct HqqPolicy {
    static constexpr int kWBytes = (kRawK / 2) * kRows;   // 64 byte rows x 128 n = 8 KiB
    static constexpr int kScaleRows = (kRawK >> GSHIFT) > 0 ? (kRawK >> GSHIFT) : 1;
    static constexpr int kRawBytes = kWBytes + 2048;       // + scales (<= 4 x 256 B) + zeros (<= 4 x 256 B)
    static constexpr bool kBF16 = BF16;
    static constexpr bool kAMajorMN = !TRANSPOSED;

    // k0: offset along the reduction dimension, n0: first of the CTA's 128 output rows
    static __device__ __forceinline__ void issue_raw(const Params& p, uint32_t dst, uint32_t bar, int k0, int n0) {
        ptx::mbar_arrive_expect_tx(bar, kWBytes + 2 * kScaleRows * 256);
        const int col = TRANSPOSED ? k0 : n0;     // position along N (the bytes' fast dimension)
        const int kk = TRANSPOSED ? n0 : k0;      // position along K (two per byte row, one scale row per group)
        ptx::tma_load_2d(dst, &p.map_w, col, kk / 2, bar);
        ptx::tma_load_2d(dst + kWBytes, &p.map_s, col, kk >> GSHIFT, bar);
        ptx::tma_load_2d(dst + kWBytes + 1024, &p.map_z, col, kk >> GSHIFT, bar);
    }

    template <int GW>
    static __device__ __forceinline__ void dequant(uint32_t raw, uint32_t a_tiles, int wi, int lane) {
        // 128 + q (bf16) or 1024 + q (fp16), exact; minus the offset gives q
        const uint32_t nib = 0x000F000Fu;
        const uint32_t magic = BF16 ? 0x43004300u : 0x64006400u;
        const uint32_t one2 = BF16 ? 0x3F803F80u : 0x3C003C00u;
        const uint32_t moff = BF16 ? 0xC300C300u : 0xE400E400u;
        const int td = wi * 32 + lane;    // GW * 32 threads share the 1024 items (64 byte rows x 16 chunks)
        const int c = td & 15;            // 8-byte chunk of the 128 n: n = 8c .. 8c + 7
        const int r_lo = td >> 4;         // byte row inside a group of GW * 2
        const uint32_t sc_addr = raw + kWBytes + c * 16;
        const uint32_t blk_off = (c >> 3) * 8192;   // 64-wide n block
        const int cc = c & 7;
#pragma unroll
        for (int q = 0; q < 32 / GW; ++q) {
            const int r = q * (GW * 2) + r_lo;   // byte row 0..63: k = 2r, 2r + 1 of the 128-k stage
            uint32_t s[4], nzs[4];
            {
                const int gi = GSHIFT >= 7 ? 0 : (2 * r) >> GSHIFT;
                const uint4 sv = ptx::lds128(sc_addr + gi * 256);
                const uint4 zv = ptx::lds128(sc_addr + 1024 + gi * 256);
                s[0] = sv.x; s[1] = sv.y; s[2] = sv.z; s[3] = sv.w;
                // -(z * s), rounded once
                nzs[0] = fma2<BF16>(zv.x, sv.x, 0u) ^ 0x80008000u;
                nzs[1] = fma2<BF16>(zv.y, sv.y, 0u) ^ 0x80008000u;
                nzs[2] = fma2<BF16>(zv.z, sv.z, 0u) ^ 0x80008000u;
                nzs[3] = fma2<BF16>(zv.w, sv.w, 0u) ^ 0x80008000u;
            }
            const uint2 wv = ptx::lds64(raw + r * 128 + c * 8);
            const uint32_t va = __byte_perm(wv.x, wv.x, 0x3120), vb = __byte_perm(wv.y, wv.y, 0x3120);
            uint32_t lo[4], hi[4];
            lo[0] = ptx::and_or(va, nib, magic);       hi[0] = ptx::and_or(va >> 4, nib, magic);
            lo[1] = ptx::and_or(va >> 8, nib, magic);  hi[1] = ptx::and_or(va >> 12, nib, magic);
            lo[2] = ptx::and_or(vb, nib, magic);       hi[2] = ptx::and_or(vb >> 4, nib, magic);
            lo[3] = ptx::and_or(vb >> 8, nib, magic);  hi[3] = ptx::and_or(vb >> 12, nib, magic);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                lo[i] = fma2<BF16>(fma2<BF16>(lo[i], one2, moff), s[i], nzs[i]);
                hi[i] = fma2<BF16>(fma2<BF16>(hi[i], one2, moff), s[i], nzs[i]);
            }
            if constexpr (TRANSPOSED) {
                // K-major tile of the 64 reduction elements that hold n = 8c..: rows are k = 2r, 2r + 1
                const uint32_t t = a_tiles + (c >> 3) * kABytes;
                const int row = 2 * r;
                ptx::sts128(t + row * 128 + ((cc ^ (row & 7)) << 4), lo[0], lo[1], lo[2], lo[3]);
                ptx::sts128(t + (row + 1) * 128 + ((cc ^ ((row + 1) & 7)) << 4), hi[0], hi[1], hi[2], hi[3]);
            } else {
                // operand tile of this 64-k block, MN-major: [n block of 64][k group of 8][k % 8][chunk ^ (k % 8)]
                const int kl = (2 * r) & 63, kg = kl >> 3, kr = kl & 7;
                const uint32_t t = a_tiles + (r >> 5) * kABytes + blk_off + kg * 1024;
                ptx::sts128(t + kr * 128 + ((cc ^ kr) << 4), lo[0], lo[1], lo[2], lo[3]);
                ptx::sts128(t + (kr + 1) * 128 + ((cc ^ (kr + 1)) << 4), hi[0], hi[1], hi[2], hi[3]);
            }
        }
    }

    // Operand in tensor memory (forward orientation only): the raw stage as above.
    static constexpr bool kRowDequant = !TRANSPOSED;
    static __device__ __forceinline__ void issue_raw_ts(const Params& p, uint32_t dst, uint32_t bar, int k0, int n0) {
        issue_raw(p, dst, bar, k0, n0);
    }
    // One thread: k = 64 h .. 64 h + 63 of weight row (column of the packed matrix) n = `row` of the CTA's 128.  Byte
    // row r of the raw stage holds, at byte n, the codes of k = 2r (low nibble) and 2r + 1 (high nibble): exactly one
    // column of the operand in tensor memory.  b * 0x1001 puts the low nibble at bits 3..0 and the high one at 19..16.
    // A warp's 32 threads read 32 consecutive bytes: one shared-memory wavefront per load, 32 loads per thread.
    static __device__ __forceinline__ void dequant_row_half(uint32_t raw, int row, int h, uint32_t t_addr) {
        const uint32_t nib = 0x000F000Fu;
        const uint32_t magic = BF16 ? 0x43004300u : 0x64006400u;
        const uint32_t one2 = BF16 ? 0x3F803F80u : 0x3C003C00u;
        const uint32_t moff = BF16 ? 0xC300C300u : 0xE400E400u;
        const uint32_t baddr = raw + (32 * h) * 128 + row;
        const uint32_t sc_addr = raw + kWBytes + row * 2;
        uint32_t col[32];
        uint32_t s2 = 0, nzs2 = 0;
#pragma unroll
        for (int kk = 0; kk < 32; ++kk) {
            // (scale, -(zero * scale)) of the group that holds k = 64 h + 2 kk, both halves of the register alike
            if (kk == 0 || (GSHIFT == 5 && (kk & 15) == 0)) {
                const int gi = GSHIFT >= 7 ? 0 : (64 * h + 2 * kk) >> GSHIFT;
                const uint32_t sv = ptx::lds_u16(sc_addr + gi * 256), zv = ptx::lds_u16(sc_addr + 1024 + gi * 256);
                s2 = sv | (sv << 16);
                const uint32_t z2 = zv | (zv << 16);
                nzs2 = fma2<BF16>(z2, s2, 0u) ^ 0x80008000u;   // -(z * s), rounded once
            }
            const uint32_t b = ptx::lds_u8(baddr + kk * 128);
            const uint32_t qv = ptx::and_or(b * 0x1001u, nib, magic);
            col[kk] = fma2<BF16>(fma2<BF16>(qv, one2, moff), s2, nzs2);   // (q - z) * s as q * s - z * s
        }
        ptx::tmem_st_32x32b_x32(t_addr, col);
    }

    static __device__ __forceinline__ int out_row(int row) { return row; }
    static __device__ __forceinline__ float row_scale(const Params&, int) { return 1.f; }
};

// forward orientation: operand in tensor memory (one token tile per CTA) or the shared-memory ring (two token tiles);
// transposed: the shared-memory ring
template <class Policy>
static int launch_hqq(const Plan& P, const Params& prm, cudaStream_t st) {
    if constexpr (Policy::kRowDequant)
        return launch_mt_ts<Policy>(P, prm, st);
    else
        return launch_mt<Policy>(P, prm, st);
}

template <bool BF16, bool TRANSPOSED>
static int launch_g(const Plan& P, int g, const Params& prm, cudaStream_t st) {
    switch (g) {
        case 32: return launch_hqq<HqqPolicy<5, BF16, TRANSPOSED>>(P, prm, st);
        case 64: return launch_hqq<HqqPolicy<6, BF16, TRANSPOSED>>(P, prm, st);
        case 128: return launch_hqq<HqqPolicy<7, BF16, TRANSPOSED>>(P, prm, st);
        default: return launch_hqq<HqqPolicy<8, BF16, TRANSPOSED>>(P, prm, st);
    }
}

static bool hqq_shape_ok(int64_t M, int64_t N, int64_t K, int g) {
    if (M < 1 || N < kRows || N % 16 != 0 || K % 128 != 0 || K < 128) return false;
    if (!(g == 32 || g == 64 || g == 128 || g == 256) || K % g != 0) return false;
    if (M > (1 << 30) || N > (1 << 30) || K > (1 << 24)) return false;
    return true;
}

// transposed form: output rows = K (>= 128, a multiple of the group), reduction = N (a multiple of 128)
static bool hqq_transposed_shape_ok(int64_t M, int64_t N, int64_t K, int g) {
    if (M < 1 || K < kRows || K % 2 != 0 || N % 128 != 0 || N < 128) return false;
    if (!(g == 32 || g == 64 || g == 128 || g == 256) || K % g != 0) return false;
    if (M > (1 << 30) || N > (1 << 24) || K > (1 << 30)) return false;
    return true;
}

}  // namespace umma
}  // namespace ao

using namespace ao;

extern "C" size_t ao_hqq_int4_linear_workspace_bytes(int64_t M, int64_t N, int64_t K, int group) {
    umma::Plan P;
    if (!umma::hqq_shape_ok(M, N, K, group) || !umma::make_plan(M, N, K, &P, true)) return 0;
    return P.ws_bytes;
}

extern "C" int ao_hqq_int4_linear(const void* a, int a_dtype, int64_t a_row_stride, const uint8_t* b_packed,
                                  const void* scales, const void* zeros, int64_t M, int64_t N, int64_t K, int group,
                                  void* c, void* workspace, size_t workspace_bytes, ao_stream_t stream) {
    if (M == 0 || N == 0) return AO_OK;
    if (a_dtype != AO_BF16 && a_dtype != AO_F16) return AO_ERR_DTYPE;
    umma::Plan P;
    if (!umma::hqq_shape_ok(M, N, K, group)) return AO_ERR_SHAPE;
    if (!umma::make_plan(M, N, K, &P, true)) return AO_ERR_UNSUPPORTED;
    if (!aligned(a, 16) || (a_row_stride * 2) % 16 != 0 || a_row_stride < K || !aligned(b_packed, 16) ||
        !aligned(scales, 16) || !aligned(zeros, 16) || !aligned(c, 2))
        return AO_ERR_ALIGN;
    if (workspace == nullptr || workspace_bytes < P.ws_bytes || !aligned(workspace, 256)) return AO_ERR_WORKSPACE;
    const bool bf16 = a_dtype == AO_BF16;
    umma::Params prm{};
    const uint32_t scale_rows = umma::kRawK / group > 0 ? umma::kRawK / group : 1;
    const CUtensorMapDataType dt16 = bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    if (!umma::make_x_map(&prm.map_x, bf16, a, K, M, a_row_stride, P.MT)) return AO_ERR_LAUNCH;
    if (!make_tensor_map_2d(&prm.map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, b_packed, (uint64_t)N, (uint64_t)(K / 2), (uint64_t)N,
                            umma::kRows, umma::kRawK / 2))
        return AO_ERR_LAUNCH;
    if (!make_tensor_map_2d(&prm.map_s, dt16, scales, (uint64_t)N, (uint64_t)(K / group), (uint64_t)N * 2, umma::kRows,
                            scale_rows))
        return AO_ERR_LAUNCH;
    if (!make_tensor_map_2d(&prm.map_z, dt16, zeros, (uint64_t)N, (uint64_t)(K / group), (uint64_t)N * 2, umma::kRows,
                            scale_rows))
        return AO_ERR_LAUNCH;
    prm.w = b_packed;
    prm.scale = scales;
    prm.y = c;
    prm.ws = static_cast<uint8_t*>(workspace);
    prm.M = (int)M;
    prm.N = (int)N;
    prm.K = (int)K;
    cudaStream_t st = as_stream(stream);
    return bf16 ? umma::launch_g<true, false>(P, group, prm, st) : umma::launch_g<false, false>(P, group, prm, st);
}

// transposed=True of the reference: c[M][K] = a[M][N] @ ((q - zeros) * scales)[N][K]^T-free form, i.e. the reduction
// runs along N.  Same operands as ao_hqq_int4_linear.
extern "C" size_t ao_hqq_int4_linear_transposed_workspace_bytes(int64_t M, int64_t N, int64_t K, int group) {
    umma::Plan P;
    if (!umma::hqq_transposed_shape_ok(M, N, K, group) || !umma::make_plan(M, K, N, &P)) return 0;
    return P.ws_bytes;
}

extern "C" int ao_hqq_int4_linear_transposed(const void* a, int a_dtype, int64_t a_row_stride, const uint8_t* b_packed,
                                             const void* scales, const void* zeros, int64_t M, int64_t N, int64_t K,
                                             int group, void* c, void* workspace, size_t workspace_bytes,
                                             ao_stream_t stream) {
    if (M == 0 || K == 0) return AO_OK;
    if (a_dtype != AO_BF16 && a_dtype != AO_F16) return AO_ERR_DTYPE;
    if (!umma::hqq_transposed_shape_ok(M, N, K, group)) return AO_ERR_SHAPE;
    umma::Plan P;
    if (!umma::make_plan(M, K, N, &P)) return AO_ERR_UNSUPPORTED;
    if (!aligned(a, 16) || (a_row_stride * 2) % 16 != 0 || a_row_stride < N || !aligned(b_packed, 16) ||
        !aligned(scales, 16) || !aligned(zeros, 16) || !aligned(c, 2))
        return AO_ERR_ALIGN;
    if (workspace == nullptr || workspace_bytes < P.ws_bytes || !aligned(workspace, 256)) return AO_ERR_WORKSPACE;
    const bool bf16 = a_dtype == AO_BF16;
    umma::Params prm{};
    const uint32_t scale_rows = umma::kRows / group > 0 ? umma::kRows / group : 1;
    const CUtensorMapDataType dt16 = bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    if (!umma::make_x_map(&prm.map_x, bf16, a, N, M, a_row_stride, P.MT)) return AO_ERR_LAUNCH;
    // boxes: 128 reduction bytes x 64 byte rows (= the CTA's 128 k); scale rows of the CTA's groups x 128 n
    if (!make_tensor_map_2d(&prm.map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, b_packed, (uint64_t)N, (uint64_t)(K / 2), (uint64_t)N,
                            umma::kRawK, umma::kRows / 2))
        return AO_ERR_LAUNCH;
    if (!make_tensor_map_2d(&prm.map_s, dt16, scales, (uint64_t)N, (uint64_t)(K / group), (uint64_t)N * 2, umma::kRawK,
                            scale_rows))
        return AO_ERR_LAUNCH;
    if (!make_tensor_map_2d(&prm.map_z, dt16, zeros, (uint64_t)N, (uint64_t)(K / group), (uint64_t)N * 2, umma::kRawK,
                            scale_rows))
        return AO_ERR_LAUNCH;
    prm.w = b_packed;
    prm.scale = scales;
    prm.y = c;
    prm.ws = static_cast<uint8_t*>(workspace);
    prm.M = (int)M;
    prm.N = (int)K;   // output rows of the pipeline
    prm.K = (int)N;   // its reduction length
    cudaStream_t st = as_stream(stream);
    return bf16 ? umma::launch_g<true, true>(P, group, prm, st) : umma::launch_g<false, true>(P, group, prm, st);
}
