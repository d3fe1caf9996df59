// Batched int4 weight-only linear (M >= 2; the dispatcher sends M >= 5 here) on the tensor_core_tiled weight layout, replacing
// aten::_weight_int4pack_mm as called at torchao/dtypes/affine_quantized_tensor.py:631 for large batches.
// The pipeline is umma_linear.cuh; this file is the weight format's policy and the host entry.
//
// Raw stage: the packed bytes of 16 tiles of 8 rows x 128 k (one TMA tile copy, 8 KiB: tile T at T * 512, the
// word j of lane t at t * 16 + j * 4 holds k = 32 j .. 32 j + 31 of row t / 4) and the (scale, zero) bf16 pairs of
// the groups inside the 128 k ([group][128 rows], one TMA tile copy).
// Dequant: a packed word already is an MMA fragment (8 codes of one row), so codes -> bf16 (128 + q) with one
// logic op per register, (q - 8) * s + z with two bf16x2 FMAs, and one stmatrix writes 8 rows x 32 k into the
// swizzled K-major operand tile.
#include "umma_linear_ts.cuh"

namespace ao {
namespace umma {

__device__ __forceinline__ uint32_t fma_bf16x2(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// GSHIFT = log2(group size): 5..8
template <int GSHIFT>
struct TinygemmPolicy {
    static constexpr int kWBytes = kRows * kRawK / 2;   // 8 KiB
    static constexpr int kScaleRows = (kRawK >> GSHIFT) > 0 ? (kRawK >> GSHIFT) : 1;
    static constexpr int kRawBytes = kWBytes + 2048;
    static constexpr bool kBF16 = true;
    static constexpr bool kAMajorMN = false;

    static __device__ __forceinline__ void issue_raw(const Params& p, uint32_t dst, uint32_t bar, int k0, int n0) {
        ptx::mbar_arrive_expect_tx(bar, kWBytes + kScaleRows * 512);
        ptx::tma_load_2d(dst, &p.map_w, k0, n0 / 8, bar);
        ptx::tma_load_2d(dst + kWBytes, &p.map_s, n0, k0 >> GSHIFT, bar);
    }

    template <int GW>
    static __device__ __forceinline__ void dequant(uint32_t raw, uint32_t a_tiles, int wi, int lane) {
        const uint32_t nib = 0x000F000Fu, magic = 0x43004300u, one2 = 0x3F803F80u, m136 = 0xC308C308u;
        // stmatrix row addresses: lane 8i + j gives row j of matrix i (k chunk i of the word's 32 k)
        const int st_r = lane & 7, st_c = lane >> 3;
        const uint32_t st_off0 = st_r * 128 + ((st_c ^ st_r) << 4);          // word 0 of a 64-k block: chunks 0..3
        const uint32_t st_off1 = st_r * 128 + (((st_c + 4) ^ st_r) << 4);    // word 1: chunks 4..7
#pragma unroll
        for (int tt = 0; tt < 16 / GW; ++tt) {
            const int tile = wi * (16 / GW) + tt;   // tiles of 8 rows x 128 k
            const uint4 w4 = ptx::lds128(raw + tile * 512 + lane * 16);
            const uint32_t w[4] = {w4.x, w4.y, w4.z, w4.w};
            const uint32_t sc_addr = raw + kWBytes + tile * 32 + (lane >> 2) * 4;
            uint32_t s2 = 0, z2 = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                // (scale, zero) of this row and of the group that holds k = 32 j of this raw stage
                if (j == 0 || (GSHIFT == 5) || (GSHIFT == 6 && j == 2)) {
                    const int gi = GSHIFT >= 7 ? 0 : (j * 32) >> GSHIFT;
                    const uint32_t sz = ptx::lds32(sc_addr + gi * (kRows * 4));
                    s2 = __byte_perm(sz, sz, 0x1010);
                    z2 = __byte_perm(sz, sz, 0x3232);
                }
                uint32_t v[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint32_t q = ptx::and_or(w[j] >> (4 * i), nib, magic);    // bf16 pair (128 + q)
                    v[i] = fma_bf16x2(fma_bf16x2(q, one2, m136), s2, z2);           // (q - 8) * s + z
                }
                ptx::stmatrix_x4(a_tiles + (j >> 1) * kABytes + tile * 1024 + ((j & 1) ? st_off1 : st_off0), v[0], v[1], v[2],
                                 v[3]);
            }
        }
    }

    // Operand in tensor memory.  The raw stage is copied as 128-byte lines with the 128-byte swizzle (p.map_z: the packed
    // weights as uint32 [N/8 tiles][K/32 lines][32 words]): line L = 4 T + r / 2 of the stage holds rows r, r + 1 of
    // tile T's lanes, and the 16-byte chunk (4 (r % 2) + c) of lane 4r + c sits at chunk position (chunk ^ (L % 8)), so
    // that the eight rows a quarter-warp reads at once fall into eight different bank groups.
    static constexpr bool kRowDequant = true;
    static __device__ __forceinline__ void issue_raw_ts(const Params& p, uint32_t dst, uint32_t bar, int k0, int n0) {
        ptx::mbar_arrive_expect_tx(bar, kWBytes + kScaleRows * 512);
        ptx::tma_load_3d(dst, &p.map_z, 0, k0 / 32, n0 / 8, bar);
        ptx::tma_load_2d(dst + kWBytes, &p.map_s, n0, k0 >> GSHIFT, bar);
    }
    // One thread: k = 64 h .. 64 h + 63 of weight row `row` of the CTA's 128.  The row's codes sit in the words of the
    // four lanes 4r .. 4r + 3 of its 8-row tile (r = row % 8): word j of lane 4r + c holds, as the pair (nibble i,
    // nibble i + 4), the codes of k = 32 j + 8 i + 2c and the next k, i.e. the content of column 16 j + 4 i + c.
    static __device__ __forceinline__ void dequant_row_half(uint32_t raw, int row, int h, uint32_t t_addr) {
        const uint32_t nib = 0x000F000Fu, magic = 0x43004300u, one2 = 0x3F803F80u, m136 = 0xC308C308u;
        const int r = row & 7, L = (row >> 3) * 4 + (r >> 1);
        const uint32_t line = raw + L * 128 + h * 8;
        const int chunk0 = 4 * (r & 1), key = L & 7;
        uint32_t w[4][2];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const uint2 v = ptx::lds64(line + (((chunk0 + c) ^ key) << 4));   // words j = 2h, 2h + 1 of lane 4r + c
            w[c][0] = v.x; w[c][1] = v.y;
        }
        // (scale, zero) of this row: group gi of the raw stage at + gi * 512
        const uint32_t sc_addr = raw + kWBytes + row * 4;
        uint32_t col[32];
        uint32_t s2 = 0, z2 = 0;
#pragma unroll
        for (int jj = 0; jj < 2; ++jj) {
            if (jj == 0 || GSHIFT == 5) {
                const int gi = GSHIFT >= 7 ? 0 : ((2 * h + jj) * 32) >> GSHIFT;
                const uint32_t sz = ptx::lds32(sc_addr + gi * (kRows * 4));
                s2 = __byte_perm(sz, sz, 0x1010);
                z2 = __byte_perm(sz, sz, 0x3232);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const uint32_t qv = ptx::and_or(w[c][jj] >> (4 * i), nib, magic);                 // bf16 pair (128 + q)
                    col[16 * jj + 4 * i + c] = fma_bf16x2(fma_bf16x2(qv, one2, m136), s2, z2);       // (q - 8) * s + z
                }
        }
        ptx::tmem_st_32x32b_x32(t_addr, col);
    }

    static __device__ __forceinline__ int out_row(int row) { return row; }
    static __device__ __forceinline__ float row_scale(const Params&, int) { return 1.f; }
};

static bool shape_ok(int64_t M, int64_t N, int64_t K, int g, int ikt) {
    if (ikt != 8 || M < 2 || N < kRows || N % 8 != 0 || K % 128 != 0 || K < 128) return false;
    if (!(g == 32 || g == 64 || g == 128 || g == 256) || K % g != 0) return false;
    if (M > (1 << 30) || N > (1 << 30) || K > (1 << 24)) return false;
    return true;
}

// 0 when this kernel does not take the shape
size_t int4_umma_workspace_bytes(int64_t M, int64_t N, int64_t K, int g, int ikt) {
    Plan P;
    if (!shape_ok(M, N, K, g, ikt) || !make_plan(M, N, K, &P, true)) return 0;
    return P.ws_bytes;
}

// AO_ERR_UNSUPPORTED: the caller falls back to row blocks through the GEMV kernel.
int int4_umma_linear(const void* x, int64_t ldx, int64_t x_cols, const int32_t* packed, const void* sz, int64_t M,
                     int64_t N, int64_t K, int g, int ikt, void* y, const void* bias, void* ws, size_t ws_bytes,
                     cudaStream_t st) {
    Plan P;
    if (!shape_ok(M, N, K, g, ikt) || !make_plan(M, N, K, &P, true)) return AO_ERR_UNSUPPORTED;
    if (!aligned(x, 16) || (ldx * 2) % 16 != 0 || x_cols < 1 || x_cols > K || !aligned(packed, 16) || !aligned(sz, 16))
        return AO_ERR_UNSUPPORTED;
    if (ws == nullptr || ws_bytes < P.ws_bytes || !aligned(ws, 256)) return AO_ERR_WORKSPACE;
    Params prm{};
    const uint32_t scale_rows = kRawK / g > 0 ? kRawK / g : 1;
    if (!make_x_map(&prm.map_x, true, x, x_cols, M, ldx, P.MT)) return AO_ERR_LAUNCH;
    // packed weights as uint32 [N/8 tiles][K words]; (scale, zero) pairs as uint32 [K/g][N]
    if (!make_tensor_map_2d(&prm.map_w, CU_TENSOR_MAP_DATA_TYPE_UINT32, packed, (uint64_t)K, (uint64_t)(N / 8),
                            (uint64_t)K * 4, kRawK, kRows / 8))
        return AO_ERR_LAUNCH;
    if (!make_tensor_map_2d(&prm.map_s, CU_TENSOR_MAP_DATA_TYPE_UINT32, sz, (uint64_t)N, (uint64_t)(K / g), (uint64_t)N * 4,
                            kRows, scale_rows))
        return AO_ERR_LAUNCH;
    // the weights again as 128-byte lines, swizzled, for the kernel that keeps the dequantised operand in tensor memory
    if (!make_tensor_map_3d(&prm.map_z, CU_TENSOR_MAP_DATA_TYPE_UINT32, packed, 32, (uint64_t)(K / 32), (uint64_t)(N / 8),
                            128, (uint64_t)K * 4, 32, kRawK / 32, kRows / 8, CU_TENSOR_MAP_SWIZZLE_128B))
        return AO_ERR_LAUNCH;
    prm.w = packed;
    prm.scale = sz;
    prm.y = y;
    prm.bias = bias;
    prm.ws = static_cast<uint8_t*>(ws);
    prm.M = (int)M;
    prm.N = (int)N;
    prm.K = (int)K;
    switch (g) {
        case 32: return launch_mt_ts<TinygemmPolicy<5>>(P, prm, st);
        case 64: return launch_mt_ts<TinygemmPolicy<6>>(P, prm, st);
        case 128: return launch_mt_ts<TinygemmPolicy<7>>(P, prm, st);
        default: return launch_mt_ts<TinygemmPolicy<8>>(P, prm, st);
    }
}

}  // namespace umma
}  // namespace ao

#if defined(AO_UMMA_TRACE) && AO_UMMA_TRACE
// trace builds: copy the timeline of this translation unit's kernels out (512 slots)
extern "C" int ao_debug_read_umma_trace(unsigned long long* host_out) {
    return (int)cudaMemcpyFromSymbol(host_out, ao::umma::g_utrace, sizeof(unsigned long long) * 512);
}
#endif
