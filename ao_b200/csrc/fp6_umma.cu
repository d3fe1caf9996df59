// Prefill-shaped FPx (e3m2 / e2m3 / e2m2 / e3m1) weight-only linear (M > 8) on the tensor-core pre-packed weight of
// torchao/prototype/quant_llm/quant_llm.py:90-106, replacing torchao::quant_llm_linear
// (torchao/csrc/cuda/fp6_llm/fp6_linear.cu:139-196) for large batches.  The pipeline is umma_linear.cuh.
//
// Raw stage: for each of the CTA's two 64-row blocks, 8 k16 tiles of the 2-bit plane (256 B per tile) and of the
// 4-bit plane (512 B per tile), four 1-D bulk copies.  Dequant: word t of every 128-byte piece is lane t's
// m16n8k16 fragment; decode_fragment gives four fp16 registers (value / 2^12) = four 8x8 matrices that one
// stmatrix writes into the swizzled K-major operand tile.  2^12 * scale[row] is applied to the fp32 accumulator.
#include "fp6_decode.cuh"
#include "umma_linear_ts.cuh"

namespace ao {
namespace umma {

template <int FMT>
struct Fp6Policy {
    static constexpr int kNBits = (FMT == fp6::kE3M2 || FMT == fp6::kE2M3) ? 6 : 5;
    static constexpr int kHi = kNBits == 6 ? 256 : 128;    // bytes of the first plane per k16 tile and 64-row block
    static constexpr int kTiles = kRawK / 16;              // k16 tiles per raw stage
    static constexpr int kP2 = kTiles * kHi, kP4 = kTiles * 512, kBlk = kP2 + kP4;   // per 64-row block
    static constexpr int kRawBytes = 2 * kBlk;             // 12 KiB (6 bits) / 10 KiB (5 bits)
    static constexpr bool kBF16 = false;
    static constexpr bool kAMajorMN = false;

    static __device__ __forceinline__ void issue_raw(const Params& p, uint32_t dst, uint32_t bar, int k0, int n0) {
        // N is a multiple of 64; a row tile entirely beyond N (the second tile of a CTA with two row tiles) copies nothing
        const int nblk = (p.N - n0) >= kRows ? 2 : ((p.N - n0) > 0 ? 1 : 0);
        // the first plane (2 bits or 1 bit per code) of every 64-row block comes first, then the 4-bit plane; inside a
        // plane the k16 tiles of one block are contiguous
        const uint8_t* plane2 = static_cast<const uint8_t*>(p.w);
        const uint8_t* plane4 = plane2 + (size_t)p.N * p.K * (kNBits - 4) / 8;
        ptx::mbar_arrive_expect_tx(bar, nblk * kBlk);
        for (int b = 0; b < nblk; ++b) {
            const size_t tile_index = (size_t)(n0 / 64 + b) * (p.K / 16) + k0 / 16;
            ptx::bulk_copy_g2s(dst + b * kBlk, plane2 + tile_index * kHi, kP2, bar);
            ptx::bulk_copy_g2s(dst + b * kBlk + kP2, plane4 + tile_index * 512, kP4, bar);
        }
    }

    // 16 units = (k16 tile, 64-row block) of 4 fragments of 16 rows each, dealt to the GW warps of a group
    template <int GW>
    static __device__ __forceinline__ void dequant(uint32_t raw, uint32_t a_tiles, int wi, int lane) {
        const fp6::Format fmt = fp6::make_format(FMT);
        // stmatrix: lane 8i + rr gives row rr of matrix i; matrix i = rows (i & 1) * 8.., k chunk (i >> 1)
        const int i = lane >> 3, rr = lane & 7;
#pragma unroll
        for (int u = wi; u < 16; u += GW) {
            const int j = u & 7, blk = u >> 3;
            const int chunk = (j & 3) * 2 + (i >> 1);
            const uint32_t st_lane = ((i & 1) * 8 + rr) * 128 + ((chunk ^ rr) << 4);
            const uint32_t tile = a_tiles + (j >> 2) * kABytes;
            const uint32_t p2 = raw + blk * kBlk + j * kHi + lane * 4;
            const uint32_t p4 = raw + blk * kBlk + kP2 + j * 512 + lane * 4;
            if constexpr (kNBits == 6) {
#pragma unroll
                for (int b = 0; b < 2; ++b) {
                    const uint32_t w2 = ptx::lds32(p2 + b * 128);
#pragma unroll
                    for (int cc = 0; cc < 2; ++cc) {
                        const uint32_t w4 = ptx::lds32(p4 + (b * 2 + cc) * 128);
                        uint32_t a[4];
                        fp6::decode_fragment(w4, cc == 0 ? w2 : (w2 << 4), fmt, a);
                        // fragment registers: a0 (rows e, k 0..7), a1 (rows e + 8, k 0..7), a2 (rows e, k 8..15), a3
                        ptx::stmatrix_x4(tile + (blk * 64 + (b * 2 + cc) * 16) * 128 + st_lane, a[0], a[1], a[2], a[3]);
                    }
                }
            } else {
                const uint32_t w1 = ptx::lds32(p2);
#pragma unroll
                for (int fr = 0; fr < 4; ++fr) {
                    const uint32_t w4 = ptx::lds32(p4 + fr * 128);
                    uint32_t a[4];
                    fp6::decode_fragment5(w4, w1, fr, fmt, a);
                    ptx::stmatrix_x4(tile + (blk * 64 + fr * 16) * 128 + st_lane, a[0], a[1], a[2], a[3]);
                }
            }
        }
    }

    // Operand in tensor memory: the raw stage as above.
    static constexpr bool kRowDequant = true;
    static __device__ __forceinline__ void issue_raw_ts(const Params& p, uint32_t dst, uint32_t bar, int k0, int n0) {
        issue_raw(p, dst, bar, k0, n0);
    }
    // One thread: k = 64 h .. 64 h + 63 (four k16 tiles) of weight row `row` of the CTA's 128.  Row = 64 blk + 16 fr +
    // 8 rh + e: in every k16 tile the four words of lanes 4e .. 4e + 3 (c = 0..3) of fragment fr hold, in bytes 1 and 3
    // (rh = 0) or 0 and 2 (rh = 1), the row's codes of k = 2c, 2c + 1 (high nibbles / fields) and 2c + 8, 2c + 9 (low
    // nibbles / fields): the contents of columns c and c + 4 of the tile's eight.  The same arithmetic as
    // decode_fragment, for one row of the fragment's two.
    static __device__ __forceinline__ void dequant_row_half(uint32_t raw, int row, int h, uint32_t t_addr) {
        const fp6::Format F = fp6::make_format(FMT);
        const int blk = row >> 6, fr = (row >> 4) & 3, rh = (row >> 3) & 1, e = row & 7;
        const uint32_t rot_a = rh ? F.rot[1] : F.rot[0], rot_b = rh ? F.rot[3] : F.rot[2];
        const uint32_t p4 = raw + blk * kBlk + kP2 + fr * 128 + e * 16;
        uint32_t col[32];
#pragma unroll
        for (int jt = 0; jt < 4; ++jt) {
            const int j = 4 * h + jt;
            const uint4 q4 = ptx::lds128(p4 + j * 512);
            const uint32_t w4[4] = {q4.x, q4.y, q4.z, q4.w};
            if constexpr (kNBits == 6) {
                const uint4 q2 = ptx::lds128(raw + blk * kBlk + j * kHi + (fr >> 1) * 128 + e * 16);
                const uint32_t w2[4] = {q2.x, q2.y, q2.z, q2.w};
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const uint32_t t = (fr & 1) ? (w2[c] << 4) : w2[c];   // this fragment's fields in bits 7..4 of every byte
                    const uint32_t v = rh ? t : (t >> 8);                 // this row's bytes in the place of bytes 0, 2
                    col[8 * jt + c] = ptx::and_or((v & fp6::kFieldHi) * F.k_hi, F.mh, fp6::rotl(w4[c], rot_a) & F.m4);
                    col[8 * jt + 4 + c] = ptx::and_or((v & fp6::kFieldLo) * F.k_lo, F.mh, fp6::rotl(w4[c], rot_b) & F.m4);
                }
            } else {
                const uint4 q1 = ptx::lds128(raw + blk * kBlk + j * kHi + e * 16);
                const uint32_t w1[4] = {q1.x, q1.y, q1.z, q1.w};
                const uint32_t sgn = 0x80008000u;
                const int sh = 8 * rh + 2 * fr;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    col[8 * jt + c] = ptx::and_or(w1[c] << sh, sgn, fp6::rotl(w4[c], rot_a) & F.m4);
                    col[8 * jt + 4 + c] = ptx::and_or(w1[c] << (sh + 1), sgn, fp6::rotl(w4[c], rot_b) & F.m4);
                }
            }
        }
        ptx::tmem_st_32x32b_x32(t_addr, col);
    }

    static __device__ __forceinline__ int out_row(int row) { return row; }
    static __device__ __forceinline__ float row_scale(const Params& p, int n) {
        return fp6::make_format(FMT).post_scale * __half2float(static_cast<const __half*>(p.scale)[n]);
    }
};

static bool fp6_shape_ok(int64_t M, int64_t N, int64_t K) {
    if (M < 2 || N < kRows || N % 64 != 0 || K % 128 != 0 || K < 128) return false;
    if (M > (1 << 30) || N > (1 << 30) || K > (1 << 22)) return false;
    return true;
}

size_t fp6_umma_workspace_bytes(int64_t M, int64_t N, int64_t K) {
    Plan P;
    if (!fp6_shape_ok(M, N, K) || !make_plan(M, N, K, &P, true)) return 0;
    return P.ws_bytes;
}

// AO_ERR_UNSUPPORTED: the caller falls back to row blocks through the decode kernel.
int fp6_umma_linear(int fmt, const void* x, int64_t ldx, const uint8_t* packed, const void* scale, int64_t M, int64_t N,
                    int64_t K, void* y, const void* bias, void* ws, size_t ws_bytes, cudaStream_t st) {
    Plan P;
    if (!fp6_shape_ok(M, N, K) || !make_plan(M, N, K, &P, true)) return AO_ERR_UNSUPPORTED;
    if (!aligned(x, 16) || (ldx * 2) % 16 != 0 || ldx < K || !aligned(packed, 16)) return AO_ERR_UNSUPPORTED;
    if (ws == nullptr || ws_bytes < P.ws_bytes || !aligned(ws, 256)) return AO_ERR_WORKSPACE;
    Params prm{};
    if (!make_x_map(&prm.map_x, false, x, K, M, ldx, P.MT)) return AO_ERR_LAUNCH;
    prm.map_w = prm.map_x;   // unused by this format
    prm.map_s = prm.map_x;
    prm.map_z = prm.map_x;
    prm.w = packed;
    prm.scale = scale;
    prm.y = y;
    prm.bias = bias;
    prm.ws = static_cast<uint8_t*>(ws);
    prm.M = (int)M;
    prm.N = (int)N;
    prm.K = (int)K;
    switch (fmt) {
        case fp6::kE3M2: return launch_mt_ts<Fp6Policy<fp6::kE3M2>>(P, prm, st);
        case fp6::kE2M3: return launch_mt_ts<Fp6Policy<fp6::kE2M3>>(P, prm, st);
        case fp6::kE2M2: return launch_mt_ts<Fp6Policy<fp6::kE2M2>>(P, prm, st);
        case fp6::kE3M1: return launch_mt_ts<Fp6Policy<fp6::kE3M1>>(P, prm, st);
    }
    return AO_ERR_UNSUPPORTED;
}

}  // namespace umma
}  // namespace ao
