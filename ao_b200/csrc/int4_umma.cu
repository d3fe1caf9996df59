// Prefill-shaped int4 weight-only linear (M > 16) on the tensor_core_tiled weight layout:
//   y[M][N] = x[M][K] @ dequant(W)[N][K]^T
// with the 5th-generation tensor cores (tcgen05.mma, accumulator in tensor memory), replacing
// aten::_weight_int4pack_mm as called at torchao/dtypes/affine_quantized_tensor.py:631 for large batches.
//
// The product is computed transposed: a CTA owns 128 weight rows (the MMA's M dimension, one tensor-memory lane
// per row) and MT activation rows (the MMA's N dimension, one fp32 column each), and walks K in blocks of 64.
//   warp 0     streams the packed int4 bytes of its 128 rows (16 KiB per 256 k, one TMA tile copy) and the groups'
//              (scale, zero) pairs into a 2-deep raw ring;
//   warp 1     streams x tiles [MT][64] bf16 with TMA in the 128-byte-swizzle layout the MMA reads;
//   warp 2     owns the tensor memory and issues the MMAs: four K=16 instructions per block, then a commit that
//              frees the block's shared-memory slot;
//   warps 3-10 dequantise: a packed word already is an MMA fragment (8 codes of one row), so codes -> bf16
//              (128 + q) with one logic op per register, (q - 8) * s + z with two bf16x2 FMAs, and one stmatrix
//              writes 8 rows x 32 k into the swizzled K-major operand tile.  After the K loop the same warps read
//              the accumulator from tensor memory and store y (bf16).
// Every wait is bounded; a wait that runs out sets the status word and the CTA still frees its tensor memory.
#include "common.cuh"
#include "ptx.cuh"
#include "tensormap.cuh"

namespace ao {
namespace umma {

constexpr int kRows = 128;            // weight rows per CTA
constexpr int kKB = 64;               // k per operand stage
constexpr int kRawK = 256;            // k per raw stage
constexpr int kRawBytes = kRows * kRawK / 2;   // 16 KiB
constexpr int kScaleBytes = 4096;     // up to 8 groups x 128 rows x (scale, zero)
constexpr int kABytes = kRows * kKB * 2;       // 16 KiB
constexpr int kDequantWarps = 8;
constexpr int kThreads = (3 + kDequantWarps) * 32;
constexpr int kWaitPolls = 2000;

template <int MT>
struct Cfg {
    static constexpr int S = MT == 256 ? 3 : 4;           // operand stages
    static constexpr int XBytes = MT * kKB * 2;
    static constexpr int TmemCols = MT < 32 ? 32 : MT;
    static constexpr int SmemBytes = 1024 + S * (kABytes + XBytes) + 2 * (kRawBytes + kScaleBytes) + 256;
};

__device__ __forceinline__ uint32_t fma_bf16x2(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

template <int MT>
__global__ void __launch_bounds__(kThreads, 1)
int4_umma_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_sz,
                 const __grid_constant__ CUtensorMap map_x, __nv_bfloat16* __restrict__ y, int* __restrict__ status,
                 int M, int N, int K, int g_shift) {
    using C = Cfg<MT>;
    constexpr int S = C::S;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = ptx::smem_addr(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;   // operand tiles need 1024-byte alignment
    uint8_t* sbase = smem_raw + (base - raw_addr);
    const uint32_t a_base = base, x_base = a_base + S * kABytes, raw_base = x_base + S * C::XBytes;
    const uint32_t sc_base = raw_base + 2 * kRawBytes, bar_base = sc_base + 2 * kScaleBytes;
    const uint32_t full_a = bar_base, full_x = full_a + 8 * S, empty = full_x + 8 * S;
    const uint32_t raw_full = empty + 8 * S, raw_empty = raw_full + 16, acc_full = raw_empty + 16;
    const uint32_t tmem_slot = acc_full + 8;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * kRows, m0 = blockIdx.y * MT;
    const int nkb = K / kKB, nraw = (K + kRawK - 1) / kRawK;
    const int gpr = kRawK >> g_shift;   // groups per raw stage

    if (tid == 0) {
        for (int s = 0; s < S; ++s) {
            ptx::mbar_init(full_a + 8 * s, kDequantWarps);
            ptx::mbar_init(full_x + 8 * s, 1);
            ptx::mbar_init(empty + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(raw_full + 8 * b, 1);
            ptx::mbar_init(raw_empty + 8 * b, kDequantWarps);
        }
        ptx::mbar_init(acc_full, 1);
        ptx::fence_mbar_init();
    }
    if (warp == 2) {
        ptx::tmem_alloc(tmem_slot, C::TmemCols);
        ptx::tmem_relinquish_alloc_permit();
    }
    ptx::tcgen05_fence_before_thread_sync();
    __syncthreads();
    ptx::tcgen05_fence_after_thread_sync();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(sbase + (tmem_slot - base));
    bool ok = true;

    if (warp == 0) {
        // ---------------- packed weights and scales ----------------
        if (lane == 0) {
            for (int r = 0; r < nraw; ++r) {
                const int b = r & 1;
                if (!ptx::mbar_wait_bounded(raw_empty + 8 * b, ((static_cast<uint32_t>(r) >> 1) & 1u) ^ 1u, kWaitPolls)) {
                    ok = false;
                    break;
                }
                ptx::mbar_arrive_expect_tx(raw_full + 8 * b, kRawBytes + gpr * 512);
                ptx::tma_load_2d(raw_base + b * kRawBytes, &map_w, r * kRawK, n0 / 8, raw_full + 8 * b);
                ptx::tma_load_2d(sc_base + b * kScaleBytes, &map_sz, n0, r * gpr, raw_full + 8 * b);
            }
        }
    } else if (warp == 1) {
        // ---------------- activations ----------------
        if (lane == 0) {
            for (int kb = 0; kb < nkb; ++kb) {
                const int s = kb % S;
                if (!ptx::mbar_wait_bounded(empty + 8 * s, (static_cast<uint32_t>(kb / S) & 1u) ^ 1u, kWaitPolls)) {
                    ok = false;
                    break;
                }
                ptx::mbar_arrive_expect_tx(full_x + 8 * s, C::XBytes);
                ptx::tma_load_2d(x_base + s * C::XBytes, &map_x, kb * kKB, m0, full_x + 8 * s);
            }
        }
    } else if (warp == 2) {
        // ---------------- MMA issue ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = ptx::umma_idesc_bf16(kRows, MT);
            for (int kb = 0; kb < nkb; ++kb) {
                const int s = kb % S;
                const uint32_t ph = static_cast<uint32_t>(kb / S) & 1u;
                if (!ptx::mbar_wait_bounded(full_a + 8 * s, ph, kWaitPolls) ||
                    !ptx::mbar_wait_bounded(full_x + 8 * s, ph, kWaitPolls)) {
                    ok = false;
                    break;
                }
                ptx::tcgen05_fence_after_thread_sync();
                const uint64_t da = ptx::umma_desc_k_sw128(a_base + s * kABytes);
                const uint64_t db = ptx::umma_desc_k_sw128(x_base + s * C::XBytes);
#pragma unroll
                for (int k4 = 0; k4 < kKB / 16; ++k4)
                    ptx::umma_f16_ss(tmem_base, da + 2 * k4, db + 2 * k4, idesc, (kb | k4) != 0 ? 1u : 0u);
                ptx::umma_commit(empty + 8 * s);
            }
            if (ok) ptx::umma_commit(acc_full);
        }
    } else {
        // ---------------- dequantise, then epilogue ----------------
        const int dw = warp - 3;
        const uint32_t nib = 0x000F000Fu, magic = 0x43004300u, one2 = 0x3F803F80u, m136 = 0xC308C308u;
        for (int kb = 0; kb < nkb && ok; ++kb) {
            const int r = kb >> 2, kbr = kb & 3, b = r & 1, s = kb % S;
            if (kbr == 0 && !ptx::mbar_wait_bounded(raw_full + 8 * b, (static_cast<uint32_t>(r) >> 1) & 1u, kWaitPolls)) {
                ok = false;
                break;
            }
            if (!ptx::mbar_wait_bounded(empty + 8 * s, (static_cast<uint32_t>(kb / S) & 1u) ^ 1u, kWaitPolls)) {
                ok = false;
                break;
            }
            const uint32_t a_stage = a_base + s * kABytes;
#pragma unroll
            for (int tt = 0; tt < 2; ++tt) {
                const int tile = 2 * dw + tt;
                const uint2 w2 = ptx::lds64(raw_base + b * kRawBytes + tile * 1024 + (kbr >> 1) * 512 + lane * 16 + (kbr & 1) * 8);
                const int row = tile * 8 + (lane >> 2);
                const int st_row = tile * 8 + (lane & 7);
#pragma unroll
                for (int wi = 0; wi < 2; ++wi) {
                    const uint32_t w = wi == 0 ? w2.x : w2.y;
                    const int gi = (kbr * 64 + wi * 32) >> g_shift;
                    const uint32_t sz = ptx::lds32(sc_base + b * kScaleBytes + (gi * kRows + row) * 4);
                    const uint32_t s2 = __byte_perm(sz, sz, 0x1010), z2 = __byte_perm(sz, sz, 0x3232);
                    uint32_t v[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint32_t q = ptx::and_or(w >> (4 * i), nib, magic);      // bf16 pair (128 + q)
                        v[i] = fma_bf16x2(fma_bf16x2(q, one2, m136), s2, z2);          // (q - 8) * s + z
                    }
                    const int chunk = wi * 4 + (lane >> 3);
                    ptx::stmatrix_x4(a_stage + st_row * 128 + ((chunk ^ (st_row & 7)) << 4), v[0], v[1], v[2], v[3]);
                }
            }
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                ptx::mbar_arrive(full_a + 8 * s);
                if (kbr == 3 || kb == nkb - 1) ptx::mbar_arrive(raw_empty + 8 * b);
            }
        }
        // epilogue: lane quarter (warp % 4) x column half (dw / 4)
        if (ok && !ptx::mbar_wait_bounded(acc_full, 0u, kWaitPolls)) ok = false;
        if (ok) {
            ptx::tcgen05_fence_after_thread_sync();
            const int q = warp & 3, half = dw >> 2;
            const int n = n0 + q * 32 + lane;
            constexpr int kColsPerWarp = MT >= 32 ? MT / 2 : MT;
            const int c_begin = MT >= 32 ? half * kColsPerWarp : 0;
            if (MT >= 32 || half == 0) {
#pragma unroll 1
                for (int c0 = c_begin; c0 < c_begin + kColsPerWarp; c0 += 16) {
                    if (m0 + c0 >= M) break;   // uniform across the warp
                    uint32_t v[16];
                    ptx::tmem_ld_32x32b_x16(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + c0, v);
                    ptx::tmem_ld_wait();
                    if (n < N) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int m = m0 + c0 + j;
                            if (m < M) y[(size_t)m * N + n] = __float2bfloat16_rn(__uint_as_float(v[j]));
                        }
                    }
                }
            }
        }
    }
    if (!ok && lane == 0) atomicExch(status, AO_ERR_TIMEOUT);
    ptx::tcgen05_fence_before_thread_sync();
    __syncthreads();
    if (warp == 2) {
        ptx::tcgen05_fence_after_thread_sync();
        ptx::tmem_dealloc(tmem_base, C::TmemCols);
    }
}

template <int MT>
static int launch(const CUtensorMap& mw, const CUtensorMap& ms, const CUtensorMap& mx, void* y, void* ws, int M, int N,
                  int K, int g_shift, cudaStream_t st) {
    auto kern = int4_umma_kernel<MT>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<MT>::SmemBytes) != cudaSuccess)
        return AO_ERR_LAUNCH;
    dim3 grid((N + kRows - 1) / kRows, (M + MT - 1) / MT);
    kern<<<grid, kThreads, Cfg<MT>::SmemBytes, st>>>(mw, ms, mx, static_cast<__nv_bfloat16*>(y), static_cast<int*>(ws), M, N,
                                                     K, g_shift);
    return launch_status();
}

// AO_ERR_UNSUPPORTED: the caller falls back to row blocks through the GEMV kernel.
int int4_umma_linear(const void* x, int64_t ldx, int64_t x_cols, const int32_t* packed, const void* sz, int64_t M,
                     int64_t N, int64_t K, int g, int ikt, void* y, void* ws, cudaStream_t st) {
    if (ikt != 8 || M <= 16 || N < kRows || N % 8 != 0 || K % 128 != 0 || K < 128) return AO_ERR_UNSUPPORTED;
    if (!(g == 32 || g == 64 || g == 128 || g == 256) || K % g != 0) return AO_ERR_UNSUPPORTED;
    if (M > (1 << 30) || N > (1 << 30) || K > (1 << 24)) return AO_ERR_UNSUPPORTED;
    if (!aligned(x, 16) || (ldx * 2) % 16 != 0 || x_cols < 1 || x_cols > K || !aligned(packed, 16) || !aligned(sz, 16))
        return AO_ERR_UNSUPPORTED;
    const int g_shift = g == 32 ? 5 : (g == 64 ? 6 : (g == 128 ? 7 : 8));
    const int MT = M > 128 ? 256 : (M > 64 ? 128 : (M > 32 ? 64 : 32));
    CUtensorMap mw, ms, mx;
    if (!make_tensor_map_2d(&mw, CU_TENSOR_MAP_DATA_TYPE_UINT32, packed, (uint64_t)K, (uint64_t)(N / 8), (uint64_t)K * 4,
                            kRawK, kRows / 8))
        return AO_ERR_LAUNCH;
    if (!make_tensor_map_2d(&ms, CU_TENSOR_MAP_DATA_TYPE_UINT32, sz, (uint64_t)N, (uint64_t)(K / g), (uint64_t)N * 4, kRows,
                            kRawK / g))
        return AO_ERR_LAUNCH;
    if (!make_tensor_map_2d(&mx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, x, (uint64_t)x_cols, (uint64_t)M, (uint64_t)ldx * 2, kKB,
                            MT, CU_TENSOR_MAP_SWIZZLE_128B))
        return AO_ERR_LAUNCH;
    switch (MT) {
        case 32: return launch<32>(mw, ms, mx, y, ws, (int)M, (int)N, (int)K, g_shift, st);
        case 64: return launch<64>(mw, ms, mx, y, ws, (int)M, (int)N, (int)K, g_shift, st);
        case 128: return launch<128>(mw, ms, mx, y, ws, (int)M, (int)N, (int)K, g_shift, st);
        default: return launch<256>(mw, ms, mx, y, ws, (int)M, (int)N, (int)K, g_shift, st);
    }
}

}  // namespace umma
}  // namespace ao
