// Prefill-shaped int4 weight-only linear (M > 16) on the tensor_core_tiled weight layout:
//   y[M][N] = x[M][K] @ dequant(W)[N][K]^T
// with the 5th-generation tensor cores (tcgen05.mma, accumulator in tensor memory), replacing
// aten::_weight_int4pack_mm as called at torchao/dtypes/affine_quantized_tensor.py:631 for large batches.
//
// The product is computed transposed: a CTA owns 128 weight rows (the MMA's M dimension, one tensor-memory lane
// per row) and MT activation rows (the MMA's N dimension, one fp32 column each), and walks K in blocks of 64.
//   warp 0     streams the packed int4 bytes of its 128 rows (8 KiB per 128 k, one TMA tile copy) and the groups'
//              (scale, zero) pairs into a 3- or 4-deep raw ring;
//   warp 1     streams x tiles [MT][64] bf16 with TMA in the 128-byte-swizzle layout the MMA reads;
//   warp 2     owns the tensor memory and issues the MMAs: four K=16 instructions per block, then a commit that
//              frees the block's shared-memory slot;
//   warps 3-10 dequantise: a packed word already is an MMA fragment (8 codes of one row), so codes -> bf16
//              (128 + q) with one logic op per register, (q - 8) * s + z with two bf16x2 FMAs, and one stmatrix
//              writes 8 rows x 32 k into the swizzled K-major operand tile.  After the K loop the same warps read
//              the accumulator from tensor memory and store y (bf16).
// When the tiles alone would leave SMs idle, K is cut into slabs over gridDim.z; fp32 partial tiles meet in the
// workspace and the CTA that completes a tile (atomic counter) adds them in slab order (deterministic).
// Every wait is bounded; a wait that runs out sets the status word and the CTA still frees its tensor memory.
#include "common.cuh"
#include "ptx.cuh"
#include "tensormap.cuh"

namespace ao {
namespace umma {

constexpr int kRows = 128;            // weight rows per CTA
constexpr int kKB = 64;               // k per operand stage (one 128-byte swizzle atom of bf16)
constexpr int kRawK = 128;            // k per raw stage = one outer tile of the packed layout = two operand stages
constexpr int kRawBytes = kRows * kRawK / 2;   // 8 KiB
constexpr int kScaleBytes = 2048;     // up to 4 groups x 128 rows x (scale, zero)
constexpr int kABytes = kRows * kKB * 2;       // 16 KiB
constexpr int kS = 4;                 // operand stages
constexpr int kDequantWarps = 8;
constexpr int kThreads = (3 + kDequantWarps) * 32;
constexpr int kWaitPolls = 2000;
constexpr int kHeaderBytes = 256;
constexpr int kMaxTiles = 16384;      // completion counters (shared region with the decode kernel's)
constexpr int kMaxSplit = 8;

template <int MT>
struct Cfg {
    static constexpr int R = MT == 256 ? 3 : 4;           // raw stages
    static constexpr int XBytes = MT * kKB * 2;
    static constexpr int TmemCols = MT < 32 ? 32 : MT;
    static constexpr int SmemBytes = 1024 + kS * (kABytes + XBytes) + R * (kRawBytes + kScaleBytes) + 256;
};

// work split of one call
struct Plan {
    int MT, nsplit, row_tiles, m_tiles;
    size_t ws_bytes;
};

static bool make_plan(int64_t M, int64_t N, int64_t K, Plan* P) {
    P->MT = M > 128 ? 256 : (M > 64 ? 128 : (M > 32 ? 64 : 32));
    P->row_tiles = (int)((N + kRows - 1) / kRows);
    P->m_tiles = (int)((M + P->MT - 1) / P->MT);
    const long long tiles = (long long)P->row_tiles * P->m_tiles;
    if (tiles > kMaxTiles) return false;
    // K slabs over gridDim.z when the tiles alone leave SMs idle; every slab keeps at least 8 iterations of 128 k
    int nsplit = (int)(kNumSMs / tiles);
    const int nit = (int)(K / kRawK);
    if (nsplit > kMaxSplit) nsplit = kMaxSplit;
    if (P->MT == 256 && nsplit > 2) nsplit = 2;
    while (nsplit > 1 && nit / nsplit < 8) --nsplit;
    if (nsplit < 1) nsplit = 1;
    P->nsplit = nsplit;
    P->ws_bytes = kHeaderBytes + (size_t)kMaxTiles * 4 +
                  (nsplit > 1 ? (size_t)tiles * nsplit * kRows * P->MT * 4 : 0);
    return true;
}

__device__ __forceinline__ uint32_t fma_bf16x2(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// GSHIFT = log2(group size): 5..8
template <int MT, int GSHIFT>
__global__ void __launch_bounds__(kThreads, 1)
int4_umma_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_sz,
                 const __grid_constant__ CUtensorMap map_x, __nv_bfloat16* __restrict__ y, uint8_t* __restrict__ ws,
                 int M, int N, int K) {
    using C = Cfg<MT>;
    constexpr int R = C::R;
    constexpr int kScaleRows = (kRawK >> GSHIFT) > 0 ? (kRawK >> GSHIFT) : 1;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = ptx::smem_addr(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;   // operand tiles need 1024-byte alignment
    uint8_t* sbase = smem_raw + (base - raw_addr);
    const uint32_t a_base = base, x_base = a_base + kS * kABytes, raw_base = x_base + kS * C::XBytes;
    const uint32_t sc_base = raw_base + R * kRawBytes, bar_base = sc_base + R * kScaleBytes;
    const uint32_t full_a = bar_base, full_x = full_a + 8 * kS, empty = full_x + 8 * kS;
    const uint32_t raw_full = empty + 8 * kS, raw_empty = raw_full + 8 * 4, acc_full = raw_empty + 8 * 4;
    const uint32_t tmem_slot = acc_full + 8, flag_slot = tmem_slot + 4;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * kRows, m0 = blockIdx.y * MT;
    const int nsplit = gridDim.z, z = blockIdx.z;
    const int nit_all = K / kRawK;
    const int it_begin = (int)(((long long)z * nit_all) / nsplit), it_end = (int)(((long long)(z + 1) * nit_all) / nsplit);
    const int nit = it_end - it_begin;     // iterations of 128 k for this CTA
    int* status = reinterpret_cast<int*>(ws);

    if (tid == 0) {
        for (int s = 0; s < kS; ++s) {
            ptx::mbar_init(full_a + 8 * s, kDequantWarps);
            ptx::mbar_init(full_x + 8 * s, 1);
            ptx::mbar_init(empty + 8 * s, 1);
        }
        for (int b = 0; b < R; ++b) {
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
        // ---------------- packed weights and scales: one raw stage per iteration ----------------
        if (lane == 0) {
            int rb = 0;
            uint32_t ph = 1;   // a fresh barrier counts as "previous phase complete"
            for (int it = 0; it < nit; ++it) {
                if (!ptx::mbar_wait_bounded(raw_empty + 8 * rb, ph, kWaitPolls)) {
                    ok = false;
                    break;
                }
                const int k0 = (it_begin + it) * kRawK;
                ptx::mbar_arrive_expect_tx(raw_full + 8 * rb, kRawBytes + kScaleRows * 512);
                ptx::tma_load_2d(raw_base + rb * kRawBytes, &map_w, k0, n0 / 8, raw_full + 8 * rb);
                ptx::tma_load_2d(sc_base + rb * kScaleBytes, &map_sz, n0, k0 >> GSHIFT, raw_full + 8 * rb);
                if (++rb == R) {
                    rb = 0;
                    ph ^= 1u;
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- activations: one operand stage per 64 k ----------------
        if (lane == 0) {
            for (int kb = 0; kb < 2 * nit; ++kb) {
                const int s = kb & (kS - 1);
                if (!ptx::mbar_wait_bounded(empty + 8 * s, (static_cast<uint32_t>(kb >> 2) & 1u) ^ 1u, kWaitPolls)) {
                    ok = false;
                    break;
                }
                ptx::mbar_arrive_expect_tx(full_x + 8 * s, C::XBytes);
                ptx::tma_load_2d(x_base + s * C::XBytes, &map_x, (2 * it_begin + kb) * kKB, m0, full_x + 8 * s);
            }
        }
    } else if (warp == 2) {
        // ---------------- MMA issue ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = ptx::umma_idesc_bf16(kRows, MT);
            for (int kb = 0; kb < 2 * nit; ++kb) {
                const int s = kb & (kS - 1);
                const uint32_t ph = static_cast<uint32_t>(kb >> 2) & 1u;
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
        // ---------------- dequantise (two tiles of 8 rows x 128 k per warp and iteration), then epilogue ----------
        const int dw = warp - 3;
        const uint32_t nib = 0x000F000Fu, magic = 0x43004300u, one2 = 0x3F803F80u, m136 = 0xC308C308u;
        // stmatrix row addresses: lane 8i + j gives row j of matrix i (k chunk i of the word's 32 k)
        const int st_r = lane & 7, st_c = lane >> 3;
        const uint32_t st_off0 = st_r * 128 + ((st_c ^ st_r) << 4);          // word 0 of a 64-k block: chunks 0..3
        const uint32_t st_off1 = st_r * 128 + (((st_c + 4) ^ st_r) << 4);    // word 1: chunks 4..7
        const uint32_t raw_lane = lane * 16;
        const uint32_t sc_lane = (lane >> 2) * 4;
        int rb = 0;
        uint32_t rph = 0;
        for (int it = 0; it < nit && ok; ++it) {
            const int s0 = (2 * it) & (kS - 1);
            const uint32_t eph = (static_cast<uint32_t>(it >> 1) & 1u) ^ 1u;
            if (!ptx::mbar_wait_bounded(raw_full + 8 * rb, rph, kWaitPolls) ||
                !ptx::mbar_wait_bounded(empty + 8 * s0, eph, kWaitPolls) ||
                !ptx::mbar_wait_bounded(empty + 8 * (s0 + 1), eph, kWaitPolls)) {
                ok = false;
                break;
            }
            const uint32_t a_stage = a_base + s0 * kABytes;
#pragma unroll
            for (int tt = 0; tt < 2; ++tt) {
                const int tile = 2 * dw + tt;
                const uint4 w4 = ptx::lds128(raw_base + rb * kRawBytes + tile * 512 + raw_lane);
                const uint32_t w[4] = {w4.x, w4.y, w4.z, w4.w};
                const uint32_t sc_addr = sc_base + rb * kScaleBytes + tile * 32 + sc_lane;
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
                    ptx::stmatrix_x4(a_stage + (j >> 1) * kABytes + tile * 1024 + ((j & 1) ? st_off1 : st_off0), v[0], v[1],
                                     v[2], v[3]);
                }
            }
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                ptx::mbar_arrive(full_a + 8 * s0);
                ptx::mbar_arrive(full_a + 8 * (s0 + 1));
                ptx::mbar_arrive(raw_empty + 8 * rb);
            }
            if (++rb == R) {
                rb = 0;
                rph ^= 1u;
            }
        }
        // ---------------- epilogue: lane quarter (warp % 4) x column half (dw / 4) ----------------
        if (ok && !ptx::mbar_wait_bounded(acc_full, 0u, kWaitPolls)) ok = false;
        const int q = warp & 3, half = dw >> 2;
        const int row = q * 32 + lane, n = n0 + row;
        constexpr int kColsPerWarp = MT / 2;
        const int c_begin = half * kColsPerWarp;
        const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
        if (nsplit == 1) {
            if (ok) {
                ptx::tcgen05_fence_after_thread_sync();
#pragma unroll 1
                for (int c0 = c_begin; c0 < c_begin + kColsPerWarp; c0 += 16) {
                    if (m0 + c0 >= M) break;   // uniform across the warp
                    uint32_t v[16];
                    ptx::tmem_ld_32x32b_x16(t_lane + c0, v);
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
        } else {
            // K slabs: fp32 partial tile [column][row] into this slab's workspace slot; the CTA that completes the
            // tile (atomic counter) adds the slabs in order and stores; the counter is left at zero.
            const int tile_id = blockIdx.y * gridDim.x + blockIdx.x;
            float* slots = reinterpret_cast<float*>(ws + kHeaderBytes + (size_t)kMaxTiles * 4);
            const size_t slot_elems = (size_t)kRows * MT;
            float* mine = slots + ((size_t)tile_id * nsplit + z) * slot_elems;
            if (ok) {
                ptx::tcgen05_fence_after_thread_sync();
#pragma unroll 1
                for (int c0 = c_begin; c0 < c_begin + kColsPerWarp; c0 += 16) {
                    if (m0 + c0 >= M) break;
                    uint32_t v[16];
                    ptx::tmem_ld_32x32b_x16(t_lane + c0, v);
                    ptx::tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; ++j) mine[(size_t)(c0 + j) * kRows + row] = __uint_as_float(v[j]);
                }
            }
            __threadfence();
            ptx::named_barrier_sync(1, kDequantWarps * 32);
            volatile int* flag = reinterpret_cast<volatile int*>(sbase + (flag_slot - base));
            if (tid == 3 * 32) {
                int* counter = reinterpret_cast<int*>(ws + kHeaderBytes) + tile_id;
                const int old = atomicAdd(counter, 1);
                *flag = (old + 1 == nsplit) ? 1 : 0;
                if (old + 1 == nsplit) *counter = 0;   // every slab has arrived: ready for the next call
            }
            ptx::named_barrier_sync(1, kDequantWarps * 32);
            if (*flag) {
                __threadfence();
                const float* tile_slots = slots + (size_t)tile_id * nsplit * slot_elems;
#pragma unroll 1
                for (int c0 = c_begin; c0 < c_begin + kColsPerWarp; c0 += 8) {
                    if (m0 + c0 >= M) break;
                    float acc[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
                    for (int zz = 0; zz < nsplit; ++zz) {
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            acc[j] += ptx::ldcg_f32(tile_slots + (size_t)zz * slot_elems + (size_t)(c0 + j) * kRows + row);
                    }
                    if (n < N) {
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const int m = m0 + c0 + j;
                            if (m < M) y[(size_t)m * N + n] = __float2bfloat16_rn(acc[j]);
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

template <int MT, int GSHIFT>
static int launch(const Plan& P, const CUtensorMap& mw, const CUtensorMap& ms, const CUtensorMap& mx, void* y, void* ws,
                  int M, int N, int K, cudaStream_t st) {
    auto kern = int4_umma_kernel<MT, GSHIFT>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<MT>::SmemBytes) != cudaSuccess)
        return AO_ERR_LAUNCH;
    dim3 grid(P.row_tiles, P.m_tiles, P.nsplit);
    kern<<<grid, kThreads, Cfg<MT>::SmemBytes, st>>>(mw, ms, mx, static_cast<__nv_bfloat16*>(y), static_cast<uint8_t*>(ws), M, N,
                                                     K);
    return launch_status();
}

template <int MT>
static int launch_g(const Plan& P, int g, const CUtensorMap& mw, const CUtensorMap& ms, const CUtensorMap& mx, void* y,
                    void* ws, int M, int N, int K, cudaStream_t st) {
    switch (g) {
        case 32: return launch<MT, 5>(P, mw, ms, mx, y, ws, M, N, K, st);
        case 64: return launch<MT, 6>(P, mw, ms, mx, y, ws, M, N, K, st);
        case 128: return launch<MT, 7>(P, mw, ms, mx, y, ws, M, N, K, st);
        default: return launch<MT, 8>(P, mw, ms, mx, y, ws, M, N, K, st);
    }
}

static bool shape_ok(int64_t M, int64_t N, int64_t K, int g, int ikt) {
    if (ikt != 8 || M <= 16 || N < kRows || N % 8 != 0 || K % 128 != 0 || K < 128) return false;
    if (!(g == 32 || g == 64 || g == 128 || g == 256) || K % g != 0) return false;
    if (M > (1 << 30) || N > (1 << 30) || K > (1 << 24)) return false;
    return true;
}

// 0 when this kernel does not take the shape
size_t int4_umma_workspace_bytes(int64_t M, int64_t N, int64_t K, int g, int ikt) {
    Plan P;
    if (!shape_ok(M, N, K, g, ikt) || !make_plan(M, N, K, &P)) return 0;
    return P.ws_bytes;
}

// AO_ERR_UNSUPPORTED: the caller falls back to row blocks through the GEMV kernel.
int int4_umma_linear(const void* x, int64_t ldx, int64_t x_cols, const int32_t* packed, const void* sz, int64_t M,
                     int64_t N, int64_t K, int g, int ikt, void* y, void* ws, size_t ws_bytes, cudaStream_t st) {
    Plan P;
    if (!shape_ok(M, N, K, g, ikt) || !make_plan(M, N, K, &P)) return AO_ERR_UNSUPPORTED;
    if (!aligned(x, 16) || (ldx * 2) % 16 != 0 || x_cols < 1 || x_cols > K || !aligned(packed, 16) || !aligned(sz, 16))
        return AO_ERR_UNSUPPORTED;
    if (ws == nullptr || ws_bytes < P.ws_bytes || !aligned(ws, 256)) return AO_ERR_WORKSPACE;
    CUtensorMap mw, ms, mx;
    const uint32_t scale_rows = kRawK / g > 0 ? kRawK / g : 1;
    if (!make_tensor_map_2d(&mw, CU_TENSOR_MAP_DATA_TYPE_UINT32, packed, (uint64_t)K, (uint64_t)(N / 8), (uint64_t)K * 4,
                            kRawK, kRows / 8))
        return AO_ERR_LAUNCH;
    if (!make_tensor_map_2d(&ms, CU_TENSOR_MAP_DATA_TYPE_UINT32, sz, (uint64_t)N, (uint64_t)(K / g), (uint64_t)N * 4, kRows,
                            scale_rows))
        return AO_ERR_LAUNCH;
    if (!make_tensor_map_2d(&mx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, x, (uint64_t)x_cols, (uint64_t)M, (uint64_t)ldx * 2, kKB,
                            P.MT, CU_TENSOR_MAP_SWIZZLE_128B))
        return AO_ERR_LAUNCH;
    switch (P.MT) {
        case 32: return launch_g<32>(P, g, mw, ms, mx, y, ws, (int)M, (int)N, (int)K, st);
        case 64: return launch_g<64>(P, g, mw, ms, mx, y, ws, (int)M, (int)N, (int)K, st);
        case 128: return launch_g<128>(P, g, mw, ms, mx, y, ws, (int)M, (int)N, (int)K, st);
        default: return launch_g<256>(P, g, mw, ms, mx, y, ws, (int)M, (int)N, (int)K, st);
    }
}

}  // namespace umma
}  // namespace ao
