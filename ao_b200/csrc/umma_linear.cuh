// Skeleton of the prefill-shaped weight-only linears (M > 8) on the 5th-generation tensor cores:
//   y[M][N] = x[M][K] @ dequant(W)[N][K]^T,   tcgen05.mma with the accumulator in tensor memory.
//
// The product is computed transposed: a CTA owns 128 weight rows (the MMA's M dimension, one tensor-memory lane
// per row) and MT activation rows (the MMA's N dimension, one fp32 column each), and walks K in iterations of
// 128 = two operand stages of 64.
//   warp 0     streams the packed weight bytes of its 128 rows x 128 k (and their scales) into a raw ring;
//   warp 1     streams x tiles [MT][64] with TMA in the 128-byte-swizzle K-major layout the MMA reads;
//   warp 2     owns the tensor memory and issues the MMAs: four K=16 instructions per operand stage, then a
//              commit that frees the stage;
//   warps 3-18 dequantise raw bytes in registers and write the 16-bit operand tile (layout chosen by the weight
//              format's policy), in groups that take alternate iterations whole; after the K loop the same warps
//              read the accumulator from tensor memory and store y;
//   warp 19    is a second MMA-issuing warp for token tiles of up to 128 columns.
// Measured on B200: a 128 x N x 16 MMA occupies the tensor pipe for max(N / 2, 45) cycles (64 x N x 16 takes the
// same time), and the issuing thread's two waits and two commits per operand stage cost it about as long as four
// such MMAs at N = 256.  Hence three forms of the K loop:
//   * MT <= 128: two issuing threads take turns, each accumulating into its own tensor-memory columns (the order of
//     additions stays fixed; the epilogue adds the two).  At MT = 32 the hand-over is per iteration of 128 k instead
//     of per operand stage: one activation stage holds both 64-k tiles, the two operand stages share one full and
//     one empty barrier, eight MMAs per pair of waits and pair of commits.
//   * MT = 256, one token tile: one issuing thread, one accumulator.
//   * several token tiles (M > 256, when it saves waves of CTAs: make_plan): the CTA keeps TWO accumulators of 256
//     columns (all of tensor memory) and issues the MMAs of two adjacent token tiles against every dequantised
//     operand stage: the dequantisation work per MMA halves (it, not the tensor pipe, sets the pace of the one-tile
//     form), at the same shared-memory footprint - the x ring simply turns over twice per operand stage.
// When the tiles alone would leave SMs idle, K is cut into slabs over gridDim.z; fp32 partial tiles meet in the
// workspace and the CTA that completes a tile (atomic counter) adds them in slab order (deterministic).
// Every wait is bounded; a wait that runs out sets the status word and the CTA still frees its tensor memory.
//
// A weight format plugs in as a Policy:
//   kRawBytes                      bytes of one raw stage (packed weights + scales of 128 rows x 128 k)
//   kBF16                          operands are bf16 (else fp16); y has the same type
//   kAMajorMN                      the dequantised operand tile is MN-major (else K-major), both 128-byte swizzle
//   issue_raw(p, dst, bar, k0, n0) one thread: expect_tx + the async copies of a raw stage
//   dequant<GW>(raw, a_tiles, wi, lane) warp wi of a group of GW warps: raw stage -> two consecutive 16 KiB
//                                  operand tiles (k 0..63, 64..127)
//   out_row(lane_row)              weight row (inside the CTA's 128) that tensor-memory lane `lane_row` holds
//   row_scale(p, n)                factor applied to the accumulator of weight row n
#pragma once
#include "common.cuh"
#include "ptx.cuh"
#include "tensormap.cuh"

namespace ao {
namespace umma {

// Device-side timeline (a build with -DAO_UMMA_TRACE=1 only): globaltimer stamps of the first CTA's roles, read back
// by ao_debug_read_umma_trace.  Slots: 16 g + 2 i (+1): dequant group g < 4, its i-th iteration, waits passed
// (dequantised and signalled); 64 + kb: the MMA thread has operand stage kb; 96 + kb: its MMAs are issued;
// 128 + it: raw stage it issued; 160: CTA start; 161: accumulator complete; 162: epilogue done; 256 + kb: the MMA
// thread has the activation stage; 288 + kb: MMAs issued, before the commits.
#if defined(AO_UMMA_TRACE) && AO_UMMA_TRACE
static __device__ unsigned long long g_utrace[512];
#define AO_UTR(cond, slot) do { if ((cond) && blockIdx.x == 0 && (slot) < 512) g_utrace[(slot)] = ptx::globaltimer_ns(); } while (0)
#else
#define AO_UTR(cond, slot) do { } while (0)
#endif

constexpr int kRows = 128;            // weight rows per CTA
constexpr int kKB = 64;               // k per operand stage (one 128-byte swizzle atom of 16-bit elements)
constexpr int kRawK = 128;            // k per raw stage / dequant iteration
constexpr int kABytes = kRows * kKB * 2;       // 16 KiB
constexpr int kDequantWarps = 16;
constexpr int kMmaWarp2 = 3 + kDequantWarps;   // second MMA-issuing warp (the first is warp 2)
constexpr int kThreads = (4 + kDequantWarps) * 32;
constexpr int kWaitPolls = 2000;
constexpr int kHeaderBytes = 256;
constexpr int kMaxTiles = 16384;      // completion counters (same workspace region as the decode kernels')
constexpr int kMaxSplit = 8;
constexpr int kSmemLimit = 227 * 1024;

struct alignas(64) Params {
    CUtensorMap map_x;   // activations [M][K]
    CUtensorMap map_w;   // packed weights (policy-specific view)
    CUtensorMap map_s;   // scales (policy-specific view)
    CUtensorMap map_z;   // zero points (policy-specific view)
    const void* w;       // raw pointers for policies that copy without tensor maps
    const void* scale;
    void* y;
    uint8_t* ws;
    int M, N, K;
    const void* bias;    // optional [N] in the output dtype: y = round(round(acc) + bias), the bits of an unfused add
    int grid_x, full_tiles, tail_split;   // the launch's schedule (Plan), filled in by launch()
};

// What a CTA works on.  The grid is one-dimensional: CTA b < full_tiles takes output tile b with the whole K range;
// after them every remaining tile appears tail_split times, once per K slab.  Tiles are numbered with the row-tile
// index fastest (tile = bx + grid_x * by).
struct Work {
    int bx, by, z, nsplit, slot_tile;   // slot_tile: index among the tiles that have K slabs (workspace slots, counters)
};
__device__ __forceinline__ Work work_of_cta(const Params& p) {
    Work w;
    int tile;
    const int b = blockIdx.x;
    if (b < p.full_tiles) {
        tile = b;
        w.z = 0;
        w.nsplit = 1;
        w.slot_tile = 0;
    } else {
        const int j = b - p.full_tiles;
        w.slot_tile = j / p.tail_split;
        w.z = j - w.slot_tile * p.tail_split;
        w.nsplit = p.tail_split;
        tile = p.full_tiles + w.slot_tile;
    }
    w.by = tile / p.grid_x;
    w.bx = tile - w.by * p.grid_x;
    return w;
}

#ifndef AO_UMMA_NG_SMALL
#define AO_UMMA_NG_SMALL 4
#endif

template <int MT, class Policy, int TT = 1>
struct Cfg {
    static constexpr int XBytes = MT * kKB * 2;
    // The narrowest token tiles (MT = 32): an MMA is short (45 cycles), so the waits and commits its issuing
    // thread executes around it decide the pace.  There everything is handed over per ITERATION of 128 k
    // instead of per operand stage of 64 k: one activation stage holds both 64-k tiles (two TMA copies on one
    // barrier), the two operand stages of an iteration share one full / one empty barrier, and the issuing thread
    // runs eight MMAs per pair of waits and pair of commits.
    static constexpr bool kIter = MT <= 32 && TT == 1;
    static constexpr int XStage = kIter ? 2 * XBytes : XBytes;
    // activation stages (a power of two): the ring has to cover the TMA latency
    static constexpr int SX = 4;
    static constexpr int SXShift = 2;
    // dequant warp groups: each group takes every NG-th iteration whole, so that the latency of one iteration
    // (copy wait, dequant, proxy fence, barrier) overlaps with the other groups' iterations; the operand ring holds
    // SA / 2 iterations (two stages each), at least one per group
    static constexpr int NG = MT <= 64 ? AO_UMMA_NG_SMALL : 2;
    static constexpr int GW = kDequantWarps / NG;
    static constexpr int SA = MT <= 64 ? 8 : 4;
    static constexpr int SAShift = MT <= 64 ? 3 : 2;
    static_assert(SA >= 2 * NG, "the operand ring needs an iteration per dequant group");
    static constexpr int Fixed = 1024 + SA * kABytes + SX * XStage + 512;
    static constexpr int Rfit = (kSmemLimit - Fixed) / Policy::kRawBytes;
    static constexpr int R = Rfit > 8 ? 8 : Rfit;         // raw stages (each covers 128 k; the ring covers the copy latency)
    // A group waits for its raw stage by phase parity, which tells two consecutive uses of a stage apart and no more:
    // the NG groups work on NG consecutive iterations at once, so these must all be different stages.
    static_assert(R >= 2 && R >= NG, "the raw ring needs a stage per dequant group");
    // MMA-issuing threads and accumulators per token tile.  For tiles of up to 128 columns two warps issue, taking
    // turns (operand stage by operand stage, or iteration by iteration for the narrow tiles), each into its own
    // accumulator so that the order of the additions stays fixed; the epilogue adds the two.
    static constexpr int NACC = (TT == 1 && MT <= 128) ? 2 : 1;
    static constexpr int TmemCols = MT * TT * NACC < 32 ? 32 : MT * TT * NACC;   // TT token tiles x NACC accumulators of MT columns
    static_assert(TmemCols <= 512, "tensor memory has 512 columns");
    static constexpr int SmemBytes = Fixed + R * Policy::kRawBytes;
};

// work split of one call
struct Plan {
    int MT, TT, row_tiles, m_tiles;   // m_tiles: CTAs along M, each covering TT token tiles of MT rows
    int RT;                           // row tiles per CTA (2 only with the operand in tensor memory)
    int grid_x;                       // CTAs along N = ceil(row_tiles / RT); output tiles = grid_x * m_tiles
    int full_tiles, tail_tiles, tail_split;   // tiles run whole / tiles cut into tail_split K slabs (see work_of_cta)
    size_t ws_bytes;
};

// operand_in_tmem: the weight format runs token tiles of up to 128 columns with the dequantised operand in tensor memory
// (umma_linear_ts.cuh); there a 128-column tile runs at the tensor pipe's pace (eight 64-cycle MMAs per iteration) and a
// 256-column tile does not, so batches that do not get two token tiles per CTA are cut into 128-column tiles.
inline bool make_plan(int64_t M, int64_t N, int64_t K, Plan* P, bool operand_in_tmem = false) {
    P->MT = M > 128 ? 256 : (M > 64 ? 128 : (M > 32 ? 64 : 32));
    P->row_tiles = (int)((N + kRows - 1) / kRows);
    // Two token tiles per CTA when that shortens the launch: a CTA with two tiles runs about 1.6 times as long as
    // one with a single tile (measured at K = 8192: it is bound by the tensor pipe, the single-tile CTA by the
    // dequantisation), and the grid runs in whole waves of one CTA per SM.
    P->TT = 1;
    if (P->MT == 256 && M > 256) {
        const long long mt1 = (M + 255) / 256;
        const long long waves1 = (P->row_tiles * mt1 + kNumSMs - 1) / kNumSMs;
        const long long waves2 = (P->row_tiles * ((mt1 + 1) / 2) + kNumSMs - 1) / kNumSMs;
        if (waves2 * 16 < waves1 * 10) P->TT = 2;
    }
    if (operand_in_tmem && P->MT == 256 && P->TT == 1) P->MT = 128;
    P->m_tiles = (int)((M + P->MT * P->TT - 1) / (P->MT * P->TT));
    if ((long long)P->row_tiles * P->m_tiles > (1ll << 30)) return false;   // (the grid is one-dimensional)
    const int nit = (int)(K / kRawK);
    // two row tiles per CTA against one activation stage, when the pairs still fill every SM: 128-column tiles on many
    // row tiles are otherwise bound by re-reading the activation tile from L2
    P->RT = 1;
    if (operand_in_tmem && P->MT == 128 && P->TT == 1 && (long long)((P->row_tiles + 1) / 2) * P->m_tiles >= kNumSMs) P->RT = 2;
    P->grid_x = (P->row_tiles + P->RT - 1) / P->RT;
    const int tiles = P->grid_x * P->m_tiles;
    // K slabs.  The grid runs in waves of one CTA per SM, so what counts is the number of waves times the length of
    // a CTA: in iterations of 128 k, nit / s plus a fixed part (set-up and epilogue; with slabs the fp32 partial tile
    // goes through the workspace, which costs more the wider the tile).  Either every tile is cut into s slabs, or only
    // the tiles of the last, partly filled wave are (the CTAs of the whole waves come first in the grid).
    P->full_tiles = tiles;
    P->tail_tiles = 0;
    P->tail_split = 1;
    if (P->TT == 1 && P->RT == 1) {
        const int smax = P->MT == 256 ? 2 : kMaxSplit;
        const double fixed1 = 6.0, fixed_s = 8.0 + P->MT / 16.0;
        const int whole = (tiles / kNumSMs) * kNumSMs;
        double best = (double)((tiles + kNumSMs - 1) / kNumSMs) * (nit + fixed1);
        for (int full = 0; full <= whole; full += (whole > 0 ? whole : 1)) {
            const int rem = tiles - full;
            if (rem == 0 || rem > kMaxTiles) continue;   // (one completion counter per tile that has slabs)
            for (int sp = 2; sp <= smax && nit / sp >= 8; ++sp) {
                const double cost = (double)(full / kNumSMs) * (nit + fixed1) +
                                    (double)((rem * sp + kNumSMs - 1) / kNumSMs) * ((double)nit / sp + fixed_s);
                if (cost < best - 1e-9) {
                    best = cost;
                    P->full_tiles = full;
                    P->tail_tiles = rem;
                    P->tail_split = sp;
                }
            }
            if (whole == 0) break;
        }
    }
    P->ws_bytes = kHeaderBytes + (size_t)kMaxTiles * 4 +
                  (P->tail_split > 1 ? (size_t)P->tail_tiles * P->tail_split * kRows * P->MT * 4 : 0);
    return true;
}

// eight accumulator columns of this thread's tensor-memory lane, added over the NACC accumulators in index order
// (nused <= NACC of them were written: a CTA with a single iteration has work for one issuing thread only)
template <int NACC, int MT>
__device__ __forceinline__ void load_acc8(uint32_t taddr, uint32_t (&v)[8], int nused) {
    ptx::tmem_ld_32x32b_x8(taddr, v);
    if constexpr (NACC > 1) {
        uint32_t w[NACC - 1][8];
#pragma unroll
        for (int a = 1; a < NACC; ++a) ptx::tmem_ld_32x32b_x8(taddr + a * MT, w[a - 1]);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int a = 1; a < NACC; ++a)
            if (a < nused) {
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) + __uint_as_float(w[a - 1][j]));
            }
    } else {
        ptx::tmem_ld_wait();
    }
}

template <bool BF16>
__device__ __forceinline__ void store_out(void* y, size_t idx, float v) {
    if constexpr (BF16)
        static_cast<__nv_bfloat16*>(y)[idx] = __float2bfloat16_rn(v);
    else
        static_cast<__half*>(y)[idx] = __float2half_rn(v);
}

// the linear's result rounded to the output dtype, then the bias added and rounded again: exactly what
// `y = linear(x, w); y += bias` produces (affine_quantized_tensor.py:638-640)
template <bool BF16>
__device__ __forceinline__ void store_out_bias(void* y, size_t idx, float v, float b) {
    if constexpr (BF16)
        static_cast<__nv_bfloat16*>(y)[idx] = __float2bfloat16_rn(__bfloat162float(__float2bfloat16_rn(v)) + b);
    else
        static_cast<__half*>(y)[idx] = __float2half_rn(__half2float(__float2half_rn(v)) + b);
}
template <bool BF16>
__device__ __forceinline__ float load_bias(const void* bias, int n) {
    if constexpr (BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(bias)[n]);
    return __half2float(static_cast<const __half*>(bias)[n]);
}

// Epilogue of the dequant warps (warps 3 .. 3 + kDequantWarps - 1): lane quarter (warp % 4) x column quarter
// ((warp - 3) / 4) of the accumulator(s) -> y, or, with K slabs, -> this slab's workspace slot, after which the CTA that
// completes the tile adds the slabs in order.  flag: a word of shared memory for the "last slab" broadcast.
template <int MT, class Policy, int NACC, int TT>
__device__ __forceinline__ void epilogue(const Params& p, const Work& wk, uint32_t tmem_base, int warp, int lane, int n0,
                                         int m0, int nacc_used, bool ok, volatile int* flag) {
    const int M = p.M, N = p.N;
    const int nsplit = wk.nsplit, z = wk.z;
    const int tid = threadIdx.x, dw = warp - 3;
    const int q = warp & 3, part = dw >> 2;
    const int row = q * 32 + lane;              // tensor-memory lane
    const int n = n0 + Policy::out_row(row);    // the weight row it holds
    const float rs = n < N ? Policy::row_scale(p, n) : 0.f;
    const bool has_bias = p.bias != nullptr;
    const float bias_n = (has_bias && n < N) ? load_bias<Policy::kBF16>(p.bias, n) : 0.f;
    constexpr int kColsPerWarp = MT / 4;
    const int c_begin = part * kColsPerWarp;
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    if (nsplit == 1) {
        if (ok) {
            ptx::tcgen05_fence_after_thread_sync();
#pragma unroll 1
            for (int cc = 0; cc < TT * kColsPerWarp; cc += 8) {
                // column cc of this warp's share: token tile cc / kColsPerWarp, column c0 inside the tile
                const int t = cc / kColsPerWarp, c0 = c_begin + (cc - t * kColsPerWarp);
                const int mt = m0 + t * MT;
                if (mt + c0 >= M) continue;   // uniform across the warp
                uint32_t v[8];
                load_acc8<NACC, MT>(t_lane + t * NACC * MT + c0, v, nacc_used);
                if (n < N) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int m = mt + c0 + j;
                        if (m < M) {
                            if (has_bias) store_out_bias<Policy::kBF16>(p.y, (size_t)m * N + n, __uint_as_float(v[j]) * rs, bias_n);
                            else store_out<Policy::kBF16>(p.y, (size_t)m * N + n, __uint_as_float(v[j]) * rs);
                        }
                    }
                }
            }
        }
    } else {
        // K slabs: fp32 partial tile [column][lane] into this slab's workspace slot; the CTA that completes the
        // tile (atomic counter) adds the slabs in order and stores; the counter is left at zero.
        const int tile_id = wk.slot_tile;
        float* slots = reinterpret_cast<float*>(p.ws + kHeaderBytes + (size_t)kMaxTiles * 4);
        const size_t slot_elems = (size_t)kRows * MT;
        float* mine = slots + ((size_t)tile_id * nsplit + z) * slot_elems;
        if (ok) {
            ptx::tcgen05_fence_after_thread_sync();
#pragma unroll 1
            for (int c0 = c_begin; c0 < c_begin + kColsPerWarp; c0 += 8) {
                if (m0 + c0 >= M) break;
                uint32_t v[8];
                load_acc8<NACC, MT>(t_lane + c0, v, nacc_used);
#pragma unroll
                for (int j = 0; j < 8; ++j) mine[(size_t)(c0 + j) * kRows + row] = __uint_as_float(v[j]);
            }
        }
        __threadfence();
        ptx::named_barrier_sync(1, kDequantWarps * 32);
                if (tid == 3 * 32) {
            int* counter = reinterpret_cast<int*>(p.ws + kHeaderBytes) + tile_id;
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
                        if (m < M) {
                            if (has_bias) store_out_bias<Policy::kBF16>(p.y, (size_t)m * N + n, acc[j] * rs, bias_n);
                            else store_out<Policy::kBF16>(p.y, (size_t)m * N + n, acc[j] * rs);
                        }
                    }
                }
            }
        }
    }
}

template <int MT, class Policy, int TT>
__global__ void __launch_bounds__(kThreads, 1) umma_linear_kernel(const __grid_constant__ Params p) {
    using C = Cfg<MT, Policy, TT>;
    constexpr int R = C::R;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = ptx::smem_addr(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;   // operand tiles need 1024-byte alignment
    uint8_t* sbase = smem_raw + (base - raw_addr);
    constexpr int SX = C::SX, kS = C::SA;
    const uint32_t a_base = base, x_base = a_base + kS * kABytes, raw_base = x_base + SX * C::XStage;
    const uint32_t bar_base = raw_base + R * Policy::kRawBytes;
    const uint32_t full_a = bar_base, empty = full_a + 8 * kS, full_x = empty + 8 * kS, x_empty = full_x + 8 * SX;
    const uint32_t raw_full = x_empty + 8 * SX, raw_empty = raw_full + 8 * 8, acc_full = raw_empty + 8 * 8;
    const uint32_t tmem_slot = acc_full + 8, flag_slot = tmem_slot + 4;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const Work wk = work_of_cta(p);
    const int n0 = wk.bx * kRows, m0 = wk.by * (MT * TT);   // first row of the CTA's first token tile
    const int nsplit = wk.nsplit, z = wk.z;
    const int nit_all = p.K / kRawK;
    const int it_begin = (int)(((long long)z * nit_all) / nsplit), it_end = (int)(((long long)(z + 1) * nit_all) / nsplit);
    const int nit = it_end - it_begin;     // iterations of 128 k for this CTA
    int* status = reinterpret_cast<int*>(p.ws);

    AO_UTR(tid == 0, 160);
    if (tid == 0) {
        for (int s = 0; s < kS; ++s) {
            ptx::mbar_init(full_a + 8 * s, C::GW);
            ptx::mbar_init(empty + 8 * s, 1);
        }
        for (int s = 0; s < SX; ++s) {
            ptx::mbar_init(full_x + 8 * s, 1);
            ptx::mbar_init(x_empty + 8 * s, 1);
        }
        for (int b = 0; b < R; ++b) {
            ptx::mbar_init(raw_full + 8 * b, 1);
            ptx::mbar_init(raw_empty + 8 * b, C::GW);
        }
        ptx::mbar_init(acc_full, C::NACC);
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
    // Programmatic dependent launch: the next kernel of the stream may start its set-up now; this one reads what the
    // previous kernel may have written (the activations) only after griddepcontrol.wait in the thread that loads them.
    // The weights never depend on a previous kernel, so their copies start at once.
    ptx::grid_launch_dependents();

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
                Policy::issue_raw(p, raw_base + rb * Policy::kRawBytes, raw_full + 8 * rb, (it_begin + it) * kRawK, n0);
                AO_UTR(it < 32, 128 + it);
                if (++rb == R) {
                    rb = 0;
                    ph ^= 1u;
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- activations: one operand stage per 64 k ----------------
        if (lane == 0) ptx::grid_dependency_wait();
        if (lane == 0 && C::kIter) {
            // one stage per iteration: the two 64-k tiles of the 128 k, one barrier
            for (int it = 0; it < nit; ++it) {
                const int s = it & (SX - 1);
                if (!ptx::mbar_wait_bounded(x_empty + 8 * s, (static_cast<uint32_t>(it >> C::SXShift) & 1u) ^ 1u, kWaitPolls)) {
                    ok = false;
                    break;
                }
                ptx::mbar_arrive_expect_tx(full_x + 8 * s, C::XStage);
                ptx::tma_load_2d(x_base + s * C::XStage, &p.map_x, 2 * (it_begin + it) * kKB, m0, full_x + 8 * s);
                ptx::tma_load_2d(x_base + s * C::XStage + C::XBytes, &p.map_x, (2 * (it_begin + it) + 1) * kKB, m0, full_x + 8 * s);
            }
        } else if (lane == 0) {
            // x stage number xi = kb * TT + t: token tile t of k block kb (a tile beyond M reads as zeros)
            for (int xi = 0; xi < 2 * nit * TT; ++xi) {
                const int s = xi & (SX - 1), kb = xi / TT, t = xi % TT;
                if (!ptx::mbar_wait_bounded(x_empty + 8 * s, (static_cast<uint32_t>(xi >> C::SXShift) & 1u) ^ 1u, kWaitPolls)) {
                    ok = false;
                    break;
                }
                ptx::mbar_arrive_expect_tx(full_x + 8 * s, C::XBytes);
                ptx::tma_load_2d(x_base + s * C::XBytes, &p.map_x, (2 * it_begin + kb) * kKB, m0 + t * MT, full_x + 8 * s);
            }
        }
    } else if (warp == 2 || warp == kMmaWarp2) {
        // ---------------- MMA issue: issuer w takes the operand stages kb = w, w + NACC, ... ----------------
        const int w = warp == 2 ? 0 : 1;
        constexpr uint32_t idesc = ptx::umma_idesc(kRows, MT, Policy::kBF16, Policy::kAMajorMN);
        constexpr uint32_t a_step = Policy::kAMajorMN ? (2048 >> 4) : (32 >> 4);   // descriptor units per k16
        // The whole warp walks the loop converged (waits, descriptors: warp-uniform values) and one elected lane issues,
        // so that the MMAs' operands stay in uniform registers: under `if (lane == 0)` an MMA cost its thread about 100
        // cycles of operand moves on a scheduler shared with four dequant warps.
        if (w < C::NACC && C::kIter) {
            // issuer w takes the iterations w, w + NACC, ...: eight MMAs per pair of waits and pair of commits
            for (int it = w; it < nit && ok; it += C::NACC) {
                const int s0 = (2 * it) & (kS - 1), sx = it & (SX - 1);
                bool got = ptx::mbar_wait_bounded(full_a + 8 * s0, static_cast<uint32_t>((2 * it) >> C::SAShift) & 1u, kWaitPolls) &&
                           ptx::mbar_wait_bounded(full_x + 8 * sx, static_cast<uint32_t>(it >> C::SXShift) & 1u, kWaitPolls);
                got = __all_sync(0xffffffffu, got);   // the warp stays converged even if a wait runs out
                if (!got) {
                    ok = false;
                    break;
                }
                ptx::tcgen05_fence_after_thread_sync();
                if (ptx::elect_one()) {
                    AO_UTR(it < 16, 64 + 2 * it);
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const uint64_t da = Policy::kAMajorMN ? ptx::umma_desc_mn_sw128(a_base + (s0 + h) * kABytes)
                                                              : ptx::umma_desc_k_sw128(a_base + (s0 + h) * kABytes);
                        const uint64_t db = ptx::umma_desc_k_sw128(x_base + sx * C::XStage + h * C::XBytes);
#pragma unroll
                        for (int k4 = 0; k4 < kKB / 16; ++k4)
                            ptx::umma_f16_ss(tmem_base + w * MT, da + a_step * k4, db + 2 * k4, idesc,
                                             (it >= C::NACC || h != 0 || k4 != 0) ? 1u : 0u);
                    }
                    ptx::umma_commit(x_empty + 8 * sx);
                    ptx::umma_commit(empty + 8 * s0);
                    AO_UTR(it < 16, 96 + 2 * it);
                }
                __syncwarp();
            }
            if (ok && ptx::elect_one()) ptx::umma_commit(acc_full);
            __syncwarp();
        } else if (w < C::NACC) {
            for (int kb = w; kb < 2 * nit && ok; kb += C::NACC) {
                const int s = kb & (kS - 1);
                const uint32_t ph = static_cast<uint32_t>(kb >> C::SAShift) & 1u;
                // the operand stage and the first token tile's activation stage: the whole warp waits; the elected lane
                // waits for the second token tile's stage itself, after it has issued the first tile's MMAs
                bool got = ptx::mbar_wait_bounded(full_a + 8 * s, ph, kWaitPolls) &&
                           ptx::mbar_wait_bounded(full_x + 8 * ((kb * TT) & (SX - 1)),
                                                  static_cast<uint32_t>((kb * TT) >> C::SXShift) & 1u, kWaitPolls);
                got = __all_sync(0xffffffffu, got);
                if (!got) {
                    ok = false;
                    break;
                }
                ptx::tcgen05_fence_after_thread_sync();
                if (ptx::elect_one()) {
                    AO_UTR(kb < 32, 64 + kb);
                    const uint64_t da = Policy::kAMajorMN ? ptx::umma_desc_mn_sw128(a_base + s * kABytes)
                                                          : ptx::umma_desc_k_sw128(a_base + s * kABytes);
#pragma unroll
                    for (int t = 0; t < TT; ++t) {
                        // token tile t: its x stage against the same operand stage, into its own accumulator columns
                        const int xi = kb * TT + t, sx = xi & (SX - 1);
                        if (t > 0) {
                            if (!ptx::mbar_wait_bounded(full_x + 8 * sx, static_cast<uint32_t>(xi >> C::SXShift) & 1u, kWaitPolls)) {
                                got = false;
                                break;
                            }
                            ptx::tcgen05_fence_after_thread_sync();
                        }
                        const uint64_t db = ptx::umma_desc_k_sw128(x_base + sx * C::XBytes);
#pragma unroll
                        for (int k4 = 0; k4 < kKB / 16; ++k4)
                            ptx::umma_f16_ss(tmem_base + (t * C::NACC + w) * MT, da + a_step * k4, db + 2 * k4, idesc,
                                             (kb >= C::NACC || k4 != 0) ? 1u : 0u);
                        ptx::umma_commit(x_empty + 8 * sx);
                    }
                    if (got) ptx::umma_commit(empty + 8 * s);
                    AO_UTR(kb < 32, 96 + kb);
                }
                if (TT > 1) {
                    got = __all_sync(0xffffffffu, got);   // (also reconverges the warp)
                    if (!got) {
                        ok = false;
                        break;
                    }
                } else {
                    __syncwarp();
                }
            }
            if (ok && ptx::elect_one()) ptx::umma_commit(acc_full);
            __syncwarp();
        }
    } else {
        // ---------------- dequantise (128 rows x 128 k per iteration), then epilogue ----------------
        const int dw = warp - 3;
        const int grp = dw / C::GW, wi = dw % C::GW;
        for (int it = grp; it < nit && ok; it += C::NG) {
            const int rb = it % R;
            const uint32_t rph = static_cast<uint32_t>(it / R) & 1u;
            const int s0 = (2 * it) & (kS - 1);
            const uint32_t eph = (static_cast<uint32_t>(it >> (C::SAShift - 1)) & 1u) ^ 1u;
            if (!ptx::mbar_wait_bounded(raw_full + 8 * rb, rph, kWaitPolls) ||
                !ptx::mbar_wait_bounded(empty + 8 * s0, eph, kWaitPolls) ||
                (!C::kIter && !ptx::mbar_wait_bounded(empty + 8 * (s0 + 1), eph, kWaitPolls))) {
                ok = false;
                break;
            }
            AO_UTR(wi == 0 && lane == 0 && it / C::NG < 8, 16 * grp + 2 * (it / C::NG));
            Policy::template dequant<C::GW>(raw_base + rb * Policy::kRawBytes, a_base + s0 * kABytes, wi, lane);
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                ptx::mbar_arrive(full_a + 8 * s0);
                if (!C::kIter) ptx::mbar_arrive(full_a + 8 * (s0 + 1));
                ptx::mbar_arrive(raw_empty + 8 * rb);
            }
            AO_UTR(wi == 0 && lane == 0 && it / C::NG < 8, 16 * grp + 2 * (it / C::NG) + 1);
        }
        // ---------------- epilogue: lane quarter (warp % 4) x column quarter (dw / 4) ----------------
        if (ok && !ptx::mbar_wait_bounded(acc_full, 0u, kWaitPolls)) ok = false;
        AO_UTR(dw == 0 && lane == 0, 161);
        const int nacc_used = C::kIter ? (nit < C::NACC ? nit : C::NACC) : C::NACC;
        epilogue<MT, Policy, C::NACC, TT>(p, wk, tmem_base, warp, lane, n0, m0, nacc_used, ok,
                                          reinterpret_cast<volatile int*>(sbase + (flag_slot - base)));
    }
    if (!ok && lane == 0) atomicExch(status, AO_ERR_TIMEOUT);
    AO_UTR(tid == 3 * 32, 162);
    ptx::tcgen05_fence_before_thread_sync();
    __syncthreads();
    if (warp == 2) {
        ptx::tcgen05_fence_after_thread_sync();
        ptx::tmem_dealloc(tmem_base, C::TmemCols);
    }
}

// launch with programmatic stream serialization allowed (see the kernels' griddepcontrol calls)
template <class Kern>
int launch_pdl(Kern kern, const Plan& P, int smem_bytes, const Params& prm_in, cudaStream_t st) {
    Params prm = prm_in;
    prm.grid_x = P.grid_x;
    prm.full_tiles = P.full_tiles;
    prm.tail_split = P.tail_split;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(P.full_tiles + P.tail_tiles * P.tail_split);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, kern, prm) != cudaSuccess) {
        (void)cudaGetLastError();
        return AO_ERR_LAUNCH;
    }
    return AO_OK;
}

template <int MT, class Policy, int TT = 1>
int launch(const Plan& P, const Params& prm, cudaStream_t st) {
    auto kern = umma_linear_kernel<MT, Policy, TT>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<MT, Policy, TT>::SmemBytes) != cudaSuccess)
        return AO_ERR_LAUNCH;
    return launch_pdl(kern, P, Cfg<MT, Policy, TT>::SmemBytes, prm, st);
}

template <class Policy>
int launch_mt(const Plan& P, const Params& prm, cudaStream_t st) {
    switch (P.MT) {
        case 32: return launch<32, Policy>(P, prm, st);
        case 64: return launch<64, Policy>(P, prm, st);
        case 128: return launch<128, Policy>(P, prm, st);
        default: return P.TT == 2 ? launch<256, Policy, 2>(P, prm, st) : launch<256, Policy>(P, prm, st);
    }
}

// x [M][x_cols] with row stride ldx elements (16-bit), box [64][MT], 128-byte swizzle; rows beyond M and columns
// beyond x_cols read as zero
inline bool make_x_map(CUtensorMap* map, bool bf16, const void* x, int64_t x_cols, int64_t M, int64_t ldx, int MT) {
    return make_tensor_map_2d(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, x,
                              (uint64_t)x_cols, (uint64_t)M, (uint64_t)ldx * 2, kKB, MT, CU_TENSOR_MAP_SWIZZLE_128B);
}

}  // namespace umma
}  // namespace ao
