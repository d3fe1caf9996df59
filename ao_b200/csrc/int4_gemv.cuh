// Decode-shaped int4 weight-only linear (M <= 16) on the tensor_core_tiled weight layout:
//   y[M][N] = x[M][K] @ dequant(W)[N][K]^T,  dequant = (q - 8) * scale + zero per group of g along K
// replacing aten::_weight_int4pack_mm as called at torchao/dtypes/affine_quantized_tensor.py:631.
//
// The kernel is HBM-bound: every packed weight byte is read exactly once.
//  * One CTA per SM.  Row pairs (16 rows = two 8-row tiles) are dealt out whole and contiguously to the
//    CTAs, so no CTA ever needs another CTA's partial sums; inside a CTA the (pair, k) work is cut
//    into one contiguous range per warp and the main loop needs no CTA-wide synchronisation.
//  * The weight of one 8-row tile is one contiguous byte stream along K: a warp streams its range
//    with 1-D bulk async copies (cp.async.bulk, 2 KiB each, completion on an mbarrier) into its own
//    ring of shared-memory stages; the group scales/zeros of the stage follow with one 16-byte
//    cp.async per lane that signals the same mbarrier.
//  * A packed word already is an m16n8k16 MMA fragment (8 codes of one row): codes become bf16
//    (128 + q) with one logic op per pair and feed mma.sync with W as the 16-row operand (two 8-row
//    tiles) and x^T as the 8-column operand, fp32 accumulate.  Scale and zero are applied per group
//    on the accumulator:  y += s * (acc - 136 * Sx) + z * Sx,  Sx = sum of x over the group.
//  * A row pair whose K range is shared by several warps is combined through shared memory at the
//    end of the CTA, in a fixed order (deterministic results).  Only when the activations of the
//    whole K range do not fit in shared memory (large M * K) is K cut into slabs handled by
//    different CTAs; their partial sums meet in fixed slots of the workspace and the CTA that
//    completes the pair (atomic counter) adds the slots in a fixed order and leaves the counter at
//    zero for the next call.
#pragma once
#include "common.cuh"
#include "ptx.cuh"

// build-time experiment knobs
#ifndef AO_GEMV_SKIP
#define AO_GEMV_SKIP 0
#endif
#ifndef AO_GEMV_TRACE
#define AO_GEMV_TRACE 0
#endif
#ifndef AO_GEMV_MULHI
#define AO_GEMV_MULHI false
#endif

namespace ao {
namespace gemv {

#if AO_GEMV_TRACE
static __device__ unsigned long long g_trace[1024 * 8];
__device__ __forceinline__ unsigned long long gtime() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define AO_TRACE(slot) do { if (threadIdx.x == 0) g_trace[(blockIdx.y * gridDim.x + blockIdx.x) * 8 + (slot)] = gtime(); } while (0)
#else
#define AO_TRACE(slot) do { } while (0)
#endif

constexpr int kMaxWarps = 16;
constexpr int kMaxThreads = kMaxWarps * 32;
constexpr int kMaxStages = 4;
constexpr bool kShiftOnFmaPipe = AO_GEMV_MULHI;  // right shifts as mul.hi (FMA pipe) instead of shf (ALU pipe)

// sub-units per unit (= per pipeline stage) for a sub-unit of UB bytes per 8-row tile: 2 KiB per tile, so
// that one bulk copy moves enough bytes to keep the copy engine's request rate off the critical path
__host__ __device__ constexpr int stage_units(int ub) { return 2048 / ub > 1 ? 2048 / ub : 1; }
constexpr int kWaitPolls = 2000;          // suspending polls (<= 0.1 ms each) of one mbarrier phase
constexpr int kXsmemBudget = 64 * 1024;   // bytes of shared memory for the activation fragments
constexpr int kHeaderBytes = 256;
constexpr int kMaxPairs = 16384;          // completion counters live in a fixed region so that calls of
                                          // different shapes can share one workspace

struct Plan {
    int M, N, K, g, ikt, NB, MR;
    int NT, NP;        // 8-row tiles, 16-row pairs
    int UK, UB;        // k values per sub-unit, bytes per sub-unit per 8-row tile
    int CH;            // sub-units per unit; one unit = one pipeline stage = one weight tile load
    int GPU;           // groups per sub-unit
    int nslabs, KS;    // K slabs (split-K across CTAs so that the x slab fits shared memory)
    int ups;           // units per pair per slab
    int G;             // CTAs per slab
    int nwarps;        // warps per CTA
    int stages, stage_bytes;  // ring depth, bytes per stage
    int KSP;           // slab length rounded up to whole units (x fragments beyond KS are zero)
    int xs_off, zero_off, sx_off, p32_off, part_off, wtab_off, pcnt_off, bar_off, smem_bytes;
    uint32_t nib_mask, magic, mul28;  // 0x000F000F, bf16x2 (128, 128), 2^28: runtime values so they stay in registers
    size_t ws_counters_off, ws_slots_off, ws_bytes;
};

int make_plan(int64_t M, int64_t N, int64_t K, int g, int ikt, Plan* P);

template <int NB>
__device__ __forceinline__ void store_rows(const Plan& P, const float (&v)[NB][4], int p, int lane,
                                           __nv_bfloat16* __restrict__ y) {
    const int row = lane >> 2, c = lane & 3;
    const int n_a = 16 * p + row, n_b = n_a + 8;
    const bool has_b = (2 * p + 1) < P.NT;
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
        const int m0 = nb * 8 + 2 * c;
        if (m0 < P.M) {
            y[(size_t)m0 * P.N + n_a] = __float2bfloat16_rn(v[nb][0]);
            if (has_b) y[(size_t)m0 * P.N + n_b] = __float2bfloat16_rn(v[nb][2]);
        }
        if (m0 + 1 < P.M) {
            y[(size_t)(m0 + 1) * P.N + n_a] = __float2bfloat16_rn(v[nb][1]);
            if (has_b) y[(size_t)(m0 + 1) * P.N + n_b] = __float2bfloat16_rn(v[nb][3]);
        }
    }
}

// One warp finishes row pair p for its CTA (which has seen the pair's whole K range inside its slab):
// a direct bf16 store, or with K slabs a partial slot plus the completion protocol.
template <int NB>
__device__ __noinline__ void finish_pair(const Plan& P, const float (&v)[NB][4], int p, int slab, int lane,
                                         __nv_bfloat16* __restrict__ y, uint8_t* __restrict__ ws) {
    if (P.nslabs == 1) {
        store_rows<NB>(P, v, p, lane, y);
        return;
    }
    float4* slots = reinterpret_cast<float4*>(ws + P.ws_slots_off);
    const size_t slot_stride = (size_t)NB * 32;  // float4 per slot
    {
        float4* mine = slots + ((size_t)slab * P.NP + p) * slot_stride;
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) mine[nb * 32 + lane] = make_float4(v[nb][0], v[nb][1], v[nb][2], v[nb][3]);
    }
    __threadfence();
    __syncwarp();
    int* counter = reinterpret_cast<int*>(ws + P.ws_counters_off) + p;
    int old = 0;
    if (lane == 0) old = atomicAdd(counter, 1);
    old = __shfl_sync(0xffffffffu, old, 0);
    if (old + 1 != P.nslabs) return;
    // this CTA completed the pair: add the slabs' partial sums in slab order
    __threadfence();
    float sum[NB][4];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int i = 0; i < 4; ++i) sum[nb][i] = 0.f;
    for (int sl0 = 0; sl0 < P.nslabs; sl0 += 4) {
        float4 v4[4][NB];
        // issue the loads of up to four slots before using any of them
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const bool live = sl0 + q < P.nslabs;
#pragma unroll
            for (int nb = 0; nb < NB; ++nb)
                v4[q][nb] = live ? ptx::ldcg_f32x4(slots + ((size_t)(sl0 + q) * P.NP + p) * slot_stride + nb * 32 + lane)
                                 : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int q = 0; q < 4; ++q)
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
                sum[nb][0] += v4[q][nb].x; sum[nb][1] += v4[q][nb].y;
                sum[nb][2] += v4[q][nb].z; sum[nb][3] += v4[q][nb].w;
            }
    }
    store_rows<NB>(P, sum, p, lane, y);
    if (lane == 0) *counter = 0;  // ready for the next call
}

template <int N_WORDS>
__device__ __forceinline__ void load_words(uint32_t addr, uint32_t (&w)[N_WORDS]) {
    if constexpr (N_WORDS == 4) {
        const uint4 v = ptx::lds128(addr);
        w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
    } else if constexpr (N_WORDS == 2) {
        const uint2 v = ptx::lds64(addr);
        w[0] = v.x; w[1] = v.y;
    } else {
        w[0] = ptx::lds32(addr);
    }
}

// Compile-time shape of the kernel: IKT inner_k_tiles of the packed weight; NB 8-column blocks of the
// batch (1 for M <= 8, 2 for M <= 16); MR batch rows held per block (1, 2, 4 or 8); G32 group size / 32.
template <int IKT, int NB, int MR, int G32>
struct Shape {
    static constexpr int HALF = IKT / 2;                                      // words per lane per outer tile
    static constexpr int UK = (IKT * 16 > 32 * G32) ? IKT * 16 : 32 * G32;    // k values per sub-unit
    static constexpr int OT = UK / (IKT * 16);                                // outer tiles per sub-unit
    static constexpr int SPU = UK / 32;                                       // k32 steps per sub-unit
    static constexpr int GPU = SPU / G32;                                     // groups per sub-unit
    static constexpr int UB = UK * 4;                                         // bytes per sub-unit per 8-row tile
    static constexpr int CH = stage_units(UB);                                // sub-units per unit (stage)
    static constexpr int MRL = MR * 4;                                        // lanes that carry a batch column
    static constexpr int XSTEP = NB * MRL * 16;                               // bytes of x fragments per k32 step
};

// Dequantise-and-multiply CNT consecutive sub-units that start at sub-unit i0 of the stage at `st`.
//   su: index (inside the K slab) of the first of these sub-units.
//   m28, m24, m20: 2^28, 2^24, 2^20 as runtime values (right shifts by 4, 8, 12 as a multiply-high).
template <int IKT, int NB, int MR, int G32, int CNT>
__device__ __forceinline__ void process_units(float (&acc)[NB][4], uint32_t st, int i0, int su, uint32_t w_lane,
                                              uint32_t sc_lane, uint32_t x_base, uint32_t x_unit_stride,
                                              uint32_t sx_base, uint32_t nib, uint32_t magic, uint32_t m28,
                                              uint32_t m24, uint32_t m20) {
    using S = Shape<IKT, NB, MR, G32>;
    constexpr uint32_t tile_b = S::CH * S::UB;
#pragma unroll
    for (int i = 0; i < CNT; ++i) {
        const uint32_t xa = x_base + (su + i) * x_unit_stride;
        const uint32_t sxa = sx_base + (su + i) * (S::GPU * NB * 32);
        const uint32_t wbase = st + (i0 + i) * (S::OT * 32 * S::HALF * 4) + w_lane;
        const uint32_t scbase = st + sc_lane + (i0 + i) * (S::GPU * 64);
        float tmp[NB][4];
#pragma unroll
        for (int o = 0; o < S::OT; ++o) {
            uint32_t wa[S::HALF], wb[S::HALF];
            load_words<S::HALF>(wbase + o * (32 * S::HALF * 4), wa);
            load_words<S::HALF>(wbase + tile_b + o * (32 * S::HALF * 4), wb);
#pragma unroll
            for (int jj = 0; jj < S::HALF; ++jj) {
                constexpr int kHalf = S::HALF;
                const int ks_rel = o * kHalf + jj;
                const uint32_t wa_ = wa[jj], wb_ = wb[jj];
                // (128 + q) as bf16 pairs: rows of tile A in a0/a2, rows of tile B in a1/a3
                uint32_t sa4, sa8, sa12, sb4, sb8, sb12;
                if constexpr (kShiftOnFmaPipe) {
                    sa4 = ptx::mulhi(wa_, m28); sa8 = ptx::mulhi(wa_, m24); sa12 = ptx::mulhi(wa_, m20);
                    sb4 = ptx::mulhi(wb_, m28); sb8 = ptx::mulhi(wb_, m24); sb12 = ptx::mulhi(wb_, m20);
                } else {
                    sa4 = wa_ >> 4; sa8 = wa_ >> 8; sa12 = wa_ >> 12;
                    sb4 = wb_ >> 4; sb8 = wb_ >> 8; sb12 = wb_ >> 12;
                }
                const uint32_t a0 = ptx::and_or(wa_, nib, magic), a2 = ptx::and_or(sa4, nib, magic);
                const uint32_t a1 = ptx::and_or(wb_, nib, magic), a3 = ptx::and_or(sb4, nib, magic);
                const uint32_t e0 = ptx::and_or(sa8, nib, magic), e2 = ptx::and_or(sa12, nib, magic);
                const uint32_t e1 = ptx::and_or(sb8, nib, magic), e3 = ptx::and_or(sb12, nib, magic);
#pragma unroll
                for (int nb = 0; nb < NB; ++nb) {
                    const uint4 xb = ptx::lds128(xa + ks_rel * S::XSTEP + nb * (S::MRL * 16));
                    if (ks_rel % G32 == 0)
                        ptx::mma_bf16_16816_zero(tmp[nb], a0, a1, a2, a3, xb.x, xb.y);
                    else
                        ptx::mma_bf16_16816(tmp[nb], a0, a1, a2, a3, xb.x, xb.y);
                    ptx::mma_bf16_16816(tmp[nb], e0, e1, e2, e3, xb.z, xb.w);
                }
                if ((ks_rel + 1) % G32 == 0) {
                    // end of a quantization group: fold scale and zero into the running sums
                    const int gq = ks_rel / G32;
                    const uint32_t sa = ptx::lds32(scbase + gq * 64);
                    const uint32_t sb = ptx::lds32(scbase + gq * 64 + 32);
                    const float s_a = __uint_as_float(sa << 16), z_a = __uint_as_float(sa & 0xffff0000u);
                    const float s_b = __uint_as_float(sb << 16), z_b = __uint_as_float(sb & 0xffff0000u);
                    const float zz_a = fmaf(-136.f, s_a, z_a), zz_b = fmaf(-136.f, s_b, z_b);
#pragma unroll
                    for (int nb = 0; nb < NB; ++nb) {
                        if constexpr (MR == 1) {
                            // a single batch row: only column 0 of the accumulator tile is meaningful
                            const float sx0 = __uint_as_float(ptx::lds32(sxa + (gq * NB + nb) * 32));
                            acc[nb][0] = fmaf(s_a, tmp[nb][0], fmaf(zz_a, sx0, acc[nb][0]));
                            acc[nb][2] = fmaf(s_b, tmp[nb][2], fmaf(zz_b, sx0, acc[nb][2]));
                        } else {
                            const uint2 sxv = ptx::lds64(sxa + (gq * NB + nb) * 32);
                            const float sx0 = __uint_as_float(sxv.x), sx1 = __uint_as_float(sxv.y);
                            acc[nb][0] = fmaf(s_a, tmp[nb][0], fmaf(zz_a, sx0, acc[nb][0]));
                            acc[nb][1] = fmaf(s_a, tmp[nb][1], fmaf(zz_a, sx1, acc[nb][1]));
                            acc[nb][2] = fmaf(s_b, tmp[nb][2], fmaf(zz_b, sx0, acc[nb][2]));
                            acc[nb][3] = fmaf(s_b, tmp[nb][3], fmaf(zz_b, sx1, acc[nb][3]));
                        }
                    }
                }
            }
        }
    }
}

template <int IKT, int NB, int MR, int G32>
__global__ void __launch_bounds__(kMaxThreads, 1)
int4_gemv_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, int Kx, const uint8_t* __restrict__ wq,
                 const uint8_t* __restrict__ sz, __nv_bfloat16* __restrict__ y, uint8_t* __restrict__ ws,
                 const __grid_constant__ Plan P) {
    using S = Shape<IKT, NB, MR, G32>;
    constexpr int UB = S::UB, UK = S::UK, MRL = S::MRL, CH = S::CH;
    constexpr int kScaleCopies = CH * S::GPU * 4;  // 16-byte pieces of one stage's scales/zeros
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nthreads = blockDim.x, nwarps = nthreads >> 5;
    const int slab = blockIdx.y, cta = blockIdx.x;
    AO_TRACE(0);
    const uint32_t smem_base = ptx::smem_addr(smem);
    const int nstages = P.stages, stage_bytes = P.stage_bytes;
    const uint32_t stage0 = smem_base + warp * nstages * stage_bytes;
    const uint32_t bars = smem_base + P.bar_off + warp * kMaxStages * 8;
    const int ups = P.ups, subs = P.KS / UK;
    int* status = reinterpret_cast<int*>(ws);

    // whole row pairs per CTA; the CTA's units (pair-major, k-minor) are cut into one range per warp
    const int pbeg = static_cast<int>((static_cast<unsigned>(cta) * static_cast<unsigned>(P.NP)) / static_cast<unsigned>(P.G));
    const int pend = static_cast<int>((static_cast<unsigned>(cta + 1) * static_cast<unsigned>(P.NP)) / static_cast<unsigned>(P.G));
    const int ubeg = pbeg * ups, Lc = (pend - pbeg) * ups;
    const int wbeg = ubeg + (warp * Lc) / nwarps, wend = ubeg + ((warp + 1) * Lc) / nwarps;

    // bring this slab of x towards L2 before the weight stream fills the memory queues
    {
        const int kx0 = slab * P.KS;
        const int xbytes = 2 * max(0, min(P.KS, Kx - kx0));
        const int lines = (xbytes + 127) >> 7;
        for (int i = tid; i < P.M * lines; i += nthreads) {
            const int m = i / lines, l = i - m * lines;
            ptx::prefetch_l2(reinterpret_cast<const uint8_t*>(x + (long long)m * ldx + kx0) + (l << 7));
        }
        int* pc = reinterpret_cast<int*>(smem + P.pcnt_off);
        for (int i = tid; i < pend - pbeg; i += nthreads) pc[i] = 0;
    }
    if (lane == 0) {
        int* wt = reinterpret_cast<int*>(smem + P.wtab_off);
        wt[warp] = wbeg;
        if (warp == nwarps - 1) wt[nwarps] = ubeg + Lc;
        // one arrival for the expect_tx of the weight copies, one per lane for its scale copies
        for (int s = 0; s < nstages; ++s) ptx::mbar_init(bars + 8 * s, 33);
        ptx::fence_mbar_init();
    }
    __syncwarp();
    AO_TRACE(6);

    // ---- producer side: one unit = one stage: [tile A bytes][tile B bytes][scales/zeros] ----------------
    //   weights: CH sub-units (fewer in the last unit of K when CH does not divide) of rows 2p and 2p+1 of the
    //            packed tensor, two 1-D bulk copies issued by lane 0;
    //   scales/zeros: CH*GPU group rows x 64 bytes ((scale, zero) of the pair's 16 rows), 16 bytes per lane;
    //            pieces past the end of K or N are zero-filled.
    int pu = wbeg, pp = wbeg / ups, pul = wbeg - pp * ups, pstage = 0, issued = 0;
    auto issue_weights = [&](int p_, int ul_, int stage) {
        const int k0 = slab * P.KS + ul_ * (CH * UK);
        const int nsub = min(CH, subs - ul_ * CH);
        const bool has_b = (2 * p_ + 1) < P.NT;
        const uint32_t wbytes = static_cast<uint32_t>(nsub * UB);
        const uint32_t dst = stage0 + stage * stage_bytes;
        const uint32_t bar = bars + 8 * stage;
        const uint8_t* src = wq + ((size_t)(2 * p_) * P.K + k0) * 4;
        ptx::mbar_arrive_expect_tx(bar, has_b ? 2u * wbytes : wbytes);
        ptx::bulk_copy_g2s(dst, src, wbytes, bar);
        if (has_b) ptx::bulk_copy_g2s(dst + CH * UB, src + (size_t)P.K * 4, wbytes, bar);
    };
    auto issue_scales = [&](int p_, int ul_, int stage) {
        const int kg0 = (slab * P.KS + ul_ * (CH * UK)) / (32 * G32);
        const uint32_t dst = stage0 + stage * stage_bytes + 2 * CH * UB;
        const int pieces_ok = (2 * p_ + 1) < P.NT ? 4 : 2;  // a lone last tile has only 32 bytes per group
#pragma unroll
        for (int c0 = 0; c0 < kScaleCopies; c0 += 32) {
            const int c = c0 + lane;
            if (kScaleCopies % 32 == 0 || c < kScaleCopies) {
                const int gi = c >> 2, piece = c & 3;
                const bool live = (kg0 + gi) * (32 * G32) < P.K && piece < pieces_ok;
                const uint8_t* src = sz + ((size_t)(live ? kg0 + gi : 0) * P.N + 16 * p_) * 4 + (live ? piece * 16 : 0);
                ptx::cp_async_16(dst + c * 16, src, live ? 16u : 0u);
            }
        }
        ptx::cp_async_mbar_arrive_noinc(bars + 8 * stage);
    };
    auto advance = [&]() {
        ++pu;
        if (++pul == ups) {
            pul = 0;
            ++pp;
        }
        if (++pstage == nstages) pstage = 0;
        ++issued;
    };
    {
        const int first = min(nstages, wend - wbeg);
        for (int s = 0; s < first; ++s) {
            if (lane == 0) issue_weights(pp, pul, pstage);
            issue_scales(pp, pul, pstage);
            advance();
        }
    }
    AO_TRACE(1);

    // ---- activation prologue: x slab -> MMA fragment order, plus per-group sums of x ----------------
    {
        const int steps = P.KSP / 32;         // fragments past the slab end (odd sub-unit count) are zero
        const int items = steps * NB * MRL;  // one item = 4 words (two k16 tiles) of one lane
        const int items_round = (items + 31) / 32 * 32;
        float* p32 = reinterpret_cast<float*>(smem + P.p32_off);
        // lanes without a batch column read zeros: one sub-unit's worth of fragment bytes
        for (int i = tid; i < S::SPU * S::XSTEP / 4; i += nthreads) reinterpret_cast<uint32_t*>(smem + P.zero_off)[i] = 0u;
        for (int it = tid; it < items_round; it += nthreads) {
            uint4 wv = make_uint4(0u, 0u, 0u, 0u);
            float psum = 0.f;
            int l = 0, blk = 0;
            if (it < items) {
                l = it % MRL;
                blk = it / MRL;  // step * NB + nb
                const int nb = blk % NB, step = blk / NB;
                const int m = nb * 8 + (l >> 2), c = l & 3;
                if (m < P.M) {
                    const int k = slab * P.KS + step * 32 + 2 * c;
                    const uint32_t* row = reinterpret_cast<const uint32_t*>(x + (long long)m * ldx);
                    uint32_t w[4];
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const int kk = k + 8 * q;
                        w[q] = (kk < Kx && step * 32 + 2 * c + 8 * q < P.KS) ? __ldg(row + (kk >> 1)) : 0u;
                    }
                    wv = make_uint4(w[0], w[1], w[2], w[3]);
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        psum += bf16_bits_to_f32(w[q] & 0xffffu) + __uint_as_float(w[q] & 0xffff0000u);
                }
                *reinterpret_cast<uint4*>(smem + P.xs_off + (size_t)it * 16) = wv;
            }
            // the four lanes (c = 0..3) of a batch column are adjacent
            psum += __shfl_xor_sync(0xffffffffu, psum, 1);
            psum += __shfl_xor_sync(0xffffffffu, psum, 2);
            if (it < items && (l & 3) == 0) p32[blk * 8 + (l >> 2)] = psum;
        }
        __syncthreads();
        float* sx = reinterpret_cast<float*>(smem + P.sx_off);
        const int groups = P.KSP / (32 * G32);
        for (int it = tid; it < groups * NB * 8; it += nthreads) {
            const int mm = it & 7, nb = (it >> 3) % NB, kg = it / (8 * NB);
            float s = 0.f;
            if (mm < MR) {
#pragma unroll
                for (int q = 0; q < G32; ++q) s += p32[((kg * G32 + q) * NB + nb) * 8 + mm];
            }
            sx[it] = s;
        }
        __syncthreads();
    }

    AO_TRACE(2);
    // ---- main loop: no CTA-wide synchronisation -----------------------------------------------------
    const bool x_lane = lane < MRL;
    const uint32_t x_base = x_lane ? smem_base + P.xs_off + lane * 16 : smem_base + P.zero_off;
    const uint32_t x_unit_stride = x_lane ? static_cast<uint32_t>(S::SPU * S::XSTEP) : 0u;
    const uint32_t sx_base = smem_base + P.sx_off + (lane & 3) * 8;
    const uint32_t w_lane = lane * (S::HALF * 4);
    const uint32_t sc_lane = 2 * CH * UB + (lane >> 2) * 4;
    const uint32_t nib = P.nib_mask, magic = P.magic, m28 = P.mul28, m24 = P.mul28 >> 4, m20 = P.mul28 >> 8;
    float4* part = reinterpret_cast<float4*>(smem + P.part_off) + warp * (2 * NB * 32);
    const float4* parts = reinterpret_cast<const float4*>(smem + P.part_off);
    const int* wtab = reinterpret_cast<const int*>(smem + P.wtab_off);  // first unit of every warp, then the end
    int* pcnt = reinterpret_cast<int*>(smem + P.pcnt_off);               // units finished, per pair of this CTA
    const float inv_units_per_warp = Lc > 0 ? static_cast<float>(nwarps) / static_cast<float>(Lc) : 0.f;
    int cstage = 0, consumed = 0;
    uint32_t phase = 0;
    bool ok = true;
    float acc[NB][4];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[nb][i] = 0.f;
    int p = wbeg / ups, ul = wbeg - p * ups, ul0 = ul;
    for (int u = wbeg; u < wend; ++u) {
        if (!ptx::mbar_wait_bounded(bars + 8 * cstage, phase, kWaitPolls)) {
            ok = false;
            break;
        }
#if AO_GEMV_SKIP != 1
        process_units<IKT, NB, MR, G32, CH>(acc, stage0 + cstage * stage_bytes, 0, ul * CH, w_lane, sc_lane, x_base,
                                            x_unit_stride, sx_base, nib, magic, m28, m24, m20);
#else
        acc[0][0] += __uint_as_float(ptx::lds32(stage0 + cstage * stage_bytes + w_lane));
#endif
        ++consumed;
        __syncwarp();  // every lane is done reading this stage
        if (pu < wend) {
            if (lane == 0) issue_weights(pp, pul, pstage);
            issue_scales(pp, pul, pstage);
            advance();
        }
        if (++cstage == nstages) {
            cstage = 0;
            phase ^= 1u;
        }
        ++ul;
        if (ul == ups || u + 1 == wend) {
            // this warp's run over row pair p ends
            if (ul0 == 0 && ul == ups) {
                // the whole K range (of this slab) of the pair was ours
                finish_pair<NB>(P, acc, p, slab, lane, y, ws);
            } else {
                // partial run: a head (started inside the pair) goes to slot 0, a tail to slot 1; the warp that
                // brings the pair's unit count to ups adds all of its runs in warp order and stores the rows
                float4* slot = part + (ul0 > 0 ? 0 : NB * 32);
#pragma unroll
                for (int nb = 0; nb < NB; ++nb)
                    slot[nb * 32 + lane] = make_float4(acc[nb][0], acc[nb][1], acc[nb][2], acc[nb][3]);
                __threadfence_block();
                __syncwarp();
                int old = 0;
                if (lane == 0) old = atomicAdd(pcnt + (p - pbeg), ul - ul0);
                old = __shfl_sync(0xffffffffu, old, 0);
                if (old + (ul - ul0) == ups) {
                    __threadfence_block();
                    const int g0 = p * ups, g1 = g0 + ups;
                    int w = min(nwarps - 1, static_cast<int>(static_cast<float>(g0 - ubeg) * inv_units_per_warp));
                    while (w > 0 && wtab[w] > g0) --w;
                    while (w + 1 < nwarps && wtab[w + 1] <= g0) ++w;
                    float sum[NB][4];
#pragma unroll
                    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
                        for (int i = 0; i < 4; ++i) sum[nb][i] = 0.f;
                    for (; w < nwarps && wtab[w] < g1; ++w) {
                        if (wtab[w + 1] <= g0) continue;  // a warp without units
                        const float4* sl = parts + w * (2 * NB * 32) + (wtab[w] > g0 ? 0 : NB * 32);
#pragma unroll
                        for (int nb = 0; nb < NB; ++nb) {
                            const float4 v = sl[nb * 32 + lane];
                            sum[nb][0] += v.x; sum[nb][1] += v.y; sum[nb][2] += v.z; sum[nb][3] += v.w;
                        }
                    }
                    finish_pair<NB>(P, sum, p, slab, lane, y, ws);
                }
            }
#pragma unroll
            for (int nb = 0; nb < NB; ++nb)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[nb][i] = 0.f;
            if (ul == ups) {
                ul = 0;
                ++p;
            }
            ul0 = ul;
        }
    }
    AO_TRACE(3);
    if (!ok) {
        // A copy never signalled.  Record it, then wait (bounded) for whatever else is in flight so that the
        // CTA's shared memory is not released under a pending copy.
        if (lane == 0) atomicExch(status, AO_ERR_TIMEOUT);
        int ss = cstage;
        uint32_t ph = phase;
        for (int q = consumed; q < issued; ++q) {
            ptx::mbar_wait_bounded(bars + 8 * ss, ph, kWaitPolls);
            if (++ss == nstages) {
                ss = 0;
                ph ^= 1u;
            }
        }
    }
    AO_TRACE(5);
}

template <int IKT, int NB, int MR, int G32>
int launch_one(const Plan& P, const void* x, long long ldx, int Kx, const void* wq, const void* sz, void* y,
               void* ws, cudaStream_t st) {
    auto kern = int4_gemv_kernel<IKT, NB, MR, G32>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, P.smem_bytes) != cudaSuccess)
        return AO_ERR_LAUNCH;
    dim3 grid(P.G, P.nslabs);
    kern<<<grid, P.nwarps * 32, P.smem_bytes, st>>>(static_cast<const __nv_bfloat16*>(x), ldx, Kx,
                                                    static_cast<const uint8_t*>(wq), static_cast<const uint8_t*>(sz),
                                                    static_cast<__nv_bfloat16*>(y), static_cast<uint8_t*>(ws), P);
    return launch_status();
}

template <int IKT, int NB, int MR>
int launch_g(const Plan& P, const void* x, long long ldx, int Kx, const void* wq, const void* sz, void* y,
             void* ws, cudaStream_t st) {
    switch (P.g) {
        case 32: return launch_one<IKT, NB, MR, 1>(P, x, ldx, Kx, wq, sz, y, ws, st);
        case 64: return launch_one<IKT, NB, MR, 2>(P, x, ldx, Kx, wq, sz, y, ws, st);
        case 128: return launch_one<IKT, NB, MR, 4>(P, x, ldx, Kx, wq, sz, y, ws, st);
        case 256: return launch_one<IKT, NB, MR, 8>(P, x, ldx, Kx, wq, sz, y, ws, st);
    }
    return AO_ERR_UNSUPPORTED;
}

// Explicitly instantiated once per inner_k_tiles value, each in its own translation unit.
template <int IKT>
int launch_ikt(const Plan& P, const void* x, long long ldx, int Kx, const void* wq, const void* sz, void* y,
               void* ws, cudaStream_t st) {
    if (P.NB == 2) return launch_g<IKT, 2, 8>(P, x, ldx, Kx, wq, sz, y, ws, st);
    switch (P.MR) {
        case 1: return launch_g<IKT, 1, 1>(P, x, ldx, Kx, wq, sz, y, ws, st);
        case 2: return launch_g<IKT, 1, 2>(P, x, ldx, Kx, wq, sz, y, ws, st);
        case 4: return launch_g<IKT, 1, 4>(P, x, ldx, Kx, wq, sz, y, ws, st);
        case 8: return launch_g<IKT, 1, 8>(P, x, ldx, Kx, wq, sz, y, ws, st);
    }
    return AO_ERR_UNSUPPORTED;
}

}  // namespace gemv
}  // namespace ao
