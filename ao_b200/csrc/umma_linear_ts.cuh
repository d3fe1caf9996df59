// The prefill-shaped weight-only linear with the DEQUANTISED WEIGHTS IN TENSOR MEMORY (tcgen05.mma with the A operand
// taken from tensor memory, the activations from shared memory), for one token tile per CTA:
//   y[M][N] = x[M][K] @ dequant(W)[N][K]^T.
// Same product orientation, warp roles, K slabs, bounded waits and epilogue as umma_linear.cuh; what differs is the path
// of the dequantised operand.  There the 16 dequant warps write a swizzled 16-bit tile to shared memory (stmatrix, proxy
// fence) and a ring of such tiles (64 - 128 KB) feeds the MMA.  Here every dequant thread owns ONE weight row of the CTA's
// 128 - the row whose tensor-memory lane it can address (lane = 32 * (warp % 4) + lane id) - turns that row's 128 k of an
// iteration into 64 registers of 16-bit pairs and stores them with tcgen05.st into 64 columns of its lane: row i in lane
// i, column c = (k = 2c, 2c + 1), exactly the layout the MMA reads for an operand in tensor memory.
// Tensor memory (512 columns): accumulators in [0, 256) (two of up to 128 columns for the two issuing warps, or one of
// 256), four operand slots of 64 columns (one iteration each) in [256, 512).
// What that buys: no operand ring in shared memory (the activation ring and the raw ring get the room: up to 16 raw
// stages in flight per SM), no stmatrix address arithmetic, no proxy fence, per-row scale loads instead of byte permutes;
// and more operand slots (4) than dequant groups (2 groups of 8 warps: two warps per lane quarter, one per 64-k half), so
// a group never waits for the MMAs that read the slot it has just filled - it goes on with its other slot.
// MMA issue.  Measured: the tensor pipe runs an MMA for max(N / 2, 45) cycles and a commit for about 50.  The issuing
// WARP walks its loop converged - waits, descriptors: warp-uniform values - and one elected lane (elect.sync) issues; a
// loop under `if (lane == 0)` instead costs about 100 cycles per MMA in operand moves on a scheduler shared with four
// dequant warps, and left the pipe idle between iterations.  Issued this way eight MMAs and their commits take 0.1 us
// and queue up ahead of the pipe.
//   * Token tiles of up to 128 columns: two warps issue alternate iterations, each into its own accumulator; the
//     epilogue adds the two in a fixed order.
//   * 256 columns (one accumulator): one warp issues.  (Two warps handing a token back and forth after ISSUING their
//     MMAs do not keep the order of the additions: MMAs of different threads are only ordered by completion.)
// Either way the order of the additions is fixed: results are bit-reproducible.
//
// Two row tiles per CTA (RT = 2, chosen by make_plan for 128-column token tiles on layers with many row tiles): every
// 128-row weight tile otherwise streams the whole activation tile from L2 (32 KB per iteration per SM at 128 columns,
// 11 TB/s over 148 SMs - the bound of such shapes).  With RT = 2 a CTA owns 256 weight rows: the work units are (k
// iteration, row tile) pairs, dequant group g and issuing warp g take row tile g of every iteration, accumulator g IS
// row tile g's output, and both multiply against the same activation stage, which is released when both have committed.
//
// A weight format takes part by providing, besides what umma_linear.cuh lists,
//   kRowDequant = true
//   issue_raw_ts(p, dst, bar, k0, n0)       as issue_raw, into the layout dequant_row_half reads
//   dequant_row_half(raw, row, h, t_addr)   one thread: k = 64 h .. 64 h + 63 of weight row `row` (0..127 inside the CTA)
//                                           of the raw stage at `raw` -> 32 columns at tensor-memory address t_addr (one
//                                           tcgen05.st, executed by the whole warp)
#pragma once
#include "umma_linear.cuh"

namespace ao {
namespace umma {

template <int MT, class Policy>
struct CfgTS {
    static constexpr int NACC = MT == 256 ? 1 : 2;            // issuing warps = accumulators (added in the epilogue)
    static constexpr int XK = MT <= 128 ? 128 : 64;           // k per activation stage
    static constexpr int XBytes = MT * kKB * 2;               // one 64-k activation tile
    static constexpr int XStage = XBytes * (XK / kKB);
    static constexpr int SX = 4, SXShift = 2;                 // activation stages (a power of two)
    static constexpr int NG = 2, GW = kDequantWarps / NG;     // dequant groups: (lane quarter, 64-k half) per warp
    // Operand slots in tensor memory (unit u uses slot u % NSLOT) behind the accumulators: a dequant group can run
    // NSLOT / NG units ahead of the MMAs.  (Six slots for the narrow token tiles were measured: no gain.)
    static constexpr int NSLOT = 4;
    static constexpr int ACol0 = 256, AColsPerIt = kRawK / 2;
    static_assert(ACol0 + NSLOT * AColsPerIt <= 512, "tensor memory has 512 columns");
    static constexpr int Fixed = 1024 + SX * XStage + 512;
    static constexpr int Rfit = (kSmemLimit - Fixed) / Policy::kRawBytes;
    // raw stages: as many as fit, up to 16.  With narrow token tiles the kernel streams weights at several TB/s and
    // the raw ring is what is in flight from HBM: 8 stages (80 KB per SM, 12 MB in all) held it to about 3.3 TB/s.
    static constexpr int kMaxRaw = 16;
    static constexpr int R = Rfit > kMaxRaw ? kMaxRaw : Rfit;
    static_assert(GW == 8, "a dequant group has two warps per lane quarter of tensor memory");
    static_assert(NSLOT % NG == 0 && R >= NG, "slots and raw stages per dequant group");
    static_assert(NACC * MT <= ACol0, "the accumulators and the operand slots share the 512 columns");
    static constexpr int SmemBytes = Fixed + R * Policy::kRawBytes;
};

template <int MT, class Policy, int RT>
__global__ void __launch_bounds__(kThreads, 1) umma_linear_ts_kernel(const __grid_constant__ Params p) {
    using C = CfgTS<MT, Policy>;
    static_assert(RT == 1 || (RT == 2 && C::NACC == 2 && C::XK == kRawK), "two row tiles: one issuing warp and accumulator each");
    constexpr int R = C::R, SX = C::SX;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = ptx::smem_addr(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;   // activation tiles need 1024-byte alignment
    uint8_t* sbase = smem_raw + (base - raw_addr);
    const uint32_t x_base = base, raw_base = x_base + SX * C::XStage;
    const uint32_t bar_base = raw_base + R * Policy::kRawBytes;
    const uint32_t full_a = bar_base, a_empty = full_a + 8 * C::NSLOT, full_x = a_empty + 8 * C::NSLOT;
    const uint32_t x_empty = full_x + 8 * SX, raw_full = x_empty + 8 * SX, raw_empty = raw_full + 8 * C::kMaxRaw;
    const uint32_t acc_full = raw_empty + 8 * C::kMaxRaw, tmem_slot = acc_full + 8, flag_slot = tmem_slot + 4;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const Work wk = work_of_cta(p);
    const int n0 = wk.bx * (kRows * RT), m0 = wk.by * MT;
    const int nsplit = wk.nsplit, z = wk.z;
    const int nit_all = p.K / kRawK;
    const int it_begin = (int)(((long long)z * nit_all) / nsplit), it_end = (int)(((long long)(z + 1) * nit_all) / nsplit);
    const int nit = it_end - it_begin;     // iterations of 128 k for this CTA
    const int nunits = nit * RT;           // work units: unit u = (iteration u / RT, row tile u % RT)
    int* status = reinterpret_cast<int*>(p.ws);

    AO_UTR(tid == 0, 160);
    if (tid == 0) {
        for (int s = 0; s < C::NSLOT; ++s) {
            ptx::mbar_init(full_a + 8 * s, C::GW);
            ptx::mbar_init(a_empty + 8 * s, 1);
        }
        for (int s = 0; s < SX; ++s) {
            ptx::mbar_init(full_x + 8 * s, 1);
            ptx::mbar_init(x_empty + 8 * s, RT);   // every issuing warp that reads the stage commits to it
        }
        for (int b = 0; b < R; ++b) {
            ptx::mbar_init(raw_full + 8 * b, 1);
            ptx::mbar_init(raw_empty + 8 * b, C::GW);
        }
        ptx::mbar_init(acc_full, C::NACC);
        ptx::fence_mbar_init();
    }
    if (warp == 2) {
        ptx::tmem_alloc(tmem_slot, 512);
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
            for (int u = 0; u < nunits; ++u) {
                if (!ptx::mbar_wait_bounded(raw_empty + 8 * rb, ph, kWaitPolls)) {
                    ok = false;
                    break;
                }
                Policy::issue_raw_ts(p, raw_base + rb * Policy::kRawBytes, raw_full + 8 * rb, (it_begin + u / RT) * kRawK,
                                     n0 + (u % RT) * kRows);
                if (++rb == R) {
                    rb = 0;
                    ph ^= 1u;
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- activations: stage xi holds XK k (one or two 64-k tiles on one barrier) ----------------
        if (lane == 0) {
            ptx::grid_dependency_wait();
            constexpr int kTiles = C::XK / kKB;
            const int nstage = nit * (kRawK / C::XK);
            for (int xi = 0; xi < nstage; ++xi) {
                const int s = xi & (SX - 1);
                if (!ptx::mbar_wait_bounded(x_empty + 8 * s, (static_cast<uint32_t>(xi >> C::SXShift) & 1u) ^ 1u, kWaitPolls)) {
                    ok = false;
                    break;
                }
                ptx::mbar_arrive_expect_tx(full_x + 8 * s, C::XStage);
#pragma unroll
                for (int h = 0; h < kTiles; ++h)
                    ptx::tma_load_2d(x_base + s * C::XStage + h * C::XBytes, &p.map_x,
                                     ((it_begin * (kRawK / C::XK) + xi) * kTiles + h) * kKB, m0, full_x + 8 * s);
            }
        }
    } else if (warp == 2 || warp == kMmaWarp2) {
        // ---------------- MMA issue: issuer w takes the units w, w + NACC, ... ----------------
        const int w = warp == 2 ? 0 : 1;
        constexpr uint32_t idesc = ptx::umma_idesc(kRows, MT, Policy::kBF16, false);
#ifndef AO_UMMA_ELECT
#define AO_UMMA_ELECT 1
#endif
        // The whole warp walks the loop (waits, descriptors: warp-uniform values) and one elected lane issues, so that
        // the operands of the MMAs can stay in uniform registers.
        if (w < C::NACC && (AO_UMMA_ELECT || lane == 0)) {
            for (int u = w; u < nunits && ok; u += C::NACC) {
                // everything this unit reads has to be there
                const int it = u / RT;
                const int slot = u % C::NSLOT;
                const int xi0 = C::XK == kKB ? 2 * it : it;          // first activation stage of the iteration
                const int sx0 = xi0 & (SX - 1), sx1 = (xi0 + 1) & (SX - 1);
                bool got = ptx::mbar_wait_bounded(full_a + 8 * slot, static_cast<uint32_t>(u / C::NSLOT) & 1u, kWaitPolls) &&
                           ptx::mbar_wait_bounded(full_x + 8 * sx0, static_cast<uint32_t>(xi0 >> C::SXShift) & 1u, kWaitPolls) &&
                           (C::XK != kKB ||
                            ptx::mbar_wait_bounded(full_x + 8 * sx1, static_cast<uint32_t>((xi0 + 1) >> C::SXShift) & 1u, kWaitPolls));
#if AO_UMMA_ELECT
                got = __all_sync(0xffffffffu, got);   // the warp stays converged even if a wait runs out
#endif
                if (!got) {
                    ok = false;
                    break;
                }
                const uint32_t a_cols = tmem_base + C::ACol0 + slot * C::AColsPerIt;
                const uint64_t db0 = ptx::umma_desc_k_sw128(x_base + sx0 * C::XStage);
                const uint64_t db1 = C::XK == kKB ? ptx::umma_desc_k_sw128(x_base + sx1 * C::XStage)
                                                  : ptx::umma_desc_k_sw128(x_base + sx0 * C::XStage + C::XBytes);
                ptx::tcgen05_fence_after_thread_sync();
                const uint32_t d_cols = tmem_base + w * MT;
                const bool first = u < C::NACC;
#if AO_UMMA_ELECT
                if (ptx::elect_one()) {
#else
                {
#endif
                AO_UTR(u < 32, 64 + u);
#pragma unroll
                for (int k4 = 0; k4 < kKB / 16; ++k4)
                    ptx::umma_f16_ts(d_cols, a_cols + k4 * 8, db0 + 2 * k4, idesc, (!first || k4 != 0) ? 1u : 0u);
                if (C::XK == kKB) ptx::umma_commit(x_empty + 8 * sx0);
#pragma unroll
                for (int k4 = 0; k4 < kKB / 16; ++k4)
                    ptx::umma_f16_ts(d_cols, a_cols + kKB / 2 + k4 * 8, db1 + 2 * k4, idesc, 1u);
                ptx::umma_commit(x_empty + 8 * (C::XK == kKB ? sx1 : sx0));
                ptx::umma_commit(a_empty + 8 * slot);
                AO_UTR(u < 32, 96 + u);
                }
#if AO_UMMA_ELECT
                __syncwarp();
#endif
            }
#if AO_UMMA_ELECT
            if (ok && ptx::elect_one()) ptx::umma_commit(acc_full);
            __syncwarp();
#else
            if (ok) ptx::umma_commit(acc_full);
#endif
        }
    } else {
        // ---------------- dequantise: group grp takes the units grp, grp + 2, ... (operand slot u % 4); every thread
        // one 64-k half of the weight row of its tensor-memory lane; then the epilogue ----------------
        const int dw = warp - 3;
        const int grp = dw >> 3, h = (dw >> 2) & 1, q = warp & 3;
        const int row = Policy::out_row(q * 32 + lane);
        const uint32_t t_lane_a = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + C::ACol0 + h * (kKB / 2);
        for (int u = grp; u < nunits && ok; u += C::NG) {
            const int rb = u % R, slot = u % C::NSLOT;
            const uint32_t rph = static_cast<uint32_t>(u / R) & 1u;
            const uint32_t eph = (static_cast<uint32_t>(u / C::NSLOT) & 1u) ^ 1u;
            if (!ptx::mbar_wait_bounded(raw_full + 8 * rb, rph, kWaitPolls) ||
                !ptx::mbar_wait_bounded(a_empty + 8 * slot, eph, kWaitPolls)) {
                ok = false;
                break;
            }
            ptx::tcgen05_fence_after_thread_sync();
            AO_UTR(dw == 8 * grp && lane == 0 && (u >> 1) < 8, 16 * grp + 2 * (u >> 1));
            Policy::dequant_row_half(raw_base + rb * Policy::kRawBytes, row, h, t_lane_a + slot * C::AColsPerIt);
            ptx::tmem_st_wait();
            ptx::tcgen05_fence_before_thread_sync();
            __syncwarp();
            if (lane == 0) {
                ptx::mbar_arrive(full_a + 8 * slot);
                ptx::mbar_arrive(raw_empty + 8 * rb);
            }
            AO_UTR(dw == 8 * grp && lane == 0 && (u >> 1) < 8, 16 * grp + 2 * (u >> 1) + 1);
        }
        if (ok && !ptx::mbar_wait_bounded(acc_full, 0u, kWaitPolls)) ok = false;
        AO_UTR(dw == 0 && lane == 0, 161);
        volatile int* flag = reinterpret_cast<volatile int*>(sbase + (flag_slot - base));
        if constexpr (RT == 2) {
            // accumulator r is row tile r's output (no K slabs in this form)
            epilogue<MT, Policy, 1, 1>(p, wk, tmem_base, warp, lane, n0, m0, 1, ok, flag);
            epilogue<MT, Policy, 1, 1>(p, wk, tmem_base + MT, warp, lane, n0 + kRows, m0, 1, ok, flag);
        } else {
            const int nacc_used = nit < C::NACC ? nit : C::NACC;   // (a single iteration leaves the second accumulator unwritten)
            epilogue<MT, Policy, C::NACC, 1>(p, wk, tmem_base, warp, lane, n0, m0, nacc_used, ok, flag);
        }
    }
    if (!ok && lane == 0) atomicExch(status, AO_ERR_TIMEOUT);
    AO_UTR(tid == 3 * 32, 162);
    ptx::tcgen05_fence_before_thread_sync();
    __syncthreads();
    if (warp == 2) {
        ptx::tcgen05_fence_after_thread_sync();
        ptx::tmem_dealloc(tmem_base, 512);
    }
}

template <int MT, class Policy, int RT = 1>
int launch_ts(const Plan& P, const Params& prm, cudaStream_t st) {
    auto kern = umma_linear_ts_kernel<MT, Policy, RT>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, CfgTS<MT, Policy>::SmemBytes) != cudaSuccess)
        return AO_ERR_LAUNCH;
    return launch_pdl(kern, P, CfgTS<MT, Policy>::SmemBytes, prm, st);
}

// one token tile per CTA: operand in tensor memory; two token tiles per CTA (both accumulators fill tensor memory):
// operand ring in shared memory
template <class Policy>
int launch_mt_ts(const Plan& P, const Params& prm, cudaStream_t st) {
    static_assert(Policy::kRowDequant, "the weight format has no per-row dequantisation");
    switch (P.MT) {
        case 32: return launch_ts<32, Policy>(P, prm, st);
        case 64: return launch_ts<64, Policy>(P, prm, st);
        case 128: return P.RT == 2 ? launch_ts<128, Policy, 2>(P, prm, st) : launch_ts<128, Policy>(P, prm, st);
        default: return P.TT == 2 ? launch<256, Policy, 2>(P, prm, st) : launch_ts<256, Policy>(P, prm, st);
    }
}

}  // namespace umma
}  // namespace ao
