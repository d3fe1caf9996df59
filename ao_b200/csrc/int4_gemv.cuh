// Decode-shaped int4 weight-only linear (M <= 16) on the tensor_core_tiled weight layout:
//   y[M][N] = x[M][K] @ dequant(W)[N][K]^T,  dequant = (q - 8) * scale + zero per group of g along K
// replacing aten::_weight_int4pack_mm as called at torchao/dtypes/affine_quantized_tensor.py:631.
//
// The kernel is HBM-bound: every packed weight byte is read exactly once.
//  * One CTA per SM.  Row pairs (16 rows = two 8-row tiles) are dealt out whole and contiguously to the
//    CTAs, so no CTA ever needs another CTA's partial sums.
//  * Warp specialisation: one producer warp streams the CTA's weights through a ring of shared-memory
//    stages; a stage is one row pair x one K chunk (up to 32 sub-units of 128 k): the bytes of each
//    8-row tile are one contiguous run in memory, so a stage is two large 1-D bulk async copies
//    (cp.async.bulk, up to 16 KiB each, completion counted on an mbarrier) plus the chunk's group
//    scales/zeros (16-byte cp.async pieces that signal the same mbarrier).  Full/empty mbarriers
//    hand the stages to the consumer warps and back.
//  * The consumer warps work in groups of eight that take the stages in turn; inside a group every warp
//    takes a contiguous run of the stage's sub-units.  A packed word already is an m16n8k16 MMA fragment
//    (8 codes of one row): codes become bf16 (128 + q) with one logic op per pair and feed mma.sync
//    with W as the 16-row operand (two 8-row tiles) and x^T as the 8-column operand, fp32 accumulate.
//    Scale and zero are applied per group on the accumulator:
//    y += s * (acc - 136 * Sx) + z * Sx,  Sx = sum of x over the group.
//  * At the end of a row pair every consumer warp leaves its partial sums in a ring of shared-memory
//    buffers; a reducer warp adds them in slot order (deterministic) and stores bf16.  Only when the
//    activations of the whole K range do not fit in shared memory (large M * K) is K cut into slabs
//    handled by different CTAs; the CTA that draws the last ticket of a pair (atomic counter, left at
//    zero for the next call) collects the others' partial sums from fixed slots of the workspace and
//    adds them in slab order (finish_pair below).
//  * Programmatic dependent launch: the kernel lets its successor start early and itself touches
//    nothing but weights before griddepcontrol.wait, so back-to-back linears overlap drain and fill.
//  * A single activation row (M = 1) whose K range spans several stages does not wait for all of x before the main
//    loop: the consumer warps fetch only the first K chunk themselves; for the later chunks the reducer warp, idle
//    at that time, issues one bulk async copy each, straight into the place the fragments live in, and the
//    consumer group that meets a chunk first turns it into fragment order in place (a 4 x 4 word transpose per
//    32 k) and publishes it on a "chunk ready" mbarrier.  The rest of x arrives behind the weight stream.
//  * Row-sharded multi-GPU use (nranks > 1): the reducer warp stages the CTA's rows and, at the end of the CTA,
//    stores them into every peer's landing area over peer-mapped memory (push_rows below).  The kernel does not
//    wait for the peers' rows: a layer must not end on the slowest rank, and its SMs should be free for the next
//    layer's weight prefetch while the rows are in flight.  Whoever needs the gathered output collects it with
//    the small gather-wait kernel (comm.cu).
#pragma once
#include <cstdlib>

#include "common.cuh"
#include "ptx.cuh"

// Build-time switch for A/B measurements (the shipped library uses the default):
//   AO_GEMV_BULKX   0: activations always fetched by the consumer warps before the main loop; 1: single-row kernels
//                   fetch the first K chunk that way and the later chunks by bulk copies behind the weight stream
#ifndef AO_GEMV_BULKX
#define AO_GEMV_BULKX 1
#endif

namespace ao {
namespace gemv {

// Device-side timeline (a build with -DAO_GEMV_TRACE=1 only): globaltimer stamps per CTA in a device array that a
// debug entry point of that build copies out.  The macros expand to nothing in the shipped library.
#if defined(AO_GEMV_TRACE) && AO_GEMV_TRACE
static __device__ unsigned long long g_trace[8 * 512 * 32];   // one per translation unit
#define AO_TR(slot) do { g_trace[((P.trace_id & 7) * 512 + blockIdx.y * gridDim.x + blockIdx.x) * 32 + (slot)] = ptx::globaltimer_ns(); } while (0)
#else
#define AO_TR(slot) do { } while (0)
#endif

constexpr int kMaxConsumerWarps = 16;
constexpr int kMaxThreads = (kMaxConsumerWarps + 2) * 32;  // + the producer warp and the reducer warp
constexpr int kMaxStages = 4;
constexpr int kMaxSubs = 32;             // sub-units per stage
constexpr int kSmemBudget = 220 * 1024;
constexpr int kWaitPolls = 2000;          // suspending polls (<= 0.1 ms each) of one mbarrier phase
constexpr int kHeaderBytes = 256;
constexpr int kMaxRanks = 8;
constexpr int kMaxXChunks = 32;          // K chunks of x with a barrier pair of their own (single-row bulk prologue)
constexpr int kMaxPairs = 16384;          // completion counters live in a fixed region so that calls of
                                          // different shapes can share one workspace

struct Plan {
    int M, N, K, g, ikt, NB, MR;
    int NT, NP;        // 8-row tiles, 16-row pairs
    int UK, UB;        // k values per sub-unit, bytes per sub-unit per 8-row tile
    int GPU;           // groups per sub-unit
    int nslabs, KS;    // K slabs (split-K across CTAs so that the x slab fits shared memory)
    int subs;          // sub-units per pair per slab
    int SUBS, cpp;     // sub-units per full stage, stages (K chunks) per pair
    int G;             // CTAs per slab
    int pair_q, pair_r;  // row pairs per CTA: NP / G, and the number of CTAs that have one more (NP % G)
    int nwarps;        // consumer warps per CTA (the CTA has one more warp, the producer)
    int GW;            // consumer warps that share one stage (nwarps / GW groups take the stages in turn)
    int nbuf;          // ring of per-pair partial-sum buffers (a power of two)
    int stages, stage_bytes;  // ring depth (a power of two), bytes per stage
    int gw_shift, stage_shift, nbuf_shift;  // log2 of GW, stages, nbuf: the per-stage bookkeeping has no divisions
    int xs_off, zero_off, sx_off, part_off, bar_off, smem_bytes;
    int trace_id;      // timeline slot of this launch (trace builds only)
    uint32_t nib_mask, magic;  // 0x000F000F, bf16x2 (128, 128): runtime values so they stay in registers
    size_t ws_counters_off, ws_slots_off, ws_bytes;
    // output exchange over peer memory (nranks > 1): every CTA sends its rows to every peer as 8-byte
    // {two bf16 rows, call number} words.  peer_ll[r]: rank r's landing area of this call site, two buffers
    // [call parity][source rank][M][N/2] of such words; the CTA's own rows also go to y_gathered [rank][M][N];
    // local_state = the call site's {CTAs of this launch that have pushed, pushes so far, ...} on this rank
    const __nv_bfloat16* bias;   // optional [N]: y = bf16(bf16(acc) + bias), the bits of `y = linear(x, w); y += bias`
    int nranks, rank;
    int ystage_off;     // shared-memory staging of the CTA's output rows [M][16 * pairs per CTA]
    int rows_cta_max;   // 16 * max pairs per CTA
    uint2* peer_ll[kMaxRanks];
    __nv_bfloat16* y_gathered;
    unsigned* local_state;
};

int make_plan(int64_t M, int64_t N, int64_t K, int g, int ikt, Plan* P);

template <int NB>
__device__ __forceinline__ void store_rows(const Plan& P, const float (&v)[NB][4], int p, int lane,
                                           __nv_bfloat16* __restrict__ y) {
    const int row = lane >> 2, c = lane & 3;
    const int n_a = 16 * p + row, n_b = n_a + 8;
    const bool has_b = (2 * p + 1) < P.NT;
    // with a bias: the result rounded to bf16, the bias added, rounded again (what the unfused add produces)
    const bool biased = P.bias != nullptr;
    const float b_a = biased ? __bfloat162float(P.bias[n_a]) : 0.f;
    const float b_b = (biased && has_b) ? __bfloat162float(P.bias[n_b]) : 0.f;
    auto out = [&](float acc, float b) {
        const __nv_bfloat16 r = __float2bfloat16_rn(acc);
        return biased ? __float2bfloat16_rn(__bfloat162float(r) + b) : r;
    };
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
        const int m0 = nb * 8 + 2 * c;
        if (m0 < P.M) {
            y[(size_t)m0 * P.N + n_a] = out(v[nb][0], b_a);
            if (has_b) y[(size_t)m0 * P.N + n_b] = out(v[nb][2], b_b);
        }
        if (m0 + 1 < P.M) {
            y[(size_t)(m0 + 1) * P.N + n_a] = out(v[nb][1], b_a);
            if (has_b) y[(size_t)(m0 + 1) * P.N + n_b] = out(v[nb][3], b_b);
        }
    }
}

// Header words of the workspace used by the K-slab hand-off: {CTAs of this launch that have finished, number of
// slab launches completed so far}.  The second is the tag the partial sums of the next launch carry.
constexpr int kCallStateOff = 16;

__device__ __forceinline__ uint2 ld_volatile_u2(const uint2* p) {
    uint2 v;
    asm volatile("ld.volatile.global.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_volatile_u2(uint2* p, uint32_t a, uint32_t b) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(a), "r"(b) : "memory");
}
// 8-byte store into a peer's memory: a plain (weak) store, which is posted without waiting for the NVLink round
// trip of the thread's previous store to that peer (volatile stores were observed to); the word is still written as
// one unit
__device__ __forceinline__ void st_peer_u2(uint2* p, uint32_t a, uint32_t b) {
    asm volatile("st.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(a), "r"(b) : "memory");
}

// One warp finishes row pair p for its CTA (which has seen the pair's whole K range inside its slab): a direct bf16
// store, or with K slabs the hand-off.  The CTAs that share a pair draw a ticket from the pair's counter when they
// start on it (the round trip is over by the time their sums are ready); the one that drew the last ticket adds the
// slabs up in slab order and stores y, the others leave their partial sums in their workspace slot as 8-byte
// {value, tag} words (tag = number of this launch; an 8-byte store is written as a unit, so a word that carries the
// tag carries the value: no fence is needed) and move on.  The finisher polls those words (bounded); it only ever
// waits for CTAs that hold a ticket, i.e. are running and have no reason to wait for it, and every CTA walks its
// pairs in the same order.
template <int NB>
__device__ __noinline__ bool finish_pair(const Plan& P, const float (&v)[NB][4], int p, int slab, int lane,
                                         __nv_bfloat16* __restrict__ y, uint8_t* __restrict__ ws, unsigned call, int ticket) {
    if (P.nslabs == 1) {
        store_rows<NB>(P, v, p, lane, y);
        return true;
    }
    uint2* slots = reinterpret_cast<uint2*>(ws + P.ws_slots_off);
    const size_t slot_stride = (size_t)NB * 4 * 32;  // words per slot: [batch block][value][lane]
    if (ticket + 1 != P.nslabs) {
        uint2* mine = slots + ((size_t)slab * P.NP + p) * slot_stride + lane;
#pragma unroll
        for (int nb = 0; nb < NB; ++nb)
#pragma unroll
            for (int i = 0; i < 4; ++i) st_volatile_u2(mine + (nb * 4 + i) * 32, __float_as_uint(v[nb][i]), call);
        return true;
    }
    if (lane == 0) *(reinterpret_cast<int*>(ws + P.ws_counters_off) + p) = 0;   // ready for the next call
    float sum[NB][4];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int i = 0; i < 4; ++i) sum[nb][i] = 0.f;
    bool ok = true;
    const uint64_t t0 = ptx::globaltimer_ns();
    for (int sl0 = 0; sl0 < P.nslabs; sl0 += 4) {
        // the loads of up to four slabs are issued before any is looked at, and all of them again while any word of
        // the warp still lacks the tag: a retry costs one round trip, not one per word
        uint2 q[4][NB][4];
        for (;;) {
            bool all = true;
#pragma unroll
            for (int h = 0; h < 4; ++h) {
                const int sl = sl0 + h;
                if (sl >= P.nslabs || sl == slab) continue;
                const uint2* src = slots + ((size_t)sl * P.NP + p) * slot_stride + lane;
#pragma unroll
                for (int nb = 0; nb < NB; ++nb)
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        q[h][nb][i] = ld_volatile_u2(src + (nb * 4 + i) * 32);
                    }
            }
#pragma unroll
            for (int h = 0; h < 4; ++h) {
                const int sl = sl0 + h;
                if (sl >= P.nslabs || sl == slab) continue;
#pragma unroll
                for (int nb = 0; nb < NB; ++nb)
#pragma unroll
                    for (int i = 0; i < 4; ++i) all = all && (q[h][nb][i].y == call);
            }
            if (__all_sync(0xffffffffu, all)) break;
            if (ptx::globaltimer_ns() - t0 > 200000000ull) {   // 0.2 s
                ok = false;
                break;
            }
        }
#pragma unroll
        for (int h = 0; h < 4; ++h) {
            const int sl = sl0 + h;
            if (sl >= P.nslabs) continue;
#pragma unroll
            for (int nb = 0; nb < NB; ++nb)
#pragma unroll
                for (int i = 0; i < 4; ++i) sum[nb][i] += (sl == slab) ? v[nb][i] : __uint_as_float(q[h][nb][i].x);
        }
    }
    store_rows<NB>(P, sum, p, lane, y);
    return ok;
}


// ---- output exchange over peer memory -------------------------------------------------------------------------

// The reducer warp keeps the CTA's finished rows in shared memory ([M][rows_cta_max] bf16) instead of storing them.
template <int NB>
__device__ __forceinline__ void stage_rows(const Plan& P, __nv_bfloat16* ys, const float (&v)[NB][4], int pi, int lane) {
    const int row = lane >> 2, c = lane & 3;
    const int r_a = 16 * pi + row, r_b = r_a + 8;
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
        const int m0 = nb * 8 + 2 * c;
        if (m0 < P.M) {
            ys[m0 * P.rows_cta_max + r_a] = __float2bfloat16_rn(v[nb][0]);
            ys[m0 * P.rows_cta_max + r_b] = __float2bfloat16_rn(v[nb][2]);
        }
        if (m0 + 1 < P.M) {
            ys[(m0 + 1) * P.rows_cta_max + r_a] = __float2bfloat16_rn(v[nb][1]);
            ys[(m0 + 1) * P.rows_cta_max + r_b] = __float2bfloat16_rn(v[nb][3]);
        }
    }
}

// One warp sends the CTA's rows (output rows 16 * pbeg .. of every batch row) to every peer and copies them into
// this rank's own block of the gathered output.  Data and "it has arrived" travel in the same 8-byte store (two bf16
// rows + the call number), which the hardware writes as one unit, so no fence and no separate flag are needed: a
// receiver polls each word of its landing area until it carries the call's number.  The landing areas are double
// buffered by the parity of the call number: a peer that is one call ahead writes into the other buffer, and it
// cannot be two ahead, because its next push of this call site comes after its own gather-wait, which needs this
// rank's push in between.
static __device__ __noinline__ void push_rows(const Plan& P, const __nv_bfloat16* ys, int pbeg, int npairs, int lane,
                                              unsigned call) {
    const int nrows = min(16 * npairs, P.N - 16 * pbeg);     // a lone last 8-row tile ends the matrix
    const int n2 = nrows / 2, half_n = P.N / 2;              // 4-byte row pairs
    const size_t block = (size_t)P.M * half_n;                // words per source rank in a landing buffer
    const size_t parity_off = (call & 1u) ? (size_t)P.nranks * block : 0;
    __syncwarp();
    for (int i = 1; i < P.nranks; ++i) {
        const int r = (P.rank + i) % P.nranks;
        uint2* dst = P.peer_ll[r] + parity_off + (size_t)P.rank * block + 8 * pbeg;
        for (int m = 0; m < P.M; ++m) {
            const uint32_t* src = reinterpret_cast<const uint32_t*>(ys + m * P.rows_cta_max);
            for (int j = lane; j < n2; j += 32) st_peer_u2(dst + (size_t)m * half_n + j, src[j], call);
        }
    }
    // local block
    {
        __nv_bfloat16* dst = P.y_gathered + (size_t)P.rank * P.M * P.N + 16 * pbeg;
        for (int m = 0; m < P.M; ++m) {
            const uint4* src = reinterpret_cast<const uint4*>(ys + m * P.rows_cta_max);
            uint4* d = reinterpret_cast<uint4*>(dst + (size_t)m * P.N);
            for (int j = lane; j < nrows / 8; j += 32) d[j] = src[j];
        }
    }
    // the last CTA to finish advances the call number for the next launch
    if (lane == 0) {
        const unsigned done = atomicAdd(P.local_state, 1u);
        if (done + 1 == gridDim.x) {
            P.local_state[0] = 0u;
            P.local_state[1] = call;
        }
    }
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
    static constexpr int MRL = MR * 4;                                        // lanes that carry a batch column
    static constexpr int XSTEP = NB * MRL * 16;                               // bytes of x fragments per k32 step
};

// Dequantise-and-multiply CNT consecutive sub-units that start at sub-unit i0 of the stage at `st`.
//   su: index (inside the K slab) of the first of these sub-units; tile_b: byte offset of tile B's bytes.
template <int IKT, int NB, int MR, int G32, int CNT>
__device__ __forceinline__ void process_units(float (&acc)[NB][4], uint32_t st, int i0, int su, uint32_t tile_b,
                                              uint32_t w_lane, uint32_t sc_lane, uint32_t x_base,
                                              uint32_t x_unit_stride, uint32_t sx_base, uint32_t nib, uint32_t magic) {
    using S = Shape<IKT, NB, MR, G32>;
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
                const uint32_t a0 = ptx::and_or(wa_, nib, magic), a2 = ptx::and_or(wa_ >> 4, nib, magic);
                const uint32_t a1 = ptx::and_or(wb_, nib, magic), a3 = ptx::and_or(wb_ >> 4, nib, magic);
                const uint32_t e0 = ptx::and_or(wa_ >> 8, nib, magic), e2 = ptx::and_or(wa_ >> 12, nib, magic);
                const uint32_t e1 = ptx::and_or(wb_ >> 8, nib, magic), e3 = ptx::and_or(wb_ >> 12, nib, magic);
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

// Single-row bulk prologue: the warps of one consumer group turn a chunk of x that a bulk copy has just landed
// (raw bf16, 64 bytes per 32 k) into MMA fragment order in place -- lane c of a fragment column reads the bf16
// pairs at k = 2c + {0, 8, 16, 24}, i.e. a 4 x 4 word transpose inside every 64-byte block, one thread per block --
// and write the per-group sums of x of the chunk's groups.  blk0: first 32-k block of the chunk inside the slab;
// k_abs0: its first k inside the activation row; elements at k >= Kx do not exist and count as zero (Kx % 8 == 0).
template <int G32>
__device__ __noinline__ void prepare_x_chunk(uint8_t* xs, float* sx, int blk0, int nblk, int k_abs0, int Kx,
                                             int wi, int GW, int lane) {
    for (int b0 = wi * 32; b0 < nblk; b0 += GW * 32) {   // uniform per warp: the shuffles need every lane
        const int b = b0 + lane;
        const bool valid = b < nblk;
        float psum = 0.f;
        if (valid) {
            uint4* blk = reinterpret_cast<uint4*>(xs + (size_t)(blk0 + b) * 64);
            const int kb = k_abs0 + 32 * b;
            uint4 q[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) q[u] = (kb + 8 * u + 8 <= Kx) ? blk[u] : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const uint32_t wv[4] = {q[u].x, q[u].y, q[u].z, q[u].w};
                float part = 0.f;
#pragma unroll
                for (int cc = 0; cc < 4; ++cc) part += bf16_bits_to_f32(wv[cc] & 0xffffu) + __uint_as_float(wv[cc] & 0xffff0000u);
                psum += part;
            }
            blk[0] = make_uint4(q[0].x, q[1].x, q[2].x, q[3].x);
            blk[1] = make_uint4(q[0].y, q[1].y, q[2].y, q[3].y);
            blk[2] = make_uint4(q[0].z, q[1].z, q[2].z, q[3].z);
            blk[3] = make_uint4(q[0].w, q[1].w, q[2].w, q[3].w);
        }
#pragma unroll
        for (int o = 1; o < G32; o <<= 1) psum += __shfl_xor_sync(0xffffffffu, psum, o);
        if (valid && (b & (G32 - 1)) == 0) sx[((blk0 + b) / G32) * 8] = psum;
    }
}

// shared-memory control block of one CTA
constexpr int kMaxPairBufs = 8;

template <int IKT, int NB, int MR, int G32>
__global__ void __launch_bounds__(kMaxThreads, 1)
int4_gemv_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, int Kx, const uint8_t* __restrict__ wq,
                 const uint8_t* __restrict__ sz, __nv_bfloat16* __restrict__ y, uint8_t* __restrict__ ws,
                 const __grid_constant__ Plan P) {
    using S = Shape<IKT, NB, MR, G32>;
    constexpr int UB = S::UB, UK = S::UK, MRL = S::MRL;
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nwarps = P.nwarps, nconsumers = nwarps * 32;
    const int slab = blockIdx.y, cta = blockIdx.x;
    const uint32_t smem_base = ptx::smem_addr(smem);
    if (tid == 0) AO_TR(0);                      // CTA start
    if (tid == P.nwarps * 32) AO_TR(1);          // producer lane start
    const int nstages = P.stages, stage_bytes = P.stage_bytes;
    const uint32_t full_bar = smem_base + P.bar_off, empty_bar = full_bar + kMaxStages * 8;
    const uint32_t pair_full_bar = empty_bar + kMaxStages * 8, pair_free_bar = pair_full_bar + kMaxPairBufs * 8;
    const uint32_t x_full_bar = pair_free_bar + kMaxPairBufs * 8, x_ready_bar = x_full_bar + kMaxXChunks * 8;
    const int subs = P.subs, SUBS = P.SUBS, cpp = P.cpp;
    // single activation row, several K chunks: chunks 1.. of x by bulk copy when its address and width allow
    constexpr bool kM1 = (NB == 1 && MR == 1);
    const bool bulk_x = kM1 && (AO_GEMV_BULKX != 0) && cpp > 1 && cpp <= kMaxXChunks &&
                        (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (Kx & 7) == 0;
    const uint32_t tile_b = SUBS * UB, sc_off = 2 * SUBS * UB;
    int* status = reinterpret_cast<int*>(ws);

    // whole row pairs per CTA, contiguous, the first pair_r CTAs one more than the others; the CTA's stream of stages
    // is (pair, K chunk), pair-major
    const int pbeg = cta * P.pair_q + min(cta, P.pair_r);
    const int pend = pbeg + P.pair_q + (cta < P.pair_r ? 1 : 0);
    const int nstage_total = (pend - pbeg) * cpp;

    // the next kernel of the stream may start its own weight prefetch as soon as SMs free up; whatever it reads or
    // writes besides weights comes after its grid_dependency_wait()
    ptx::grid_launch_dependents();
    if (tid == nconsumers) {
        for (int s = 0; s < nstages; ++s) {
            ptx::mbar_init(full_bar + 8 * s, 33);       // expect_tx arrival + one cp.async arrival per producer lane
            ptx::mbar_init(empty_bar + 8 * s, P.GW);    // one arrival per consumer warp of the stage's group
        }
        const int nslots_init = min(nwarps >> P.gw_shift, cpp) << P.gw_shift;
        for (int i = 0; i < P.nbuf; ++i) {
            ptx::mbar_init(pair_full_bar + 8 * i, nslots_init);  // one arrival per warp that worked on the pair
            ptx::mbar_init(pair_free_bar + 8 * i, 1);            // the reducer hands the buffer back
        }
        if (bulk_x) {
            for (int c = 1; c < cpp; ++c) {
                ptx::mbar_init(x_full_bar + 8 * c, 1);           // the bulk copy of chunk c of x (expect_tx arrival)
                ptx::mbar_init(x_ready_bar + 8 * c, 1 << P.gw_shift);   // the warps that put it into fragment order
            }
        }
        ptx::fence_mbar_init();
    }
    // the producer warp only announces that the barriers exist and goes straight to its first copies
    if (warp == nwarps) {
        __syncwarp();
        ptx::named_barrier_arrive(2, blockDim.x);
    } else {
        ptx::named_barrier_sync(2, blockDim.x);
    }
    if (tid == 0) AO_TR(5);                      // consumers past the barrier-ready barrier

    if (warp == nwarps) {
        // =============================== producer warp =================================================
        // stage = [tile A bytes][tile B bytes][scales/zeros: one 64-byte row per group]
        int pi = 0, c = 0, s = 0;
        uint32_t phase = 1;  // a fresh barrier counts as "previous phase complete"
        const uint64_t stream_once = ptx::l2_policy_evict_first();   // every weight byte is read exactly once
        bool ok = true;
        for (int t = 0; t < nstage_total; ++t) {
            if (!ptx::mbar_wait_bounded(empty_bar + 8 * s, phase, kWaitPolls)) {
                ok = false;
                break;
            }
            const int p = pbeg + pi;
            const int sub0 = c * SUBS;
            const int nsub = min(SUBS, subs - sub0);
            const int k0 = slab * P.KS + sub0 * UK;
            const bool has_b = (2 * p + 1) < P.NT;
            const uint32_t dst = smem_base + s * stage_bytes;
            const uint32_t bar = full_bar + 8 * s;
            if (lane == 0) {
                const uint32_t wbytes = static_cast<uint32_t>(nsub * UB);
                const uint8_t* src = wq + ((size_t)(2 * p) * P.K + k0) * 4;
                ptx::mbar_arrive_expect_tx(bar, has_b ? 2u * wbytes : wbytes);
                ptx::bulk_copy_g2s_hint(dst, src, wbytes, bar, stream_once);
                if (has_b) ptx::bulk_copy_g2s_hint(dst + tile_b, src + (size_t)P.K * 4, wbytes, bar, stream_once);
                if (t == 0) AO_TR(8);            // first stage's bulk copies issued
            }
            {
                // 64 bytes ((scale, zero) of the pair's 16 rows) per group; a lone last tile has only 32
                const int kg0 = k0 / (32 * G32);
                const int pieces = nsub * S::GPU * 4;
                const int piece_ok = has_b ? 4 : 2;
                for (int q = lane; q < pieces; q += 32) {
                    const int gi = q >> 2, piece = q & 3;
                    const bool live = piece < piece_ok;
                    const uint8_t* src = sz + ((size_t)(kg0 + gi) * P.N + 16 * p) * 4 + (live ? piece * 16 : 0);
                    ptx::cp_async_16(dst + sc_off + q * 16, src, live ? 16u : 0u);
                }
                ptx::cp_async_mbar_arrive_noinc(bar);
            }
            if (++c == cpp) {
                c = 0;
                ++pi;
            }
            if (++s == nstages) {
                s = 0;
                phase ^= 1u;
            }
        }
        if (lane == 0) AO_TR(9);                 // last stage issued
        if (!ok && lane == 0) {
            ptx::grid_dependency_wait();
            atomicExch(status, AO_ERR_TIMEOUT);
        }
        return;
    }

    if (warp == nwarps + 1) {
        // =============================== reducer warp ==================================================
        if (lane == 0) AO_TR(10);      // reducer at the dependency wait
        ptx::grid_dependency_wait();   // y, the workspace and the exchange state may be in use by earlier kernels
        if (lane == 0) AO_TR(11);      // dependency wait passed
        if (bulk_x && lane == 0) {
            // x may be the previous kernel's output, hence after the wait: one bulk copy per K chunk, straight
            // into the place where the fragments live (the consumers reorder each chunk in place)
            const uint64_t keep = ptx::l2_policy_evict_last();   // every CTA reads the same activations
            const int CK = SUBS * UK;
            for (int c = 1; c < cpp; ++c) {
                const int k0 = slab * P.KS + c * CK;                         // first k of the chunk in the row
                const int nk = max(0, min(min(CK, P.KS - c * CK), Kx - k0));  // elements that exist
                const uint32_t bar = x_full_bar + 8 * c;
                if (nk > 0) {
                    ptx::mbar_arrive_expect_tx(bar, static_cast<uint32_t>(nk) * 2u);
                    ptx::bulk_copy_g2s_hint(smem_base + P.xs_off + c * CK * 2, x + k0, static_cast<uint32_t>(nk) * 2u, bar, keep);
                } else {
                    ptx::mbar_arrive(bar);
                }
            }
        }
        // adds the consumer warps' partial sums of each finished pair in slot order and stores the rows
        const int NGr = nwarps >> P.gw_shift;
        const int nslots = min(NGr, cpp) << P.gw_shift;
        const int nbuf_mask = P.nbuf - 1, nbuf_shift = P.nbuf_shift;
        const float4* parts = reinterpret_cast<const float4*>(smem + P.part_off);
        bool ok = true;
        // number of this call of the exchange (all CTAs of a launch read the same value: it changes when the last
        // CTA of the launch finishes)
        const unsigned call = P.nranks > 1 ? *reinterpret_cast<volatile unsigned*>(P.local_state + 1) + 1u : 0u;
        // tag of this launch's slab partial sums (all CTAs read the same value: it changes when the last one finishes)
        unsigned* call_state = reinterpret_cast<unsigned*>(ws + kCallStateOff);
        const unsigned slab_call = P.nslabs > 1 ? *reinterpret_cast<volatile unsigned*>(call_state + 1) + 1u : 0u;
        for (int pi = 0; pi < pend - pbeg; ++pi) {
            const int buf = pi & nbuf_mask;
            // issued before the wait: the ticket that decides who finishes the pair
            int ticket = 0;
            if (P.nslabs > 1 && lane == 0) ticket = atomicAdd(reinterpret_cast<int*>(ws + P.ws_counters_off) + pbeg + pi, 1);
            if (!ptx::mbar_wait_bounded(pair_full_bar + 8 * buf, static_cast<uint32_t>(pi >> nbuf_shift) & 1u, kWaitPolls)) {
                ok = false;
                break;
            }
            float sum[NB][4];
#pragma unroll
            for (int nb = 0; nb < NB; ++nb)
#pragma unroll
                for (int i = 0; i < 4; ++i) sum[nb][i] = 0.f;
            // nslots is a multiple of 8: eight slots' loads are issued before any is used
            const float4* src = parts + (buf * nslots) * (NB * 32) + lane;
            for (int w0 = 0; w0 < nslots; w0 += 8) {
                float4 v[8][NB];
#pragma unroll
                for (int q = 0; q < 8; ++q)
#pragma unroll
                    for (int nb = 0; nb < NB; ++nb) v[q][nb] = src[((w0 + q) * NB + nb) * 32];
#pragma unroll
                for (int q = 0; q < 8; ++q)
#pragma unroll
                    for (int nb = 0; nb < NB; ++nb) {
                        sum[nb][0] += v[q][nb].x; sum[nb][1] += v[q][nb].y;
                        sum[nb][2] += v[q][nb].z; sum[nb][3] += v[q][nb].w;
                    }
            }
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(pair_free_bar + 8 * buf);
            if (P.nranks > 1)
                stage_rows<NB>(P, reinterpret_cast<__nv_bfloat16*>(smem + P.ystage_off), sum, pi, lane);
            else if (!finish_pair<NB>(P, sum, pbeg + pi, slab, lane, y, ws, slab_call, __shfl_sync(0xffffffffu, ticket, 0)))
                ok = false;
        }
        if (P.nslabs > 1 && lane == 0) {
            // the last CTA of the launch to finish advances the launch number
            const unsigned done = atomicAdd(call_state, 1u);
            if (done + 1 == gridDim.x * gridDim.y) {
                call_state[0] = 0u;
                call_state[1] = slab_call;
            }
        }
        if (P.nranks > 1) {
            // even after a failed wait the rows are sent, so that the other ranks are not left waiting for this one
            push_rows(P, reinterpret_cast<const __nv_bfloat16*>(smem + P.ystage_off), pbeg, pend - pbeg, lane, call);
        }
        if (lane == 0) AO_TR(12);      // reducer done: last rows stored
        if (!ok && lane == 0) atomicExch(status, AO_ERR_TIMEOUT);
        return;
    }

    // ================================= consumer warps ==================================================
    ptx::grid_dependency_wait();       // x may be the output of the previous kernel
    // ---- activation prologue: x slab (with later chunks by bulk copy: its first chunk) -> MMA fragment order,
    // ---- plus per-group sums of x ----------------------------------------------------------------------
    {
        // lanes without a batch column read zeros: one sub-unit's worth of fragment bytes
        for (int i = tid; i < S::SPU * S::XSTEP / 4; i += nconsumers) reinterpret_cast<uint32_t*>(smem + P.zero_off)[i] = 0u;
        // One item = 8 consecutive k of one batch row (16 bytes, one vector load: every CTA reads all of x, so the
        // number of L2 requests per CTA is what this prologue costs).  Its four bf16 pairs go to the four lanes
        // c = 0..3 of the row's fragment column; the g / 8 items of a quantization group sit in adjacent lanes and
        // add up their x with shuffles.
        constexpr int G8 = G32 * 4;                 // items per quantization group
        const int octs = (bulk_x ? min(SUBS * UK, P.KS) : P.KS) / 8;   // items per batch row (a multiple of G8)
        const int items = octs * (NB * MR);         // rows at and beyond M are zeros
        const int items_round = (items + 31) / 32 * 32;
        float* sx = reinterpret_cast<float*>(smem + P.sx_off);
        if constexpr (MR < 8) {
            // group sums of the fragment columns that carry no batch row
            const int groups = P.KS / (32 * G32);
            for (int i = tid; i < groups * NB * 8; i += nconsumers)
                if ((i & 7) >= MR) sx[i] = 0.f;
        }
        // x stays in L2 while the weights stream through.  The loads of four rounds of items are issued before any
        // is used, so the prologue costs one memory latency, not one per round.
        const uint64_t keep = ptx::l2_policy_evict_last();
        const bool vec_ok = ((reinterpret_cast<uintptr_t>(x) & 15) == 0) && ((ldx & 7) == 0);
        constexpr int kRounds = 4;
        for (int it0 = tid; it0 < items_round; it0 += kRounds * nconsumers) {
            uint4 w[kRounds];
#pragma unroll
            for (int u = 0; u < kRounds; ++u) {
                const int it = it0 + u * nconsumers;
                w[u] = make_uint4(0u, 0u, 0u, 0u);
                if (it < items) {
                    const int rr = it / octs, j = it - rr * octs;
                    const int m = (rr / MR) * 8 + (rr % MR);
                    if (m < P.M) {
                        const int k = slab * P.KS + 8 * j;
                        const __nv_bfloat16* row = x + (long long)m * ldx;
                        if (vec_ok && k + 8 <= Kx) {
                            w[u] = ptx::ldg_u32x4_hint(row + k, keep);
                        } else {
                            const uint32_t* row32 = reinterpret_cast<const uint32_t*>(row);
                            if (k < Kx) w[u].x = ptx::ldg_u32_hint(row32 + (k >> 1), keep);
                            if (k + 2 < Kx) w[u].y = ptx::ldg_u32_hint(row32 + (k >> 1) + 1, keep);
                            if (k + 4 < Kx) w[u].z = ptx::ldg_u32_hint(row32 + (k >> 1) + 2, keep);
                            if (k + 6 < Kx) w[u].w = ptx::ldg_u32_hint(row32 + (k >> 1) + 3, keep);
                        }
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < kRounds; ++u) {
                const int it = it0 + u * nconsumers;
                if (it >= items_round) break;   // uniform over the warp: items_round is a multiple of 32
                const uint32_t wv[4] = {w[u].x, w[u].y, w[u].z, w[u].w};
                float psum = 0.f;
#pragma unroll
                for (int c = 0; c < 4; ++c) psum += bf16_bits_to_f32(wv[c] & 0xffffu) + __uint_as_float(wv[c] & 0xffff0000u);
#pragma unroll
                for (int o = 1; o < G8; o <<= 1) psum += __shfl_xor_sync(0xffffffffu, psum, o);
                if (it < items) {
                    const int rr = it / octs, j = it - rr * octs;
                    const int nb = rr / MR, mm = rr % MR;
                    // pair c of octet j is word (j & 3) of lane (mm, c) at k32 step j / 4
                    uint32_t* dst = reinterpret_cast<uint32_t*>(smem + P.xs_off) + (((j >> 2) * NB + nb) * MRL + mm * 4) * 4 + (j & 3);
#pragma unroll
                    for (int c = 0; c < 4; ++c) dst[c * 4] = wv[c];
                    if ((j & (G8 - 1)) == 0) sx[((j / G8) * NB + nb) * 8 + mm] = psum;
                }
            }
        }
        ptx::named_barrier_sync(1, nconsumers);
    }
    if (tid == 0) AO_TR(13);                     // activations staged

    // ---- main loop: sub-units of the CTA's stream are dealt round-robin to the consumer warps ---------
    const bool x_lane = lane < MRL;
    const uint32_t x_base = x_lane ? smem_base + P.xs_off + lane * 16 : smem_base + P.zero_off;
    const uint32_t x_unit_stride = x_lane ? static_cast<uint32_t>(S::SPU * S::XSTEP) : 0u;
    const uint32_t sx_base = smem_base + P.sx_off + (lane & 3) * 8;
    const uint32_t w_lane = lane * (S::HALF * 4);
    const uint32_t sc_lane = sc_off + (lane >> 2) * 4;
    const uint32_t nib = P.nib_mask, magic = P.magic;
    float4* parts = reinterpret_cast<float4*>(smem + P.part_off);  // [pair parity][warp][NB][32]
    float acc[NB][4];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[nb][i] = 0.f;
    // Consumer warps form NG groups of GW warps; the stages of the CTA's stream go to the groups in turn, and
    // inside a group every warp takes a contiguous run of the stage's sub-units (unrolled four at a time).
    // GW, the number of groups NG, the ring depth and the number of pair buffers are powers of two
    const int gw_shift = P.gw_shift, GW = 1 << gw_shift, NG = nwarps >> gw_shift, ng_mask = NG - 1;
    const int grp = warp >> gw_shift, wi = warp & (GW - 1);
    const int npairs = pend - pbeg;
    bool ok = true;
    const int ncontrib = min(NG, cpp);           // groups that work on one pair
    const int nslots = ncontrib << gw_shift;     // warps whose partial sums make up one pair
    const int stage_mask = nstages - 1, stage_shift = P.stage_shift;
    const int nbuf_mask = P.nbuf - 1, nbuf_shift = P.nbuf_shift;
    uint32_t x_seen = 1u;                        // chunks of x this warp knows to be in fragment order
    for (int pi = 0, t0 = 0; pi < npairs && ok; ++pi, t0 += cpp) {
        // the pair's stages t0 .. t0 + cpp - 1 go to groups t0 % NG, t0 % NG + 1, ...
        const int ordinal = (grp - t0) & ng_mask;
        if (ordinal >= ncontrib) continue;       // this warp's group has no stage of this pair
        for (int c = ordinal; c < cpp; c += NG) {
            const int t = t0 + c;
            const int s = t & stage_mask;
            const uint32_t phase = static_cast<uint32_t>(t >> stage_shift) & 1u;
            const int sub0 = c * SUBS;
            const int nsub = min(SUBS, subs - sub0);
            if (!ptx::mbar_wait_bounded(full_bar + 8 * s, phase, kWaitPolls)) {
                ok = false;
                break;
            }
            if (tid == 0 && t == 0) AO_TR(14);   // warp 0 sees its first stage full
            if (bulk_x && !((x_seen >> c) & 1u)) {
                // chunk c of x: whoever meets it first (the group that has stage c of the CTA's first pair) puts
                // it into fragment order; everybody else waits until that has happened
                if (pi == 0) {
                    if (!ptx::mbar_wait_bounded(x_full_bar + 8 * c, 0u, kWaitPolls)) {
                        ok = false;
                        break;
                    }
                    prepare_x_chunk<G32>(smem + P.xs_off, reinterpret_cast<float*>(smem + P.sx_off), sub0 * (UK / 32),
                                         nsub * (UK / 32), slab * P.KS + sub0 * UK, Kx, wi, GW, lane);
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(x_ready_bar + 8 * c);
                }
                if (!ptx::mbar_wait_bounded(x_ready_bar + 8 * c, 0u, kWaitPolls)) {
                    ok = false;
                    break;
                }
                x_seen |= 1u << c;
            }
            const uint32_t st = smem_base + s * stage_bytes;
            int j = (wi * nsub) >> gw_shift;
            const int jend = ((wi + 1) * nsub) >> gw_shift;
            for (; j + 4 <= jend; j += 4)
                process_units<IKT, NB, MR, G32, 4>(acc, st, j, sub0 + j, tile_b, w_lane, sc_lane, x_base, x_unit_stride,
                                                   sx_base, nib, magic);
            for (; j < jend; ++j)
                process_units<IKT, NB, MR, G32, 1>(acc, st, j, sub0 + j, tile_b, w_lane, sc_lane, x_base, x_unit_stride,
                                                   sx_base, nib, magic);
            __syncwarp();  // every lane is done reading this stage
            if (lane == 0) ptx::mbar_arrive(empty_bar + 8 * s);
        }
        if (!ok) break;
        // the pair is complete for this warp: leave the partial sums for the reducer warp
        const int buf = pi & nbuf_mask;
        // the buffer must have been handed back after the pair that used it before
        if (!ptx::mbar_wait_bounded(pair_free_bar + 8 * buf, (static_cast<uint32_t>(pi >> nbuf_shift) & 1u) ^ 1u, kWaitPolls)) {
            ok = false;
            break;
        }
        float4* slot = parts + (buf * nslots + (ordinal << gw_shift) + wi) * (NB * 32);
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
            slot[nb * 32 + lane] = make_float4(acc[nb][0], acc[nb][1], acc[nb][2], acc[nb][3]);
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[nb][i] = 0.f;
        }
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(pair_full_bar + 8 * buf);
    }
    if (tid == 0) AO_TR(15);                     // warp 0 leaves the main loop
    if (!ok && lane == 0) atomicExch(status, AO_ERR_TIMEOUT);
}

template <int IKT, int NB, int MR, int G32>
int launch_one(const Plan& P, const void* x, long long ldx, int Kx, const void* wq, const void* sz, void* y,
               void* ws, cudaStream_t st) {
    auto kern = int4_gemv_kernel<IKT, NB, MR, G32>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, P.smem_bytes) != cudaSuccess)
        return AO_ERR_LAUNCH;
    // programmatic dependent launch: this kernel may begin (barrier set-up, weight prefetch) while the previous
    // kernel of the stream drains; everything else waits inside the kernel
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(P.G, P.nslabs);
    cfg.blockDim = dim3((P.nwarps + 2) * 32);
    cfg.dynamicSmemBytes = P.smem_bytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, kern, static_cast<const __nv_bfloat16*>(x), ldx, Kx, static_cast<const uint8_t*>(wq),
                           static_cast<const uint8_t*>(sz), static_cast<__nv_bfloat16*>(y), static_cast<uint8_t*>(ws),
                           P) != cudaSuccess) {
        (void)cudaGetLastError();
        return AO_ERR_LAUNCH;
    }
    return AO_OK;
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
