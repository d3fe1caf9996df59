// Decode-shaped FP6 (e3m2) weight-only linear, M <= 16:
//   y[M][N] = x[M][K] (fp16) @ (decode(W)[N][K] * scale[N])^T      -> fp16
// on the tensor-core pre-packed weight of torchao/prototype/quant_llm/quant_llm.py:90-106, replacing
// torchao::quant_llm_linear (torchao/ops.py:15-37, torchao/csrc/cuda/fp6_llm/fp6_linear.cu:139-196) for
// decode shapes.
//
// Layout facts used here (derived from the packer): for a block of 64 output rows `a` and a 16-wide k tile
// `f` the 2-bit plane holds 256 contiguous bytes and the 4-bit plane 512; all k tiles of one row block are
// contiguous, so a row block is two byte streams (16*K and 32*K bytes).  Inside (a, f), word t of each
// 128-byte piece belongs to warp lane t and already is the m16n8k16 A fragment of that lane: the four
// bytes of the 4-bit word are (row e+8 | row e) x (col 2c | col 2c+1), high nibble column j, low nibble
// column j+8 (e = t/4, c = t%4); the 2-bit word has the same byte meaning with the two 16-row halves of a
// 32-row piece in bits 7..4 and 3..0.
//
// Structure: one CTA per SM; a producer warp streams (row block, K chunk) stages with two 1-D bulk async
// copies each through a full/empty mbarrier ring; groups of eight consumer warps take the stages in turn,
// every warp a contiguous run of k tiles; codes become fp16 bit patterns (sign, exponent and mantissa bits
// land in fp16's fields, a factor 2^12 short) with logic ops and one integer multiply per register, and
// feed mma.sync (fp16 operands, fp32 accumulate) with W as the 16-row operand.  A reducer warp adds the
// consumer warps' partial sums in slot order, applies 2^12 * scale[row] and stores fp16.  K is cut into
// slabs over CTAs when there are too few row blocks to fill the machine or the activations do not fit
// in shared memory; slab partial sums meet in workspace slots and the CTA that completes a row block
// (atomic counter) adds them in slab order.
#include <cstdlib>

#include "common.cuh"
#include "ptx.cuh"
#include "fp6_decode.cuh"

namespace ao {
namespace fp6 {

constexpr int kConsumerWarps = 16;
constexpr int kGroupWarps = 8;
constexpr int kThreads = (kConsumerWarps + 2) * 32;
constexpr int kMaxStages = 4;
constexpr int kMaxTiles = 32;   // k16 tiles per stage (512 k)
constexpr int kMaxBlockBufs = 4;
constexpr int kWaitPolls = 2000;
constexpr int kHeaderBytes = 256;
constexpr int kMaxBlocks = 16384;

struct Plan {
    int M, N, K, NB, MR;
    int NA;            // 64-row blocks
    int nslabs, KS;    // K slabs
    int tiles;         // k16 tiles per slab
    int TILES, cpb;    // k16 tiles per full stage, stages (K chunks) per row block
    int G;             // CTAs per slab
    int stages, stage_bytes;
    int nbuf;          // ring of per-row-block partial-sum buffers (a power of two)
    int stage_shift, nbuf_shift;  // log2 of stages and nbuf: no divisions in the per-stage bookkeeping
    int xs_off, zero_off, part_off, bar_off, smem_bytes;
    Format fmt;        // decode constants of the 6-bit format, runtime values (kept in registers)
    size_t ws_counters_off, ws_slots_off, ws_bytes;
    const __half* bias;   // optional [N]: y = round(round(acc * scale) + bias), the bits of `out += bias` after the op
};

static int make_plan(int64_t M, int64_t N, int64_t K, int fmt_id, Plan* P) {
    P->fmt = make_format(fmt_id);
    P->bias = nullptr;
    const int tile_bytes = P->fmt.nbits == 6 ? 768 : 640;   // packed bytes of 64 rows x 16 k
    if (M < 1 || M > 16) return AO_ERR_SHAPE;
    if (N < 64 || N % 64 != 0 || K < 64 || K % 64 != 0) return AO_ERR_SHAPE;
    if (N > 64 * kMaxBlocks || K > (1 << 22)) return AO_ERR_SHAPE;
    P->M = (int)M; P->N = (int)N; P->K = (int)K;
    P->NB = M > 8 ? 2 : 1;
    P->MR = M > 4 ? 8 : (M > 2 ? 4 : (M > 1 ? 2 : 1));
    P->NA = (int)(N / 64);
    // K slabs: the x fragments of a slab (KS * MR * NB * 2 bytes) must fit next to a ring of two stages; among
    // those the split with the shortest estimated time of the busiest CTA
    const int ngroups = kConsumerWarps / kGroupWarps;
    int best = 0;
    double best_cost = 0.0;
    for (int ns = 1; ns <= 32; ++ns) {
        if (K % (64 * ns) != 0) continue;
        const int ks = (int)(K / ns);
        const int tl = ks / 16, TL = tl < kMaxTiles ? tl : kMaxTiles, cb = (tl + TL - 1) / TL;
        const int slots = (ngroups < cb ? ngroups : cb) * kGroupWarps;
        const long long need = 2LL * TL * tile_bytes + (long long)ks * P->MR * P->NB * 2 + 4 * P->NB * P->MR * 32 +
                               2LL * slots * 4 * P->NB * 512 + 512;
        if (need > 220 * 1024) continue;
        int g = kNumSMs / ns;
        if (g < 1) continue;
        if (g > P->NA) g = P->NA;
        const int per = (P->NA + g - 1) / g;
        // time of the busiest CTA in units of one full stage: its (block, slab) units, each the unit's stages plus
        // about one and a half stages of fixed cost (pipeline hand-over, partial sums, hand-off), plus the
        // finisher's collection of the other slabs.  Measured on 4096 x 4096 / 11008 x 4096 (1, 2, 4, 8 slabs):
        // 9.7 / 16.9, 8.2 / 15.1, 10.7 / 21.9, 22.3 / 51.1 us.
        const double cost = per * (tl / (double)kMaxTiles + 1.5) + 0.5 * (ns - 1);
        if (best == 0 || cost < best_cost) {
            best_cost = cost;
            best = ns;
        }
    }
    if (best == 0) return AO_ERR_UNSUPPORTED;
    P->nslabs = best;
    P->KS = (int)(K / best);
    P->tiles = P->KS / 16;
    P->TILES = P->tiles < kMaxTiles ? P->tiles : kMaxTiles;
    P->cpb = (P->tiles + P->TILES - 1) / P->TILES;
    P->stage_bytes = P->TILES * tile_bytes;
    int G = kNumSMs / best;
    if (G > P->NA) G = P->NA;
    P->G = G;
    const int xs_bytes = P->KS * P->MR * P->NB * 2;  // per k16 tile: NB * MR*4 lanes * 8 bytes
    const int zero_bytes = 4 * P->NB * P->MR * 32;
    const int nslots = (ngroups < P->cpb ? ngroups : P->cpb) * kGroupWarps;
    int nbuf = (64 * 1024) / (nslots * 4 * P->NB * 512);
    if (nbuf > kMaxBlockBufs) nbuf = kMaxBlockBufs;
    if (nbuf < 2) nbuf = 2;
    int stages = kMaxStages;
    auto total = [&](int st, int nb_) {
        return (long long)st * P->stage_bytes + xs_bytes + zero_bytes + (long long)nb_ * nslots * 4 * P->NB * 512 + 512;
    };
    nbuf = nbuf >= 4 ? 4 : 2;
    while (total(stages, nbuf) > 220 * 1024) {
        if (nbuf > 2) nbuf = 2;
        else if (stages > 2) stages = 2;
        else return AO_ERR_UNSUPPORTED;
    }
    P->nbuf = nbuf;
    P->nbuf_shift = nbuf == 4 ? 2 : 1;
    P->stage_shift = stages == 4 ? 2 : 1;
    const int part_bytes = nbuf * nslots * 4 * P->NB * 512;
    P->stages = stages;
    int off = stages * P->stage_bytes;
    P->xs_off = off;
    off += xs_bytes;
    P->zero_off = off;
    off += zero_bytes;
    P->part_off = off;
    off += part_bytes;
    P->bar_off = off;
    off += 2 * kMaxStages * 8 + 2 * kMaxBlockBufs * 8;
    P->smem_bytes = off;
    P->ws_counters_off = kHeaderBytes;
    P->ws_slots_off = kHeaderBytes + (size_t)kMaxBlocks * 4;
    P->ws_bytes = P->ws_slots_off + (best > 1 ? (size_t)best * P->NA * 4 * P->NB * 1024 : 0);   // {value, tag} words
    return AO_OK;
}

// post_scale * scale[row] of the eight rows this lane stores of row block a (fragment fr: rows e and e + 8)
struct RowScales {
    float s0[4], s1[4];
    float b0[4], b1[4];   // bias of the same rows (0 without a bias)
};
__device__ __forceinline__ RowScales load_row_scales(const Plan& P, int a, int lane, const __half* __restrict__ scale) {
    RowScales r;
    const int row = lane >> 2;
#pragma unroll
    for (int fr = 0; fr < 4; ++fr) {
        const int n0 = a * 64 + fr * 16 + row;
        r.s0[fr] = P.fmt.post_scale * __half2float(scale[n0]);
        r.s1[fr] = P.fmt.post_scale * __half2float(scale[n0 + 8]);
        r.b0[fr] = P.bias != nullptr ? __half2float(P.bias[n0]) : 0.f;
        r.b1[fr] = P.bias != nullptr ? __half2float(P.bias[n0 + 8]) : 0.f;
    }
    return r;
}

// the product rounded to fp16, then (with a bias) the bias added and rounded again: what
// `out = quant_llm_linear(...); out += bias` produces (quant_llm.py:433-445)
__device__ __forceinline__ __half out_f16(float v, float bias, bool has_bias) {
    const __half h = __float2half_rn(v);
    return has_bias ? __float2half_rn(__half2float(h) + bias) : h;
}

// rows of fragment fr (16 rows) of row block a: store y = acc * 2^12 * scale[row]
template <int NB>
__device__ __forceinline__ void store_block(const Plan& P, const float (&v)[4][NB][4], int a, int lane, const RowScales& rs,
                                            __half* __restrict__ y) {
    const int row = lane >> 2, c = lane & 3;
    const bool hb = P.bias != nullptr;
#pragma unroll
    for (int fr = 0; fr < 4; ++fr) {
        const int n0 = a * 64 + fr * 16 + row, n1 = n0 + 8;
        const float s0 = rs.s0[fr], s1 = rs.s1[fr], b0 = rs.b0[fr], b1 = rs.b1[fr];
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
            const int m0 = nb * 8 + 2 * c;
            if (m0 < P.M) {
                y[(size_t)m0 * P.N + n0] = out_f16(v[fr][nb][0] * s0, b0, hb);
                y[(size_t)m0 * P.N + n1] = out_f16(v[fr][nb][2] * s1, b1, hb);
            }
            if (m0 + 1 < P.M) {
                y[(size_t)(m0 + 1) * P.N + n0] = out_f16(v[fr][nb][1] * s0, b0, hb);
                y[(size_t)(m0 + 1) * P.N + n1] = out_f16(v[fr][nb][3] * s1, b1, hb);
            }
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

// K slabs.  The CTAs that share row block a draw a ticket from the block's counter when they start on it (the
// round trip is over by the time their sums are ready); the one that drew the last ticket adds the slabs up and
// stores y, the others leave their partial sums in their workspace slot as 8-byte {value, tag} words (tag = number of
// this launch; an 8-byte store is written as a unit, so a word that carries the tag carries the value: no fence is
// needed) and move on.  The finisher polls those words (bounded); it only ever waits for CTAs that hold a ticket,
// i.e. are running and have no reason to wait for it, and every CTA walks the blocks in the same order.
template <int NB>
__device__ __noinline__ bool finish_block(const Plan& P, const float (&v)[4][NB][4], int a, int slab, int lane,
                                          const RowScales& rs, __half* __restrict__ y, uint8_t* __restrict__ ws,
                                          unsigned call, int ticket) {
    if (P.nslabs == 1) {
        store_block<NB>(P, v, a, lane, rs, y);
        return true;
    }
    uint2* slots = reinterpret_cast<uint2*>(ws + P.ws_slots_off);
    const size_t slot_stride = (size_t)4 * NB * 4 * 32;  // words per slot: [fragment][batch block][value][lane]
    if (ticket + 1 != P.nslabs) {
        uint2* mine = slots + ((size_t)slab * P.NA + a) * slot_stride + lane;
#pragma unroll
        for (int fr = 0; fr < 4; ++fr)
#pragma unroll
            for (int nb = 0; nb < NB; ++nb)
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    st_volatile_u2(mine + ((fr * NB + nb) * 4 + i) * 32, __float_as_uint(v[fr][nb][i]), call);
        return true;
    }
    if (lane == 0) *(reinterpret_cast<int*>(ws + P.ws_counters_off) + a) = 0;   // ready for the next call
    float sum[4][NB][4];
#pragma unroll
    for (int fr = 0; fr < 4; ++fr)
#pragma unroll
        for (int nb = 0; nb < NB; ++nb)
#pragma unroll
            for (int i = 0; i < 4; ++i) sum[fr][nb][i] = 0.f;
    bool ok = true;
    const uint64_t t0 = ptx::globaltimer_ns();
    for (int sl = 0; sl < P.nslabs; ++sl) {
        if (sl == slab) {
#pragma unroll
            for (int fr = 0; fr < 4; ++fr)
#pragma unroll
                for (int nb = 0; nb < NB; ++nb)
#pragma unroll
                    for (int i = 0; i < 4; ++i) sum[fr][nb][i] += v[fr][nb][i];
            continue;
        }
        const uint2* src = slots + ((size_t)sl * P.NA + a) * slot_stride + lane;
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
            uint2 q[4][4];
            // the sixteen loads of a batch block are issued before any is looked at, and all of them again while any
            // word of the warp still lacks the tag: a retry costs one round trip, not one per word
            for (;;) {
                bool all = true;
#pragma unroll
                for (int fr = 0; fr < 4; ++fr)
#pragma unroll
                    for (int i = 0; i < 4; ++i) q[fr][i] = ld_volatile_u2(src + ((fr * NB + nb) * 4 + i) * 32);
#pragma unroll
                for (int fr = 0; fr < 4; ++fr)
#pragma unroll
                    for (int i = 0; i < 4; ++i) all = all && (q[fr][i].y == call);
                if (__all_sync(0xffffffffu, all)) break;
                if (ptx::globaltimer_ns() - t0 > 200000000ull) {   // 0.2 s
                    ok = false;
                    break;
                }
            }
#pragma unroll
            for (int fr = 0; fr < 4; ++fr)
#pragma unroll
                for (int i = 0; i < 4; ++i) sum[fr][nb][i] += __uint_as_float(q[fr][i].x);
        }
    }
    store_block<NB>(P, sum, a, lane, rs, y);
    return __all_sync(0xffffffffu, ok);
}

template <int NB, int MR, int NBITS>
__global__ void __launch_bounds__(kThreads, 1)
fp6_gemv_kernel(const __half* __restrict__ x, long long ldx, const uint8_t* __restrict__ wq,
                const __half* __restrict__ scale, __half* __restrict__ y, uint8_t* __restrict__ ws,
                const __grid_constant__ Plan P) {
    constexpr int MRL = MR * 4;
    constexpr int XT = NB * MRL * 8;  // bytes of x fragments per k16 tile
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    constexpr int nwarps = kConsumerWarps, nconsumers = nwarps * 32;
    const int slab = blockIdx.y, cta = blockIdx.x;
    const uint32_t smem_base = ptx::smem_addr(smem);
    const int nstages = P.stages, stage_bytes = P.stage_bytes;
    const uint32_t full_bar = smem_base + P.bar_off, empty_bar = full_bar + kMaxStages * 8;
    const uint32_t blk_full_bar = empty_bar + kMaxStages * 8, blk_free_bar = blk_full_bar + kMaxBlockBufs * 8;
    const int tiles = P.tiles, TILES = P.TILES, cpb = P.cpb;
    constexpr int HI = NBITS == 6 ? 256 : 128;   // bytes of the first plane per k16 tile
    const uint32_t plane4_off = TILES * HI;
    int* status = reinterpret_cast<int*>(ws);

    const int abeg = static_cast<int>((static_cast<unsigned>(cta) * static_cast<unsigned>(P.NA)) / static_cast<unsigned>(P.G));
    const int aend = static_cast<int>((static_cast<unsigned>(cta + 1) * static_cast<unsigned>(P.NA)) / static_cast<unsigned>(P.G));
    const int nstage_total = (aend - abeg) * cpb;
    constexpr int NG = kConsumerWarps / kGroupWarps;
    const int ncontrib = min(NG, cpb), nslots = ncontrib * kGroupWarps;

    // programmatic dependent launch: the next kernel of the stream may start its weight prefetch while this one
    // drains; everything it reads or writes besides weights comes after its grid_dependency_wait()
    ptx::grid_launch_dependents();
    if (tid == nconsumers) {
        for (int s = 0; s < nstages; ++s) {
            ptx::mbar_init(full_bar + 8 * s, 1);
            ptx::mbar_init(empty_bar + 8 * s, kGroupWarps);
        }
        for (int i = 0; i < P.nbuf; ++i) {
            ptx::mbar_init(blk_full_bar + 8 * i, nslots);
            ptx::mbar_init(blk_free_bar + 8 * i, 1);
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

    if (warp == nwarps) {
        // =============================== producer warp =================================================
        // stage = [2-bit plane bytes of the chunk: 256 per k tile][4-bit plane bytes: 512 per k tile]
        if (lane == 0) {
            const uint8_t* plane2 = wq;
            const uint8_t* plane4 = wq + (size_t)P.N * P.K * (NBITS - 4) / 8;
            int ai = 0, c = 0, s = 0;
            uint32_t phase = 1;
            bool ok = true;
            const uint64_t stream_once = ptx::l2_policy_evict_first();   // every weight byte is read exactly once
            for (int t = 0; t < nstage_total; ++t) {
                if (!ptx::mbar_wait_bounded(empty_bar + 8 * s, phase, kWaitPolls)) {
                    ok = false;
                    break;
                }
                const int a = abeg + ai;
                const int f0 = slab * tiles + c * TILES;             // first k tile, counted over the whole K
                const int nf = min(TILES, tiles - c * TILES);
                const size_t tile_index = (size_t)a * (P.K / 16) + f0;
                const uint32_t dst = smem_base + s * stage_bytes;
                const uint32_t bar = full_bar + 8 * s;
                ptx::mbar_arrive_expect_tx(bar, nf * (HI + 512u));
                ptx::bulk_copy_g2s_hint(dst, plane2 + tile_index * HI, nf * HI, bar, stream_once);
                ptx::bulk_copy_g2s_hint(dst + plane4_off, plane4 + tile_index * 512, nf * 512u, bar, stream_once);
                if (++c == cpb) {
                    c = 0;
                    ++ai;
                }
                if (++s == nstages) {
                    s = 0;
                    phase ^= 1u;
                }
            }
            if (!ok) {
                ptx::grid_dependency_wait();
                atomicExch(status, AO_ERR_TIMEOUT);
            }
        }
        return;
    }

    const float4* parts_ro = reinterpret_cast<const float4*>(smem + P.part_off);
    if (warp == nwarps + 1) {
        // =============================== reducer warp ==================================================
        ptx::grid_dependency_wait();   // y and the workspace may be in use by earlier kernels
        bool ok = true;
        // tag of this launch's partial sums (all CTAs read the same value: it changes when the last one finishes)
        unsigned* call_state = reinterpret_cast<unsigned*>(ws + kCallStateOff);
        const unsigned call = P.nslabs > 1 ? *reinterpret_cast<volatile unsigned*>(call_state + 1) + 1u : 0u;
        for (int ai = 0; ai < aend - abeg; ++ai) {
            const int buf = ai & (P.nbuf - 1);
            // issued before the wait: the ticket that decides who finishes the block, and the rows' scales
            int ticket = 0;
            if (P.nslabs > 1 && lane == 0) ticket = atomicAdd(reinterpret_cast<int*>(ws + P.ws_counters_off) + abeg + ai, 1);
            const RowScales rs = load_row_scales(P, abeg + ai, lane, scale);
            if (!ptx::mbar_wait_bounded(blk_full_bar + 8 * buf, static_cast<uint32_t>(ai >> P.nbuf_shift) & 1u, kWaitPolls)) {
                ok = false;
                break;
            }
            float sum[4][NB][4];
#pragma unroll
            for (int fr = 0; fr < 4; ++fr)
#pragma unroll
                for (int nb = 0; nb < NB; ++nb)
#pragma unroll
                    for (int i = 0; i < 4; ++i) sum[fr][nb][i] = 0.f;
            const float4* src = parts_ro + (size_t)(buf * nslots) * (4 * NB * 32) + lane;
            // nslots is a multiple of 8; the loads of two slots are issued before either is used
            for (int w = 0; w < nslots; w += 2) {
                float4 q[2][4][NB];
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int fr = 0; fr < 4; ++fr)
#pragma unroll
                        for (int nb = 0; nb < NB; ++nb) q[h][fr][nb] = src[(size_t)((w + h) * 4 * NB + fr * NB + nb) * 32];
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int fr = 0; fr < 4; ++fr)
#pragma unroll
                        for (int nb = 0; nb < NB; ++nb) {
                            sum[fr][nb][0] += q[h][fr][nb].x; sum[fr][nb][1] += q[h][fr][nb].y;
                            sum[fr][nb][2] += q[h][fr][nb].z; sum[fr][nb][3] += q[h][fr][nb].w;
                        }
            }
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(blk_free_bar + 8 * buf);
            if (!finish_block<NB>(P, sum, abeg + ai, slab, lane, rs, y, ws, call, __shfl_sync(0xffffffffu, ticket, 0))) ok = false;
        }
        if (P.nslabs > 1 && lane == 0) {
            // the last CTA of the launch to finish advances the launch number
            const unsigned done = atomicAdd(call_state, 1u);
            if (done + 1 == gridDim.x * gridDim.y) {
                call_state[0] = 0u;
                call_state[1] = call;
            }
        }
        if (!ok && lane == 0) atomicExch(status, AO_ERR_TIMEOUT);
        return;
    }

    // ================================= consumer warps ==================================================
    ptx::grid_dependency_wait();       // x may be the output of the previous kernel
    // x slab -> MMA B-fragment order: per k16 tile and lane (batch column m = lane/4, c = lane%4) the words
    // x[m][k0+2c .. +1] and x[m][k0+2c+8 .. +9]
    {
        // One item = 8 consecutive k of one batch row (a 16-byte vector load: every CTA reads all of x, so the number
        // of L2 requests is what this prologue costs); its four pairs go to lanes c = 0..3 of the row's column.
        // The loads of four rounds of items are issued before any is used.
        const int octs = P.KS / 8;
        const int items = octs * (NB * MR);         // rows at and beyond M are zeros
        for (int i = tid; i < 4 * XT / 4; i += nconsumers) reinterpret_cast<uint32_t*>(smem + P.zero_off)[i] = 0u;
        const uint64_t keep = ptx::l2_policy_evict_last();   // x stays in L2 while the weights stream through
        const bool vec_ok = ((reinterpret_cast<uintptr_t>(x) & 15) == 0) && ((ldx & 7) == 0);
        constexpr int kRounds = 4;
        for (int it0 = tid; it0 < items; it0 += kRounds * nconsumers) {
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
                        const __half* row = x + (long long)m * ldx;
                        if (vec_ok) {
                            w[u] = ptx::ldg_u32x4_hint(row + k, keep);
                        } else {
                            const uint32_t* row32 = reinterpret_cast<const uint32_t*>(row) + (k >> 1);
                            w[u].x = ptx::ldg_u32_hint(row32, keep);
                            w[u].y = ptx::ldg_u32_hint(row32 + 1, keep);
                            w[u].z = ptx::ldg_u32_hint(row32 + 2, keep);
                            w[u].w = ptx::ldg_u32_hint(row32 + 3, keep);
                        }
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < kRounds; ++u) {
                const int it = it0 + u * nconsumers;
                if (it < items) {
                    const int rr = it / octs, j = it - rr * octs;
                    const int nb = rr / MR, mm = rr % MR;
                    // pair c of octet j is word (j & 1) of lane (mm, c) at k16 tile j / 2
                    uint32_t* dst = reinterpret_cast<uint32_t*>(smem + P.xs_off) + (((j >> 1) * NB + nb) * MRL + mm * 4) * 2 + (j & 1);
                    dst[0] = w[u].x; dst[2] = w[u].y; dst[4] = w[u].z; dst[6] = w[u].w;
                }
            }
        }
        ptx::named_barrier_sync(1, nconsumers);
    }

    const bool x_lane = lane < MRL;
    const uint32_t x_base = x_lane ? smem_base + P.xs_off + lane * 8 : smem_base + P.zero_off;
    const uint32_t x_tile_stride = x_lane ? static_cast<uint32_t>(XT) : 0u;
    const Format fmt = P.fmt;
    float4* parts = reinterpret_cast<float4*>(smem + P.part_off);
    const int grp = warp / kGroupWarps, wi = warp - grp * kGroupWarps;
    float acc[4][NB][4];
#pragma unroll
    for (int fr = 0; fr < 4; ++fr)
#pragma unroll
        for (int nb = 0; nb < NB; ++nb)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[fr][nb][i] = 0.f;
    bool ok = true;
    for (int ai = 0; ai < aend - abeg && ok; ++ai) {
        const int first_grp = (ai * cpb) % NG;
        int ordinal = grp - first_grp;
        if (ordinal < 0) ordinal += NG;
        if (ordinal >= ncontrib) continue;
        for (int c = ordinal; c < cpb; c += NG) {
            const int t = ai * cpb + c;
            const int s = t & (nstages - 1);
            const uint32_t phase = static_cast<uint32_t>(t >> P.stage_shift) & 1u;
            const int nf = min(TILES, tiles - c * TILES);
            if (!ptx::mbar_wait_bounded(full_bar + 8 * s, phase, kWaitPolls)) {
                ok = false;
                break;
            }
            const uint32_t st = smem_base + s * stage_bytes;
            const int j0 = (wi * nf) / kGroupWarps, j1 = ((wi + 1) * nf) / kGroupWarps;
#pragma unroll 2
            for (int j = j0; j < j1; ++j) {
                const uint32_t p2 = st + j * HI + lane * 4;
                const uint32_t p4 = st + plane4_off + j * 512 + lane * 4;
                const uint32_t xa = x_base + (c * TILES + j) * x_tile_stride;
                uint2 xb[NB];
#pragma unroll
                for (int nb = 0; nb < NB; ++nb) xb[nb] = ptx::lds64(xa + nb * (MRL * 8));
                if constexpr (NBITS == 6) {
#pragma unroll
                    for (int b = 0; b < 2; ++b) {
                        const uint32_t w2 = ptx::lds32(p2 + b * 128);
#pragma unroll
                        for (int cc = 0; cc < 2; ++cc) {
                            const uint32_t w4 = ptx::lds32(p4 + (b * 2 + cc) * 128);
                            uint32_t a[4];
                            decode_fragment(w4, cc == 0 ? w2 : (w2 << 4), fmt, a);
#pragma unroll
                            for (int nb = 0; nb < NB; ++nb)
                                ptx::mma_f16_16816(acc[b * 2 + cc][nb], a[0], a[1], a[2], a[3], xb[nb].x, xb[nb].y);
                        }
                    }
                } else {
                    const uint32_t w1 = ptx::lds32(p2);   // the signs of all 64 rows of this lane's column pair
#pragma unroll
                    for (int fr = 0; fr < 4; ++fr) {
                        const uint32_t w4 = ptx::lds32(p4 + fr * 128);
                        uint32_t a[4];
                        decode_fragment5(w4, w1, fr, fmt, a);
#pragma unroll
                        for (int nb = 0; nb < NB; ++nb)
                            ptx::mma_f16_16816(acc[fr][nb], a[0], a[1], a[2], a[3], xb[nb].x, xb[nb].y);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(empty_bar + 8 * s);
        }
        if (!ok) break;
        const int buf = ai & (P.nbuf - 1);
        if (!ptx::mbar_wait_bounded(blk_free_bar + 8 * buf, (static_cast<uint32_t>(ai >> P.nbuf_shift) & 1u) ^ 1u, kWaitPolls)) {
            ok = false;
            break;
        }
        float4* slot = parts + (size_t)(buf * nslots + ordinal * kGroupWarps + wi) * (4 * NB * 32);
#pragma unroll
        for (int fr = 0; fr < 4; ++fr)
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
                slot[(fr * NB + nb) * 32 + lane] = make_float4(acc[fr][nb][0], acc[fr][nb][1], acc[fr][nb][2], acc[fr][nb][3]);
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[fr][nb][i] = 0.f;
            }
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(blk_full_bar + 8 * buf);
    }
    if (!ok && lane == 0) atomicExch(status, AO_ERR_TIMEOUT);
}

template <int NB, int MR, int NBITS>
static int launch_bits(const Plan& P, const void* x, long long ldx, const void* wq, const void* scale, void* y, void* ws,
                  cudaStream_t st) {
    auto kern = fp6_gemv_kernel<NB, MR, NBITS>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, P.smem_bytes) != cudaSuccess)
        return AO_ERR_LAUNCH;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(P.G, P.nslabs);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = P.smem_bytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, kern, static_cast<const __half*>(x), ldx, static_cast<const uint8_t*>(wq),
                           static_cast<const __half*>(scale), static_cast<__half*>(y), static_cast<uint8_t*>(ws),
                           P) != cudaSuccess) {
        (void)cudaGetLastError();
        return AO_ERR_LAUNCH;
    }
    return AO_OK;
}

template <int NB, int MR>
static int launch(const Plan& P, const void* x, long long ldx, const void* wq, const void* scale, void* y, void* ws,
                  cudaStream_t st) {
    return P.fmt.nbits == 6 ? launch_bits<NB, MR, 6>(P, x, ldx, wq, scale, y, ws, st)
                            : launch_bits<NB, MR, 5>(P, x, ldx, wq, scale, y, ws, st);
}

}  // namespace fp6
}  // namespace ao

namespace ao {
namespace umma {
size_t fp6_umma_workspace_bytes(int64_t M, int64_t N, int64_t K);
int fp6_umma_linear(int fmt, const void* x, int64_t ldx, const uint8_t* packed, const void* scale, int64_t M, int64_t N,
                    int64_t K, void* y, const void* bias, void* ws, size_t ws_bytes, cudaStream_t st);
}  // namespace umma
}  // namespace ao

using namespace ao;
using ao::fp6::Format;

namespace {

// A 9..16-row call whose activations and partial sums cannot share one SM's shared memory with the stage ring
// runs as two calls of at most 8 rows.
size_t gemv_workspace_bytes(int64_t M, int64_t N, int64_t K, int fmt = ao::fp6::kE3M2) {
    fp6::Plan P;
    int rc = fp6::make_plan(M, N, K, fmt, &P);
    if (rc == AO_ERR_UNSUPPORTED && M > 8) {
        const size_t a = gemv_workspace_bytes(8, N, K, fmt), b = gemv_workspace_bytes(M - 8, N, K, fmt);
        return a == 0 || b == 0 ? 0 : (a > b ? a : b);
    }
    return rc == AO_OK ? P.ws_bytes : 0;
}

int gemv(int fmt, const void* x_f16, int64_t x_row_stride, const uint8_t* packed, const void* scale_f16, int64_t M,
         int64_t N, int64_t K, void* y_f16, const void* bias_f16, void* workspace, size_t workspace_bytes,
         ao_stream_t stream) {
    if (M == 0 || N == 0) return AO_OK;
    fp6::Plan P;
    int rc = fp6::make_plan(M, N, K, fmt, &P);
    if (rc == AO_ERR_UNSUPPORTED && M > 8) {
        rc = gemv(fmt, x_f16, x_row_stride, packed, scale_f16, 8, N, K, y_f16, bias_f16, workspace, workspace_bytes, stream);
        if (rc) return rc;
        return gemv(fmt, static_cast<const __half*>(x_f16) + 8 * x_row_stride, x_row_stride, packed, scale_f16, M - 8, N, K,
                    static_cast<__half*>(y_f16) + 8 * N, bias_f16, workspace, workspace_bytes, stream);
    }
    if (rc) return rc;
    if (!aligned(bias_f16, 2)) return AO_ERR_ALIGN;
    P.bias = static_cast<const __half*>(bias_f16);
    if (x_row_stride < K || x_row_stride % 2 != 0) return AO_ERR_SHAPE;
    if (!aligned(x_f16, 4) || !aligned(packed, 16) || !aligned(scale_f16, 2) || !aligned(y_f16, 2) ||
        !aligned(workspace, 256))
        return AO_ERR_ALIGN;
    if (workspace == nullptr || workspace_bytes < P.ws_bytes) return AO_ERR_WORKSPACE;
    cudaStream_t st = as_stream(stream);
    if (P.NB == 2) return fp6::launch<2, 8>(P, x_f16, x_row_stride, packed, scale_f16, y_f16, workspace, st);
    switch (P.MR) {
        case 1: return fp6::launch<1, 1>(P, x_f16, x_row_stride, packed, scale_f16, y_f16, workspace, st);
        case 2: return fp6::launch<1, 2>(P, x_f16, x_row_stride, packed, scale_f16, y_f16, workspace, st);
        case 4: return fp6::launch<1, 4>(P, x_f16, x_row_stride, packed, scale_f16, y_f16, workspace, st);
        case 8: return fp6::launch<1, 8>(P, x_f16, x_row_stride, packed, scale_f16, y_f16, workspace, st);
    }
    return AO_ERR_UNSUPPORTED;
}

// A single row and the smallest batches go to the GEMV kernel, larger batches to the tcgen05 kernel, the rest in row
// blocks of 16.  Measured on B200 (e3m2, 12288x4096 / 4096x4096 / 11008x4096 / 4096x11008): the tcgen05 kernel at 16
// columns takes 17.1 / 8.4 / 17.0 / 15.2 us whatever M <= 16 is, the GEMV 16.4 / 9.3 / 16.5 / 17.6 at M = 4 and 17.7 /
// 10.6 / 17.6 / 25.2 at M = 8: so M >= 5 always, and from M = 2 on long reductions (K >= 2 N).
bool prefers_tcgen05(int64_t M, int64_t N, int64_t K) { return M >= 5 || (M >= 2 && K >= 2 * N); }

size_t linear_workspace_bytes(int64_t M, int64_t N, int64_t K) {
    if (M <= 8 && !prefers_tcgen05(M, N, K)) return gemv_workspace_bytes(M, N, K);
    size_t need = umma::fp6_umma_workspace_bytes(M, N, K);
    for (int m = 1; m <= 16; m *= 2) {
        const size_t b = gemv_workspace_bytes(m, N, K);
        if (b == 0) return 0;
        need = b > need ? b : need;
    }
    return need;
}

int linear(int fmt, const void* x_f16, int64_t x_row_stride, const uint8_t* packed, const void* scale_f16, int64_t M,
           int64_t N, int64_t K, void* y_f16, const void* bias_f16, void* workspace, size_t workspace_bytes,
           ao_stream_t stream) {
    if (M < 0 || N < 0) return AO_ERR_SHAPE;
    if (M <= 8 && !prefers_tcgen05(M, N, K))
        return gemv(fmt, x_f16, x_row_stride, packed, scale_f16, M, N, K, y_f16, bias_f16, workspace, workspace_bytes, stream);
    if (workspace == nullptr || workspace_bytes < 256 || !aligned(workspace, 256)) return AO_ERR_WORKSPACE;
    {
        const int rc = umma::fp6_umma_linear(fmt, x_f16, x_row_stride, packed, scale_f16, M, N, K, y_f16, bias_f16, workspace,
                                             workspace_bytes, as_stream(stream));
        if (rc != AO_ERR_UNSUPPORTED) return rc;
    }
    if (M <= 16)
        return gemv(fmt, x_f16, x_row_stride, packed, scale_f16, M, N, K, y_f16, bias_f16, workspace, workspace_bytes, stream);
    const auto* x = static_cast<const __half*>(x_f16);
    auto* y = static_cast<__half*>(y_f16);
    for (int64_t m0 = 0; m0 < M; m0 += 16) {
        const int64_t mb = M - m0 < 16 ? M - m0 : 16;
        int rc = gemv(fmt, x + m0 * x_row_stride, x_row_stride, packed, scale_f16, mb, N, K, y + m0 * N, bias_f16, workspace,
                      workspace_bytes, stream);
        if (rc) return rc;
    }
    return AO_OK;
}

}  // namespace

extern "C" size_t ao_fp6_gemv_workspace_bytes(int64_t M, int64_t N, int64_t K) { return gemv_workspace_bytes(M, N, K); }

extern "C" int ao_fp6_gemv(const void* x_f16, int64_t x_row_stride, const uint8_t* packed, const void* scale_f16,
                           int64_t M, int64_t N, int64_t K, void* y_f16, void* workspace, size_t workspace_bytes,
                           ao_stream_t stream) {
    return gemv(ao::fp6::kE3M2, x_f16, x_row_stride, packed, scale_f16, M, N, K, y_f16, nullptr, workspace, workspace_bytes, stream);
}

// torchao::quant_llm_linear for e3m2
extern "C" size_t ao_fp6_linear_workspace_bytes(int64_t M, int64_t N, int64_t K) { return linear_workspace_bytes(M, N, K); }

extern "C" int ao_fp6_linear(const void* x_f16, int64_t x_row_stride, const uint8_t* packed, const void* scale_f16,
                             int64_t M, int64_t N, int64_t K, void* y_f16, void* workspace, size_t workspace_bytes,
                             ao_stream_t stream) {
    return linear(ao::fp6::kE3M2, x_f16, x_row_stride, packed, scale_f16, M, N, K, y_f16, nullptr, workspace, workspace_bytes, stream);
}

// torchao::quant_llm_linear: (EXPONENT, MANTISSA) = (3, 2), (2, 3), (2, 2) or (3, 1)
extern "C" int ao_fpx_linear(int ebits, int mbits, const void* x_f16, int64_t x_row_stride, const uint8_t* packed,
                             const void* scale_f16, int64_t M, int64_t N, int64_t K, void* y_f16, void* workspace,
                             size_t workspace_bytes, ao_stream_t stream) {
    const int fmt = ao::fp6::format_id(ebits, mbits);
    if (fmt < 0) return AO_ERR_UNSUPPORTED;
    return linear(fmt, x_f16, x_row_stride, packed, scale_f16, M, N, K, y_f16, nullptr, workspace, workspace_bytes, stream);
}

// the same with the bias add of the reference's linear dispatch (quant_llm.py:444-445) fused into the stores:
// bias_f16 [N] fp16 or null; y = round_f16(round_f16(x @ W^T) + bias)
extern "C" int ao_fpx_linear_bias(int ebits, int mbits, const void* x_f16, int64_t x_row_stride, const uint8_t* packed,
                                  const void* scale_f16, const void* bias_f16, int64_t M, int64_t N, int64_t K, void* y_f16,
                                  void* workspace, size_t workspace_bytes, ao_stream_t stream) {
    const int fmt = ao::fp6::format_id(ebits, mbits);
    if (fmt < 0) return AO_ERR_UNSUPPORTED;
    return linear(fmt, x_f16, x_row_stride, packed, scale_f16, M, N, K, y_f16, bias_f16, workspace, workspace_bytes, stream);
}
