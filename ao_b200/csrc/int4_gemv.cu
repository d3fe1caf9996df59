// Decode-shaped int4 weight-only linear (M <= 16) on the tensor_core_tiled weight layout:
//   y[M][N] = x[M][K] @ dequant(W)[N][K]^T,  dequant = (q - 8) * scale + zero per group of g along K
// replacing aten::_weight_int4pack_mm as called at torchao/dtypes/affine_quantized_tensor.py:631.
//
// The kernel is HBM-bound: every packed weight byte is read exactly once.
//  * The weight of one 8-row tile is one contiguous byte stream along K, so every warp owns a
//    contiguous range of (row-pair, k-unit) work and streams it with 1-D bulk async copies
//    (cp.async.bulk, completion on an mbarrier) into its own ring of shared-memory stages; the
//    group scales/zeros of the range ride along in the same stage.  No CTA-wide barrier is needed in
//    the main loop.
//  * A packed word already is the B/A fragment of an m16n8k16 MMA (8 codes of one row): codes become
//    bf16 (128 + q) with one logic op per pair and feed mma.sync with W as the 16-row operand (two
//    8-row tiles) and x^T as the 8-column operand, fp32 accumulate.  Scale and zero are applied per
//    group on the accumulator:  y += s * (acc - 136 * Sx) + z * Sx,  Sx = sum of x over the group.
//  * Split-K partial sums go to fixed slots in the workspace; the warp that completes a row pair
//    (atomic unit counter) adds the slots in a fixed order and writes bf16 — deterministic, and the
//    counters are left at zero for the next call.
#include "common.cuh"
#include "ptx.cuh"

namespace ao {
namespace gemv {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kStages = 4;
constexpr int kCtasPerSm = 2;
constexpr int kSpinLimit = 1 << 22;       // polls of one mbarrier phase before giving up
constexpr int kXsmemBudget = 64 * 1024;   // bytes of shared memory for the activation fragments
constexpr uint32_t kMagic = 0x43004300u;  // bf16x2 (128.0, 128.0)
constexpr uint32_t kNib = 0x000F000Fu;
constexpr int kHeaderBytes = 256;
constexpr int kMaxPairs = 16384;         // completion counters live in a fixed region so that calls of
                                         // different shapes can share one workspace

struct Plan {
    int M, N, K, g, ikt, NB, MR;
    int NT, NP;        // 8-row tiles, 16-row pairs
    int UK, UB;        // k values per unit, bytes per unit per 8-row tile
    int CH;            // units per stage
    int GPU;           // groups per unit
    int nslabs, KS;    // K slabs (split-K across CTAs so that the x slab fits shared memory)
    int ups;           // units per pair per slab
    int Gx, Ws, R;     // CTAs per slab, warps per slab, partial slots per (slab, pair)
    long long Us;      // units per slab
    int stage_bytes, scale_off;
    int xs_off, sx_off, p32_off, bar_off, smem_bytes;
    size_t ws_counters_off, ws_slots_off, ws_bytes;
};

static int make_plan(int64_t M, int64_t N, int64_t K, int g, int ikt, Plan* P) {
    if (M < 1 || M > 16) return AO_ERR_SHAPE;
    if (!(ikt == 2 || ikt == 4 || ikt == 8)) return AO_ERR_ARG;
    if (!(g == 32 || g == 64 || g == 128 || g == 256)) return AO_ERR_UNSUPPORTED;
    if (N < 8 || N % 8 != 0 || K < 32 || K % (ikt * 16) != 0 || K % g != 0) return AO_ERR_SHAPE;
    if (N > 16 * kMaxPairs || K > (1 << 24)) return AO_ERR_SHAPE;
    P->M = (int)M; P->N = (int)N; P->K = (int)K; P->g = g; P->ikt = ikt;
    P->NB = M > 8 ? 2 : 1;
    P->MR = M > 4 ? 8 : (M > 2 ? 4 : (M > 1 ? 2 : 1));
    P->NT = (int)(N / 8);
    P->NP = (P->NT + 1) / 2;
    P->UK = ikt * 16 > g ? ikt * 16 : g;
    P->UB = P->UK * 4;
    P->GPU = P->UK / g;
    P->CH = 1024 / P->UB > 1 ? 1024 / P->UB : 1;
    while (P->CH > 1 && P->CH * P->GPU > 30) P->CH /= 2;
    if (P->CH * P->GPU > 30) return AO_ERR_UNSUPPORTED;
    // K slabs: the x fragments of one slab take 2 * KS * MR * NB bytes
    const int ks_max = kXsmemBudget / (2 * P->MR * P->NB);
    int nslabs = 1;
    while (!(K % nslabs == 0 && (K / nslabs) % P->UK == 0 && K / nslabs <= ks_max)) {
        ++nslabs;
        if (nslabs > K / P->UK) return AO_ERR_UNSUPPORTED;
    }
    P->nslabs = nslabs;
    P->KS = (int)(K / nslabs);
    P->ups = P->KS / P->UK;
    P->Us = (long long)P->NP * P->ups;
    int gx = kNumSMs * kCtasPerSm / nslabs;
    if (gx < 1) gx = 1;
    const long long need = (P->Us + kWarps - 1) / kWarps;
    if (gx > need) gx = (int)need;
    P->Gx = gx;
    P->Ws = gx * kWarps;
    P->R = P->Ws / P->NP + 3;
    P->scale_off = 2 * P->CH * P->UB;
    P->stage_bytes = P->scale_off + P->CH * P->GPU * 64;
    int off = kWarps * kStages * P->stage_bytes;
    P->xs_off = off;
    off += 2 * P->KS * P->MR * P->NB;
    P->sx_off = off;
    off += (P->KS / g) * P->NB * 8 * 4;
    P->p32_off = off;
    off += (P->KS / 32) * P->NB * 8 * 4;
    P->bar_off = off;
    off += kWarps * kStages * 8;
    P->smem_bytes = off;
    if (P->smem_bytes > 227 * 1024) return AO_ERR_UNSUPPORTED;
    P->ws_counters_off = kHeaderBytes;
    P->ws_slots_off = kHeaderBytes + (size_t)kMaxPairs * 4;
    P->ws_bytes = P->ws_slots_off + (size_t)nslabs * P->NP * P->R * P->NB * 512;
    return AO_OK;
}

// first unit of warp j, and the warp that owns unit u, for the even split of Us units over Ws warps
__device__ __forceinline__ long long range_start(long long j, long long Us, int Ws) { return (j * Us) / Ws; }
__device__ __forceinline__ int range_owner(long long u, long long Us, int Ws) {
    return static_cast<int>(((u + 1) * Ws + Us - 1) / Us - 1);
}

template <int NB>
struct Acc {
    float v[NB][4];
};

// Ends the accumulation of row pair p by this warp: direct bf16 store when the warp saw the whole K
// range, otherwise a partial slot plus the completion protocol.
template <int NB>
__device__ __forceinline__ void flush_pair(const Plan& P, const Acc<NB>& acc, int p, int units_done, int slab, int j,
                                           int lane, __nv_bfloat16* __restrict__ y, uint8_t* __restrict__ ws) {
    const int row = lane >> 2, c = lane & 3;
    const int n_a = 16 * p + row, n_b = n_a + 8;
    const bool has_b = (2 * p + 1) < P.NT;
    if (P.nslabs == 1 && units_done == P.ups) {
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
            const int m0 = nb * 8 + 2 * c;
            if (m0 < P.M) {
                y[(size_t)m0 * P.N + n_a] = __float2bfloat16_rn(acc.v[nb][0]);
                if (has_b) y[(size_t)m0 * P.N + n_b] = __float2bfloat16_rn(acc.v[nb][2]);
            }
            if (m0 + 1 < P.M) {
                y[(size_t)(m0 + 1) * P.N + n_a] = __float2bfloat16_rn(acc.v[nb][1]);
                if (has_b) y[(size_t)(m0 + 1) * P.N + n_b] = __float2bfloat16_rn(acc.v[nb][3]);
            }
        }
        return;
    }
    const long long u0 = (long long)p * P.ups;
    const int jf = range_owner(u0, P.Us, P.Ws);
    const int jl = range_owner(u0 + P.ups - 1, P.Us, P.Ws);
    int* status = reinterpret_cast<int*>(ws);
    if (j - jf >= P.R || jl - jf >= P.R) {  // cannot happen with R = Ws/NP + 3; never write out of bounds
        if (lane == 0) atomicExch(status, AO_ERR_WORKSPACE);
        return;
    }
    float4* slots = reinterpret_cast<float4*>(ws + P.ws_slots_off);
    const size_t slot_stride = (size_t)NB * 32;  // float4 per slot
    {
        float4* mine = slots + (((size_t)slab * P.NP + p) * P.R + (j - jf)) * slot_stride;
#pragma unroll
        for (int nb = 0; nb < NB; ++nb)
            mine[nb * 32 + lane] = make_float4(acc.v[nb][0], acc.v[nb][1], acc.v[nb][2], acc.v[nb][3]);
    }
    __threadfence();
    __syncwarp();
    int* counter = reinterpret_cast<int*>(ws + P.ws_counters_off) + p;
    int old = 0;
    if (lane == 0) old = atomicAdd(counter, units_done);
    old = __shfl_sync(0xffffffffu, old, 0);
    if (old + units_done != P.ups * P.nslabs) return;
    // this warp completed the pair: add all partial slots in a fixed order
    __threadfence();
    float sum[NB][4];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int i = 0; i < 4; ++i) sum[nb][i] = 0.f;
    for (int sl = 0; sl < P.nslabs; ++sl) {
        for (int jj = jf; jj <= jl; ++jj) {
            if (range_start(jj, P.Us, P.Ws) == range_start(jj + 1, P.Us, P.Ws)) continue;  // warp without work
            const float4* s = slots + (((size_t)sl * P.NP + p) * P.R + (jj - jf)) * slot_stride;
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
                const float4 v = ptx::ldcg_f32x4(s + nb * 32 + lane);
                sum[nb][0] += v.x; sum[nb][1] += v.y; sum[nb][2] += v.z; sum[nb][3] += v.w;
            }
        }
    }
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
        const int m0 = nb * 8 + 2 * c;
        if (m0 < P.M) {
            y[(size_t)m0 * P.N + n_a] = __float2bfloat16_rn(sum[nb][0]);
            if (has_b) y[(size_t)m0 * P.N + n_b] = __float2bfloat16_rn(sum[nb][2]);
        }
        if (m0 + 1 < P.M) {
            y[(size_t)(m0 + 1) * P.N + n_a] = __float2bfloat16_rn(sum[nb][1]);
            if (has_b) y[(size_t)(m0 + 1) * P.N + n_b] = __float2bfloat16_rn(sum[nb][3]);
        }
    }
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

// IKT: inner_k_tiles of the packed weight; NB: 8-column blocks of the batch (1 for M <= 8, 2 for M <= 16);
// G32: group size / 32.
template <int IKT, int NB, int G32>
__global__ void __launch_bounds__(kThreads, kCtasPerSm)
int4_gemv_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, int Kx, const uint8_t* __restrict__ wq,
                 const uint8_t* __restrict__ sz, __nv_bfloat16* __restrict__ y, uint8_t* __restrict__ ws, const Plan P) {
    constexpr int HALF = IKT / 2;                               // words per lane per outer tile
    constexpr int UK = (IKT * 16 > 32 * G32) ? IKT * 16 : 32 * G32;
    constexpr int OT = UK / (IKT * 16);                          // outer tiles per unit
    constexpr int SPU = UK / 32;                                 // k32 steps per unit
    constexpr int GPU = SPU / G32;                               // groups per unit
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int slab = blockIdx.y;
    const int j = blockIdx.x * kWarps + warp;
    const uint32_t smem_base = ptx::smem_addr(smem);
    const uint32_t stage0 = smem_base + warp * kStages * P.stage_bytes;
    const uint32_t bars = smem_base + P.bar_off + warp * kStages * 8;
    const uint32_t xs = smem_base + P.xs_off;
    const uint32_t sxs = smem_base + P.sx_off;
    const long long ubeg = range_start(j, P.Us, P.Ws), uend = range_start(j + 1, P.Us, P.Ws);
    const int CH = P.CH, ups = P.ups, UB = P.UB;
    int* status = reinterpret_cast<int*>(ws);

    if (lane == 0) {
        for (int s = 0; s < kStages; ++s) ptx::mbar_init(bars + 8 * s, 1);
        ptx::fence_mbar_init();
    }
    __syncwarp();

    // one stage = up to CH consecutive units of one row pair: [tile A bytes][tile B bytes][scales/zeros]
    auto issue = [&](long long u, int s) -> int {
        const int p = static_cast<int>(u / ups);
        const int ul = static_cast<int>(u - (long long)p * ups);
        int cnt = CH;
        if (uend - u < cnt) cnt = static_cast<int>(uend - u);
        if (ups - ul < cnt) cnt = ups - ul;
        const long long k0 = (long long)slab * P.KS + (long long)ul * UK;
        const bool has_b = (2 * p + 1) < P.NT;
        const int ngr = cnt * GPU;
        const uint32_t wbytes = static_cast<uint32_t>(cnt * UB);
        const uint32_t sbytes = has_b ? 64u : 32u;
        const uint32_t total = wbytes * (has_b ? 2u : 1u) + ngr * sbytes;
        const uint32_t dst = stage0 + s * P.stage_bytes;
        const uint32_t bar = bars + 8 * s;
        if (lane == 0) ptx::mbar_arrive_expect_tx(bar, total);
        __syncwarp();
        if (lane == 0) {
            ptx::bulk_copy_g2s(dst, wq + ((long long)(2 * p) * P.K + k0) * 4, wbytes, bar);
        } else if (lane == 1) {
            if (has_b) ptx::bulk_copy_g2s(dst + CH * UB, wq + ((long long)(2 * p + 1) * P.K + k0) * 4, wbytes, bar);
        } else if (lane - 2 < ngr) {
            const int gi = lane - 2;
            const long long kg = k0 / (32 * G32) + gi;
            ptx::bulk_copy_g2s(dst + P.scale_off + gi * 64, sz + (kg * P.N + 16LL * p) * 4, sbytes, bar);
        }
        return cnt;
    };

    long long u_prod = ubeg;
    int issued = 0;
    for (int s = 0; s < kStages && u_prod < uend; ++s) {
        u_prod += issue(u_prod, s);
        ++issued;
    }

    // ---- activation prologue: x slab -> MMA fragment order, plus per-group sums of x ----------------
    {
        const int MRL = P.MR * 4;                 // lanes that carry a batch column
        const int steps = P.KS / 32;
        const int items = steps * NB * MRL;       // one item = 4 words (two k16 tiles) of one lane
        const int items_round = (items + 31) / 32 * 32;
        float* p32 = reinterpret_cast<float*>(smem + P.p32_off);
        for (int it = tid; it < items_round; it += kThreads) {
            uint4 wv = make_uint4(0u, 0u, 0u, 0u);
            float psum = 0.f;
            int l = 0, blk = 0;
            if (it < items) {
                l = it % MRL;
                blk = it / MRL;                   // step * NB + nb
                const int nb = blk % NB, step = blk / NB;
                const int m = nb * 8 + (l >> 2), c = l & 3;
                if (m < P.M) {
                    const long long k = (long long)slab * P.KS + step * 32 + 2 * c;
                    const uint32_t* row = reinterpret_cast<const uint32_t*>(x + (long long)m * ldx);
                    uint32_t w[4];
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const long long kk = k + 8 * q;
                        w[q] = (kk < Kx) ? __ldg(row + (kk >> 1)) : 0u;
                    }
                    wv = make_uint4(w[0], w[1], w[2], w[3]);
#pragma unroll
                    for (int q = 0; q < 4; ++q) psum += bf16_bits_to_f32(w[q] & 0xffffu) + __uint_as_float(w[q] & 0xffff0000u);
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
        const int groups = P.KS / (32 * G32);
        for (int it = tid; it < groups * NB * 8; it += kThreads) {
            const int mm = it & 7, nb = (it >> 3) % NB, kg = it / (8 * NB);
            float s = 0.f;
            if (mm < P.MR) {
#pragma unroll
                for (int q = 0; q < G32; ++q) s += p32[((kg * G32 + q) * NB + nb) * 8 + mm];
            }
            sx[it] = s;
        }
        __syncthreads();
    }

    // ---- main loop ------------------------------------------------------------------------------
    Acc<NB> acc;
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc.v[nb][i] = 0.f;
    int cur_p = -1, cur_units = 0;
    int s = 0, consumed = 0;
    uint32_t phase = 0;
    const int MRL = P.MR * 4;
    const bool x_lane = lane < MRL;
    const int c2 = (lane & 3) * 2;
    bool ok = true;
    for (long long u = ubeg; u < uend;) {
        const int p = static_cast<int>(u / ups);
        const int ul = static_cast<int>(u - (long long)p * ups);
        int cnt = CH;
        if (uend - u < cnt) cnt = static_cast<int>(uend - u);
        if (ups - ul < cnt) cnt = ups - ul;
        if (p != cur_p) {
            if (cur_p >= 0) flush_pair<NB>(P, acc, cur_p, cur_units, slab, j, lane, y, ws);
            cur_p = p;
            cur_units = 0;
#pragma unroll
            for (int nb = 0; nb < NB; ++nb)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc.v[nb][i] = 0.f;
        }
        if (!ptx::mbar_wait_bounded(bars + 8 * s, phase, kSpinLimit)) {
            ok = false;
            break;
        }
        const bool has_b = (2 * p + 1) < P.NT;
        const uint32_t st = stage0 + s * P.stage_bytes;
        for (int i = 0; i < cnt; ++i) {
            const int ks0 = (ul + i) * SPU;  // first k32 step of the unit inside the slab
            float tmp[NB][4];
#pragma unroll
            for (int nb = 0; nb < NB; ++nb)
#pragma unroll
                for (int q = 0; q < 4; ++q) tmp[nb][q] = 0.f;
#pragma unroll
            for (int o = 0; o < OT; ++o) {
                uint32_t wa[HALF], wb[HALF];
                const uint32_t woff = ((i * OT + o) * 32 + lane) * (HALF * 4);
                load_words<HALF>(st + woff, wa);
                load_words<HALF>(st + CH * UB + woff, wb);
                if (!has_b) {
#pragma unroll
                    for (int q = 0; q < HALF; ++q) wb[q] = 0u;
                }
#pragma unroll
                for (int jj = 0; jj < HALF; ++jj) {
                    constexpr int dummy = 0;
                    (void)dummy;
                    const int ks_rel = o * HALF + jj;
                    const uint32_t a = wa[jj], b = wb[jj];
                    const uint32_t a0 = (a & kNib) | kMagic, a2 = ((a >> 4) & kNib) | kMagic;
                    const uint32_t a1 = (b & kNib) | kMagic, a3 = ((b >> 4) & kNib) | kMagic;
                    const uint32_t e0 = ((a >> 8) & kNib) | kMagic, e2 = ((a >> 12) & kNib) | kMagic;
                    const uint32_t e1 = ((b >> 8) & kNib) | kMagic, e3 = ((b >> 12) & kNib) | kMagic;
#pragma unroll
                    for (int nb = 0; nb < NB; ++nb) {
                        uint4 xb = make_uint4(0u, 0u, 0u, 0u);
                        if (x_lane) xb = ptx::lds128(xs + (((ks0 + ks_rel) * NB + nb) * MRL + lane) * 16);
                        ptx::mma_bf16_16816(tmp[nb], a0, a1, a2, a3, xb.x, xb.y);
                        ptx::mma_bf16_16816(tmp[nb], e0, e1, e2, e3, xb.z, xb.w);
                    }
                    if ((ks_rel + 1) % G32 == 0) {
                        // end of a quantization group: fold scale and zero into the running sums
                        const int gq = ks_rel / G32;
                        const uint32_t sa = ptx::lds32(st + P.scale_off + (i * GPU + gq) * 64 + (lane >> 2) * 4);
                        const uint32_t sb = ptx::lds32(st + P.scale_off + (i * GPU + gq) * 64 + 32 + (lane >> 2) * 4);
                        const float s_a = __uint_as_float(sa << 16), z_a = __uint_as_float(sa & 0xffff0000u);
                        const float s_b = __uint_as_float(sb << 16), z_b = __uint_as_float(sb & 0xffff0000u);
                        const float zz_a = fmaf(-136.f, s_a, z_a), zz_b = fmaf(-136.f, s_b, z_b);
                        const int kgl = (ks0 + ks_rel) / G32;
#pragma unroll
                        for (int nb = 0; nb < NB; ++nb) {
                            const uint2 sxv = ptx::lds64(sxs + ((kgl * NB + nb) * 8 + c2) * 4);
                            const float sx0 = __uint_as_float(sxv.x), sx1 = __uint_as_float(sxv.y);
                            acc.v[nb][0] = fmaf(s_a, tmp[nb][0], fmaf(zz_a, sx0, acc.v[nb][0]));
                            acc.v[nb][1] = fmaf(s_a, tmp[nb][1], fmaf(zz_a, sx1, acc.v[nb][1]));
                            acc.v[nb][2] = fmaf(s_b, tmp[nb][2], fmaf(zz_b, sx0, acc.v[nb][2]));
                            acc.v[nb][3] = fmaf(s_b, tmp[nb][3], fmaf(zz_b, sx1, acc.v[nb][3]));
#pragma unroll
                            for (int q = 0; q < 4; ++q) tmp[nb][q] = 0.f;
                        }
                    }
                }
            }
        }
        cur_units += cnt;
        ++consumed;
        __syncwarp();  // every lane is done reading this stage
        if (u_prod < uend) {
            u_prod += issue(u_prod, s);
            ++issued;
        }
        u += cnt;
        if (++s == kStages) {
            s = 0;
            phase ^= 1u;
        }
    }
    if (ok) {
        if (cur_p >= 0) flush_pair<NB>(P, acc, cur_p, cur_units, slab, j, lane, y, ws);
    } else {
        // A copy never signalled.  Record it, then wait (bounded) for whatever else is in flight so the
        // CTA's shared memory is not released under a pending copy.
        if (lane == 0) atomicExch(status, AO_ERR_TIMEOUT);
        int ss = s;
        uint32_t ph = phase;
        for (int q = consumed; q < issued; ++q) {
            ptx::mbar_wait_bounded(bars + 8 * ss, ph, kSpinLimit);
            if (++ss == kStages) {
                ss = 0;
                ph ^= 1u;
            }
        }
    }
}

template <int IKT, int NB, int G32>
static int launch_one(const Plan& P, const void* x, long long ldx, int Kx, const void* wq, const void* sz, void* y,
                      void* ws, cudaStream_t st) {
    auto kern = int4_gemv_kernel<IKT, NB, G32>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, P.smem_bytes) != cudaSuccess)
        return AO_ERR_LAUNCH;
    dim3 grid(P.Gx, P.nslabs);
    kern<<<grid, kThreads, P.smem_bytes, st>>>(static_cast<const __nv_bfloat16*>(x), ldx, Kx,
                                               static_cast<const uint8_t*>(wq), static_cast<const uint8_t*>(sz),
                                               static_cast<__nv_bfloat16*>(y), static_cast<uint8_t*>(ws), P);
    return launch_status();
}

template <int IKT, int NB>
static int launch_g(const Plan& P, const void* x, long long ldx, int Kx, const void* wq, const void* sz, void* y,
                    void* ws, cudaStream_t st) {
    switch (P.g) {
        case 32: return launch_one<IKT, NB, 1>(P, x, ldx, Kx, wq, sz, y, ws, st);
        case 64: return launch_one<IKT, NB, 2>(P, x, ldx, Kx, wq, sz, y, ws, st);
        case 128: return launch_one<IKT, NB, 4>(P, x, ldx, Kx, wq, sz, y, ws, st);
        case 256: return launch_one<IKT, NB, 8>(P, x, ldx, Kx, wq, sz, y, ws, st);
    }
    return AO_ERR_UNSUPPORTED;
}

template <int IKT>
static int launch_nb(const Plan& P, const void* x, long long ldx, int Kx, const void* wq, const void* sz, void* y,
                     void* ws, cudaStream_t st) {
    return P.NB == 1 ? launch_g<IKT, 1>(P, x, ldx, Kx, wq, sz, y, ws, st)
                     : launch_g<IKT, 2>(P, x, ldx, Kx, wq, sz, y, ws, st);
}

}  // namespace gemv
}  // namespace ao

using namespace ao;

extern "C" size_t ao_int4_gemv_workspace_bytes(int64_t M, int64_t N, int64_t K, int group, int inner_k_tiles) {
    gemv::Plan P;
    if (gemv::make_plan(M, N, K, group, inner_k_tiles, &P) != AO_OK) return 0;
    return P.ws_bytes;
}

extern "C" int ao_int4_gemv(const void* x_bf16, int64_t x_row_stride, int64_t x_cols, const int32_t* packed,
                            const void* scale_and_zero, int64_t M, int64_t N, int64_t K, int group, int inner_k_tiles,
                            void* y_bf16, void* workspace, size_t workspace_bytes, ao_stream_t stream) {
    if (M == 0 || N == 0) return AO_OK;
    gemv::Plan P;
    int rc = gemv::make_plan(M, N, K, group, inner_k_tiles, &P);
    if (rc) return rc;
    if (x_cols < 2 || x_cols > K || x_cols % 2 != 0 || x_row_stride < x_cols || x_row_stride % 2 != 0) return AO_ERR_SHAPE;
    if (!aligned(x_bf16, 4) || !aligned(packed, 16) || !aligned(scale_and_zero, 16) || !aligned(y_bf16, 2) ||
        !aligned(workspace, 256))
        return AO_ERR_ALIGN;
    if (workspace == nullptr || workspace_bytes < P.ws_bytes) return AO_ERR_WORKSPACE;
    cudaStream_t st = as_stream(stream);
    switch (inner_k_tiles) {
        case 8: return gemv::launch_nb<8>(P, x_bf16, x_row_stride, (int)x_cols, packed, scale_and_zero, y_bf16, workspace, st);
        case 4: return gemv::launch_nb<4>(P, x_bf16, x_row_stride, (int)x_cols, packed, scale_and_zero, y_bf16, workspace, st);
        case 2: return gemv::launch_nb<2>(P, x_bf16, x_row_stride, (int)x_cols, packed, scale_and_zero, y_bf16, workspace, st);
    }
    return AO_ERR_ARG;
}
