// Host side of the int4 decode GEMV: the launch plan (work split, shared-memory and workspace layout)
// and the C entry points.  The kernel lives in int4_gemv.cuh and is instantiated per inner_k_tiles
// value in int4_gemv_ikt{8,4,2}.cu.
#include "int4_gemv.cuh"

namespace ao {
namespace gemv {

#ifdef AO_B200_DEV_KNOBS
// Tuning sweeps only (a build with -DAO_B200_DEV_KNOBS): an integer from the environment, clamped to [lo, hi].
static int dev_knob(const char* name, int dflt, int lo, int hi) {
    const char* e = getenv(name);
    if (!e) return dflt;
    const int v = atoi(e);
    return v < lo ? lo : (v > hi ? hi : v);
}
#endif

int make_plan(int64_t M, int64_t N, int64_t K, int g, int ikt, Plan* P) {
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
    // K slabs: as few as possible such that the x fragments of one slab (2 * KS * MR * NB bytes), a ring of two
    // stages and the smallest set of partial-sum buffers still fit in shared memory
    int nslabs = 1;
    for (;; ++nslabs) {
        if (nslabs > K / P->UK) return AO_ERR_UNSUPPORTED;
        if (K % nslabs != 0 || (K / nslabs) % P->UK != 0) continue;
        const int ks = (int)(K / nslabs);
        const int subs_ = ks / P->UK, SUBS_ = subs_ < kMaxSubs ? subs_ : kMaxSubs;
        const int stage_ = ((2 * SUBS_ * P->UB + SUBS_ * P->GPU * 64 + 127) / 128) * 128;
        const long long need = 2LL * ks * P->MR * P->NB + (P->UK / 32) * P->NB * P->MR * 64 + (ks / g) * P->NB * 32 +
                               2 * 8 * P->NB * 512 + 1024 + 2 * stage_;
        if (need <= kSmemBudget) break;
    }
    P->nslabs = nslabs;
    P->KS = (int)(K / nslabs);
    // a stage holds one row pair x up to kMaxSubs sub-units of K
    P->subs = P->KS / P->UK;
    P->SUBS = P->subs < kMaxSubs ? P->subs : kMaxSubs;
#ifdef AO_B200_DEV_KNOBS
    P->SUBS = dev_knob("AO_GEMV_SUBS", P->SUBS, 1, P->SUBS);
#endif
    P->cpp = (P->subs + P->SUBS - 1) / P->SUBS;
    if ((long long)P->NP * P->cpp > (1LL << 30)) return AO_ERR_SHAPE;
    const int stage_raw = 2 * P->SUBS * P->UB + P->SUBS * P->GPU * 64;
    P->stage_bytes = ((stage_raw + 127) / 128) * 128;
    // shared memory: stage ring, x fragments, zero block, group sums of x, partial sums (two pair parities),
    // control block, barriers.  As many consumer warps (24, 16, 8) and as deep a ring (4 .. 2) as fit.
    const int xs_bytes = 2 * P->KS * P->MR * P->NB, zero_bytes = (P->UK / 32) * P->NB * P->MR * 64;
    const int sx_bytes = (P->KS / g) * P->NB * 32;
    int nwarps = kMaxConsumerWarps, stages = kMaxStages;
#ifdef AO_B200_DEV_KNOBS
    nwarps = dev_knob("AO_GEMV_NWARPS", nwarps, 8, kMaxConsumerWarps) / 8 * 8;
    stages = dev_knob("AO_GEMV_STAGES", stages, 2, kMaxStages) >= 4 ? 4 : 2;
#endif
    for (;;) {
        const int total = xs_bytes + zero_bytes + sx_bytes + 2 * nwarps * P->NB * 512 + 1024 +
                          stages * P->stage_bytes;
        if (total <= kSmemBudget) break;
        if (stages > 2) stages = 2;   // the ring depth stays a power of two
        else if (nwarps > 8) nwarps -= 8;
        else return AO_ERR_UNSUPPORTED;
    }
    P->nwarps = nwarps;
    P->stages = stages;
    int off = stages * P->stage_bytes;
    P->xs_off = off;
    off += xs_bytes;
    P->zero_off = off;
    P->trace_id = 0;
    off += zero_bytes;
    P->sx_off = off;
    off += sx_bytes;
    int G = kNumSMs / nslabs;
    if (G < 1) G = 1;
    if (G > P->NP) G = P->NP;
    P->G = G;
    P->pair_q = P->NP / G;
    P->pair_r = P->NP % G;
    // groups of 8 warps (four sub-units per warp and stage, unrolled) when the CTA has enough stages to keep
    // every group busy; otherwise all warps share each stage
    const int stages_per_cta = ((P->NP + G - 1) / G) * P->cpp;
    P->GW = (stages_per_cta >= 2 * (nwarps / 8) && P->SUBS >= kMaxSubs) ? 8 : nwarps;
    // ring of pair buffers: within the budget of two buffers of all warps, at most kMaxPairBufs
    const int NG = nwarps / P->GW;
    const int nslots = (NG < P->cpp ? NG : P->cpp) * P->GW;
    int nbuf = (2 * nwarps) / nslots;  // 2, 4 or more; kept a power of two
    nbuf = nbuf >= 8 ? 8 : (nbuf >= 4 ? 4 : 2);
    P->nbuf = nbuf;
    P->nbuf_shift = nbuf == 8 ? 3 : (nbuf == 4 ? 2 : 1);
    P->gw_shift = P->GW == 16 ? 4 : 3;
    P->stage_shift = stages == 4 ? 2 : 1;
    P->part_off = off;
    off += nbuf * nslots * P->NB * 512;
    P->bar_off = off;
    off += 2 * kMaxStages * 8 + 2 * kMaxPairBufs * 8 + 2 * kMaxXChunks * 8;
    // staging of the CTA's output rows for the peer exchange (used only when nranks > 1; small)
    P->rows_cta_max = 16 * ((P->NP + G - 1) / G);
    P->ystage_off = (off + 15) / 16 * 16;
    off = P->ystage_off + ((P->M * P->rows_cta_max * 2 + 15) / 16) * 16;
    P->bias = nullptr;
    P->nranks = 1;
    P->rank = 0;
    P->local_state = nullptr;
    P->y_gathered = nullptr;
    for (int r = 0; r < kMaxRanks; ++r) P->peer_ll[r] = nullptr;
    P->smem_bytes = off;
    P->nib_mask = 0x000F000Fu;
    P->magic = 0x43004300u;
    P->ws_counters_off = kHeaderBytes;
    P->ws_slots_off = kHeaderBytes + (size_t)kMaxPairs * 4;
    P->ws_bytes = P->ws_slots_off + (nslabs > 1 ? (size_t)nslabs * P->NP * P->NB * 1024 : 0);   // {value, tag} words
    return AO_OK;
}

extern template int launch_ikt<8>(const Plan&, const void*, long long, int, const void*, const void*,
                                  void*, void*, cudaStream_t);
extern template int launch_ikt<4>(const Plan&, const void*, long long, int, const void*, const void*,
                                  void*, void*, cudaStream_t);
extern template int launch_ikt<2>(const Plan&, const void*, long long, int, const void*, const void*,
                                  void*, void*, cudaStream_t);

}  // namespace gemv
}  // namespace ao

using namespace ao;

extern "C" size_t ao_int4_gemv_workspace_bytes(int64_t M, int64_t N, int64_t K, int group, int inner_k_tiles) {
    gemv::Plan P;
    if (gemv::make_plan(M, N, K, group, inner_k_tiles, &P) != AO_OK) return 0;
    return P.ws_bytes;
}

static int int4_gemv_impl(const void* x_bf16, int64_t x_row_stride, int64_t x_cols, const int32_t* packed,
                         const void* scale_and_zero, int64_t M, int64_t N, int64_t K, int group, int inner_k_tiles,
                         void* y_bf16, const void* bias_bf16, void* workspace, size_t workspace_bytes, ao_stream_t stream) {
    if (M == 0 || N == 0) return AO_OK;
    gemv::Plan P;
    int rc = gemv::make_plan(M, N, K, group, inner_k_tiles, &P);
    if (rc) return rc;
    if (bias_bf16 != nullptr && !aligned(bias_bf16, 2)) return AO_ERR_ALIGN;
    P.bias = static_cast<const __nv_bfloat16*>(bias_bf16);
    if (x_cols < 2 || x_cols > K || x_cols % 2 != 0 || x_row_stride < x_cols || x_row_stride % 2 != 0) return AO_ERR_SHAPE;
    if (!aligned(x_bf16, 4) || !aligned(packed, 16) || !aligned(scale_and_zero, 16) || !aligned(y_bf16, 2) ||
        !aligned(workspace, 256))
        return AO_ERR_ALIGN;
    if (workspace == nullptr || workspace_bytes < P.ws_bytes) return AO_ERR_WORKSPACE;
#if defined(AO_GEMV_TRACE) && AO_GEMV_TRACE
    P.trace_id = N == 6144 ? 0 : (N == 28672 ? 2 : (K == 14336 ? 3 : 1));   // the four layers of the decode set
#endif
    cudaStream_t st = as_stream(stream);
    switch (inner_k_tiles) {
        case 8: return gemv::launch_ikt<8>(P, x_bf16, x_row_stride, (int)x_cols, packed, scale_and_zero, y_bf16, workspace, st);
        case 4: return gemv::launch_ikt<4>(P, x_bf16, x_row_stride, (int)x_cols, packed, scale_and_zero, y_bf16, workspace, st);
        case 2: return gemv::launch_ikt<2>(P, x_bf16, x_row_stride, (int)x_cols, packed, scale_and_zero, y_bf16, workspace, st);
    }
    return AO_ERR_ARG;
}

extern "C" int ao_int4_gemv(const void* x_bf16, int64_t x_row_stride, int64_t x_cols, const int32_t* packed,
                            const void* scale_and_zero, int64_t M, int64_t N, int64_t K, int group, int inner_k_tiles,
                            void* y_bf16, void* workspace, size_t workspace_bytes, ao_stream_t stream) {
    return int4_gemv_impl(x_bf16, x_row_stride, x_cols, packed, scale_and_zero, M, N, K, group, inner_k_tiles, y_bf16,
                          nullptr, workspace, workspace_bytes, stream);
}

// ao_int4_gemv with the bias add of the linear fused into the store (used by ao_int4_tinygemm_linear_bias)
extern "C" int ao_int4_gemv_bias(const void* x_bf16, int64_t x_row_stride, int64_t x_cols, const int32_t* packed,
                                 const void* scale_and_zero, int64_t M, int64_t N, int64_t K, int group,
                                 int inner_k_tiles, void* y_bf16, const void* bias_bf16, void* workspace,
                                 size_t workspace_bytes, ao_stream_t stream) {
    return int4_gemv_impl(x_bf16, x_row_stride, x_cols, packed, scale_and_zero, M, N, K, group, inner_k_tiles, y_bf16,
                          bias_bf16, workspace, workspace_bytes, stream);
}

// The same kernel with the output exchange of a row-sharded layer in its epilogue: every CTA sends its rows to every
// peer's landing area through peer-mapped memory (NVLink) and returns without waiting; ao_gather_wait (comm.cu)
// collects the peers' rows.  ao_int4_gemv_gather enqueues both for one call site.
extern "C" int ao_int4_gemv_push(const void* x_bf16, int64_t x_row_stride, int64_t x_cols, const int32_t* packed,
                                   const void* scale_and_zero, int64_t M, int64_t N, int64_t K, int group,
                                 int inner_k_tiles, int nranks, int rank, void* const* peer_landing,
                                 void* y_gathered, void* site_state, void* workspace, size_t workspace_bytes,
                                 ao_stream_t stream) {
    if (M == 0 || N == 0) return AO_OK;
    if (nranks < 1 || nranks > gemv::kMaxRanks || rank < 0 || rank >= nranks || !peer_landing || !y_gathered || !site_state)
        return AO_ERR_ARG;
    gemv::Plan P;
    int rc = gemv::make_plan(M, N, K, group, inner_k_tiles, &P);
    if (rc) return rc;
    if (P.nslabs != 1) return AO_ERR_UNSUPPORTED;   // the exchange epilogue needs whole rows per CTA
    if (P.smem_bytes > 227 * 1024) return AO_ERR_UNSUPPORTED;
    if (x_cols < 2 || x_cols > K || x_cols % 2 != 0 || x_row_stride < x_cols || x_row_stride % 2 != 0) return AO_ERR_SHAPE;
    if (!aligned(x_bf16, 4) || !aligned(packed, 16) || !aligned(scale_and_zero, 16) || !aligned(workspace, 256) ||
        !aligned(site_state, 16) || !aligned(y_gathered, 16))
        return AO_ERR_ALIGN;
    if (workspace == nullptr || workspace_bytes < P.ws_bytes) return AO_ERR_WORKSPACE;
    P.nranks = nranks;
    P.rank = rank;
    P.local_state = static_cast<unsigned*>(site_state);
    P.y_gathered = static_cast<__nv_bfloat16*>(y_gathered);
    for (int r = 0; r < nranks; ++r) {
        if (!peer_landing[r] || !aligned(peer_landing[r], 16)) return AO_ERR_ALIGN;
        P.peer_ll[r] = static_cast<uint2*>(peer_landing[r]);
    }
    cudaStream_t st = as_stream(stream);
    switch (inner_k_tiles) {
        case 8: return gemv::launch_ikt<8>(P, x_bf16, x_row_stride, (int)x_cols, packed, scale_and_zero, y_gathered, workspace, st);
        case 4: return gemv::launch_ikt<4>(P, x_bf16, x_row_stride, (int)x_cols, packed, scale_and_zero, y_gathered, workspace, st);
        case 2: return gemv::launch_ikt<2>(P, x_bf16, x_row_stride, (int)x_cols, packed, scale_and_zero, y_gathered, workspace, st);
    }
    return AO_ERR_ARG;
}

extern "C" int ao_gather_exchange(int nsites, void* const* peer_landing, void* const* y_gathered, void* const* state,
                                  const int64_t* M, const int64_t* N, int nranks, int rank, int push, void* workspace,
                                  ao_stream_t stream);

extern "C" int ao_int4_gemv_gather(const void* x_bf16, int64_t x_row_stride, int64_t x_cols, const int32_t* packed,
                                   const void* scale_and_zero, int64_t M, int64_t N, int64_t K, int group,
                                   int inner_k_tiles, int nranks, int rank, void* const* peer_landing,
                                   void* y_gathered, void* site_state, void* workspace, size_t workspace_bytes,
                                   ao_stream_t stream) {
    if (M == 0 || N == 0) return AO_OK;
    int rc = ao_int4_gemv_push(x_bf16, x_row_stride, x_cols, packed, scale_and_zero, M, N, K, group, inner_k_tiles, nranks,
                               rank, peer_landing, y_gathered, site_state, workspace, workspace_bytes, stream);
    if (rc || nranks < 2) return rc;
    return ao_gather_exchange(1, peer_landing, &y_gathered, &site_state, &M, &N, nranks, rank, /*push=*/0, workspace, stream);
}
