// Peer-memory plumbing for the output exchange of row-sharded linears: export a CUDA IPC handle of a device
// allocation, open another process's handle.  Set-up code (called once per process group), not on the hot path.
#include <cuda.h>

#include "common.cuh"

namespace {

using GetAddressRangeFn = CUresult (*)(CUdeviceptr*, size_t*, CUdeviceptr);

GetAddressRangeFn address_range_fn() {
    static GetAddressRangeFn fn = []() -> GetAddressRangeFn {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            return nullptr;
        return reinterpret_cast<GetAddressRangeFn>(p);
    }();
    return fn;
}

}  // namespace

// handle_out: 64 bytes (cudaIpcMemHandle_t) of the allocation that contains ptr; offset_out: ptr - allocation base.
extern "C" int ao_comm_export(const void* ptr, void* handle_out, int64_t* offset_out) {
    if (!ptr || !handle_out || !offset_out) return AO_ERR_ARG;
    GetAddressRangeFn range = address_range_fn();
    if (!range) return AO_ERR_LAUNCH;
    CUdeviceptr base = 0;
    size_t size = 0;
    if (range(&base, &size, reinterpret_cast<CUdeviceptr>(ptr)) != CUDA_SUCCESS) return AO_ERR_ARG;
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base)) != cudaSuccess) {
        (void)cudaGetLastError();
        return AO_ERR_LAUNCH;
    }
    static_assert(sizeof(h) == 64, "IPC handle size");
    memcpy(handle_out, &h, sizeof(h));
    *offset_out = static_cast<int64_t>(reinterpret_cast<CUdeviceptr>(ptr) - base);
    return AO_OK;
}

// Maps another process's allocation into this process (current device); *base_out is the mapped allocation base.
extern "C" int ao_comm_import(const void* handle, void** base_out) {
    if (!handle || !base_out) return AO_ERR_ARG;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void* p = nullptr;
    if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
        (void)cudaGetLastError();
        return AO_ERR_LAUNCH;
    }
    *base_out = p;
    return AO_OK;
}

extern "C" int ao_comm_close(void* base) {
    if (!base) return AO_OK;
    if (cudaIpcCloseMemHandle(base) != cudaSuccess) {
        (void)cudaGetLastError();
        return AO_ERR_LAUNCH;
    }
    return AO_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// Gather exchange: the all-gather of row-sharded decode outputs over peer memory, for several layers in one launch.
//
// Every rank's rows travel as 8-byte {two bf16 rows, call number} words - data and "it has arrived" in one store
// that the hardware writes as a unit, so there is no fence and no separate flag - into a landing area in the
// receiver's memory that is double buffered by the parity of the call number.  The kernel has two halves:
//   push  (optional)  reads this rank's own block [M][N] of each site's gathered output and stores it into every
//                     peer's landing area.  Skipped for sites whose rows the GEMV epilogue (ao_int4_gemv_push) has
//                     already sent.
//   wait              polls every word of the call's landing buffer until it carries the call's number (bounded:
//                     0.2 s, then AO_ERR_TIMEOUT in the status word) and writes the rows into the gathered output
//                     [rank][M][N].
// Up to kMaxSites call sites (layers) share one launch: a decode step is a chain of microsecond-sized kernels, and
// what an exchange costs there is its fixed part - one more kernel boundary, and the NVLink write acknowledgement
// that a kernel's completion waits for - so the layers of a step whose outputs nobody needs before the step ends
// are exchanged together.  The kernel runs on a few dozen small CTAs, starts behind the kernels before it
// (griddepcontrol.wait, executed before it reads anything, so the stream's order of completion holds for everything
// that follows) and lets the next launch start early.
// ---------------------------------------------------------------------------------------------------------------
namespace ao {
namespace gather {

// Device-side timeline (a build with -DAO_COMM_TRACE=1 only): globaltimer stamps of CTA 0, thread 0, of the most
// recent launch, copied out by a debug entry point of that build.  Nothing in the shipped library.
#if defined(AO_COMM_TRACE) && AO_COMM_TRACE
static __device__ unsigned long long g_comm_trace[16];
#define AO_CTR(slot) do { if (blockIdx.x == 0 && threadIdx.x == 0) { unsigned long long t_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_)); g_comm_trace[slot] = t_; } } while (0)
#else
#define AO_CTR(slot) do { } while (0)
#endif

constexpr int kMaxSites = 8;
constexpr int kMaxRanks = 8;
constexpr int kThreads = 256;
constexpr int kCtas = 64;   // at least; see the launch

struct Site {
    uint2* peer_landing[kMaxRanks];   // the site's landing area in every rank's buffer: [parity][source rank][M][N/2] words
    __nv_bfloat16* y;                 // this rank's gathered output [nranks][M][N]
    unsigned* state;                  // the site's {pushed CTAs, pushes so far, CTAs done waiting, waits so far}
    int M, N;
};
struct Args {
    Site site[kMaxSites];
    int nsites, nranks, rank, push;
    int* status;
};

__device__ __forceinline__ uint2 ld_volatile_u2(const uint2* p) {
    uint2 v;
    asm volatile("ld.volatile.global.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}
// 8-byte store into a peer's memory.  A plain (weak) store on purpose: the word is written as one unit whatever its
// qualifier, and a thread's consecutive volatile stores to a peer were observed to wait for one another's NVLink
// round trip (about 2.5 us each), while plain stores are posted back to back.
__device__ __forceinline__ void st_peer_u2(uint2* p, uint32_t a, uint32_t b) {
    asm volatile("st.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__global__ void __launch_bounds__(kThreads) gather_exchange_kernel(const __grid_constant__ Args Ap) {
    AO_CTR(0);
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // Everything that depends only on the arguments happens before the dependency wait, while the kernel before
    // this one is still running: the arguments move from constant memory (a cold miss per 64-byte line, one after
    // the other along dependent index arithmetic) into shared memory, and the thread works out what it will send.
    __shared__ Args A;
    __shared__ long long first_push[kMaxSites + 1], first_wait[kMaxSites + 1];
    {
        const uint32_t* src = reinterpret_cast<const uint32_t*>(&Ap);
        uint32_t* dst = reinterpret_cast<uint32_t*>(&A);
        for (int i = threadIdx.x; i < static_cast<int>(sizeof(Args) / 4); i += kThreads) dst[i] = src[i];
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        first_push[0] = first_wait[0] = 0;
        for (int s = 0; s < kMaxSites; ++s) {
            const long long block = s < A.nsites ? (long long)A.site[s].M * (A.site[s].N / 2) : 0;
            first_push[s + 1] = first_push[s] + block;
            first_wait[s + 1] = first_wait[s] + (long long)(A.nranks - 1) * block;
        }
    }
    __syncthreads();
    const int tid = blockIdx.x * kThreads + threadIdx.x, nthreads = gridDim.x * kThreads;
    const int nsites = A.nsites, nranks = A.nranks, rank = A.rank;
    auto site_of = [&](const long long* first, long long i) {
        int s = 0;
        for (int t = 1; t < nsites; ++t)
            if (i >= first[t]) s = t;
        return s;
    };
    // The words of all sites form one index space that the threads stride through, so that the sites are pushed
    // and polled together: a round of polling costs one memory latency for the whole launch, not one per site.
    // This thread's first words to send: where they come from, and where they go in every peer's landing area
    // (up to the parity of the call number, which is not known yet).
    constexpr int kAhead = 4;
    const uint32_t* asrc[kAhead];
    int asite[kAhead];
    long long aoff[kAhead];
    const long long push_total = A.push ? first_push[nsites] : 0;
#pragma unroll
    for (int k = 0; k < kAhead; ++k) {
        const long long i = tid + (long long)k * nthreads;
        asrc[k] = nullptr;
        asite[k] = 0;
        aoff[k] = 0;
        if (i < push_total) {
            const int s = site_of(first_push, i);
            const Site& S = A.site[s];
            const long long block = (long long)S.M * (S.N / 2), w = i - first_push[s];
            asite[k] = s;
            asrc[k] = reinterpret_cast<const uint32_t*>(S.y + (size_t)rank * S.M * S.N) + w;
            aoff[k] = (long long)rank * block + w;
        }
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");   // the kernels before this one have completed
    AO_CTR(1);
    // the words to send and the call numbers are independent trips to the L2: both are on their way before either
    // is used
    uint32_t ahead[kAhead];
#pragma unroll
    for (int k = 0; k < kAhead; ++k) ahead[k] = asrc[k] ? *asrc[k] : 0u;
    // numbers of this push and this wait (all CTAs read the same values: they change when the last CTA of the
    // launch finishes); one thread per site reads the site's four counters in one load, the CTA shares them
    __shared__ uint4 counters[kMaxSites];
    if (threadIdx.x < nsites) {
        uint4 c;
        asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(c.x), "=r"(c.y), "=r"(c.z), "=r"(c.w)
                     : "l"(A.site[threadIdx.x].state) : "memory");
        counters[threadIdx.x] = c;
    }
    __syncthreads();
    unsigned pcall[kMaxSites], wcall[kMaxSites];
#pragma unroll
    for (int s = 0; s < kMaxSites; ++s) {
        pcall[s] = wcall[s] = 0u;
        if (s < nsites) {
            pcall[s] = counters[s].y + 1u;
            wcall[s] = counters[s].w + 1u;
        }
    }
    if (A.push) {
#pragma unroll
        for (int k = 0; k < kAhead; ++k) {
            if (asrc[k] == nullptr) continue;
            const Site& S = A.site[asite[k]];
            unsigned call = pcall[0];
#pragma unroll
            for (int t = 1; t < kMaxSites; ++t) call = (asite[k] == t) ? pcall[t] : call;
            const size_t off = ((call & 1u) ? (size_t)nranks * S.M * (S.N / 2) : 0) + (size_t)aoff[k];
            for (int d = 1; d < nranks; ++d) {
                const int r = (rank + d) % nranks;
                st_peer_u2(S.peer_landing[r] + off, ahead[k], call);
            }
        }
        for (long long i = tid + (long long)kAhead * nthreads; i < push_total; i += nthreads) {
            const int s = site_of(first_push, i);
            const Site& S = A.site[s];
            const long long block = (long long)S.M * (S.N / 2), w = i - first_push[s];
            unsigned call = pcall[0];
#pragma unroll
            for (int t = 1; t < kMaxSites; ++t) call = (s == t) ? pcall[t] : call;
            const size_t off = ((call & 1u) ? (size_t)nranks * block : 0) + (size_t)rank * block + w;
            const uint32_t v = reinterpret_cast<const uint32_t*>(S.y + (size_t)rank * S.M * S.N)[w];
            for (int d = 1; d < nranks; ++d) {
                const int r = (rank + d) % nranks;
                st_peer_u2(S.peer_landing[r] + off, v, call);
            }
        }
    }
    AO_CTR(2);
    bool ok = true;
    const uint64_t t0 = globaltimer_ns();
    const long long total = first_wait[nsites];
    // a thread owns up to eight words at a time and re-reads all that are still missing together
    for (long long b0 = tid; b0 < total && ok; b0 += (long long)nthreads * 8) {
        const uint2* src[8];
        uint32_t* dst[8];
        unsigned want[8];
        unsigned pending = 0u;
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const long long i = b0 + (long long)q * nthreads;
            src[q] = nullptr;
            dst[q] = nullptr;
            want[q] = 0u;
            if (i < total) {
                const int s = site_of(first_wait, i);
                const Site& S = A.site[s];
                const long long block = (long long)S.M * (S.N / 2), w = i - first_wait[s];
                const int si = (int)(w / block);
                const long long rem = w - (long long)si * block;
                const int r = si + (si >= rank ? 1 : 0);        // the source ranks other than this one, in order
                unsigned call = wcall[0];
#pragma unroll
                for (int t = 1; t < kMaxSites; ++t) call = (s == t) ? wcall[t] : call;
                src[q] = S.peer_landing[rank] + ((call & 1u) ? (size_t)nranks * block : 0) + (size_t)r * block + rem;
                dst[q] = reinterpret_cast<uint32_t*>(S.y + (size_t)r * S.M * S.N) + rem;
                want[q] = call;
                pending |= 1u << q;
            }
        }
        while (pending) {
            uint2 v[8];
#pragma unroll
            for (int q = 0; q < 8; ++q)
                if (pending & (1u << q)) v[q] = ld_volatile_u2(src[q]);
#pragma unroll
            for (int q = 0; q < 8; ++q)
                if ((pending & (1u << q)) && v[q].y == want[q]) {
                    *dst[q] = v[q].x;
                    pending &= ~(1u << q);
                }
            if (pending && globaltimer_ns() - t0 > 200000000ull) {   // 0.2 s
                ok = false;
                break;
            }
        }
    }
    AO_CTR(3);
    if (!ok) atomicExch(A.status, AO_ERR_TIMEOUT);
    __syncthreads();
    AO_CTR(4);
    if (threadIdx.x < nsites) {
        // the last CTA to finish advances the call numbers of the sites for the next launch (one thread per site)
        unsigned* st = A.site[threadIdx.x].state;
        __threadfence();
        const unsigned done = atomicAdd(st + 2, 1u);
        if (done + 1 == gridDim.x) {
            st[2] = 0u;
            if (A.push) st[1] = *reinterpret_cast<volatile unsigned*>(st + 1) + 1u;
            __threadfence();
            st[3] = *reinterpret_cast<volatile unsigned*>(st + 3) + 1u;
        }
    }
    AO_CTR(5);
}

}  // namespace gather
}  // namespace ao

#if defined(AO_COMM_TRACE) && AO_COMM_TRACE
extern "C" int ao_debug_read_comm_trace(unsigned long long* host_out) {
    return (int)cudaMemcpyFromSymbol(host_out, ao::gather::g_comm_trace, sizeof(unsigned long long) * 16);
}
#endif

extern "C" int ao_gather_exchange(int nsites, void* const* peer_landing, void* const* y_gathered, void* const* state,
                                  const int64_t* M, const int64_t* N, int nranks, int rank, int push, void* workspace,
                                  ao_stream_t stream) {
    using namespace ao;
    if (nsites < 1 || nsites > gather::kMaxSites || nranks < 2 || nranks > gather::kMaxRanks || rank < 0 || rank >= nranks)
        return AO_ERR_ARG;
    if (!peer_landing || !y_gathered || !state || !M || !N || !workspace) return AO_ERR_ARG;
    gather::Args A = {};
    for (int s = 0; s < nsites; ++s) {
        if (!y_gathered[s] || !state[s]) return AO_ERR_ARG;
        if (M[s] < 1 || M[s] > 64 || N[s] < 8 || N[s] % 8 != 0) return AO_ERR_SHAPE;
        if (!aligned(y_gathered[s], 16) || !aligned(state[s], 16)) return AO_ERR_ALIGN;
        for (int r = 0; r < nranks; ++r) {
            void* p = peer_landing[s * nranks + r];
            if (!p) return AO_ERR_ARG;
            if (!aligned(p, 16)) return AO_ERR_ALIGN;
            A.site[s].peer_landing[r] = static_cast<uint2*>(p);
        }
        A.site[s].y = static_cast<__nv_bfloat16*>(y_gathered[s]);
        A.site[s].state = static_cast<unsigned*>(state[s]);
        A.site[s].M = (int)M[s];
        A.site[s].N = (int)N[s];
    }
    A.nsites = nsites;
    A.nranks = nranks;
    A.rank = rank;
    A.push = push ? 1 : 0;
    A.status = static_cast<int*>(workspace);
    cudaLaunchConfig_t cfg = {};
    // CTAs: a thread polls up to eight words per round, and a round costs one memory latency, so as many CTAs as give
    // every word a thread in the first round, between kCtas and one per SM
    long long wait_words = 0;
    for (int s = 0; s < nsites; ++s) wait_words += (long long)(nranks - 1) * M[s] * (N[s] / 2);
    long long ctas = (wait_words + gather::kThreads * 8 - 1) / (gather::kThreads * 8);
    ctas = ctas < gather::kCtas ? gather::kCtas : (ctas > kNumSMs ? kNumSMs : ctas);
    cfg.gridDim = dim3((unsigned)ctas);
    cfg.blockDim = dim3(gather::kThreads);
    cfg.stream = as_stream(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, gather::gather_exchange_kernel, A) != cudaSuccess) {
        (void)cudaGetLastError();
        return AO_ERR_LAUNCH;
    }
    return AO_OK;
}
