// ao_int4_gemv_static_scratch: the int4 decode GEMV for callers that cannot hand over a workspace.
//
// Some hosts of this library have no way to give a kernel scratch memory: a plug-in boundary whose operator
// signature is fixed (inputs, weights, output, stream and nothing else), or a plain C serving loop that owns no
// device allocator and must not call one while requests are in flight, because an allocation may synchronise the
// device or fail under memory pressure in the middle of serving.  For them the scratch lives in this library's own
// image: one file-scope device array per GPU, of a fixed and modest size, so this entry point never allocates.
//
// Consequences the caller has to know:
//   * the first call on a device looks up the array's device address (and may load the module); make that call
//     once per device during start-up, before any stream capture;
//   * requests whose scratch need exceeds kStaticScratchBytes are rejected with AO_ERR_WORKSPACE
//     (ao_int4_gemv_static_scratch_max_bytes() reports the limit, ao_int4_gemv_workspace_bytes() the need);
//   * every call on a device uses the same array, which still holds what the previous call left there.  The
//     part that has to start at zero (status word and completion counters) is cleared on the stream at the
//     start of each call.  The launch counter next to the status word is deliberately NOT cleared: the K-slab
//     hand-off tags its partial sums with the launch number, so the number must keep growing from call to call or
//     a finisher could mistake the previous call's partial sums (still in the array) for this call's.  Two calls
//     that overlap on the GPU (different streams) race on the array and must be serialised by the caller, or use
//     ao_int4_gemv with workspaces of their own;
//   * the array that is used belongs to the device that is current when the entry point is called; the stream
//     must be a stream of that device.
#include <mutex>

#include "int4_gemv.cuh"

namespace ao {
namespace gemv {

extern template int launch_ikt<8>(const Plan&, const void*, long long, int, const void*, const void*,
                                  void*, void*, cudaStream_t);
extern template int launch_ikt<4>(const Plan&, const void*, long long, int, const void*, const void*,
                                  void*, void*, cudaStream_t);
extern template int launch_ikt<2>(const Plan&, const void*, long long, int, const void*, const void*,
                                  void*, void*, cudaStream_t);

constexpr size_t kStaticScratchBytes = 2u << 20;  // 2 MiB per device
constexpr int kMaxDevices = 64;

static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

static std::mutex g_setup_mutex;
static void* g_scratch_ptr[kMaxDevices] = {};

// Device address of the scratch array on the current device; looked up once per device.
static int scratch_for_current_device(void** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) return AO_ERR_LAUNCH;
    if (dev < 0 || dev >= kMaxDevices) return AO_ERR_UNSUPPORTED;   // more devices than the address table holds
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_scratch_ptr[dev] == nullptr) {
        void* ptr = nullptr;
        if (cudaGetSymbolAddress((void**)&ptr, g_static_scratch) != cudaSuccess || ptr == nullptr) {
            (void)cudaGetLastError();
            return AO_ERR_LAUNCH;
        }
        g_scratch_ptr[dev] = ptr;
    }
    *out = g_scratch_ptr[dev];
    return AO_OK;
}

}  // namespace gemv
}  // namespace ao

using namespace ao;

extern "C" size_t ao_int4_gemv_static_scratch_max_bytes(void) { return gemv::kStaticScratchBytes; }

extern "C" int ao_int4_gemv_static_scratch(const void* x_bf16, int64_t x_row_stride, int64_t x_cols,
                                           const int32_t* packed, const void* scale_and_zero, int64_t M, int64_t N,
                                           int64_t K, int group, int inner_k_tiles, void* y_bf16, ao_stream_t stream) {
    if (M == 0 || N == 0) return AO_OK;
    gemv::Plan P;
    int rc = gemv::make_plan(M, N, K, group, inner_k_tiles, &P);
    if (rc) return rc;
    if (P.ws_bytes > gemv::kStaticScratchBytes) return AO_ERR_WORKSPACE;  // beyond the stated maximum
    if (x_cols < 2 || x_cols > K || x_cols % 2 != 0 || x_row_stride < x_cols || x_row_stride % 2 != 0) return AO_ERR_SHAPE;
    if (!aligned(x_bf16, 4) || !aligned(packed, 16) || !aligned(scale_and_zero, 16) || !aligned(y_bf16, 2))
        return AO_ERR_ALIGN;
    void* scratch = nullptr;
    rc = gemv::scratch_for_current_device(&scratch);
    if (rc) return rc;
    cudaStream_t st = as_stream(stream);
    // what must start at zero: the status word and, with K slabs, the completion counters of this call's row
    // pairs.  Bytes [kCallStateOff, kCallStateOff + 8) -- the finished-CTA counter, which every launch leaves at
    // zero itself, and the launch number that tags the slab partial sums -- persist from call to call.
    static_assert(gemv::kCallStateOff >= 4, "the status word is cleared on its own");
    unsigned char* base = static_cast<unsigned char*>(scratch);
    bool ok = cudaMemsetAsync(base, 0, 4, st) == cudaSuccess;
    if (ok && P.nslabs > 1) ok = cudaMemsetAsync(base + P.ws_counters_off, 0, (size_t)P.NP * 4, st) == cudaSuccess;
    if (!ok) {
        (void)cudaGetLastError();
        return AO_ERR_LAUNCH;
    }
    switch (inner_k_tiles) {
        case 8: return gemv::launch_ikt<8>(P, x_bf16, x_row_stride, (int)x_cols, packed, scale_and_zero, y_bf16, scratch, st);
        case 4: return gemv::launch_ikt<4>(P, x_bf16, x_row_stride, (int)x_cols, packed, scale_and_zero, y_bf16, scratch, st);
        case 2: return gemv::launch_ikt<2>(P, x_bf16, x_row_stride, (int)x_cols, packed, scale_and_zero, y_bf16, scratch, st);
    }
    return AO_ERR_ARG;
}
