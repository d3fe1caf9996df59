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
