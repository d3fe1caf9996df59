// int4 decode GEMV kernels for packed weights with inner_k_tiles = 8.
#include "int4_gemv.cuh"

namespace ao {
namespace gemv {
template int launch_ikt<8>(const Plan&, const void*, long long, int, const void*, const void*, void*, void*,
                            cudaStream_t);
}
}  // namespace ao


#if defined(AO_GEMV_TRACE) && AO_GEMV_TRACE
// trace builds: copy the timeline of the kernels of this translation unit out (8 launches x 512 CTAs x 32 slots)
extern "C" int ao_debug_read_trace(unsigned long long* host_out, int n) {
    return (int)cudaMemcpyFromSymbol(host_out, ao::gemv::g_trace, sizeof(unsigned long long) * n);
}
#endif
