// int4 decode GEMV kernels for packed weights with inner_k_tiles = 8.
#include "int4_gemv.cuh"

namespace ao {
namespace gemv {
template int launch_ikt<8>(const Plan&, const void*, long long, int, const void*, const void*, void*, void*,
                            cudaStream_t);
}
}  // namespace ao

