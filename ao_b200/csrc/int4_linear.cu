// Dispatcher of the int4 tensor_core_tiled linear: a single row and the smallest batches go to the GEMV kernel,
// larger batches to the tcgen05 kernel; shapes that kernel does not take run as row blocks of 16 through the GEMV.
// Where the line is (measured on B200, both kernels on the same weights): the tcgen05 kernel at 16 columns costs
// 8.3 / 7.2 / 23.5 / 13.3 us on the Llama-3-8B layers (qkv, o, gate_up, down) whatever M <= 16 is; the GEMV costs
// 7.3 / 6.2 / 19.2 / 16.3 us at M = 2, 8.7 / 7.4 / 20.5 / 20.2 at M = 4 and 11.0 / 9.8 / 24.1 / 21.2 at M = 8.  So: M >= 5
// always, and from M = 2 where the reduction is long against the number of rows (K >= 2 N: the GEMV then needs K
// slabs or long activation prologues).
#include "common.cuh"

namespace ao {
namespace umma {
size_t int4_umma_workspace_bytes(int64_t M, int64_t N, int64_t K, int g, int ikt);
int int4_umma_linear(const void* x, int64_t ldx, int64_t x_cols, const int32_t* packed, const void* sz, int64_t M,
                     int64_t N, int64_t K, int g, int ikt, void* y, const void* bias, void* ws, size_t ws_bytes,
                     cudaStream_t st);
}
}  // namespace ao

static bool prefers_tcgen05(int64_t M, int64_t N, int64_t K) { return M >= 5 || (M >= 2 && K >= 2 * N); }

extern "C" size_t ao_int4_tinygemm_linear_workspace_bytes(int64_t M, int64_t N, int64_t K, int group,
                                                          int inner_k_tiles) {
    if (M <= 8 && !prefers_tcgen05(M, N, K)) return ao_int4_gemv_workspace_bytes(M, N, K, group, inner_k_tiles);
    // larger batches: the tcgen05 kernel's need, and the decode kernel's for shapes that fall back to row blocks
    size_t need = ao::umma::int4_umma_workspace_bytes(M, N, K, group, inner_k_tiles);
    for (int m = 1; m <= 16; m *= 2) {
        const size_t b = ao_int4_gemv_workspace_bytes(m, N, K, group, inner_k_tiles);
        if (b == 0) return 0;
        need = b > need ? b : need;
    }
    return need;
}

extern "C" int ao_int4_gemv_bias(const void* x_bf16, int64_t x_row_stride, int64_t x_cols, const int32_t* packed,
                                 const void* scale_and_zero, int64_t M, int64_t N, int64_t K, int group,
                                 int inner_k_tiles, void* y_bf16, const void* bias_bf16, void* workspace,
                                 size_t workspace_bytes, ao_stream_t stream);

extern "C" int ao_int4_tinygemm_linear_bias(const void* x_bf16, int64_t x_row_stride, int64_t x_cols,
                                            const int32_t* packed, const void* scale_and_zero, int64_t M, int64_t N,
                                            int64_t K, int group, int inner_k_tiles, void* y_bf16,
                                            const void* bias_bf16, void* workspace, size_t workspace_bytes,
                                            ao_stream_t stream) {
    if (M < 0 || N < 0) return AO_ERR_SHAPE;
    if (M <= 8 && !prefers_tcgen05(M, N, K))
        return ao_int4_gemv_bias(x_bf16, x_row_stride, x_cols, packed, scale_and_zero, M, N, K, group, inner_k_tiles, y_bf16,
                                 bias_bf16, workspace, workspace_bytes, stream);
    if (workspace == nullptr || workspace_bytes < 256 || !ao::aligned(workspace, 256)) return AO_ERR_WORKSPACE;
    {
        const int rc = ao::umma::int4_umma_linear(x_bf16, x_row_stride, x_cols, packed, scale_and_zero, M, N, K, group,
                                                  inner_k_tiles, y_bf16, bias_bf16, workspace, workspace_bytes, ao::as_stream(stream));
        if (rc != AO_ERR_UNSUPPORTED) return rc;
    }
    if (M <= 16)
        return ao_int4_gemv_bias(x_bf16, x_row_stride, x_cols, packed, scale_and_zero, M, N, K, group, inner_k_tiles, y_bf16,
                                 bias_bf16, workspace, workspace_bytes, stream);
    // row blocks of 16 through the same kernel, back to back on the stream
    const auto* x = static_cast<const __nv_bfloat16*>(x_bf16);
    auto* y = static_cast<__nv_bfloat16*>(y_bf16);
    for (int64_t m0 = 0; m0 < M; m0 += 16) {
        const int64_t mb = M - m0 < 16 ? M - m0 : 16;
        // every block uses the 16-row plan's workspace layout only if mb == 16; smaller tails need less
        int rc = ao_int4_gemv_bias(x + m0 * x_row_stride, x_row_stride, x_cols, packed, scale_and_zero, mb, N, K, group,
                                   inner_k_tiles, y + m0 * N, bias_bf16, workspace, workspace_bytes, stream);
        if (rc) return rc;
    }
    return AO_OK;
}

extern "C" int ao_int4_tinygemm_linear(const void* x_bf16, int64_t x_row_stride, int64_t x_cols,
                                       const int32_t* packed, const void* scale_and_zero, int64_t M, int64_t N,
                                       int64_t K, int group, int inner_k_tiles, void* y_bf16, void* workspace,
                                       size_t workspace_bytes, ao_stream_t stream) {
    return ao_int4_tinygemm_linear_bias(x_bf16, x_row_stride, x_cols, packed, scale_and_zero, M, N, K, group, inner_k_tiles,
                                        y_bf16, nullptr, workspace, workspace_bytes, stream);
}
