// PyTorch dispatcher binding of the C ABI (include/ao_b200.h): the seam the reference's Python reaches the kernels
// through.
//   torchao::quant_llm_linear            schema of torchao/csrc/fp6_llm.cpp:5-8, CUDA implementation in the place of
//                                        torchao/csrc/cuda/fp6_llm/fp6_linear.cu:139-200
//   torchao::_weight_int4pack_mm         twins of aten::_weight_int4pack_mm / aten::_convert_weight_to_int4pack as the
//   torchao::_convert_weight_to_int4pack reference calls them (torchao/dtypes/affine_quantized_tensor.py:461, 631);
//                                        PyTorch's own operators cannot be overridden in place
// Conventions kept from fp6_linear.cu: inputs are borrowed and never mutated; the callee allocates the output (and its
// scratch) with the caching allocator on the input's device; everything is enqueued on
// at::cuda::getCurrentCUDAStream() without synchronising, so the operators can be captured in CUDA graphs; shape
// errors are TORCH_CHECK failures.  Unlike the reference, a non-zero status of the kernel layer is an error too.
// The fake (meta) implementations live in Python (ao_b200/_torch_ops.py), as the reference's do (torchao/ops.py).
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include <mutex>
#include <unordered_map>

#include "../../../include/ao_b200.h"

namespace {

// Zero-initialised scratch per (device, stream), grown on demand and kept: the kernels leave it ready for the next
// call.  It is a raw device allocation, not a tensor of the caching allocator: under torch.compile's CUDA-graph trees
// every live allocation made while the compiled function runs must be one of its outputs, and this buffer outlives
// the call by design.  The first call on a stream allocates and clears it, which cannot happen inside a stream
// capture: make one call during warm-up (the graph trees' own warm-up run counts).  A buffer that is outgrown is
// kept alive, because captured graphs may still point at it.
void* workspace(size_t nbytes, int device_index, cudaStream_t stream, size_t* size_out) {
    struct Buf { void* ptr; size_t size; };
    static std::mutex mu;
    static std::unordered_map<uint64_t, Buf> cache;
    const uint64_t key = (static_cast<uint64_t>(device_index) << 56) ^ reinterpret_cast<uint64_t>(stream);
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end() && it->second.size >= nbytes) {
        *size_out = it->second.size;
        return it->second.ptr;
    }
    cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
    TORCH_CHECK(cudaStreamIsCapturing(stream, &capturing) == cudaSuccess && capturing == cudaStreamCaptureStatusNone,
                "the first call of a torchao:: operator on a stream sets up its scratch buffer and cannot be captured in a "
                "CUDA graph: run the operator once on this stream before capturing");
    const size_t size = nbytes < (1u << 20) ? (1u << 20) : nbytes;
    void* ptr = nullptr;
    TORCH_CHECK(cudaMalloc(&ptr, size) == cudaSuccess, "out of device memory for the operators' scratch buffer (", size, " bytes)");
    TORCH_CHECK(cudaMemsetAsync(ptr, 0, size, stream) == cudaSuccess, "clearing the operators' scratch buffer failed");
    cache[key] = Buf{ptr, size};
    *size_out = size;
    return ptr;
}

void check_status(int rc, const char* what) {
    TORCH_CHECK(rc == AO_OK, what, ": ", ao_status_string(rc), " (status ", rc, ")");
}

at::Tensor quant_llm_linear_cuda(int64_t EXPONENT, int64_t MANTISSA, at::Tensor _in_feats, at::Tensor _weights,
                                 at::Tensor _scales, int64_t splitK) {
    (void)splitK;   // the kernel chooses its own K split
    TORCH_CHECK(_in_feats.dim() == 2 && _weights.dim() == 2 && _scales.dim() == 1, "quant_llm_linear: expected 2-D input, 2-D weight, 1-D scale");
    TORCH_CHECK(_in_feats.scalar_type() == at::kHalf && _weights.scalar_type() == at::kByte && _scales.scalar_type() == at::kHalf,
                "quant_llm_linear: expected fp16 input, uint8 weight, fp16 scale");
    const int64_t NBITS = 1 + EXPONENT + MANTISSA;
    const int64_t BS = _in_feats.size(0), IC = _in_feats.size(1), OC = _weights.size(0);
    TORCH_CHECK(IC % 64 == 0, "Expected in_features to be a multiple of 64, but received ", IC);
    TORCH_CHECK((IC / 8 * NBITS) == _weights.size(1), "Dimensions mismatched");
    TORCH_CHECK(OC == _scales.size(0), "Dimensions mismatched");
    TORCH_CHECK((EXPONENT == 3 && MANTISSA == 2) || (EXPONENT == 2 && MANTISSA == 3) || (EXPONENT == 2 && MANTISSA == 2) ||
                    (EXPONENT == 3 && MANTISSA == 1),
                "FP", NBITS, " E", EXPONENT, "M", MANTISSA, " is not supported.");
    c10::cuda::CUDAGuard guard(_in_feats.device());
    at::Tensor x = (_in_feats.stride(1) == 1 && _in_feats.stride(0) % 2 == 0) ? _in_feats : _in_feats.contiguous();
    at::Tensor w = _weights.contiguous(), s = _scales.contiguous();
    at::Tensor out = at::empty({BS, OC}, x.options());
    if (BS == 0) return out;
    auto stream = at::cuda::getCurrentCUDAStream().stream();
    const size_t need = ao_fp6_linear_workspace_bytes(BS, OC, IC);
    TORCH_CHECK(need > 0, "quant_llm_linear: unsupported shape BS=", BS, " OC=", OC, " IC=", IC);
    size_t ws_size = 0;
    void* ws = workspace(need, x.device().index(), stream, &ws_size);
    check_status(ao_fpx_linear((int)EXPONENT, (int)MANTISSA, x.data_ptr(), x.stride(0), w.data_ptr<uint8_t>(), s.data_ptr(), BS,
                               OC, IC, out.data_ptr(), ws, ws_size, stream),
                 "quant_llm_linear");
    return out;
}

at::Tensor weight_int4pack_mm_cuda(at::Tensor x, at::Tensor w, int64_t qGroupSize, at::Tensor qScaleAndZeros) {
    TORCH_CHECK(x.dim() == 2 && x.scalar_type() == at::kBFloat16, "_weight_int4pack_mm: x must be a 2-D bfloat16 tensor");
    TORCH_CHECK(w.dim() == 4 && w.scalar_type() == at::kInt && w.size(2) == 32,
                "_weight_int4pack_mm: w must be int32 [N/8][K/(innerKTiles*16)][32][innerKTiles/2]");
    TORCH_CHECK(qScaleAndZeros.dim() == 3 && qScaleAndZeros.size(2) == 2 && qScaleAndZeros.scalar_type() == at::kBFloat16,
                "_weight_int4pack_mm: qScaleAndZeros must be bfloat16 [K/group][N][2]");
    const int64_t ikt = w.size(3) * 2, N = w.size(0) * 8, K = w.size(1) * ikt * 16, M = x.size(0);
    TORCH_CHECK(x.size(1) <= K, "_weight_int4pack_mm: x has ", x.size(1), " columns, the weight only ", K);
    TORCH_CHECK(qScaleAndZeros.size(0) == K / qGroupSize && qScaleAndZeros.size(1) == N,
                "_weight_int4pack_mm: qScaleAndZeros does not match K/group and N");
    c10::cuda::CUDAGuard guard(x.device());
    at::Tensor xc = x;
    if (x.stride(1) != 1 || x.stride(0) % 2 != 0 || x.size(1) % 2 != 0 || reinterpret_cast<uintptr_t>(x.data_ptr()) % 4 != 0)
        xc = at::constant_pad_nd(x, {0, x.size(1) % 2}).contiguous();
    at::Tensor wc = w.contiguous(), sz = qScaleAndZeros.contiguous();
    at::Tensor y = at::empty({M, N}, x.options());
    if (M == 0) return y;
    auto stream = at::cuda::getCurrentCUDAStream().stream();
    const size_t need = ao_int4_tinygemm_linear_workspace_bytes(M, N, K, (int)qGroupSize, (int)ikt);
    TORCH_CHECK(need > 0, "_weight_int4pack_mm: unsupported shape M=", M, " N=", N, " K=", K, " group=", qGroupSize);
    size_t ws_size = 0;
    void* ws = workspace(need, x.device().index(), stream, &ws_size);
    check_status(ao_int4_tinygemm_linear(xc.data_ptr(), xc.stride(0), xc.size(1), wc.data_ptr<int32_t>(), sz.data_ptr(), M, N, K,
                                         (int)qGroupSize, (int)ikt, y.data_ptr(), ws, ws_size, stream),
                 "_weight_int4pack_mm");
    return y;
}

at::Tensor convert_weight_to_int4pack_cuda(at::Tensor int_data, int64_t innerKTiles) {
    TORCH_CHECK(int_data.dim() == 2, "_convert_weight_to_int4pack: int_data must be 2-D [n][k]");
    TORCH_CHECK(innerKTiles == 2 || innerKTiles == 4 || innerKTiles == 8, "innerKTiles must be 2, 4, or 8");
    c10::cuda::CUDAGuard guard(int_data.device());
    at::Tensor codes = int_data.to(at::kInt).contiguous();
    const int64_t N = codes.size(0), K = codes.size(1);
    TORCH_CHECK(N % 8 == 0, "expect N to be a multiple of 8, got ", N);
    TORCH_CHECK(K % (innerKTiles * 16) == 0, "expect K to be a multiple of ", innerKTiles * 16, ", got ", K);
    at::Tensor out = at::empty({N / 8, K / (innerKTiles * 16), 32, innerKTiles / 2}, codes.options());
    check_status(ao_pack_tinygemm_int4(codes.data_ptr<int32_t>(), N, K, (int)innerKTiles, out.data_ptr<int32_t>(),
                                       at::cuda::getCurrentCUDAStream().stream()),
                 "_convert_weight_to_int4pack");
    return out;
}

}  // namespace

TORCH_LIBRARY_FRAGMENT(torchao, m) {
    m.impl_abstract_pystub("ao_b200._torch_ops");   // where the fake implementations are registered
    m.def("quant_llm_linear(int EXPONENT, int MANTISSA, Tensor _in_feats, Tensor _weights, Tensor _scales, int splitK) -> Tensor");
    m.def("_weight_int4pack_mm(Tensor x, Tensor w, int qGroupSize, Tensor qScaleAndZeros) -> Tensor");
    m.def("_convert_weight_to_int4pack(Tensor int_data, int innerKTiles) -> Tensor");
}

TORCH_LIBRARY_IMPL(torchao, CUDA, m) {
    m.impl("torchao::quant_llm_linear", &quant_llm_linear_cuda);
    m.impl("torchao::_weight_int4pack_mm", &weight_int4pack_mm_cuda);
    m.impl("torchao::_convert_weight_to_int4pack", &convert_weight_to_int4pack_cuda);
}
