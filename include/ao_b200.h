/*
 * ao_b200 — C ABI of the B200 (sm_100a) weight-only quantized-linear path.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream, enqueues
 * its kernels on that stream and returns a status code.  Nothing here allocates,
 * synchronises or throws; the caller owns every buffer, including workspaces whose
 * size comes from the matching *_workspace_bytes query.  Calls are thread-safe as
 * long as concurrent calls use distinct output / workspace buffers.
 *
 * Each declaration cites the reference (torchao 0.3.1) interface it stands in for,
 * by the file's path inside the reference project.
 */
#ifndef AO_B200_H
#define AO_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* CUDA stream handle (cudaStream_t) passed as an opaque pointer. */
typedef void* ao_stream_t;

/* status codes */
enum {
    AO_OK = 0,
    AO_ERR_SHAPE = 1,       /* a size / divisibility requirement is not met          */
    AO_ERR_ALIGN = 2,       /* a pointer is not aligned as the kernel requires        */
    AO_ERR_DTYPE = 3,       /* unsupported dtype code or dtype combination            */
    AO_ERR_LAUNCH = 4,      /* the CUDA runtime rejected a launch (see cudaGetLastError) */
    AO_ERR_TIMEOUT = 5,     /* a bounded device-side wait ran out                     */
    AO_ERR_UNSUPPORTED = 6, /* valid request that this build has no kernel for        */
    AO_ERR_WORKSPACE = 7,   /* workspace missing or too small                         */
    AO_ERR_ARG = 8          /* an argument the reference would reject (ValueError)    */
};

/* dtype codes */
enum { AO_F32 = 0, AO_F16 = 1, AO_BF16 = 2, AO_I32 = 3, AO_I64 = 4, AO_I8 = 5, AO_U8 = 6, AO_I16 = 7 };

/* MappingType / ZeroPointDomain (torchao/quantization/quant_primitives.py:24-47) */
enum { AO_MAP_SYMMETRIC = 0, AO_MAP_ASYMMETRIC = 1 };
enum { AO_ZP_INT = 0, AO_ZP_FLOAT = 1 };

#define AO_MAX_DIMS 8

const char* ao_status_string(int status);
int ao_abi_version(void);

/* ------------------------------------------------------------------------------------------
 * Affine quantization primitives.  Tensors are contiguous, described by `ndim` sizes and a
 * block_size of the same rank (block[i] divides sizes[i]); scale / zero_point hold one value
 * per block in the row-major order of (sizes[i] / block[i]).
 * ---------------------------------------------------------------------------------------- */

/* choose_qparams_affine — torchao/quantization/quant_primitives.py:278-367.
 * Returns AO_ERR_ARG for the combinations the reference raises on (symmetric without
 * preserve_zero, symmetric with a FLOAT zero point, asymmetric non-preserving INT domain). */
int ao_choose_qparams_affine(const void* input, int input_dtype, int ndim, const int64_t* sizes,
                             const int64_t* block_size, int mapping_type, int64_t quant_min,
                             int64_t quant_max, int has_eps, double eps, int scale_dtype,
                             int zero_point_dtype, int preserve_zero, int zero_point_domain,
                             void* scale_out, void* zero_point_out, ao_stream_t stream);

/* quantize_affine — torchao/quantization/quant_primitives.py:134-206. */
int ao_quantize_affine(const void* input, int input_dtype, int ndim, const int64_t* sizes,
                       const int64_t* block_size, const void* scale, int scale_dtype,
                       const void* zero_point, int zero_point_dtype, int64_t quant_min,
                       int64_t quant_max, int zero_point_domain, void* out, int out_dtype,
                       ao_stream_t stream);

/* dequantize_affine — torchao/quantization/quant_primitives.py:208-276.
 * zero_point may be NULL. */
int ao_dequantize_affine(const void* input, int input_dtype, int ndim, const int64_t* sizes,
                         const int64_t* block_size, const void* scale, int scale_dtype,
                         const void* zero_point, int zero_point_dtype, int64_t quant_min,
                         int64_t quant_max, int zero_point_domain, void* out, int out_dtype,
                         ao_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * int4 weight-only fast path (asymmetric uint4, groups of `group` along K, bf16 scale and
 * float zero point) — what int4_weight_only() configures,
 * torchao/quantization/quant_api.py:362-387 and
 * AffineQuantizedTensor.from_float, torchao/dtypes/affine_quantized_tensor.py:184-229.
 * ---------------------------------------------------------------------------------------- */

/* One pass over W bf16 [N][K]: per-group scale / zero (bf16 [N][K/group]) and codes.
 * Any of scale_out, zero_out, codes_i32_out (int32 [N][K]), codes_u8_out (uint8 [N][K]) may be
 * NULL.  group in {32, 64, 128, 256}, K % group == 0, W 16-byte aligned.
 * Replaces choose_qparams_affine + quantize_affine as called at
 * affine_quantized_tensor.py:212-213 with the int4_weight_only parameter set. */
int ao_int4_groupwise_quantize(const void* w_bf16, int64_t N, int64_t K, int group, void* scale_out,
                               void* zero_out, int32_t* codes_i32_out, uint8_t* codes_u8_out,
                               ao_stream_t stream);

/* W bf16 [N][K] -> tensor_core_tiled weight int32 [N/8][K/(ikt*16)][32][ikt/2] and
 * scale_and_zero bf16 [K/group][N][2] in one pass (no int32 codes are materialised).
 * N % 8 == 0, K % (ikt*16) == 0, K % group == 0, group in {32,64,128,256}.
 * Replaces from_float + TensorCoreTiledAQTLayout.from_plain,
 * affine_quantized_tensor.py:212-213, 460-465. */
int ao_int4_quantize_pack_tinygemm(const void* w_bf16, int64_t N, int64_t K, int group,
                                   int inner_k_tiles, int32_t* packed_out, void* scale_and_zero_out,
                                   ao_stream_t stream);

/* aten::_convert_weight_to_int4pack as the reference calls it (int32 codes [N][K]),
 * affine_quantized_tensor.py:461.  out: int32 [N/8][K/(ikt*16)][32][ikt/2]. */
int ao_pack_tinygemm_int4(const int32_t* codes, int64_t N, int64_t K, int inner_k_tiles,
                          int32_t* packed_out, ao_stream_t stream);

/* Inverse of the above: what TensorCoreTiledAQTLayout.get_plain needs,
 * affine_quantized_tensor.py:509-537. */
int ao_unpack_tinygemm_int4(const int32_t* packed, int64_t N, int64_t K, int inner_k_tiles,
                            int32_t* codes_out, ao_stream_t stream);

/* pack_tinygemm_scales_and_zeros / unpack — torchao/quantization/utils.py:310-328.
 * scale, zero: bf16 [N][G]; scale_and_zero: bf16 [G][N][2]. */
int ao_pack_tinygemm_scales_and_zeros(const void* scale, const void* zero, int64_t N, int64_t G,
                                      void* scale_and_zero_out, ao_stream_t stream);
int ao_unpack_tinygemm_scales_and_zeros(const void* scale_and_zero, int64_t N, int64_t G,
                                        void* scale_out, void* zero_out, ao_stream_t stream);

/* pack_2xint4 — torchao/prototype/hqq/mixed_mm.py:13-33.  t: uint8 [R][C] -> uint8 [R/2][C],
 * row 2r in the low nibble, row 2r+1 in the high nibble. */
int ao_pack_2xint4(const uint8_t* t, int64_t R, int64_t C, uint8_t* out, ao_stream_t stream);

/* Codes uint8 [N][K] (one per byte, row-major) -> the HQQ operand layout uint8 [K/2][N]
 * (pack_2xint4 applied to the transpose, as test/hqq/test_triton_mm.py:100-106 prepares it). */
int ao_pack_hqq_int4_from_rowmajor(const uint8_t* codes, int64_t N, int64_t K, uint8_t* out,
                                   ao_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * FPx (e3m2 and friends) codec and the FP6 tensor-core pre-packed layout.
 * ---------------------------------------------------------------------------------------- */

/* _f32_to_fpx_unpacked / _fpx_unpacked_to_f32 — torchao/prototype/custom_fp_utils.py:27-140, 145-229 */
int ao_f32_to_fpx_unpacked(const float* x, int64_t n, int ebits, int mbits, uint8_t* out,
                           ao_stream_t stream);
int ao_fpx_unpacked_to_f32(const uint8_t* codes, int64_t n, int ebits, int mbits, float* out,
                           ao_stream_t stream);

/* pack_tc_fpx(codes, 6) / unpack_tc_fpx(packed, 6) — torchao/prototype/quant_llm/quant_llm.py:90-113,
 * 172-200.  codes: uint8 [M][N] (low 6 bits used); packed: uint8 [M][N*6/8]. */
int ao_pack_tc_fp6(const uint8_t* codes, int64_t M, int64_t N, uint8_t* packed_out, ao_stream_t stream);
int ao_unpack_tc_fp6(const uint8_t* packed, int64_t M, int64_t N, uint8_t* codes_out, ao_stream_t stream);

/* to_scaled_tc_fpx(w, 3, 2) — quant_llm.py:116-130: per-row absmax/28 scale (fp16 out),
 * e3m2 encode, pre-pack.  w dtype F32 / F16 / BF16, [M][N]. */
int ao_to_scaled_tc_fp6(const void* w, int w_dtype, int64_t M, int64_t N, uint8_t* packed_out,
                        void* scale_f16_out, ao_stream_t stream);

/* from_scaled_tc_fpx(packed, 3, 2, scale) — quant_llm.py:203-208.  scale_f16 may be NULL. */
int ao_from_scaled_tc_fp6(const uint8_t* packed, int64_t M, int64_t N, const void* scale_f16,
                          float* out, ao_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Mixed-precision linears.
 * ---------------------------------------------------------------------------------------- */

/* aten::_weight_int4pack_mm as the reference calls it — affine_quantized_tensor.py:631.
 * x bf16 [M][K] (row stride x_row_stride elements; columns >= x_cols are read as zero, which
 * stands in for the reference's per-call zero padding of the activation to the padded K,
 * affine_quantized_tensor.py:625-627), packed int32 tensor_core_tiled (inner_k_tiles 8/4/2),
 * scale_and_zero bf16 [K/group][N][2] -> y bf16 [M][N] contiguous.
 * A single row and the smallest batches run the HBM-bound GEMV kernel; M >= 5 (M >= 2 when K >= 2 N) the tcgen05
 * kernels (inner_k_tiles 8, N >= 128, 16-byte aligned activation rows), anything else is processed in row blocks of 16
 * by the GEMV kernel.  The two kernels add their fp32 sums in different orders: results agree within the tolerance of
 * the operator, not bit for bit; ao_int4_gemv is the GEMV alone.
 *
 * Workspace: ao_int4_tinygemm_linear_workspace_bytes(...) bytes, 256-byte aligned.  It holds a
 * status word (int at offset 0: AO_OK, or the code of a device-side failure such as a copy
 * that never completed), the number of K-slab launches so far (bytes 16..23; it tags the partial
 * sums that CTAs hand to one another), split-K completion counters and partial-sum slots.  It must
 * be zero-filled once before its first use; every call that completes leaves it ready for the
 * next one; after a non-zero status word it must be zero-filled again.  Calls that may overlap on
 * the GPU need workspaces of their own. */
size_t ao_int4_tinygemm_linear_workspace_bytes(int64_t M, int64_t N, int64_t K, int group,
                                               int inner_k_tiles);
int ao_int4_tinygemm_linear(const void* x_bf16, int64_t x_row_stride, int64_t x_cols,
                            const int32_t* packed, const void* scale_and_zero, int64_t M, int64_t N,
                            int64_t K, int group, int inner_k_tiles, void* y_bf16, void* workspace,
                            size_t workspace_bytes, ao_stream_t stream);

/* The same with the bias add of the linear fused into the kernels' stores (affine_quantized_tensor.py:638-640 adds it
 * as a separate pass).  bias_bf16: bf16 [N] or NULL.  The result has the bits of the unfused sequence: the linear's
 * output rounded to bf16, the bias added in fp32, rounded to bf16 again. */
int ao_int4_tinygemm_linear_bias(const void* x_bf16, int64_t x_row_stride, int64_t x_cols,
                                 const int32_t* packed, const void* scale_and_zero, int64_t M, int64_t N,
                                 int64_t K, int group, int inner_k_tiles, void* y_bf16, const void* bias_bf16,
                                 void* workspace, size_t workspace_bytes, ao_stream_t stream);
int ao_int4_gemv_bias(const void* x_bf16, int64_t x_row_stride, int64_t x_cols, const int32_t* packed,
                      const void* scale_and_zero, int64_t M, int64_t N, int64_t K, int group, int inner_k_tiles,
                      void* y_bf16, const void* bias_bf16, void* workspace, size_t workspace_bytes,
                      ao_stream_t stream);

/* The GEMV kernel alone (1 <= M <= 16), same arguments and workspace rules. */
size_t ao_int4_gemv_workspace_bytes(int64_t M, int64_t N, int64_t K, int group, int inner_k_tiles);
int ao_int4_gemv(const void* x_bf16, int64_t x_row_stride, int64_t x_cols, const int32_t* packed,
                 const void* scale_and_zero, int64_t M, int64_t N, int64_t K, int group,
                 int inner_k_tiles, void* y_bf16, void* workspace, size_t workspace_bytes,
                 ao_stream_t stream);

/* Output all-gather of row-sharded decode linears over peer memory (no counterpart in the reference, which has no
 * multi-GPU path for this operator).  Rank `rank` of `nranks` holds N rows of each weight and computes y_r [M][N];
 * every rank ends up with y_gathered [nranks][M][N].  Rows cross NVLink as 8-byte words {two bf16 rows, call number}
 * - data and arrival in one store, no fence - into a landing area in the receiver's memory.
 *
 * ao_gather_exchange: for up to 8 call sites (layers) in one small kernel: with push != 0 it first stores this
 *   rank's own block of each site's y_gathered (e.g. written there by ao_int4_gemv with y_bf16 = y_gathered +
 *   rank * M * N) into every peer's landing area; then it polls the words of each site's landing buffer until they
 *   carry the call's number (bounded: at most 0.2 s, then AO_ERR_TIMEOUT in the status word at workspace[0]) and
 *   writes the peers' blocks of y_gathered.  When it completes, the gathered outputs are complete on this GPU.
 * ao_int4_gemv_push: the GEMV whose CTAs send their rows themselves, as they finish, and write this rank's own block
 *   of y_gathered; it does not wait for the peers.  Follow it with ao_gather_exchange(push = 0).  (A kernel's
 *   completion waits for the acknowledgement of its NVLink writes - about 2.5 us on an NVSwitch node - so in a chain
 *   of dependent microsecond kernels one exchange per step is cheaper than a push per layer; the fused push pays
 *   when other work follows the GEMV that does not need its completion.)
 * ao_int4_gemv_gather: ao_int4_gemv_push + ao_gather_exchange(push = 0) for one call site.
 *
 * Per call site (one per sharded layer and batch size; ao_gather_exchange takes 1 <= M <= 64, the GEMV forms M <= 8), the
 * same on every rank:
 *   peer_landing[r]  rank r's landing area of the site: 2 * nranks * M * N / 2 words of 8 bytes (two buffers, used
 *                    alternately by the parity of the call number), zero before the first call; the entry of `rank`
 *                    is this rank's own area.  ao_gather_exchange takes nsites * nranks pointers, site-major
 *   y_gathered       this rank's output, bf16 [nranks][M][N], 16-byte aligned; overwritten by the site's next call
 *   site_state       this rank's unsigned[4] {pushed CTAs, pushes so far, CTAs done waiting, waits so far}, zero
 *                    before the first call, 16-byte aligned
 * Every rank must issue the same sequence of calls with the same shapes, and each push of a site must be followed by
 * its wait before the site's next push (the wait may come later in the stream, after pushes of other sites).  The
 * GEMV push needs K small enough for the activations to fit in shared memory (otherwise AO_ERR_UNSUPPORTED).  The
 * current device must be the stream's device. */
int ao_gather_exchange(int nsites, void* const* peer_landing, void* const* y_gathered, void* const* state,
                       const int64_t* M, const int64_t* N, int nranks, int rank, int push, void* workspace,
                       ao_stream_t stream);
int ao_int4_gemv_push(const void* x_bf16, int64_t x_row_stride, int64_t x_cols, const int32_t* packed,
                      const void* scale_and_zero, int64_t M, int64_t N, int64_t K, int group, int inner_k_tiles,
                      int nranks, int rank, void* const* peer_landing, void* y_gathered, void* site_state,
                      void* workspace, size_t workspace_bytes, ao_stream_t stream);
int ao_int4_gemv_gather(const void* x_bf16, int64_t x_row_stride, int64_t x_cols, const int32_t* packed,
                        const void* scale_and_zero, int64_t M, int64_t N, int64_t K, int group,
                        int inner_k_tiles, int nranks, int rank, void* const* peer_landing,
                        void* y_gathered, void* site_state, void* workspace, size_t workspace_bytes,
                        ao_stream_t stream);

/* Set-up helpers for the exchange (CUDA IPC): export the 64-byte handle of the allocation that contains ptr and
 * ptr's offset in it; map another process's allocation; unmap it.  Not for the hot path. */
int ao_comm_export(const void* ptr, void* handle_out, int64_t* offset_out);
int ao_comm_import(const void* handle, void** base_out);
int ao_comm_close(void* base);

/* The same GEMV without a workspace argument.  This entry point has no counterpart in the reference.
 * It is for callers that cannot pass scratch memory and must not allocate (a fixed operator signature,
 * a C serving loop without a device allocator): the scratch is a device array inside the library, one per
 * GPU, of ao_int4_gemv_static_scratch_max_bytes() bytes (2 MiB).  Nothing is allocated by the call.
 *  - The first call on a device performs a one-time set-up (address look-up of the array); make it
 *    during start-up, before any stream capture.
 *  - A shape whose ao_int4_gemv_workspace_bytes() exceeds the maximum returns AO_ERR_WORKSPACE.
 *  - All calls on a device share the array; the call clears the part that has to start at zero on
 *    `stream` itself (and keeps the launch counter that tags split-K partial sums growing across calls), but
 *    calls that overlap on the GPU race on it: serialise them, or use ao_int4_gemv.
 *  - The array of the device that is current at the call is used: `stream` must belong to that device. */
size_t ao_int4_gemv_static_scratch_max_bytes(void);
int ao_int4_gemv_static_scratch(const void* x_bf16, int64_t x_row_stride, int64_t x_cols,
                                const int32_t* packed, const void* scale_and_zero, int64_t M, int64_t N,
                                int64_t K, int group, int inner_k_tiles, void* y_bf16, ao_stream_t stream);

/* hqq_quants_to_torch_quants — torchao/prototype/hqq/hqq_tinygemm_linear.py:173-208 (4 bits).  HQQ codes wq uint8
 * [groups][group_size] with scale / zero per group (dtype = AO_BF16, AO_F16 or AO_F32: the reference's compute dtype)
 * -> int32 codes of the tinygemm convention and new_zeros = scale * 8 - zero * scale; the scales are unchanged.
 * Every operation is rounded to the dtype like the reference's tensor expressions. */
int ao_hqq_quants_to_tinygemm(const uint8_t* wq, const void* scales, const void* zeros, int dtype,
                              int64_t groups, int group_size, int32_t* q_out, void* new_zeros_out,
                              ao_stream_t stream);

/* triton_mixed_mm(a, b, scales, zeros, group_size) — torchao/prototype/hqq/mixed_mm.py:36-173 with the kernel
 * torchao/prototype/hqq/kernels.py:162-387 (non-transposed form): c[M][N] = a[M][K] @ ((q - zeros) * scales)[K][N].
 * a: bf16 or fp16 (a_dtype = AO_BF16 / AO_F16) [M][K], row stride a_row_stride elements; b_packed uint8 [K/2][N]
 * as produced by ao_pack_2xint4 on the [K][N] codes; scales, zeros [K/group][N] contiguous in a's dtype;
 * c [M][N] contiguous in a's dtype.  N % 16 == 0, N >= 128, K % 128 == 0, group in {32, 64, 128, 256}, any M >= 1.
 * Runs on the tcgen05 tensor cores (fp32 accumulate).  Workspace rules as for ao_int4_tinygemm_linear. */
size_t ao_hqq_int4_linear_workspace_bytes(int64_t M, int64_t N, int64_t K, int group);
int ao_hqq_int4_linear(const void* a, int a_dtype, int64_t a_row_stride, const uint8_t* b_packed,
                       const void* scales, const void* zeros, int64_t M, int64_t N, int64_t K, int group,
                       void* c, void* workspace, size_t workspace_bytes, ao_stream_t stream);

/* The transposed form of triton_mixed_mm (transposed=True, used for the backward pass): c[M][K] = a[M][N] @ W[N][K]
 * with the same b_packed [K/2][N], scales and zeros [K/group][N]; the reduction runs along N.  N % 128 == 0,
 * K >= 128, K % group == 0. */
size_t ao_hqq_int4_linear_transposed_workspace_bytes(int64_t M, int64_t N, int64_t K, int group);
int ao_hqq_int4_linear_transposed(const void* a, int a_dtype, int64_t a_row_stride, const uint8_t* b_packed,
                                  const void* scales, const void* zeros, int64_t M, int64_t N, int64_t K,
                                  int group, void* c, void* workspace, size_t workspace_bytes,
                                  ao_stream_t stream);

/* pack_tc_fpx / unpack_tc_fpx for 5- and 6-bit codes (quant_llm.py:60-113, 134-200): a 5-bit code is split into a
 * 1-bit and a 4-bit plane, a 6-bit code into a 2-bit and a 4-bit plane.  packed: uint8 [M][N * nbits / 8]. */
int ao_pack_tc_fpx(const uint8_t* codes, int64_t M, int64_t N, int nbits, uint8_t* packed_out, ao_stream_t stream);
int ao_unpack_tc_fpx(const uint8_t* packed, int64_t M, int64_t N, int nbits, uint8_t* codes_out, ao_stream_t stream);

/* The same two for the formats the reference's linear dispatches: (ebits, mbits) = (3, 2), (2, 3), (2, 2), (3, 1)
 * (to_scaled_tc_fpx / from_scaled_tc_fpx, quant_llm.py:116-130, 203-208; the bit packing is format-independent).
 * With a workspace of at least M * 4 bytes (no initialisation needed) the work runs as two well-parallel kernels;
 * workspace may be NULL. */
int ao_to_scaled_tc_fpx(const void* w, int w_dtype, int64_t M, int64_t N, int ebits, int mbits,
                        uint8_t* packed_out, void* scale_f16_out, void* workspace, size_t workspace_bytes,
                        ao_stream_t stream);
int ao_from_scaled_tc_fpx(const uint8_t* packed, int64_t M, int64_t N, int ebits, int mbits,
                          const void* scale_f16, float* out, ao_stream_t stream);

/* torchao::quant_llm_linear(3, 2, x, w, s, splitK) — torchao/ops.py:15-37, schema
 * torchao/csrc/fp6_llm.cpp:5-8, CUDA entry torchao/csrc/cuda/fp6_llm/fp6_linear.cu:139-196.
 * x fp16 [M][K] (row stride x_row_stride), packed uint8 [N][K*6/8] as produced by
 * ao_pack_tc_fp6 / ao_to_scaled_tc_fp6, scale fp16 [N] -> y fp16 [M][N].  N % 64 == 0,
 * K % 64 == 0.  The K split is chosen by the kernel (the reference's splitK argument has no
 * counterpart).  Workspace rules as for ao_int4_tinygemm_linear. */
size_t ao_fp6_linear_workspace_bytes(int64_t M, int64_t N, int64_t K);
int ao_fp6_linear(const void* x_f16, int64_t x_row_stride, const uint8_t* packed, const void* scale_f16,
                  int64_t M, int64_t N, int64_t K, void* y_f16, void* workspace,
                  size_t workspace_bytes, ao_stream_t stream);

/* torchao::quant_llm_linear(EXPONENT, MANTISSA, ...) — the dispatch of
 * torchao/csrc/cuda/fp6_llm/fp6_linear.cu:175-193: (3, 2), (2, 3) (6 bits), (2, 2), (3, 1) (5 bits); anything else
 * returns AO_ERR_UNSUPPORTED.  packed: uint8 [N][K * nbits / 8].  Same arguments and workspace
 * (ao_fp6_linear_workspace_bytes) as ao_fp6_linear. */
int ao_fpx_linear(int ebits, int mbits, const void* x_f16, int64_t x_row_stride, const uint8_t* packed,
                  const void* scale_f16, int64_t M, int64_t N, int64_t K, void* y_f16, void* workspace,
                  size_t workspace_bytes, ao_stream_t stream);

/* ao_fpx_linear with the bias add of the reference's linear dispatch fused into the stores
 * (torchao/prototype/quant_llm/quant_llm.py:433-445: `out = quant_llm_linear(...); out += bias`): bias_f16 [N] fp16 or
 * NULL; y = round_f16(round_f16(x @ W^T) + bias), the bits the separate add gives. */
int ao_fpx_linear_bias(int ebits, int mbits, const void* x_f16, int64_t x_row_stride, const uint8_t* packed,
                       const void* scale_f16, const void* bias_f16, int64_t M, int64_t N, int64_t K, void* y_f16,
                       void* workspace, size_t workspace_bytes, ao_stream_t stream);

/* The decode kernel alone (1 <= M <= 16). */
size_t ao_fp6_gemv_workspace_bytes(int64_t M, int64_t N, int64_t K);
int ao_fp6_gemv(const void* x_f16, int64_t x_row_stride, const uint8_t* packed, const void* scale_f16,
                int64_t M, int64_t N, int64_t K, void* y_f16, void* workspace, size_t workspace_bytes,
                ao_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* AO_B200_H */
