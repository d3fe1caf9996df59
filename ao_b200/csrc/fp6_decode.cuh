// FP6 (e3m2) codes of the tensor-core pre-packed layout -> fp16 bit patterns, shared by the decode and the prefill
// kernels.  The result is the code's value divided by 2^12: sign, exponent and mantissa bits are moved into
// fp16's fields (exponent bias 15 instead of 3), which leaves a factor 2^(15-3) for the epilogue.
#pragma once
#include "ptx.cuh"

namespace ao {
namespace fp6 {

// The four A-fragment registers (m16n8k16: rows e / e + 8, columns 2c.. / 2c + 8..) of one 16-row fragment.
//   w4: the lane's word of the 4-bit plane; t: the lane's word of the 2-bit plane with this fragment's fields in
//   bits 7..4 of every byte.  m4 = 0x0F000F00, mh = 0x90009000, f_hi = 0x00C000C0, f_lo = 0x00300030,
//   k_hi = 0x140, k_lo = 0x500 (passed as values so that they can live in registers).
__device__ __forceinline__ void decode_fragment(uint32_t w4, uint32_t t, uint32_t m4, uint32_t mh, uint32_t f_hi,
                                                uint32_t f_lo, uint32_t k_hi, uint32_t k_lo, uint32_t (&a)[4]) {
    const uint32_t v = t >> 8;  // bytes 1, 3 (row e) moved to the place of bytes 0, 2 (row e + 8)
    // sign -> bit 15, top exponent bit -> bit 12 (both halves), low four bits -> bits 11..8
    a[0] = ptx::and_or((v & f_hi) * k_hi, mh, (w4 >> 4) & m4);   // row e,     cols 2c, 2c+1
    a[1] = ptx::and_or((t & f_hi) * k_hi, mh, (w4 << 4) & m4);   // row e + 8, cols 2c, 2c+1
    a[2] = ptx::and_or((v & f_lo) * k_lo, mh, w4 & m4);          // row e,     cols 2c+8, 2c+9
    a[3] = ptx::and_or((t & f_lo) * k_lo, mh, (w4 << 8) & m4);   // row e + 8, cols 2c+8, 2c+9
}

}  // namespace fp6
}  // namespace ao
