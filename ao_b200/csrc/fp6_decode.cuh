// 6-bit float codes (e3m2, e2m3) of the tensor-core pre-packed layout -> fp16 bit patterns, shared by the decode and
// the prefill kernels.  Sign, exponent and mantissa bits are moved into fp16's fields; the exponent bias (15
// instead of the format's) leaves a power-of-two factor for the epilogue.
#pragma once
#include "ptx.cuh"

namespace ao {
namespace fp6 {

// Constants of a 6-bit format whose code splits into a 2-bit piece (sign + top exponent bit) and a 4-bit piece:
//   e3m2 (s eee mm): sign -> bit 15, e2 -> bit 12, (e1 e0 m1 m0) -> bits 11..8;   value = fp16 * 2^12
//   e2m3 (s ee mmm): sign -> bit 15, e1 -> bit 11, (e0 m2 m1 m0) -> bits 10..7;   value = fp16 * 2^14
struct Format {
    uint32_t m4, mh;          // where the 4-bit piece / the two top bits land (both halves)
    uint32_t k_hi, k_lo;      // multipliers that move the 2-bit field from bits 7..6 / 5..4 to its two places
    uint32_t sr0, sl1, sr2, sl3;   // shifts that move the four nibbles of the 4-bit word under m4
    float post_scale;         // 2^(15 - bias)
};
constexpr uint32_t kFieldHi = 0x00C000C0u, kFieldLo = 0x00300030u;

__host__ __device__ constexpr Format format_e3m2() {
    return Format{0x0F000F00u, 0x90009000u, 0x140u, 0x500u, 4u, 4u, 0u, 8u, 4096.f};
}
__host__ __device__ constexpr Format format_e2m3() {
    return Format{0x07800780u, 0x88008800u, 0x120u, 0x480u, 5u, 3u, 1u, 7u, 16384.f};
}

// The four A-fragment registers (m16n8k16: rows e / e + 8, columns 2c.. / 2c + 8..) of one 16-row fragment.
//   w4: the lane's word of the 4-bit plane; t: the lane's word of the 2-bit plane with this fragment's fields in
//   bits 7..4 of every byte.  The format's constants are passed as values so that they can live in registers.
__device__ __forceinline__ void decode_fragment(uint32_t w4, uint32_t t, const Format& F, uint32_t (&a)[4]) {
    const uint32_t v = t >> 8;  // bytes 1, 3 (row e) moved to the place of bytes 0, 2 (row e + 8)
    a[0] = ptx::and_or((v & kFieldHi) * F.k_hi, F.mh, (w4 >> F.sr0) & F.m4);   // row e,     cols 2c, 2c+1
    a[1] = ptx::and_or((t & kFieldHi) * F.k_hi, F.mh, (w4 << F.sl1) & F.m4);   // row e + 8, cols 2c, 2c+1
    a[2] = ptx::and_or((v & kFieldLo) * F.k_lo, F.mh, (w4 >> F.sr2) & F.m4);   // row e,     cols 2c+8, 2c+9
    a[3] = ptx::and_or((t & kFieldLo) * F.k_lo, F.mh, (w4 << F.sl3) & F.m4);   // row e + 8, cols 2c+8, 2c+9
}

}  // namespace fp6
}  // namespace ao
