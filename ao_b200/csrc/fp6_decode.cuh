// 5- and 6-bit float codes (e3m2, e2m3, e2m2, e3m1) of the tensor-core pre-packed layout -> fp16 bit patterns, shared by the decode and
// the prefill kernels.  Sign, exponent and mantissa bits are moved into fp16's fields; the exponent bias (15
// instead of the format's) leaves a power-of-two factor for the epilogue.
#pragma once
#include "ptx.cuh"

namespace ao {
namespace fp6 {

// Constants of a format.  6-bit codes split into a 2-bit piece (sign + top exponent bit) and a 4-bit piece, 5-bit
// codes into the sign bit and a 4-bit piece:
//   e3m2 (s eee mm): sign -> bit 15, e2 -> bit 12, (e1 e0 m1 m0) -> bits 11..8;   value = fp16 * 2^12
//   e2m3 (s ee mmm): sign -> bit 15, e1 -> bit 11, (e0 m2 m1 m0) -> bits 10..7;   value = fp16 * 2^14
//   e2m2 (s ee mm):  sign -> bit 15, (e1 e0 m1 m0) -> bits 11..8;                 value = fp16 * 2^14
//   e3m1 (s eee m):  sign -> bit 15, (e2 e1 e0 m0) -> bits 12..9;                 value = fp16 * 2^12
struct Format {
    uint32_t m4, mh;          // where the 4-bit piece / the two top bits (6-bit codes) land, both halves
    uint32_t k_hi, k_lo;      // 6-bit codes: multipliers that move the 2-bit field from bits 7..6 / 5..4 to its places
    uint32_t rot[4];          // left rotations that bring the four nibbles of the 4-bit word under m4
    float post_scale;         // 2^(15 - bias)
    int nbits;
};
constexpr uint32_t kFieldHi = 0x00C000C0u, kFieldLo = 0x00300030u;

enum { kE3M2 = 0, kE2M3 = 1, kE2M2 = 2, kE3M1 = 3 };

__host__ __device__ constexpr Format make_format(int id) {
    return id == kE3M2   ? Format{0x0F000F00u, 0x90009000u, 0x140u, 0x500u, {28u, 4u, 0u, 8u}, 4096.f, 6}
           : id == kE2M3 ? Format{0x07800780u, 0x88008800u, 0x120u, 0x480u, {27u, 3u, 31u, 7u}, 16384.f, 6}
           : id == kE2M2 ? Format{0x0F000F00u, 0u, 0u, 0u, {28u, 4u, 0u, 8u}, 16384.f, 5}
                         : Format{0x1E001E00u, 0u, 0u, 0u, {29u, 5u, 1u, 9u}, 4096.f, 5};
}

// (ebits, mbits) -> format id, or -1
__host__ __device__ constexpr int format_id(int ebits, int mbits) {
    return (ebits == 3 && mbits == 2) ? kE3M2 : (ebits == 2 && mbits == 3) ? kE2M3 : (ebits == 2 && mbits == 2) ? kE2M2
           : (ebits == 3 && mbits == 1) ? kE3M1 : -1;
}

__device__ __forceinline__ uint32_t rotl(uint32_t v, uint32_t r) { return __funnelshift_l(v, v, r); }

// The four A-fragment registers (m16n8k16: rows e / e + 8, columns 2c.. / 2c + 8..) of one 16-row fragment of a
// 6-bit format.  w4: the lane's word of the 4-bit plane; t: the lane's word of the 2-bit plane with this fragment's
// fields in bits 7..4 of every byte.  The format's constants are passed as values so that they can live in registers.
__device__ __forceinline__ void decode_fragment(uint32_t w4, uint32_t t, const Format& F, uint32_t (&a)[4]) {
    const uint32_t v = t >> 8;  // bytes 1, 3 (row e) moved to the place of bytes 0, 2 (row e + 8)
    a[0] = ptx::and_or((v & kFieldHi) * F.k_hi, F.mh, rotl(w4, F.rot[0]) & F.m4);   // row e,     cols 2c, 2c+1
    a[1] = ptx::and_or((t & kFieldHi) * F.k_hi, F.mh, rotl(w4, F.rot[1]) & F.m4);   // row e + 8, cols 2c, 2c+1
    a[2] = ptx::and_or((v & kFieldLo) * F.k_lo, F.mh, rotl(w4, F.rot[2]) & F.m4);   // row e,     cols 2c+8, 2c+9
    a[3] = ptx::and_or((t & kFieldLo) * F.k_lo, F.mh, rotl(w4, F.rot[3]) & F.m4);   // row e + 8, cols 2c+8, 2c+9
}

// The same for a 5-bit format.  w1: the lane's word of the 1-bit plane (64 rows x one column pair x both k halves):
// the sign of fragment fr's row (c ? e + 8 : e), column half g, element hb sits at bit
// hb * 16 + (1 - c) * 8 + (3 - fr) * 2 + (1 - g), so one shift brings both elements' signs to bits 15 and 31.
__device__ __forceinline__ void decode_fragment5(uint32_t w4, uint32_t w1, int fr, const Format& F, uint32_t (&a)[4]) {
    const uint32_t sgn = 0x80008000u;
    a[0] = ptx::and_or(w1 << (2 * fr), sgn, rotl(w4, F.rot[0]) & F.m4);        // c = 0, g = 0
    a[1] = ptx::and_or(w1 << (8 + 2 * fr), sgn, rotl(w4, F.rot[1]) & F.m4);    // c = 1, g = 0
    a[2] = ptx::and_or(w1 << (2 * fr + 1), sgn, rotl(w4, F.rot[2]) & F.m4);    // c = 0, g = 1
    a[3] = ptx::and_or(w1 << (9 + 2 * fr), sgn, rotl(w4, F.rot[3]) & F.m4);    // c = 1, g = 1
}

}  // namespace fp6
}  // namespace ao
