/*
 * CPU oracle for the weight-only quantized-linear path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is a plain-C restatement of the
 * reference's (torchao 0.3.1) algorithms for the path; it is the checker for
 * the CUDA kernels and the timed CPU baseline.  Nothing in the product package
 * may import, link or call it.
 *
 * Conventions
 *  - Floating tensors travel as fp32 arrays whose values are exactly
 *    representable in their logical dtype (DT_F32 / DT_F16 / DT_BF16); every
 *    arithmetic step is evaluated in fp32 and then rounded to the dtype eager
 *    PyTorch would produce for that step ("compute in fp32, round to the result
 *    dtype"), which is what makes codes / scales / zero points bit-exact.
 *  - Blocks are rows: callers canonicalise an n-d block_size to [nblocks][block]
 *    (see oracle.py), so scale/zero_point are one value per row here.
 *
 * Reference citations (paths inside the reference project):
 *   torchao/quantization/quant_primitives.py:278-367  choose_qparams_affine
 *   torchao/quantization/quant_primitives.py:134-206  quantize_affine
 *   torchao/quantization/quant_primitives.py:208-276  dequantize_affine
 *   torchao/quantization/utils.py:310-323             pack_tinygemm_scales_and_zeros
 *   torchao/prototype/custom_fp_utils.py:27-140       _f32_to_fpx_unpacked
 *   torchao/prototype/custom_fp_utils.py:145-229      _fpx_unpacked_to_f32
 *   torchao/prototype/quant_llm/quant_llm.py:90-130   _pack_tc_fp6 / to_scaled_tc_fpx
 *   torchao/prototype/quant_llm/quant_llm.py:172-208  _unpack_tc_fp6 / from_scaled_tc_fpx
 *   torchao/prototype/hqq/mixed_mm.py:13-33           pack_2xint4
 *   torchao/dtypes/affine_quantized_tensor.py:460-465 tensor_core_tiled from_plain
 *     (calls aten::_convert_weight_to_int4pack, PyTorch ATen, pinned to the
 *      torch 2.11.0 build on the GPU box; its output layout is restated in
 *      orc_pack_tinygemm and pinned by a fixture generated with that op)
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

enum { DT_F32 = 0, DT_F16 = 1, DT_BF16 = 2, DT_I32 = 3, DT_I64 = 4, DT_I8 = 5, DT_U8 = 6, DT_I16 = 7 };
enum { MAP_SYMMETRIC = 0, MAP_ASYMMETRIC = 1 };
enum { ZP_INT = 0, ZP_FLOAT = 1 };

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* fp32 -> bf16 -> fp32, round to nearest even (NaN kept quiet) */
static inline float rbf16(float f) {
    uint32_t u = f2u(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return u2f(u | 0x00400000u);
    u += 0x7fffu + ((u >> 16) & 1u);
    return u2f(u & 0xffff0000u);
}

/* fp32 -> fp16 bits, round to nearest even */
static inline uint16_t f32_to_f16_bits(float f) {
    uint32_t x = f2u(f);
    uint32_t sign = (x >> 16) & 0x8000u;
    x &= 0x7fffffffu;
    if (x >= 0x7f800000u) return (uint16_t)(sign | (x > 0x7f800000u ? 0x7e00u : 0x7c00u));
    if (x >= 0x477ff000u) { /* >= 65520 rounds to inf */
        return (uint16_t)(sign | 0x7c00u);
    }
    if (x < 0x38800000u) { /* subnormal half or zero */
        double d = (double)u2f(x) * 16777216.0; /* in units of 2^-24, the fp16 subnormal step */
        double fl = floor(d);
        double diff = d - fl;
        uint32_t q = (uint32_t)fl;
        if (diff > 0.5 || (diff == 0.5 && (q & 1u))) q++;
        return (uint16_t)(sign | q);
    }
    uint32_t mant_odd = (x >> 13) & 1u;
    x += ((uint32_t)(15 - 127) << 23) + 0xfffu;
    x += mant_odd;
    return (uint16_t)(sign | (x >> 13));
}

static inline float f16_bits_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t e = (h >> 10) & 0x1fu, m = h & 0x3ffu;
    if (e == 0) {
        if (m == 0) return u2f(sign);
        float v = (float)m * 5.9604644775390625e-08f; /* 2^-24 */
        return sign ? -v : v;
    }
    if (e == 31) return u2f(sign | 0x7f800000u | (m << 13));
    return u2f(sign | ((e + 112u) << 23) | (m << 13));
}

static inline float rf16(float f) { return f16_bits_to_f32(f32_to_f16_bits(f)); }

static inline float rnd(int dt, float f) {
    if (dt == DT_BF16) return rbf16(f);
    if (dt == DT_F16) return rf16(f);
    return f;
}

static inline int promote(int a, int b) {
    if (a == b) return a;
    return DT_F32; /* f32 with anything, or f16 with bf16 */
}
static inline int is_float_dt(int dt) { return dt == DT_F32 || dt == DT_F16 || dt == DT_BF16; }

static inline float dt_eps(int dt) {
    if (dt == DT_BF16) return 0.0078125f;
    if (dt == DT_F16) return 0.0009765625f;
    return 1.1920928955078125e-07f;
}

/* conversion of a float that PyTorch would .to() an integer dtype: truncation */
static inline float to_int_like(int dt, float v) {
    if (is_float_dt(dt)) return rnd(dt, v);
    return truncf(v);
}

/* exported helpers so tests can pin the rounding primitives themselves */
float orc_round_bf16(float f) { return rbf16(f); }
float orc_round_f16(float f) { return rf16(f); }

/* ------------------------------------------------------------------ */
/* choose_qparams_affine — quant_primitives.py:278-367                 */
/* x: [nb][be] values of dtype in_dt.  scale_out/zp_out: [nb] values    */
/* of scale_dt / zp_dt (integers for an integer zp_dt).                 */
/* returns 0, or a negative code for the reference's ValueError cases. */
/* ------------------------------------------------------------------ */
int orc_choose_qparams(const float* x, int64_t nb, int64_t be, int in_dt, int mapping,
                       int64_t qmin, int64_t qmax, int has_eps, double eps_in, int scale_dt,
                       int zp_dt, int preserve_zero, int zp_domain, float* scale_out,
                       float* zp_out) {
    if (mapping == MAP_SYMMETRIC && !preserve_zero) return -1;                 /* :348-349 */
    if (mapping == MAP_SYMMETRIC && zp_domain != ZP_INT) return -2;            /* :350-351 */
    if (mapping == MAP_ASYMMETRIC && !preserve_zero && zp_domain != ZP_FLOAT) return -3; /* :359 */
    const float eps = rnd(in_dt, has_eps ? (float)eps_in : dt_eps(in_dt));     /* :363-365 */
    const float mid = (float)((double)(qmax + qmin + 1) / 2.0);
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < nb; ++b) {
        const float* r = x + b * be;
        float mn = r[0], mx = r[0];
        for (int64_t i = 1; i < be; ++i) {
            float v = r[i];
            mn = v < mn ? v : mn;
            mx = v > mx ? v : mx;
        }
        float mnn = mn, mxp = mx;
        if (preserve_zero) {                                                   /* :335-340 */
            mnn = mn < 0.f ? mn : 0.f;
            mxp = mx > 0.f ? mx : 0.f;
        }
        float scale, zp;
        if (mapping == MAP_SYMMETRIC) {                                        /* :345-352 */
            float a = -mnn;
            mxp = a > mxp ? a : mxp;
            float div = (float)((double)(qmax - qmin) / 2.0);
            scale = rnd(in_dt, mxp / div);
            zp = rnd(in_dt, (float)(int64_t)((double)(qmax + qmin + 1) / 2.0));
        } else {
            float d = rnd(in_dt, mxp - mnn);                                   /* :354 */
            scale = rnd(in_dt, d / (float)(qmax - qmin));
            if (preserve_zero) {                                               /* :355-357 */
                float q = rnd(in_dt, mnn / scale);
                q = nearbyintf(q);
                zp = rnd(in_dt, (float)qmin - q);
                zp = zp < (float)qmin ? (float)qmin : zp;
                zp = zp > (float)qmax ? (float)qmax : zp;
            } else {                                                           /* :359-361 */
                float sm = rnd(in_dt, scale * mid);
                zp = rnd(in_dt, mnn + sm);
            }
        }
        scale = scale < eps ? eps : scale;                                     /* :365 (NaN-free inputs) */
        scale_out[b] = rnd(scale_dt, scale);                                   /* :367 */
        zp_out[b] = to_int_like(zp_dt, zp);
    }
    return 0;
}

static inline float clampf(float v, float lo, float hi) { return v < lo ? lo : (v > hi ? hi : v); }

/* ------------------------------------------------------------------ */
/* quantize_affine — quant_primitives.py:134-206                       */
/* out: int32 codes [nb][be] (the caller narrows to the output dtype).  */
/* zp may be NULL only in the INT domain (treated as absent => error in */
/* the reference, so callers never pass NULL).                          */
/* ------------------------------------------------------------------ */
void orc_quantize(const float* x, int64_t nb, int64_t be, int in_dt, const float* scale,
                  int scale_dt, const float* zp, int zp_dt, int64_t qmin, int64_t qmax,
                  int zp_domain, int32_t* out) {
    const float mid = (float)((double)(qmax + qmin + 1) / 2.0);
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < nb; ++b) {
        const float* r = x + b * be;
        int32_t* o = out + b * be;
        const float s = scale[b];
        const float z = zp[b];
        if (zp_domain == ZP_INT) {                                             /* :191-194 */
            const float inv = rnd(scale_dt, 1.0f / s);
            const int p1 = promote(in_dt, scale_dt);
            const int p2 = is_float_dt(zp_dt) ? promote(p1, zp_dt) : p1;
            for (int64_t i = 0; i < be; ++i) {
                float v = rnd(p1, r[i] * inv);
                v = nearbyintf(v);
                v = rnd(p2, v + z);
                v = clampf(v, (float)qmin, (float)qmax);
                o[i] = (int32_t)v;
            }
        } else {                                                               /* :195-203 */
            const float sm = rnd(scale_dt, s * mid);
            const int pm = is_float_dt(zp_dt) ? promote(zp_dt, scale_dt) : scale_dt;
            const float minv = rnd(pm, z - sm);
            const int p3 = promote(in_dt, pm);
            const int p4 = promote(p3, scale_dt);
            for (int64_t i = 0; i < be; ++i) {
                float v = rnd(p3, r[i] - minv);
                v = rnd(p4, v / s);
                v = nearbyintf(v);
                v = clampf(v, (float)qmin, (float)qmax);
                o[i] = (int32_t)v;
            }
        }
    }
}

/* ------------------------------------------------------------------ */
/* dequantize_affine — quant_primitives.py:208-276                     */
/* q: int32 codes; zp: values of zp_dt, may be NULL.                    */
/* ------------------------------------------------------------------ */
void orc_dequantize(const int32_t* q, int64_t nb, int64_t be, const float* scale, int scale_dt,
                    const float* zp, int zp_dt, int64_t qmin, int64_t qmax, int zp_domain,
                    int out_dt, float* out) {
    (void)scale_dt; (void)zp_dt;
    const float mid = (float)((double)(qmax + qmin + 1) / 2.0);
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < nb; ++b) {
        const int32_t* r = q + b * be;
        float* o = out + b * be;
        const float s = scale[b];
        if (zp_domain == ZP_INT) {                                             /* :258-265 */
            const int32_t zi = zp ? (int32_t)zp[b] : 0;
            for (int64_t i = 0; i < be; ++i) {
                float v = rnd(out_dt, (float)(r[i] - zi));
                o[i] = rnd(out_dt, v * s);
            }
        } else {                                                               /* :266-274 */
            for (int64_t i = 0; i < be; ++i) {
                float v = rnd(out_dt, (float)r[i] - mid);
                v = rnd(out_dt, v * s);
                if (zp) v = rnd(out_dt, v + zp[b]);
                o[i] = v;
            }
        }
    }
}

/* ------------------------------------------------------------------ */
/* pack_tinygemm_scales_and_zeros — quantization/utils.py:310-323       */
/* scale, zero: [N][G] (uint16 bf16 bits) -> out [G][N][2]               */
/* ------------------------------------------------------------------ */
void orc_pack_scales_and_zeros(const uint16_t* scale, const uint16_t* zero, int64_t N, int64_t G,
                               uint16_t* out) {
    for (int64_t n = 0; n < N; ++n)
        for (int64_t g = 0; g < G; ++g) {
            out[(g * N + n) * 2 + 0] = scale[n * G + g];
            out[(g * N + n) * 2 + 1] = zero[n * G + g];
        }
}

/* ------------------------------------------------------------------ */
/* tensor_core_tiled weight layout (aten::_convert_weight_to_int4pack). */
/* codes: int32 [N][K], values 0..15.  out: int32                       */
/* [N/8][K/(ikt*16)][32][ikt/2].  One output word holds, for lane t of a */
/* warp (row n = tile*8 + t/4, c = t%4), the eight codes at k offsets    */
/* {2c, 2c+1, 2c+8, 2c+9} of two consecutive 16-wide k tiles A and B;    */
/* nibble order (lsb first): A[2c], A[2c+8], B[2c], B[2c+8],            */
/* A[2c+1], A[2c+9], B[2c+1], B[2c+9].                                   */
/* ------------------------------------------------------------------ */
int orc_pack_tinygemm(const int32_t* codes, int64_t N, int64_t K, int ikt, int32_t* out) {
    if (!(ikt == 2 || ikt == 4 || ikt == 8)) return -1;
    if (N % 8 || K % (ikt * 16)) return -2;
    const int64_t NT = N / 8, KO = K / (ikt * 16);
    for (int64_t nt = 0; nt < NT; ++nt)
        for (int64_t ko = 0; ko < KO; ++ko)
            for (int t = 0; t < 32; ++t)
                for (int j = 0; j < ikt / 2; ++j) {
                    const int64_t n = nt * 8 + t / 4;
                    const int c = t % 4;
                    const int64_t kA = (ko * ikt + 2 * j) * 16, kB = kA + 16;
                    const int32_t* r = codes + n * K;
                    uint32_t v0 = r[kA + 2 * c], v1 = r[kA + 2 * c + 1];
                    uint32_t v2 = r[kA + 2 * c + 8], v3 = r[kA + 2 * c + 9];
                    uint32_t v4 = r[kB + 2 * c], v5 = r[kB + 2 * c + 1];
                    uint32_t v6 = r[kB + 2 * c + 8], v7 = r[kB + 2 * c + 9];
                    uint32_t w = (v7 << 28) | (v5 << 24) | (v3 << 20) | (v1 << 16) | (v6 << 12) |
                                 (v4 << 8) | (v2 << 4) | v0;
                    out[((nt * KO + ko) * 32 + t) * (ikt / 2) + j] = (int32_t)w;
                }
    return 0;
}

int orc_unpack_tinygemm(const int32_t* packed, int64_t N, int64_t K, int ikt, int32_t* codes) {
    if (!(ikt == 2 || ikt == 4 || ikt == 8)) return -1;
    if (N % 8 || K % (ikt * 16)) return -2;
    const int64_t NT = N / 8, KO = K / (ikt * 16);
    for (int64_t nt = 0; nt < NT; ++nt)
        for (int64_t ko = 0; ko < KO; ++ko)
            for (int t = 0; t < 32; ++t)
                for (int j = 0; j < ikt / 2; ++j) {
                    const int64_t n = nt * 8 + t / 4;
                    const int c = t % 4;
                    const int64_t kA = (ko * ikt + 2 * j) * 16, kB = kA + 16;
                    int32_t* r = codes + n * K;
                    uint32_t w = (uint32_t)packed[((nt * KO + ko) * 32 + t) * (ikt / 2) + j];
                    r[kA + 2 * c] = w & 15;            r[kA + 2 * c + 8] = (w >> 4) & 15;
                    r[kB + 2 * c] = (w >> 8) & 15;     r[kB + 2 * c + 8] = (w >> 12) & 15;
                    r[kA + 2 * c + 1] = (w >> 16) & 15; r[kA + 2 * c + 9] = (w >> 20) & 15;
                    r[kB + 2 * c + 1] = (w >> 24) & 15; r[kB + 2 * c + 9] = (w >> 28) & 15;
                }
    return 0;
}

/* ------------------------------------------------------------------ */
/* pack_2xint4 — prototype/hqq/mixed_mm.py:13-33                        */
/* t: uint8 [R][C] (R even) -> out uint8 [R/2][C]; row 2r -> low nibble, */
/* row 2r+1 -> high nibble.  The HQQ path calls it on W_q.T ([K][N]).    */
/* ------------------------------------------------------------------ */
void orc_pack_2xint4(const uint8_t* t, int64_t R, int64_t C, uint8_t* out) {
    for (int64_t r = 0; r < R / 2; ++r)
        for (int64_t c = 0; c < C; ++c)
            out[r * C + c] = (uint8_t)((t[(2 * r) * C + c] & 0xF) | (t[(2 * r + 1) * C + c] << 4));
}

/* ------------------------------------------------------------------ */
/* fp32 <-> ExMy codec — prototype/custom_fp_utils.py:27-140, 145-229   */
/* ------------------------------------------------------------------ */
static inline uint8_t f32_to_fpx_one(float xf, int ebits, int mbits) {
    const int MB = 23, EB = 8, BIAS32 = 127;
    const int exp_bias = (1 << (ebits - 1)) - 1;
    const int max_int = (1 << (ebits + mbits)) - 1;
    const uint32_t sign_mask = 1u << (ebits + mbits);
    const uint32_t magic_adder = (1u << (MB - mbits - 1)) - 1;
    const float max_normal =
        ldexpf(1.0f, ((1 << ebits) - 1) - exp_bias) * ((float)((1 << (mbits + 1)) - 1) / (float)(1 << mbits));
    const float min_normal = ldexpf(1.0f, 1 - exp_bias);
    const int denorm_exp = (BIAS32 - exp_bias) + (MB - mbits) + 1;
    const uint32_t denorm_mask_int = (uint32_t)denorm_exp << MB;
    const float denorm_mask_float = u2f(denorm_mask_int);

    uint32_t xb = f2u(xf);
    uint32_t sign = xb & 0x80000000u;
    xb ^= sign;
    float x = u2f(xb);
    uint8_t res;
    if (x >= max_normal) {
        res = (uint8_t)max_int;
    } else if (x < min_normal) {
        float d = x + denorm_mask_float;
        uint32_t di = f2u(d) - denorm_mask_int;
        res = (uint8_t)di;
    } else {
        uint32_t nx = xb;
        uint32_t mant_odd = (nx >> (MB - mbits)) & 1u;
        nx += ((uint32_t)(exp_bias - BIAS32) << MB) + magic_adder;
        nx += mant_odd;
        nx >>= (MB - mbits);
        res = (uint8_t)nx;
    }
    uint32_t sign_lp = (sign >> (MB + EB - mbits - ebits)) & sign_mask;
    return (uint8_t)(res | sign_lp);
}

static inline float fpx_to_f32_one(uint8_t c, int ebits, int mbits) {
    const int MB = 23, BIAS32 = 127;
    const uint32_t sign_mask = 1u << (ebits + mbits);
    const int exp_bias = (1 << (ebits - 1)) - 1;
    uint32_t sign = c & sign_mask;
    uint32_t pos = c ^ sign;
    uint32_t e = pos >> mbits, m = pos & ((1u << mbits) - 1);
    uint32_t res;
    if (pos == 0) {
        res = 0;
    } else if (e == 0) {
        /* subnormal: value = m * 2^(1-bias-mbits) */
        res = f2u(ldexpf((float)m, 1 - exp_bias - mbits));
    } else {
        res = ((e - exp_bias + BIAS32) << MB) | (m << (MB - mbits));
    }
    res |= sign << (31 - (ebits + mbits));
    return u2f(res);
}

void orc_f32_to_fpx(const float* x, int64_t n, int ebits, int mbits, uint8_t* out) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) out[i] = f32_to_fpx_one(x[i], ebits, mbits);
}
void orc_fpx_to_f32(const uint8_t* c, int64_t n, int ebits, int mbits, float* out) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) out[i] = fpx_to_f32_one(c[i], ebits, mbits);
}

/* ------------------------------------------------------------------ */
/* _pack_tc_fp6 — prototype/quant_llm/quant_llm.py:90-106               */
/* codes uint8 [M][N] (6 significant bits) -> out uint8 [M*N*6/8]:      */
/* all 2-bit bytes (M*N/4) then all 4-bit bytes (M*N/2).                */
/* ------------------------------------------------------------------ */
int orc_pack_tc_fp6(const uint8_t* codes, int64_t M, int64_t N, uint8_t* out) {
    if (M % 64 || N % 64) return -1;
    const int64_t F = N / 16;
    uint8_t* o2 = out;
    uint8_t* o4 = out + M * N / 4;
    memset(out, 0, (size_t)(M * N * 3 / 4));
    for (int64_t a = 0; a < M / 64; ++a)
        for (int b = 0; b < 2; ++b)
            for (int c = 0; c < 2; ++c)
                for (int d = 0; d < 2; ++d)
                    for (int e = 0; e < 8; ++e)
                        for (int64_t f = 0; f < F; ++f)
                            for (int g = 0; g < 2; ++g)
                                for (int h = 0; h < 8; ++h) {
                                    /* the view is flipped along d before the permutes (:94) */
                                    int64_t row = a * 64 + b * 32 + c * 16 + (1 - d) * 8 + e;
                                    int64_t col = f * 16 + g * 8 + h;
                                    uint8_t v = codes[row * N + col];
                                    /* 2-bit plane: order (a,f,b,e,h,d,c,g) (:97) */
                                    int64_t i2 = ((((((a * F + f) * 2 + b) * 8 + e) * 8 + h) * 2 + d) * 2 + c) * 2 + g;
                                    o2[i2 >> 2] |= (uint8_t)(((v >> 4) & 3) << (6 - 2 * (i2 & 3)));
                                    /* 4-bit plane: order (a,f,b,c,e,h,d,g) (:101) */
                                    int64_t i4 = ((((((a * F + f) * 2 + b) * 2 + c) * 8 + e) * 8 + h) * 2 + d) * 2 + g;
                                    o4[i4 >> 1] |= (uint8_t)((v & 15) << (4 - 4 * (i4 & 1)));
                                }
    return 0;
}

int orc_unpack_tc_fp6(const uint8_t* packed, int64_t M, int64_t N, uint8_t* codes) {
    if (M % 64 || N % 64) return -1;
    const int64_t F = N / 16;
    const uint8_t* o2 = packed;
    const uint8_t* o4 = packed + M * N / 4;
    for (int64_t a = 0; a < M / 64; ++a)
        for (int b = 0; b < 2; ++b)
            for (int c = 0; c < 2; ++c)
                for (int d = 0; d < 2; ++d)
                    for (int e = 0; e < 8; ++e)
                        for (int64_t f = 0; f < F; ++f)
                            for (int g = 0; g < 2; ++g)
                                for (int h = 0; h < 8; ++h) {
                                    int64_t row = a * 64 + b * 32 + c * 16 + (1 - d) * 8 + e;
                                    int64_t col = f * 16 + g * 8 + h;
                                    int64_t i2 = ((((((a * F + f) * 2 + b) * 8 + e) * 8 + h) * 2 + d) * 2 + c) * 2 + g;
                                    int64_t i4 = ((((((a * F + f) * 2 + b) * 2 + c) * 8 + e) * 8 + h) * 2 + d) * 2 + g;
                                    uint8_t hi = (o2[i2 >> 2] >> (6 - 2 * (i2 & 3))) & 3;
                                    uint8_t lo = (o4[i4 >> 1] >> (4 - 4 * (i4 & 1))) & 15;
                                    codes[row * N + col] = (uint8_t)((hi << 4) | lo);
                                }
    return 0;
}

/* ------------------------------------------------------------------ */
/* to_scaled_tc_fpx — quant_llm.py:116-130 (6-bit case).                */
/* w: fp32 [M][N] (already .float()).  scale_out: fp16 bits [M].        */
/* codes_out (optional): unpacked codes [M][N].                          */
/* ------------------------------------------------------------------ */
int orc_to_scaled_tc_fp6(const float* w, int64_t M, int64_t N, int ebits, int mbits,
                         uint8_t* packed, uint16_t* scale_out, uint8_t* codes_out) {
    if (M % 64 || N % 64 || ebits + mbits != 5) return -1;
    const int exp_bias = (1 << (ebits - 1)) - 1;
    const float max_normal =
        ldexpf(1.0f, ((1 << ebits) - 1) - exp_bias) * ((float)((1 << (mbits + 1)) - 1) / (float)(1 << mbits));
    uint8_t* codes = codes_out ? codes_out : (uint8_t*)malloc((size_t)(M * N));
#pragma omp parallel for schedule(static)
    for (int64_t m = 0; m < M; ++m) {
        float amax = 0.f;
        for (int64_t n = 0; n < N; ++n) {
            float a = fabsf(w[m * N + n]);
            amax = a > amax ? a : amax;
        }
        amax = amax < 1e-12f ? 1e-12f : amax;
        float s = amax / max_normal;
        for (int64_t n = 0; n < N; ++n) codes[m * N + n] = f32_to_fpx_one(w[m * N + n] / s, ebits, mbits);
        scale_out[m] = f32_to_f16_bits(s);
    }
    int rc = orc_pack_tc_fp6(codes, M, N, packed);
    if (!codes_out) free(codes);
    return rc;
}

/* from_scaled_tc_fpx — quant_llm.py:203-208 (6-bit): fp32 [M][N] = decode * scale.float() */
int orc_from_scaled_tc_fp6(const uint8_t* packed, int64_t M, int64_t N, int ebits, int mbits,
                           const uint16_t* scale, float* out) {
    uint8_t* codes = (uint8_t*)malloc((size_t)(M * N));
    int rc = orc_unpack_tc_fp6(packed, M, N, codes);
    if (rc == 0) {
#pragma omp parallel for schedule(static)
        for (int64_t m = 0; m < M; ++m) {
            float s = scale ? f16_bits_to_f32(scale[m]) : 1.0f;
            for (int64_t n = 0; n < N; ++n) {
                float v = fpx_to_f32_one(codes[m * N + n], ebits, mbits);
                out[m * N + n] = scale ? v * s : v;
            }
        }
    }
    free(codes);
    return rc;
}

/* ------------------------------------------------------------------ */
/* y[M][N] = x[M][K] @ w[N][K]^T, all fp32 in memory, accumulated in    */
/* double: the "fp32 dequant-matmul" the GEMM tolerance is stated        */
/* against (the accumulation order of a BLAS is not part of the spec).  */
/* ------------------------------------------------------------------ */
void orc_linear_f32(const float* x, const float* w, int64_t M, int64_t N, int64_t K, float* y) {
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        const float* wr = w + n * K;
        for (int64_t m = 0; m < M; ++m) {
            const float* xr = x + m * K;
            double acc = 0.0;
            for (int64_t k = 0; k < K; ++k) acc += (double)xr[k] * (double)wr[k];
            y[m * N + n] = (float)acc;
        }
    }
}

/* ------------------------------------------------------------------ */
/* Timed CPU baseline for the int4 path: what F.linear does for an       */
/* AffineQuantizedTensor on CPU in the reference — dequantize the whole  */
/* weight to the activation dtype (affine_quantized_tensor.py:683-690,   */
/* dequantize_affine FLOAT domain) and then a dense matmul.  codes are   */
/* one per byte, scale/zero fp32-carried bf16 [N][K/g].  wbuf: [N][K]    */
/* scratch (bf16 values in fp32).  y: bf16-rounded values.               */
/* ------------------------------------------------------------------ */
void orc_int4_linear_dequant_then_matmul(const float* x, const uint8_t* codes, const float* scale,
                                         const float* zero, int64_t M, int64_t N, int64_t K,
                                         int64_t g, float* wbuf, float* y) {
    const int64_t G = K / g;
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        for (int64_t gi = 0; gi < G; ++gi) {
            const float s = scale[n * G + gi], z = zero[n * G + gi];
            const uint8_t* c = codes + n * K + gi * g;
            float* o = wbuf + n * K + gi * g;
            for (int64_t i = 0; i < g; ++i) {
                float v = (float)c[i] - 8.0f;
                v = rbf16(v * s);
                o[i] = rbf16(v + z);
            }
        }
    }
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        const float* wr = wbuf + n * K;
        for (int64_t m = 0; m < M; ++m) {
            const float* xr = x + m * K;
            float acc = 0.f;
            for (int64_t k = 0; k < K; ++k) acc += xr[k] * wr[k];
            y[m * N + n] = rbf16(acc);
        }
    }
}

/* Thread count of the OpenMP loops above: a launcher may have exported OMP_NUM_THREADS=1 for its child
 * processes (torch.distributed.run does); the timed CPU baseline sets the count it reports explicitly. */
void orc_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
