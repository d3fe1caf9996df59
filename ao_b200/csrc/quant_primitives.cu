// Affine quantization primitives: choose_qparams_affine / quantize_affine / dequantize_affine.
//
// Two families:
//  * general kernels: any contiguous n-d tensor with any block_size the reference accepts, any
//    of the supported dtype combinations; arithmetic follows eager PyTorch step by step (compute
//    in fp32, round to the dtype PyTorch's type promotion gives that step) so results are
//    bit-identical to torchao/quantization/quant_primitives.py:134-367.
//  * the int4 weight-only fast path (bf16 weight, groups of 32..256 along K, float zero point):
//    128-bit loads, sub-warp shuffle min/max, one pass.
#include "common.cuh"

namespace ao {

struct BlockView {
    int ndim;
    int rowblock;  // blocks are contiguous runs of block_elems elements
    int64_t size[AO_MAX_DIMS], block[AO_MAX_DIMS], nblk[AO_MAX_DIMS], stride[AO_MAX_DIMS];
    int64_t numel, nblocks, block_elems;
};

static int make_view(int ndim, const int64_t* sizes, const int64_t* block, BlockView* v) {
    if (ndim < 1 || ndim > AO_MAX_DIMS) return AO_ERR_SHAPE;
    v->ndim = ndim;
    v->numel = 1;
    v->nblocks = 1;
    v->block_elems = 1;
    for (int i = ndim - 1; i >= 0; --i) {
        if (sizes[i] < 1 || block[i] < 1 || sizes[i] % block[i] != 0) return AO_ERR_SHAPE;
        v->size[i] = sizes[i];
        v->block[i] = block[i];
        v->nblk[i] = sizes[i] / block[i];
        v->stride[i] = v->numel;
        v->numel *= sizes[i];
        v->nblocks *= v->nblk[i];
        v->block_elems *= block[i];
    }
    // contiguous blocks: block == 1 up to some dim j, anything at j, full size after j
    int j = 0;
    while (j < ndim && block[j] == 1) ++j;
    bool rb = true;
    for (int i = j + 1; i < ndim; ++i) rb = rb && (block[i] == sizes[i]);
    v->rowblock = rb ? 1 : 0;
    return AO_OK;
}

// offset of element e of block b
__device__ __forceinline__ int64_t element_offset(const BlockView& v, int64_t b, int64_t e) {
    if (v.rowblock) return b * v.block_elems + e;
    int64_t off = 0;
    for (int i = v.ndim - 1; i >= 0; --i) {
        int64_t bi = b % v.nblk[i];
        b /= v.nblk[i];
        int64_t ei = e % v.block[i];
        e /= v.block[i];
        off += (bi * v.block[i] + ei) * v.stride[i];
    }
    return off;
}

// block index of the element at linear offset i
__device__ __forceinline__ int64_t block_of(const BlockView& v, int64_t i) {
    if (v.rowblock) return i / v.block_elems;
    int64_t b = 0, mul = 1;
    for (int d = v.ndim - 1; d >= 0; --d) {
        int64_t c = i % v.size[d];
        i /= v.size[d];
        b += (c / v.block[d]) * mul;
        mul *= v.nblk[d];
    }
    return b;
}

struct QParamsArgs {
    int in_dt, mapping, scale_dt, zp_dt, preserve_zero, zp_domain;
    float qmin, qmax, eps, mid, sym_div, asym_div, sym_zp;
};

// one warp per block
__global__ void __launch_bounds__(256) choose_qparams_kernel(const void* __restrict__ x, BlockView v,
                                                             QParamsArgs a, void* __restrict__ scale_out,
                                                             void* __restrict__ zp_out) {
    const int lane = threadIdx.x & 31;
    const int64_t warps_per_grid = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
    for (int64_t b = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); b < v.nblocks;
         b += warps_per_grid) {
        float mn = INFINITY, mx = -INFINITY;
        for (int64_t e = lane; e < v.block_elems; e += 32) {
            float f = load_as_f32(x, a.in_dt, element_offset(v, b, e));
            mn = fminf(mn, f);
            mx = fmaxf(mx, f);
        }
        mn = warp_min(mn, 32);
        mx = warp_max(mx, 32);
        if (lane != 0) continue;
        float mnn = mn, mxp = mx;
        if (a.preserve_zero) {
            mnn = fminf(mn, 0.f);
            mxp = fmaxf(mx, 0.f);
        }
        float scale, zp;
        if (a.mapping == AO_MAP_SYMMETRIC) {
            mxp = fmaxf(-mnn, mxp);
            scale = round_to(a.in_dt, __fdiv_rn(mxp, a.sym_div));
            zp = round_to(a.in_dt, a.sym_zp);
        } else {
            float d = round_to(a.in_dt, __fsub_rn(mxp, mnn));
            scale = round_to(a.in_dt, __fdiv_rn(d, a.asym_div));
            if (a.preserve_zero) {
                float q = rintf(round_to(a.in_dt, __fdiv_rn(mnn, scale)));
                zp = round_to(a.in_dt, __fsub_rn(a.qmin, q));
                zp = fminf(fmaxf(zp, a.qmin), a.qmax);
            } else {
                float sm = round_to(a.in_dt, __fmul_rn(scale, a.mid));
                zp = round_to(a.in_dt, __fadd_rn(mnn, sm));
            }
        }
        scale = fmaxf(scale, a.eps);
        store_from_f32(scale_out, a.scale_dt, b, round_to(a.scale_dt, scale));
        store_from_f32(zp_out, a.zp_dt, b, is_float_dtype(a.zp_dt) ? round_to(a.zp_dt, zp) : truncf(zp));
    }
}

struct QuantArgs {
    int in_dt, scale_dt, zp_dt, zp_domain, out_dt, has_zp;
    float qmin, qmax, mid;
};

__global__ void __launch_bounds__(256) quantize_kernel(const void* __restrict__ x, BlockView v, QuantArgs a,
                                                       const void* __restrict__ scale,
                                                       const void* __restrict__ zp, void* __restrict__ out) {
    const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
    const int p1 = promote_dtype(a.in_dt, a.scale_dt);
    const int p2 = is_float_dtype(a.zp_dt) ? promote_dtype(p1, a.zp_dt) : p1;
    const int pm = promote_dtype(is_float_dtype(a.zp_dt) ? a.zp_dt : a.scale_dt, a.scale_dt);
    const int p3 = promote_dtype(a.in_dt, pm);
    const int p4 = promote_dtype(p3, a.scale_dt);
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < v.numel; i += step) {
        const int64_t b = block_of(v, i);
        const float s = load_as_f32(scale, a.scale_dt, b);
        const float z = load_as_f32(zp, a.zp_dt, b);
        const float xv = load_as_f32(x, a.in_dt, i);
        float r;
        if (a.zp_domain == AO_ZP_INT) {
            const float inv = round_to(a.scale_dt, __fdiv_rn(1.0f, s));
            r = rintf(round_to(p1, __fmul_rn(xv, inv)));
            r = round_to(p2, __fadd_rn(r, z));
        } else {
            const float sm = round_to(a.scale_dt, __fmul_rn(s, a.mid));
            const float minv = round_to(pm, __fsub_rn(z, sm));
            r = round_to(p3, __fsub_rn(xv, minv));
            r = rintf(round_to(p4, __fdiv_rn(r, s)));
        }
        r = fminf(fmaxf(r, a.qmin), a.qmax);
        store_from_f32(out, a.out_dt, i, r);
    }
}

__global__ void __launch_bounds__(256) dequantize_kernel(const void* __restrict__ q, int q_dt, BlockView v,
                                                         QuantArgs a, const void* __restrict__ scale,
                                                         const void* __restrict__ zp, void* __restrict__ out) {
    const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < v.numel; i += step) {
        const int64_t b = block_of(v, i);
        const float s = load_as_f32(scale, a.scale_dt, b);
        const int32_t qi = load_as_i32(q, q_dt, i);
        float r;
        if (a.zp_domain == AO_ZP_INT) {
            const int32_t zi = a.has_zp ? load_as_i32(zp, a.zp_dt, b) : 0;
            r = round_to(a.out_dt, static_cast<float>(qi - zi));
            r = round_to(a.out_dt, __fmul_rn(r, s));
        } else {
            r = round_to(a.out_dt, __fsub_rn(static_cast<float>(qi), a.mid));
            r = round_to(a.out_dt, __fmul_rn(r, s));
            if (a.has_zp) r = round_to(a.out_dt, __fadd_rn(r, load_as_f32(zp, a.zp_dt, b)));
        }
        store_from_f32(out, a.out_dt, i, r);
    }
}

// ---------------------------------------------------------------------------------------------
// Vectorised variants of the three general kernels for the common layout: blocks are contiguous runs of B elements
// (B a multiple of 8), every thread owns 8 consecutive elements (128-bit loads for 16-bit inputs), block constants
// are computed once per thread, group min / max by sub-warp shuffles.  Same arithmetic, same rounding steps.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void unpack8_bf16(const uint4& v, float (&f)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

template <int DT>
__device__ __forceinline__ void load8(const void* p, int64_t v8, float (&f)[8]) {
    if constexpr (DT == AO_F32) {
        const float4 a = __ldg(static_cast<const float4*>(p) + 2 * v8), b = __ldg(static_cast<const float4*>(p) + 2 * v8 + 1);
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    } else if constexpr (DT == AO_BF16) {
        unpack8_bf16(__ldg(static_cast<const uint4*>(p) + v8), f);
    } else if constexpr (DT == AO_F16) {
        const uint4 v = __ldg(static_cast<const uint4*>(p) + v8);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
            f[2 * i] = __low2float(h);
            f[2 * i + 1] = __high2float(h);
        }
    } else if constexpr (DT == AO_I32) {
        const int4 a = __ldg(static_cast<const int4*>(p) + 2 * v8), b = __ldg(static_cast<const int4*>(p) + 2 * v8 + 1);
        f[0] = (float)a.x; f[1] = (float)a.y; f[2] = (float)a.z; f[3] = (float)a.w;
        f[4] = (float)b.x; f[5] = (float)b.y; f[6] = (float)b.z; f[7] = (float)b.w;
    } else {   // AO_U8 / AO_I8
        const uint2 v = __ldg(static_cast<const uint2*>(p) + v8);
        const uint32_t w[2] = {v.x, v.y};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t b = (w[i >> 2] >> (8 * (i & 3))) & 0xffu;
            f[i] = DT == AO_U8 ? static_cast<float>(b) : static_cast<float>(static_cast<int8_t>(b));
        }
    }
}

// values are already rounded to the dtype / integral
template <int DT>
__device__ __forceinline__ void store8(void* p, int64_t v8, const float (&f)[8]) {
    if constexpr (DT == AO_F32) {
        static_cast<float4*>(p)[2 * v8] = make_float4(f[0], f[1], f[2], f[3]);
        static_cast<float4*>(p)[2 * v8 + 1] = make_float4(f[4], f[5], f[6], f[7]);
    } else if constexpr (DT == AO_BF16 || DT == AO_F16) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if constexpr (DT == AO_BF16) {
                const __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
                w[i] = *reinterpret_cast<const uint32_t*>(&h);
            } else {
                const __half2 h = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
                w[i] = *reinterpret_cast<const uint32_t*>(&h);
            }
        }
        static_cast<uint4*>(p)[v8] = make_uint4(w[0], w[1], w[2], w[3]);
    } else if constexpr (DT == AO_I32) {
        static_cast<int4*>(p)[2 * v8] = make_int4((int)f[0], (int)f[1], (int)f[2], (int)f[3]);
        static_cast<int4*>(p)[2 * v8 + 1] = make_int4((int)f[4], (int)f[5], (int)f[6], (int)f[7]);
    } else {   // AO_U8 / AO_I8
        uint32_t w[2] = {0u, 0u};
#pragma unroll
        for (int i = 0; i < 8; ++i) w[i >> 2] |= (static_cast<uint32_t>(static_cast<int>(f[i])) & 0xffu) << (8 * (i & 3));
        static_cast<uint2*>(p)[v8] = make_uint2(w[0], w[1]);
    }
}

__device__ __forceinline__ void qparams_from_minmax(const QParamsArgs& a, float mn, float mx, float* scale_out, float* zp_out) {
    float mnn = mn, mxp = mx;
    if (a.preserve_zero) {
        mnn = fminf(mn, 0.f);
        mxp = fmaxf(mx, 0.f);
    }
    float scale, zp;
    if (a.mapping == AO_MAP_SYMMETRIC) {
        mxp = fmaxf(-mnn, mxp);
        scale = round_to(a.in_dt, __fdiv_rn(mxp, a.sym_div));
        zp = round_to(a.in_dt, a.sym_zp);
    } else {
        float d = round_to(a.in_dt, __fsub_rn(mxp, mnn));
        scale = round_to(a.in_dt, __fdiv_rn(d, a.asym_div));
        if (a.preserve_zero) {
            float q = rintf(round_to(a.in_dt, __fdiv_rn(mnn, scale)));
            zp = round_to(a.in_dt, __fsub_rn(a.qmin, q));
            zp = fminf(fmaxf(zp, a.qmin), a.qmax);
        } else {
            float sm = round_to(a.in_dt, __fmul_rn(scale, a.mid));
            zp = round_to(a.in_dt, __fadd_rn(mnn, sm));
        }
    }
    *scale_out = fmaxf(scale, a.eps);
    *zp_out = zp;
}

// L = B / 8 lanes share a block (L a power of two <= 32); nvec = numel / 8
template <int DT>
__global__ void __launch_bounds__(256) choose_qparams_vec_kernel(const void* __restrict__ x, int64_t nvec, int L,
                                                                 QParamsArgs a, void* __restrict__ scale_out,
                                                                 void* __restrict__ zp_out) {
    const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
    const int64_t rounded = (nvec + 31) / 32 * 32;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < rounded; i += step) {
        float f[8];
        float mn = INFINITY, mx = -INFINITY;
        if (i < nvec) {
            load8<DT>(x, i, f);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                mn = fminf(mn, f[k]);
                mx = fmaxf(mx, f[k]);
            }
        }
        mn = warp_min(mn, L);
        mx = warp_max(mx, L);
        if (i < nvec && (i % L) == 0) {
            float scale, zp;
            qparams_from_minmax(a, mn, mx, &scale, &zp);
            const int64_t b = i / L;
            store_from_f32(scale_out, a.scale_dt, b, round_to(a.scale_dt, scale));
            store_from_f32(zp_out, a.zp_dt, b, is_float_dtype(a.zp_dt) ? round_to(a.zp_dt, zp) : truncf(zp));
        }
    }
}

// one warp per block of B elements (any B that is a multiple of 8)
template <int DT>
__global__ void __launch_bounds__(256) choose_qparams_row_kernel(const void* __restrict__ x, int64_t nblocks, int64_t vec_per_block,
                                                                 QParamsArgs a, void* __restrict__ scale_out,
                                                                 void* __restrict__ zp_out) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
    for (int64_t b = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); b < nblocks; b += warps) {
        float mn = INFINITY, mx = -INFINITY;
        for (int64_t e = lane; e < vec_per_block; e += 32) {
            float f[8];
            load8<DT>(x, b * vec_per_block + e, f);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                mn = fminf(mn, f[k]);
                mx = fmaxf(mx, f[k]);
            }
        }
        mn = warp_min(mn, 32);
        mx = warp_max(mx, 32);
        if (lane == 0) {
            float scale, zp;
            qparams_from_minmax(a, mn, mx, &scale, &zp);
            store_from_f32(scale_out, a.scale_dt, b, round_to(a.scale_dt, scale));
            store_from_f32(zp_out, a.zp_dt, b, is_float_dtype(a.zp_dt) ? round_to(a.zp_dt, zp) : truncf(zp));
        }
    }
}

template <int IN_DT, int OUT_DT>
__global__ void __launch_bounds__(256) quantize_vec_kernel(const void* __restrict__ x, int64_t nvec, int64_t vec_per_block,
                                                           QuantArgs a, const void* __restrict__ scale,
                                                           const void* __restrict__ zp, void* __restrict__ out) {
    const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
    const int p1 = promote_dtype(a.in_dt, a.scale_dt);
    const int p2 = is_float_dtype(a.zp_dt) ? promote_dtype(p1, a.zp_dt) : p1;
    const int pm = promote_dtype(is_float_dtype(a.zp_dt) ? a.zp_dt : a.scale_dt, a.scale_dt);
    const int p3 = promote_dtype(a.in_dt, pm);
    const int p4 = promote_dtype(p3, a.scale_dt);
    // with bf16 operands the division below equals a multiplication by the correctly rounded reciprocal
    // (see int4_code_bf16)
    const bool rcp_ok = IN_DT == AO_BF16 && a.scale_dt == AO_BF16 && p3 == AO_BF16 && p4 == AO_BF16;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += step) {
        const int64_t b = i / vec_per_block;
        const float s = load_as_f32(scale, a.scale_dt, b);
        const float z = load_as_f32(zp, a.zp_dt, b);
        float f[8];
        load8<IN_DT>(x, i, f);
        if (a.zp_domain == AO_ZP_INT) {
            const float inv = round_to(a.scale_dt, __fdiv_rn(1.0f, s));
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                float r = rintf(round_to(p1, __fmul_rn(f[k], inv)));
                r = round_to(p2, __fadd_rn(r, z));
                f[k] = fminf(fmaxf(r, a.qmin), a.qmax);
            }
        } else {
            const float sm = round_to(a.scale_dt, __fmul_rn(s, a.mid));
            const float minv = round_to(pm, __fsub_rn(z, sm));
            const float rs = __frcp_rn(s);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                float r = round_to(p3, __fsub_rn(f[k], minv));
                r = rintf(round_to(p4, rcp_ok ? __fmul_rn(r, rs) : __fdiv_rn(r, s)));
                f[k] = fminf(fmaxf(r, a.qmin), a.qmax);
            }
        }
        store8<OUT_DT>(out, i, f);
    }
}

template <int Q_DT, int OUT_DT>
__global__ void __launch_bounds__(256) dequantize_vec_kernel(const void* __restrict__ q, int64_t nvec, int64_t vec_per_block,
                                                             QuantArgs a, const void* __restrict__ scale,
                                                             const void* __restrict__ zp, void* __restrict__ out) {
    const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += step) {
        const int64_t b = i / vec_per_block;
        const float s = load_as_f32(scale, a.scale_dt, b);
        float f[8];
        load8<Q_DT>(q, i, f);
        if (a.zp_domain == AO_ZP_INT) {
            const float zi = a.has_zp ? static_cast<float>(load_as_i32(zp, a.zp_dt, b)) : 0.f;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                float r = round_to(OUT_DT, f[k] - zi);   // small integers: the difference is exact in fp32
                f[k] = round_to(OUT_DT, __fmul_rn(r, s));
            }
        } else {
            const float z = a.has_zp ? load_as_f32(zp, a.zp_dt, b) : 0.f;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                float r = round_to(OUT_DT, __fsub_rn(f[k], a.mid));
                r = round_to(OUT_DT, __fmul_rn(r, s));
                if (a.has_zp) r = round_to(OUT_DT, __fadd_rn(r, z));
                f[k] = r;
            }
        }
        store8<OUT_DT>(out, i, f);
    }
}

// ---------------------------------------------------------------------------------------------
// int4 weight-only fast path
// ---------------------------------------------------------------------------------------------
struct Int4Params {
    float s, zp, minv, rs;   // rs = 1 / s, correctly rounded
};

// the int4_weight_only parameter set: asymmetric, qmin 0, qmax 15, mid 8, eps 1e-6 (as bf16),
// zero point in the float domain, everything bf16
__device__ __forceinline__ Int4Params int4_qparams_bf16(float mn, float mx) {
    Int4Params p;
    const float d = round_bf16(__fsub_rn(mx, mn));
    const float s0 = round_bf16(__fdiv_rn(d, 15.0f));
    p.zp = round_bf16(__fadd_rn(mn, round_bf16(__fmul_rn(s0, 8.0f))));  // uses the unclamped scale
    p.s = fmaxf(s0, __uint_as_float(0x35860000u));                      // bf16(1e-6)
    p.minv = round_bf16(__fsub_rn(p.zp, round_bf16(__fmul_rn(p.s, 8.0f))));
    p.rs = __frcp_rn(p.s);
    return p;
}

// round_bf16((x - minv) / s) with the division done as a multiplication by 1 / s.  Both operands are bf16 values
// (8-bit significands), so the exact quotient is either a bf16 value itself or at least 2^-18 (relative) away from
// every midpoint between two bf16 values; the product's error (< 2^-22) cannot move it across one: the bf16
// result is the same as that of the correctly rounded fp32 division the reference performs.
__device__ __forceinline__ int int4_code_bf16(float x, const Int4Params& p) {
    float r = round_bf16(__fsub_rn(x, p.minv));
    r = rintf(round_bf16(__fmul_rn(r, p.rs)));
    return static_cast<int>(fminf(fmaxf(r, 0.f), 15.f));
}

// G/8 lanes share a group; each lane owns 8 consecutive elements (one 128-bit load).
template <int G>
__global__ void __launch_bounds__(256) int4_groupwise_quantize_kernel(const uint4* __restrict__ w, int64_t n_vec,
                                                                      __nv_bfloat16* __restrict__ scale_out,
                                                                      __nv_bfloat16* __restrict__ zero_out,
                                                                      int32_t* __restrict__ codes_i32,
                                                                      uint8_t* __restrict__ codes_u8) {
    constexpr int L = G / 8;  // lanes per group: 4, 8, 16, 32
    const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
    // n_vec is a multiple of L and blockDim a multiple of 32, so whole sub-warps stay together
    const int64_t n_round = (n_vec + 31) / 32 * 32;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_round; i += step) {
        const bool live = i < n_vec;
        float f[8];
        if (live) {
            unpack8_bf16(__ldg(w + i), f);
        } else {
#pragma unroll
            for (int k = 0; k < 8; ++k) f[k] = 0.f;
        }
        float mn = f[0], mx = f[0];
#pragma unroll
        for (int k = 1; k < 8; ++k) {
            mn = fminf(mn, f[k]);
            mx = fmaxf(mx, f[k]);
        }
        mn = warp_min(mn, L);
        mx = warp_max(mx, L);
        if (!live) continue;
        const Int4Params p = int4_qparams_bf16(mn, mx);
        if ((i % L) == 0) {
            if (scale_out) scale_out[i / L] = __float2bfloat16_rn(p.s);
            if (zero_out) zero_out[i / L] = __float2bfloat16_rn(p.zp);
        }
        int c[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) c[k] = int4_code_bf16(f[k], p);
        if (codes_i32) {
            int4* o = reinterpret_cast<int4*>(codes_i32) + 2 * i;
            o[0] = make_int4(c[0], c[1], c[2], c[3]);
            o[1] = make_int4(c[4], c[5], c[6], c[7]);
        }
        if (codes_u8) {
            uint2 o;
            o.x = c[0] | (c[1] << 8) | (c[2] << 16) | (c[3] << 24);
            o.y = c[4] | (c[5] << 8) | (c[6] << 16) | (c[7] << 24);
            reinterpret_cast<uint2*>(codes_u8)[i] = o;
        }
    }
}

// Fused W -> tensor_core_tiled packed weight + interleaved scale/zero, no shared memory.
// A warp owns 8 rows x U columns (U = the larger of the group and the packed layout's outer tile of IKT * 16 k);
// lane = row * 4 + c reads, for every 32-k span, the 8 values k = 8c .. 8c + 7 of its row (one 16-byte load) -
// which is exactly the lane numbering of the packed layout.  Group min / max are quad reductions; the 8 codes of a
// span live as nibbles of one register; a packed word takes byte c (codes 2c, 2c + 1) of the four registers of
// its quad (shuffles), puts the low nibbles in bits 15..0 and the high nibbles in bits 31..16, and the lane's
// IKT / 2 words of an outer tile leave as one vector store.
template <int G, int IKT>
__global__ void __launch_bounds__(256) int4_quantize_pack_kernel(const __nv_bfloat16* __restrict__ w, int64_t N,
                                                                 int64_t K, int32_t* __restrict__ packed,
                                                                 __nv_bfloat16* __restrict__ scale_and_zero) {
    constexpr int OT = IKT * 16;                 // k per outer tile
    constexpr int U = G > OT ? G : OT;           // k per warp unit
    constexpr int S = U / 32;                    // 32-k spans per unit
    constexpr int SPG = G / 32;                  // spans per group
    constexpr int HALF = IKT / 2;                // words per lane per outer tile = spans per outer tile
    const int lane = threadIdx.x & 31, row = lane >> 2, c = lane & 3;
    const int64_t upr = K / U;                   // units per tile row
    const int64_t unit = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= (N / 8) * upr) return;           // whole warps leave together
    const int64_t nt = unit / upr, k0 = (unit % upr) * U;
    const int64_t n = nt * 8 + row;
    const __nv_bfloat16* src = w + n * K + k0 + 8 * c;
    float f[S][8];
#pragma unroll
    for (int s = 0; s < S; ++s) unpack8_bf16(__ldg(reinterpret_cast<const uint4*>(src + 32 * s)), f[s]);
    uint32_t ch[S];
#pragma unroll
    for (int gi = 0; gi < S / SPG; ++gi) {
        float mn = f[gi * SPG][0], mx = mn;
#pragma unroll
        for (int s = gi * SPG; s < (gi + 1) * SPG; ++s)
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                mn = fminf(mn, f[s][k]);
                mx = fmaxf(mx, f[s][k]);
            }
        mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, 2));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const Int4Params p = int4_qparams_bf16(mn, mx);
        if (c == 0) {
            __nv_bfloat162 sz;
            sz.x = __float2bfloat16_rn(p.s);
            sz.y = __float2bfloat16_rn(p.zp);
            reinterpret_cast<__nv_bfloat162*>(scale_and_zero)[(k0 / G + gi) * N + n] = sz;
        }
#pragma unroll
        for (int s = gi * SPG; s < (gi + 1) * SPG; ++s) {
            uint32_t v = 0;
#pragma unroll
            for (int k = 0; k < 8; ++k) v |= static_cast<uint32_t>(int4_code_bf16(f[s][k], p)) << (4 * k);
            ch[s] = v;
        }
    }
    // byte c of a register holds codes 2c, 2c + 1 of that 8-k chunk
    const uint32_t sel01 = static_cast<uint32_t>(c) | (static_cast<uint32_t>(4 + c) << 4) | 0x8800u;  // upper bytes: zero
    const int quad = lane & ~3;
    const int64_t KO = K / OT;
    int32_t* dst = packed + ((nt * KO + k0 / OT) * 32 + lane) * HALF;
#pragma unroll
    for (int o = 0; o < U / OT; ++o) {
        uint32_t words[HALF];
#pragma unroll
        for (int j = 0; j < HALF; ++j) {
            const uint32_t v = ch[o * HALF + j];
            const uint32_t c0 = __shfl_sync(0xffffffffu, v, quad), c1 = __shfl_sync(0xffffffffu, v, quad + 1);
            const uint32_t c2 = __shfl_sync(0xffffffffu, v, quad + 2), c3 = __shfl_sync(0xffffffffu, v, quad + 3);
            // P = bytes (chunk 0, chunk 1, chunk 2, chunk 3) = k 2c.., 2c + 8.., 2c + 16.., 2c + 24..
            const uint32_t p01 = __byte_perm(c0, c1, sel01), p23 = __byte_perm(c2, c3, sel01);
            const uint32_t P = __byte_perm(p01, p23, 0x5410);
            uint32_t lo = P & 0x0F0F0F0Fu, hi = (P >> 4) & 0x0F0F0F0Fu;
            lo = (lo | (lo >> 4)) & 0x00FF00FFu;
            lo = (lo | (lo >> 8)) & 0x0000FFFFu;
            hi = (hi | (hi >> 4)) & 0x00FF00FFu;
            hi = (hi | (hi >> 8)) & 0x0000FFFFu;
            words[j] = lo | (hi << 16);
        }
        int32_t* d = dst + static_cast<int64_t>(o) * 32 * HALF;
        if constexpr (HALF == 4)
            *reinterpret_cast<uint4*>(d) = make_uint4(words[0], words[1], words[2], words[3]);
        else if constexpr (HALF == 2)
            *reinterpret_cast<uint2*>(d) = make_uint2(words[0], words[1]);
        else
            *reinterpret_cast<uint32_t*>(d) = words[0];
    }
}

static int grid_for(int64_t work_items, int threads) {
    int64_t g = (work_items + threads - 1) / threads;
    const int64_t cap = static_cast<int64_t>(kNumSMs) * 16;
    if (g > cap) g = cap;
    if (g < 1) g = 1;
    return static_cast<int>(g);
}

}  // namespace ao

using namespace ao;

extern "C" int ao_choose_qparams_affine(const void* input, int input_dtype, int ndim, const int64_t* sizes,
                                        const int64_t* block_size, int mapping_type, int64_t quant_min,
                                        int64_t quant_max, int has_eps, double eps, int scale_dtype,
                                        int zero_point_dtype, int preserve_zero, int zero_point_domain,
                                        void* scale_out, void* zero_point_out, ao_stream_t stream) {
    if (!is_float_dtype(input_dtype) || !is_float_dtype(scale_dtype)) return AO_ERR_DTYPE;
    if (zero_point_dtype < AO_F32 || zero_point_dtype > AO_I16) return AO_ERR_DTYPE;
    if (mapping_type != AO_MAP_SYMMETRIC && mapping_type != AO_MAP_ASYMMETRIC) return AO_ERR_ARG;
    if (mapping_type == AO_MAP_SYMMETRIC && (!preserve_zero || zero_point_domain != AO_ZP_INT)) return AO_ERR_ARG;
    if (mapping_type == AO_MAP_ASYMMETRIC && !preserve_zero && zero_point_domain != AO_ZP_FLOAT) return AO_ERR_ARG;
    BlockView v;
    int rc = make_view(ndim, sizes, block_size, &v);
    if (rc) return rc;
    QParamsArgs a;
    a.in_dt = input_dtype;
    a.mapping = mapping_type;
    a.scale_dt = scale_dtype;
    a.zp_dt = zero_point_dtype;
    a.preserve_zero = preserve_zero;
    a.zp_domain = zero_point_domain;
    a.qmin = static_cast<float>(quant_min);
    a.qmax = static_cast<float>(quant_max);
    float e = has_eps ? static_cast<float>(eps)
                      : (input_dtype == AO_BF16 ? 0.0078125f : input_dtype == AO_F16 ? 0.0009765625f : 1.1920928955078125e-07f);
    // clamp(min=eps) compares in the tensor's dtype
    if (input_dtype == AO_BF16) e = __bfloat162float(__float2bfloat16_rn(e));
    if (input_dtype == AO_F16) e = __half2float(__float2half_rn(e));
    a.eps = e;
    a.mid = static_cast<float>(static_cast<double>(quant_max + quant_min + 1) / 2.0);
    a.sym_div = static_cast<float>(static_cast<double>(quant_max - quant_min) / 2.0);
    a.asym_div = static_cast<float>(quant_max - quant_min);
    a.sym_zp = static_cast<float>(static_cast<int64_t>(static_cast<double>(quant_max + quant_min + 1) / 2.0));
    cudaStream_t st = as_stream(stream);
    if (v.rowblock && v.block_elems % 8 == 0 && aligned(input, 16)) {
        // vectorised: B / 8 lanes per block when that is a power of two up to 32, else one warp per block
        const int64_t vpb = v.block_elems / 8, nvec = v.numel / 8;
        const bool sub = vpb <= 32 && (vpb & (vpb - 1)) == 0;
        const int grid = sub ? grid_for(nvec, 256) : grid_for(v.nblocks * 32, 256);
#define AO_CHOOSE(DT_)                                                                                               \
    if (sub) choose_qparams_vec_kernel<DT_><<<grid, 256, 0, st>>>(input, nvec, (int)vpb, a, scale_out, zero_point_out); \
    else choose_qparams_row_kernel<DT_><<<grid, 256, 0, st>>>(input, v.nblocks, vpb, a, scale_out, zero_point_out)
        switch (input_dtype) {
            case AO_BF16: AO_CHOOSE(AO_BF16); break;
            case AO_F16: AO_CHOOSE(AO_F16); break;
            default: AO_CHOOSE(AO_F32); break;
        }
#undef AO_CHOOSE
        return launch_status();
    }
    const int grid = grid_for(v.nblocks * 32, 256);
    choose_qparams_kernel<<<grid, 256, 0, st>>>(input, v, a, scale_out, zero_point_out);
    return launch_status();
}

static int fill_quant_args(QuantArgs* a, int in_dt, int scale_dt, int zp_dt, int zp_domain, int out_dt,
                           const void* zp, int64_t qmin, int64_t qmax) {
    if (!is_float_dtype(scale_dt)) return AO_ERR_DTYPE;
    if (zp_domain != AO_ZP_INT && zp_domain != AO_ZP_FLOAT) return AO_ERR_ARG;
    a->in_dt = in_dt;
    a->scale_dt = scale_dt;
    a->zp_dt = zp_dt;
    a->zp_domain = zp_domain;
    a->out_dt = out_dt;
    a->has_zp = zp != nullptr;
    a->qmin = static_cast<float>(qmin);
    a->qmax = static_cast<float>(qmax);
    a->mid = static_cast<float>(static_cast<double>(qmax + qmin + 1) / 2.0);
    return AO_OK;
}

extern "C" int ao_quantize_affine(const void* input, int input_dtype, int ndim, const int64_t* sizes,
                                  const int64_t* block_size, const void* scale, int scale_dtype,
                                  const void* zero_point, int zero_point_dtype, int64_t quant_min,
                                  int64_t quant_max, int zero_point_domain, void* out, int out_dtype,
                                  ao_stream_t stream) {
    if (!is_float_dtype(input_dtype)) return AO_ERR_DTYPE;
    if (is_float_dtype(out_dtype) || out_dtype > AO_I16) return AO_ERR_DTYPE;
    if (zero_point == nullptr) return AO_ERR_ARG;
    BlockView v;
    int rc = make_view(ndim, sizes, block_size, &v);
    if (rc) return rc;
    QuantArgs a;
    rc = fill_quant_args(&a, input_dtype, scale_dtype, zero_point_dtype, zero_point_domain, out_dtype, zero_point,
                         quant_min, quant_max);
    if (rc) return rc;
    cudaStream_t st = as_stream(stream);
    if (v.rowblock && v.block_elems % 8 == 0 && aligned(input, 16) && aligned(out, 16) &&
        (out_dtype == AO_I32 || out_dtype == AO_U8 || out_dtype == AO_I8)) {
        const int64_t vpb = v.block_elems / 8, nvec = v.numel / 8;
        const int grid = grid_for(nvec, 256);
#define AO_QUANT(IN_, OUT_) quantize_vec_kernel<IN_, OUT_><<<grid, 256, 0, st>>>(input, nvec, vpb, a, scale, zero_point, out)
#define AO_QUANT_IN(IN_)                                  \
    switch (out_dtype) {                                  \
        case AO_I32: AO_QUANT(IN_, AO_I32); break;        \
        case AO_U8: AO_QUANT(IN_, AO_U8); break;          \
        default: AO_QUANT(IN_, AO_I8); break;             \
    }
        switch (input_dtype) {
            case AO_BF16: AO_QUANT_IN(AO_BF16); break;
            case AO_F16: AO_QUANT_IN(AO_F16); break;
            default: AO_QUANT_IN(AO_F32); break;
        }
#undef AO_QUANT_IN
#undef AO_QUANT
        return launch_status();
    }
    quantize_kernel<<<grid_for(v.numel, 256), 256, 0, st>>>(input, v, a, scale, zero_point, out);
    return launch_status();
}

extern "C" int ao_dequantize_affine(const void* input, int input_dtype, int ndim, const int64_t* sizes,
                                    const int64_t* block_size, const void* scale, int scale_dtype,
                                    const void* zero_point, int zero_point_dtype, int64_t quant_min,
                                    int64_t quant_max, int zero_point_domain, void* out, int out_dtype,
                                    ao_stream_t stream) {
    if (is_float_dtype(input_dtype) || input_dtype > AO_I16) return AO_ERR_DTYPE;
    if (!is_float_dtype(out_dtype)) return AO_ERR_DTYPE;
    BlockView v;
    int rc = make_view(ndim, sizes, block_size, &v);
    if (rc) return rc;
    QuantArgs a;
    rc = fill_quant_args(&a, AO_F32, scale_dtype, zero_point_dtype, zero_point_domain, out_dtype, zero_point,
                         quant_min, quant_max);
    if (rc) return rc;
    cudaStream_t st = as_stream(stream);
    const bool small_codes = quant_min >= -(1LL << 23) && quant_max <= (1LL << 23);
    if (v.rowblock && v.block_elems % 8 == 0 && aligned(input, 16) && aligned(out, 16) && small_codes &&
        (input_dtype == AO_I32 || input_dtype == AO_U8 || input_dtype == AO_I8)) {
        const int64_t vpb = v.block_elems / 8, nvec = v.numel / 8;
        const int grid = grid_for(nvec, 256);
#define AO_DEQ(Q_, OUT_) dequantize_vec_kernel<Q_, OUT_><<<grid, 256, 0, st>>>(input, nvec, vpb, a, scale, zero_point, out)
#define AO_DEQ_Q(Q_)                                      \
    switch (out_dtype) {                                  \
        case AO_BF16: AO_DEQ(Q_, AO_BF16); break;         \
        case AO_F16: AO_DEQ(Q_, AO_F16); break;           \
        default: AO_DEQ(Q_, AO_F32); break;               \
    }
        switch (input_dtype) {
            case AO_I32: AO_DEQ_Q(AO_I32); break;
            case AO_U8: AO_DEQ_Q(AO_U8); break;
            default: AO_DEQ_Q(AO_I8); break;
        }
#undef AO_DEQ_Q
#undef AO_DEQ
        return launch_status();
    }
    dequantize_kernel<<<grid_for(v.numel, 256), 256, 0, st>>>(input, input_dtype, v, a, scale, zero_point, out);
    return launch_status();
}

extern "C" int ao_int4_groupwise_quantize(const void* w_bf16, int64_t N, int64_t K, int group, void* scale_out,
                                          void* zero_out, int32_t* codes_i32_out, uint8_t* codes_u8_out,
                                          ao_stream_t stream) {
    if (N < 1 || K < 1 || K % group != 0) return AO_ERR_SHAPE;
    if (!aligned(w_bf16, 16) || (codes_i32_out && !aligned(codes_i32_out, 16)) ||
        (codes_u8_out && !aligned(codes_u8_out, 8)))
        return AO_ERR_ALIGN;
    const int64_t n_vec = N * K / 8;
    const int grid = grid_for(n_vec, 256);
    auto* s = static_cast<__nv_bfloat16*>(scale_out);
    auto* z = static_cast<__nv_bfloat16*>(zero_out);
    const uint4* w = static_cast<const uint4*>(w_bf16);
    cudaStream_t st = as_stream(stream);
    switch (group) {
        case 32: int4_groupwise_quantize_kernel<32><<<grid, 256, 0, st>>>(w, n_vec, s, z, codes_i32_out, codes_u8_out); break;
        case 64: int4_groupwise_quantize_kernel<64><<<grid, 256, 0, st>>>(w, n_vec, s, z, codes_i32_out, codes_u8_out); break;
        case 128: int4_groupwise_quantize_kernel<128><<<grid, 256, 0, st>>>(w, n_vec, s, z, codes_i32_out, codes_u8_out); break;
        case 256: int4_groupwise_quantize_kernel<256><<<grid, 256, 0, st>>>(w, n_vec, s, z, codes_i32_out, codes_u8_out); break;
        default: return AO_ERR_UNSUPPORTED;
    }
    return launch_status();
}

extern "C" int ao_int4_quantize_pack_tinygemm(const void* w_bf16, int64_t N, int64_t K, int group, int inner_k_tiles,
                                              int32_t* packed_out, void* scale_and_zero_out, ao_stream_t stream) {
    if (!(inner_k_tiles == 2 || inner_k_tiles == 4 || inner_k_tiles == 8)) return AO_ERR_ARG;
    if (N < 8 || N % 8 != 0 || K < 1 || K % group != 0 || K % (inner_k_tiles * 16) != 0 || K % 32 != 0)
        return AO_ERR_SHAPE;
    if (!aligned(w_bf16, 16) || !aligned(scale_and_zero_out, 4) || !aligned(packed_out, 16)) return AO_ERR_ALIGN;
    const auto* w = static_cast<const __nv_bfloat16*>(w_bf16);
    auto* sz = static_cast<__nv_bfloat16*>(scale_and_zero_out);
    cudaStream_t st = as_stream(stream);
    const int ot = inner_k_tiles * 16, unit_k = group > ot ? group : ot;
    const int64_t units = (N / 8) * (K / unit_k);
    if ((units + 7) / 8 > 2147483647LL) return AO_ERR_SHAPE;
    const unsigned grid = static_cast<unsigned>((units + 7) / 8);
#define AO_LAUNCH_QP(G_, I_) int4_quantize_pack_kernel<G_, I_><<<grid, 256, 0, st>>>(w, N, K, packed_out, sz)
#define AO_LAUNCH_QP_G(G_)                                  \
    switch (inner_k_tiles) {                                \
        case 8: AO_LAUNCH_QP(G_, 8); break;                 \
        case 4: AO_LAUNCH_QP(G_, 4); break;                 \
        default: AO_LAUNCH_QP(G_, 2); break;                \
    }
    switch (group) {
        case 32: AO_LAUNCH_QP_G(32); break;
        case 64: AO_LAUNCH_QP_G(64); break;
        case 128: AO_LAUNCH_QP_G(128); break;
        case 256: AO_LAUNCH_QP_G(256); break;
        default: return AO_ERR_UNSUPPORTED;
    }
#undef AO_LAUNCH_QP_G
#undef AO_LAUNCH_QP
    return launch_status();
}
