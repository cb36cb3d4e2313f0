// Device-side building blocks of the fused 4-bit AdamW step for sm_100a: the two 16-entry code
// books with their 15-entry midpoint tables (shared-memory resident), nibble pack/unpack, 128-bit
// parameter/gradient access, the element-wise AdamW arithmetic with every rounding explicit, and
// the warp-level abs-max reductions.
//
// Arithmetic contract (matches the reference's PyTorch path operator for operator,
// optim/adamw_fourbit_triton.py:415, :455-473, and its scaling helpers :618-630, :834-863):
//   p1  = rn(p * decay)
//   m   = fma(w1, rn(g - m_old), m_old)
//   v   = fma(rn(w2 * g), g, rn(beta2 * v_old))
//   den = rn(rn(sqrt(v) / bc2s) + eps)
//   p   = rn(p1 + rn(rn(neg_step * m) / den))
//   x_m = rn(m / max|m| over the 128-block),  x_v = rn(v / scale_v),  code = #{midpoints < x}
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/quantfour_b200.h"

namespace qf {

constexpr int kWarpsPerCta = 8;
constexpr int kThreads = kWarpsPerCta * 32;
constexpr int kPanelCols = 256;   // columns one warp covers: 32 lanes x 8 elements = two 128-blocks
constexpr int kRowsPerItem = 16;  // rows (of kPanelCols elements) one warp work item covers
constexpr int kMainRowsPerItem = 64;  // rows of one item of the second pass over a rank-1 panel: longer items
                                      // amortise the per-item set-up (column maxima into shared memory); a launch
                                      // with too few such items to give every warp slot of the device one takes
                                      // 32 or 16 rows per item instead (always an even number: rows go in pairs)
constexpr int kPreRowsPerItem = 64;  // the same for the first pass over a rank-1 panel: each item ends with one
                                     // red.max per column, so longer items mean fewer contended atomics
constexpr unsigned kFull = 0xffffffffu;

// Code books.  Literals as in optim/cuda_adamw_kernels.cu:25-98 (= optim/adamw_fourbit_triton.py:16-97):
// decimal constants rounded once to fp32.  The midpoint tables are the reference's own literals, not
// recomputed from the maps (they differ by one ulp at +-0.145).
__device__ __constant__ float c_qm[16] = {-0.8875f, -0.6625f, -0.4375f, -0.2125f, -0.0775f, -0.0325f,
                                          -0.0055f, 0.0f,     0.0055f,  0.0325f,  0.0775f,  0.2125f,
                                          0.4375f,  0.6625f,  0.8875f,  1.0f};
__device__ __constant__ float c_mm[16] = {-0.775f, -0.55f, -0.325f, -0.145f, -0.055f, -0.019f, -0.00275f, 0.00275f,
                                          0.019f,  0.055f, 0.145f,  0.325f,  0.55f,   0.775f,  0.94375f,
                                          __builtin_huge_valf()};
__device__ __constant__ float c_qv[16] = {0.0625f, 0.125f, 0.1875f, 0.25f, 0.3125f, 0.375f, 0.4375f, 0.5f,
                                          0.5625f, 0.625f, 0.6875f, 0.75f, 0.8125f, 0.875f, 0.9375f, 1.0f};
__device__ __constant__ float c_mv[16] = {0.09375f, 0.15625f, 0.21875f, 0.28125f, 0.34375f, 0.40625f,
                                          0.46875f, 0.53125f, 0.59375f, 0.65625f, 0.71875f, 0.78125f,
                                          0.84375f, 0.90625f, 0.96875f, __builtin_huge_valf()};

// Shared-memory copy of the tables, one per CTA.
struct Tables {
    float qm[16], mm[16], qv[16], mv[16];
};

__device__ __forceinline__ void load_tables(Tables& s) {
    if (threadIdx.x < 16) {
        s.qm[threadIdx.x] = c_qm[threadIdx.x];
        s.mm[threadIdx.x] = c_mm[threadIdx.x];
        s.qv[threadIdx.x] = c_qv[threadIdx.x];
        s.mv[threadIdx.x] = c_mv[threadIdx.x];
    }
    __syncthreads();
}

// Nearest-code search, ties to the lower code: the number of midpoints strictly below x.  Same result
// as the reference's q_mapping / bsearch including the end clamps (optim/cuda_adamw_kernels.cu:167-194,
// optim/adamw_fourbit_triton.py:1020-1047).  Branch-free 4-step binary search in shared memory; a NaN
// input yields code 0.
__device__ __forceinline__ uint32_t search16(float x, const float* __restrict__ mid) {
    uint32_t c = (mid[7] < x) ? 8u : 0u;
    c += (mid[c + 3] < x) ? 4u : 0u;
    c += (mid[c + 1] < x) ? 2u : 0u;
    c += (mid[c] < x) ? 1u : 0u;
    return c;
}

// x / s with the all-zero-group rule: scale 0 means every value of the group is 0 and maps to x = 0.
__device__ __forceinline__ float scaled(float x, float s) { return s == 0.0f ? 0.0f : __fdiv_rn(x, s); }

__device__ __forceinline__ void adamw_elem(float& p, float g, float& m, float& v, const QfHyper& h) {
    const float p1 = __fmul_rn(p, h.decay);
    m = __fmaf_rn(h.w1, __fsub_rn(g, m), m);
    v = __fmaf_rn(__fmul_rn(h.w2, g), g, __fmul_rn(h.beta2, v));
    const float den = __fadd_rn(__fdiv_rn(__fsqrt_rn(v), h.bc2s), h.eps);
    p = __fadd_rn(p1, __fdiv_rn(__fmul_rn(h.neg_step, m), den));
}

// The second-moment update alone; the first pass over a rank-1 tensor needs only this.
__device__ __forceinline__ float v_update(float g, float v_old, const QfHyper& h) {
    return __fmaf_rn(__fmul_rn(h.w2, g), g, __fmul_rn(h.beta2, v_old));
}

// ---- 8-element access -------------------------------------------------------------------------

template <typename T>
struct Elem;

template <>
struct Elem<float> {
    static __device__ __forceinline__ void load8(const char* base, int64_t e, float (&x)[8]) {
        const float4* q = reinterpret_cast<const float4*>(base + e * 4);
        const float4 a = q[0], b = q[1];
        x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
        x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
    }
    static __device__ __forceinline__ void store8(char* base, int64_t e, const float (&x)[8]) {
        float4* q = reinterpret_cast<float4*>(base + e * 4);
        q[0] = make_float4(x[0], x[1], x[2], x[3]);
        q[1] = make_float4(x[4], x[5], x[6], x[7]);
    }
    static __device__ __forceinline__ float load1(const char* base, int64_t e) {
        return reinterpret_cast<const float*>(base)[e];
    }
    static __device__ __forceinline__ void store1(char* base, int64_t e, float x) {
        reinterpret_cast<float*>(base)[e] = x;
    }
};

template <>
struct Elem<__nv_bfloat16> {
    static __device__ __forceinline__ void load8(const char* base, int64_t e, float (&x)[8]) {
        const uint4 r = *reinterpret_cast<const uint4*>(base + e * 2);
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            x[2 * k] = __uint_as_float(w[k] << 16);
            x[2 * k + 1] = __uint_as_float(w[k] & 0xffff0000u);
        }
    }
    static __device__ __forceinline__ void store8(char* base, int64_t e, const float (&x)[8]) {
        uint32_t w[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(x[2 * k], x[2 * k + 1]);  // nearest even
            w[k] = *reinterpret_cast<const uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(base + e * 2) = make_uint4(w[0], w[1], w[2], w[3]);
    }
    static __device__ __forceinline__ float load1(const char* base, int64_t e) {
        return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[e]);
    }
    static __device__ __forceinline__ void store1(char* base, int64_t e, float x) {
        reinterpret_cast<__nv_bfloat16*>(base)[e] = __float2bfloat16_rn(x);
    }
};

// fp16 parameters and gradients (the reference's launcher dispatches half as well, optim/cuda_adamw_kernels.cu:443):
// widened exactly, rounded to nearest even on the way back.  Tensors of this dtype always take the flat mapping.
template <>
struct Elem<__half> {
    static __device__ __forceinline__ void load8(const char* base, int64_t e, float (&x)[8]) {
        const uint4 r = *reinterpret_cast<const uint4*>(base + e * 2);
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[k]));
            x[2 * k] = f.x;
            x[2 * k + 1] = f.y;
        }
    }
    static __device__ __forceinline__ void store8(char* base, int64_t e, const float (&x)[8]) {
        uint32_t w[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const __half2 h = __floats2half2_rn(x[2 * k], x[2 * k + 1]);  // nearest even
            w[k] = *reinterpret_cast<const uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(base + e * 2) = make_uint4(w[0], w[1], w[2], w[3]);
    }
    static __device__ __forceinline__ float load1(const char* base, int64_t e) {
        return __half2float(reinterpret_cast<const __half*>(base)[e]);
    }
    static __device__ __forceinline__ void store1(char* base, int64_t e, float x) {
        reinterpret_cast<__half*>(base)[e] = __float2half_rn(x);
    }
};

// Eight elements as loaded, not yet widened: lets a loop fetch the next row before it works on this one.
template <typename T>
struct Raw8;
template <>
struct Raw8<float> {
    float4 a, b;
    __device__ __forceinline__ void load(const char* base, int64_t e) {
        const float4* q = reinterpret_cast<const float4*>(base + e * 4);
        a = q[0];
        b = q[1];
    }
    // staged layout: two arrays of 32 16-byte vectors, lane-major (see main_panel)
    __device__ __forceinline__ void from_shared(const char* arr, int lane) {
        a = *reinterpret_cast<const float4*>(arr + lane * 16);
        b = *reinterpret_cast<const float4*>(arr + (32 + lane) * 16);
    }
    __device__ __forceinline__ void widen(float (&x)[8]) const {
        x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
        x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
    }
};
template <>
struct Raw8<__nv_bfloat16> {
    uint4 r;
    __device__ __forceinline__ void from_shared(const char* arr, int lane) {
        r = *reinterpret_cast<const uint4*>(arr + lane * 16);
    }
    __device__ __forceinline__ void load(const char* base, int64_t e) { r = *reinterpret_cast<const uint4*>(base + e * 2); }
    __device__ __forceinline__ void widen(float (&x)[8]) const {
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            // byte permutes: a plain shift tends to be placed on the multiply-add pipe, which these kernels fill anyway
            asm("prmt.b32 %0, %1, 0, 0x1044;" : "=f"(x[2 * k]) : "r"(w[k]));
            asm("prmt.b32 %0, %1, 0, 0x3244;" : "=f"(x[2 * k + 1]) : "r"(w[k]));
        }
    }
};

template <>
struct Raw8<__half> {
    uint4 r;
    __device__ __forceinline__ void from_shared(const char* arr, int lane) {
        r = *reinterpret_cast<const uint4*>(arr + lane * 16);
    }
    __device__ __forceinline__ void load(const char* base, int64_t e) { r = *reinterpret_cast<const uint4*>(base + e * 2); }
    __device__ __forceinline__ void widen(float (&x)[8]) const {
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[k]));
            x[2 * k] = f.x;
            x[2 * k + 1] = f.y;
        }
    }
};

__device__ __forceinline__ void load8f(const float* base, int64_t e, float (&x)[8]) {
    Elem<float>::load8(reinterpret_cast<const char*>(base), e, x);
}

// Element k of a 32-bit word of eight codes (element 2j -> low nibble of byte j).
__device__ __forceinline__ uint32_t nib(uint32_t w, int k) { return (w >> (4 * k)) & 15u; }

// Partial (tail) load of up to 8 codes starting at even element e: bytes beyond the buffer read as 0.
__device__ __forceinline__ uint32_t load_codes_tail(const uint8_t* c, int64_t e, int nv) {
    uint32_t w = 0;
    const int nbytes = (nv + 1) >> 1;
    for (int b = 0; b < nbytes; ++b) w |= static_cast<uint32_t>(c[(e >> 1) + b]) << (8 * b);
    return w;
}
__device__ __forceinline__ void store_codes_tail(uint8_t* c, int64_t e, int nv, uint32_t w) {
    const int nbytes = (nv + 1) >> 1;
    for (int b = 0; b < nbytes; ++b) c[(e >> 1) + b] = static_cast<uint8_t>(w >> (8 * b));
}

// ---- reductions ---------------------------------------------------------------------------------

// Max over the 16 lanes that hold one 128-element block (8 elements per lane).
__device__ __forceinline__ float max16(float x) {
    x = fmaxf(x, __shfl_xor_sync(kFull, x, 1));
    x = fmaxf(x, __shfl_xor_sync(kFull, x, 2));
    x = fmaxf(x, __shfl_xor_sync(kFull, x, 4));
    x = fmaxf(x, __shfl_xor_sync(kFull, x, 8));
    return x;
}

// Non-negative floats order like their bit patterns, so maxima of |x| can be combined with integer
// max: one redux instruction across a warp and one red.max per address in global memory.  A NaN has a
// larger pattern than +inf and therefore survives the reduction.
__device__ __forceinline__ uint32_t absbits(float x) { return __float_as_uint(x) & 0x7fffffffu; }

__device__ __forceinline__ void atomic_max_nonneg(float* addr, uint32_t bits) {
    atomicMax(reinterpret_cast<unsigned int*>(addr), bits);
}

__device__ __forceinline__ bool nonfinite(float x) { return !(fabsf(x) < __builtin_huge_valf()); }

}  // namespace qf
