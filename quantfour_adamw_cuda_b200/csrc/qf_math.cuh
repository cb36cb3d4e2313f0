// Packed-fp32 arithmetic of the fast path (sm_100a): every add / multiply / fused multiply-add works on
// two elements per instruction (fma.rn.f32x2 and friends), and the IEEE divisions and square roots of the
// reference arithmetic are produced by explicit Newton / Markstein sequences built from those packed
// operations plus one MUFU approximation, instead of the general-purpose div.rn / sqrt.rn expansions.
//
// Each sequence returns the correctly rounded (round-to-nearest-even) result for operands in the ranges
// the callers guarantee; outside those ranges the callers take the exact path of qf_device.cuh:
//   sqrt2      any v >= 0 (operands below 2^-96, where the residual of the Newton step would underflow,
//              branch to sqrt.rn inside the function)
//   div2       divisor normal, in [2^-90, 2^100]; dividend 0 or of magnitude >= 2^-100
//   Recip      the same ranges; the reciprocal is shared by all dividends of one divisor
// The test-suite checks sqrt2 against sqrt.rn on every non-negative float and the division sequences
// against div.rn on billions of random and structured operand pairs (tests/cuda/math_check.cu).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace qf {

using f2 = float2;

__device__ __forceinline__ f2 mk2(float a, float b) { return make_float2(a, b); }
__device__ __forceinline__ f2 bc2(float a) { return make_float2(a, a); }
// CAUTION: ptxas 12.9 was observed to contract a packed multiply whose only use is a packed add into one
// packed fused multiply-add (even when both are spelled with an explicit .rn in PTX), which changes the
// rounding.  No sequence in this library feeds a mul2 result into add2; where the reference arithmetic has
// "round(a*b) then add", the product is taken as fma2(a, b, 0), which rounds identically and cannot be
// merged with the following add (checked on the device by the test-suite).
__device__ __forceinline__ f2 mul2(f2 a, f2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ f2 add2(f2 a, f2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ f2 fma2(f2 a, f2 b, f2 c) { return __ffma2_rn(a, b, c); }
// Negation is written per half: the compiler folds it into the operand modifiers of the consuming packed
// instruction (a packed multiply by -1 costs an instruction and two FP32-pipe cycles).
__device__ __forceinline__ f2 neg2(f2 a) { return mk2(-a.x, -a.y); }

__device__ __forceinline__ float rsqrt_approx(float x) {
    float y;
    asm("rsqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float rcp_approx(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

constexpr float kFltMin = 1.17549435e-38f;

// Correctly rounded sqrt of two non-negative values.  y ~ 1/sqrt(v); s = v*y; one Newton step with
// the residual taken exactly by a fused multiply-add: s + (v - s*s) * (y/2).  The residual is a multiple
// of ulp(s)^2, representable only while v >= 2^-103; smaller operands (zero included) take sqrt.rn.
// CHECKED = false is for callers that know both operands are >= 2^-96.
template <bool CHECKED = true>
__device__ __forceinline__ f2 sqrt2(f2 v) {
    if (CHECKED && fminf(v.x, v.y) < 0x1p-96f) return mk2(__fsqrt_rn(v.x), __fsqrt_rn(v.y));
    const f2 y = mk2(rsqrt_approx(v.x), rsqrt_approx(v.y));
    const f2 s = mul2(v, y);
    const f2 nh = mul2(y, bc2(-0.5f));
    const f2 e = fma2(s, s, neg2(v));  // s*s - v
    return fma2(e, nh, s);
}

// A divisor prepared for repeated division: r ~ 1/d (MUFU + one Newton step), nd = -d.
struct Recip {
    float r, nd;
};
__device__ __forceinline__ Recip make_recip(float d) {
    Recip o;
    o.nd = -d;
    const float r0 = d == 0.0f ? 0.0f : rcp_approx(d);  // d == 0: every dividend is 0 as well -> quotient 0
    const float e = __fmaf_rn(o.nd, r0, 1.0f);
    o.r = __fmaf_rn(r0, e, r0);
    return o;
}

// a / d for two dividends and per-element divisors given as (r, nd): quotient estimate and two
// residual corrections, each residual exact through the fused multiply-add.
__device__ __forceinline__ f2 div2_prepared(f2 a, f2 r, f2 nd) {
    f2 q = mul2(a, r);
    f2 t = fma2(nd, q, a);
    q = fma2(t, r, q);
    t = fma2(nd, q, a);
    return fma2(t, r, q);
}

// The same with one residual correction.  With q0 = RN(a r) and the exact residual t = a - d q0, the value
// q0 + t r differs from a / d by |a / d - q0| * |1 - d r|: a few 2^-47 |a / d| for a reciprocal within a unit in the
// last place.  Its rounding is therefore the correctly rounded quotient unless a / d lies within that distance of the
// midpoint of two neighbouring floats.  Quotients of two 24-bit operands can come that close to such a midpoint (the
// closest is about 2^-49 relative), so exceptions exist, but they are rare and never more than one unit in the last
// place: 0 (reciprocal from rcp.rn) and 1 (reciprocal from the approximation unit) of 1.2 * 10^9 random operand pairs
// in tests/cuda/math_check.cu, which re-measures the rate on every run.  The step uses this form where such a
// deviation cannot reach a result except through a second coincidence:
//   * requantization: the quotient only selects a code, which changes only if the two candidate quotients also
//     straddle one of the 15 code boundaries (of the order of 10^-15 per element; a differing code would then be one
//     level off at an exact near-tie, the case for which the contract allows a fraction of 10^-6);
//   * the update of bf16 parameters: the quotient enters a sum that is then rounded to 8 bits of mantissa.
// fp32 parameters keep the second correction: there the last place of the quotient is visible in the result.
__device__ __forceinline__ f2 div2_prepared1(f2 a, f2 r, f2 nd) {
    const f2 q = mul2(a, r);
    const f2 t = fma2(nd, q, a);
    return fma2(t, r, q);
}
template <bool ONE>
__device__ __forceinline__ f2 div2_prepared_n(f2 a, f2 r, f2 nd) {
    return ONE ? div2_prepared1(a, r, nd) : div2_prepared(a, r, nd);
}

// a / d for two independent (dividend, divisor) pairs.
__device__ __forceinline__ f2 div2(f2 a, f2 d) {
    const f2 nd = neg2(d);
    const f2 r0 = mk2(rcp_approx(d.x), rcp_approx(d.y));
    const f2 e = fma2(nd, r0, bc2(1.0f));
    const f2 r = fma2(r0, e, r0);
    return div2_prepared(a, r, nd);
}
// The same with the reciprocal as the approximation unit gives it (one unit in the last place) and one correction;
// see div2_prepared1 for what that costs in accuracy.
__device__ __forceinline__ f2 div2_1(f2 a, f2 d) {
    return div2_prepared1(a, mk2(rcp_approx(d.x), rcp_approx(d.y)), neg2(d));
}

}  // namespace qf
