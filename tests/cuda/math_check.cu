// Device-side checks of the packed fast-path arithmetic (quantfour_adamw_cuda_b200/csrc/qf_math.cuh and the
// table / closed-form searches of qf_kernels.cuh) against the plain IEEE intrinsics and the 4-step binary
// search.  Test infrastructure: built into tests/cuda/libqf_mathcheck.so, loaded only by the test-suite.
#include <cstdint>
#include <cstdio>

#include "../../quantfour_adamw_cuda_b200/csrc/qf_kernels.cuh"

namespace {

struct Report {
    unsigned long long checked, bad;
    unsigned int first_a, first_b;
};

__device__ void note(Report* r, uint32_t a, uint32_t b) {
    if (atomicAdd(&r->bad, 1ull) == 0) {
        r->first_a = a;
        r->first_b = b;
    }
}

// sqrt2 against sqrt.rn for every float bit pattern in [lo, hi).
__global__ void k_sqrt(uint32_t lo, uint64_t count, Report* r) {
    for (uint64_t i = (blockIdx.x * (uint64_t)blockDim.x + threadIdx.x) * 2; i < count; i += (uint64_t)gridDim.x * blockDim.x * 2) {
        const float a = __uint_as_float(lo + (uint32_t)i), b = __uint_as_float(lo + (uint32_t)i + 1);
        const qf::f2 s = qf::sqrt2(qf::mk2(a, b));
        if (__float_as_uint(s.x) != __float_as_uint(__fsqrt_rn(a))) note(r, __float_as_uint(a), __float_as_uint(s.x));
        if (i + 1 < count && __float_as_uint(s.y) != __float_as_uint(__fsqrt_rn(b))) note(r, __float_as_uint(b), __float_as_uint(s.y));
    }
}

__device__ uint64_t splitmix(uint64_t& x) {
    uint64_t z = (x += 0x9e3779b97f4a7c15ull);
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}

// A float with random sign (if sgn), random mantissa and an exponent drawn from [emin, emax] (unbiased).
__device__ float rnd_float(uint64_t& st, int emin, int emax, bool sgn, int mant_mode) {
    const uint64_t z = splitmix(st);
    uint32_t mant = (uint32_t)z & 0x7fffffu;
    if (mant_mode == 1) mant = 0x7fffffu - ((uint32_t)(z >> 40) & 0xffu);   // mantissa near all ones
    if (mant_mode == 2) mant = (uint32_t)(z >> 40) & 0xffu;                  // mantissa near zero
    const int e = emin + (int)((z >> 23) % (uint64_t)(emax - emin + 1));
    uint32_t bits = ((uint32_t)(e + 127) << 23) | mant;
    if (sgn && (z >> 63)) bits |= 0x80000000u;
    return __uint_as_float(bits);
}

// mode 0: div2 (independent divisors, MUFU reciprocal);  mode 1: div2_prepared with r = rcp.rn(d);
// mode 2: div2_prepared with r = RN(1/d) and a restricted dividend range (|a| <= d, the quantize case).
__global__ void k_div(uint64_t seed, uint64_t per_thread, int mode, int a_emin, int a_emax, int d_emin, int d_emax,
                      int mant_mode, Report* r) {
    uint64_t st = seed ^ ((blockIdx.x * (uint64_t)blockDim.x + threadIdx.x) * 0x2545f4914f6cdd1dull);
    for (uint64_t i = 0; i < per_thread; ++i) {
        const float d0 = rnd_float(st, d_emin, d_emax, false, mant_mode), d1 = rnd_float(st, d_emin, d_emax, false, mant_mode);
        float a0 = rnd_float(st, a_emin, a_emax, true, (int)(i & 1) * mant_mode), a1 = rnd_float(st, a_emin, a_emax, true, 0);
        if (mode == 2) {
            a0 = a0 * d0;
            a1 = a1 * d1;
        }
        qf::f2 q;
        if (mode == 0) {
            q = qf::div2(qf::mk2(a0, a1), qf::mk2(d0, d1));
        } else {
            q = qf::div2_prepared(qf::mk2(a0, a1), qf::mk2(__frcp_rn(d0), __frcp_rn(d1)), qf::mk2(-d0, -d1));
        }
        if (__float_as_uint(q.x) != __float_as_uint(__fdiv_rn(a0, d0))) note(r, __float_as_uint(a0), __float_as_uint(d0));
        if (__float_as_uint(q.y) != __float_as_uint(__fdiv_rn(a1, d1))) note(r, __float_as_uint(a1), __float_as_uint(d1));
    }
}

// The single-correction forms (div2_prepared1 with r = rcp.rn(d) in mode 0, div2_1 in mode 1): `bad` counts quotients
// that differ from div.rn, `checked` those that differ by more than one unit in the last place (must stay 0).  With
// codes != 0 the quotient is additionally turned into a first-moment code (table search) and a second-moment code
// (closed form) and first_a / first_b count the codes that differ from those of the exact quotient.
__global__ void k_div1(uint64_t seed, uint64_t per_thread, int mode, int a_emin, int a_emax, int d_emin, int d_emax,
                       int mant_mode, int codes, Report* r) {
    __shared__ qf::Smem s;
    qf::load_smem(s);
    uint64_t st = seed ^ ((blockIdx.x * (uint64_t)blockDim.x + threadIdx.x) * 0x2545f4914f6cdd1dull);
    for (uint64_t i = 0; i < per_thread; ++i) {
        const float d[2] = {rnd_float(st, d_emin, d_emax, false, mant_mode), rnd_float(st, d_emin, d_emax, false, mant_mode)};
        float a[2] = {rnd_float(st, a_emin, a_emax, true, (int)(i & 1) * mant_mode), rnd_float(st, a_emin, a_emax, true, 0)};
        if (codes) {
            a[0] *= d[0];
            a[1] *= d[1];
        }
        const qf::f2 q = mode == 0 ? qf::div2_prepared1(qf::mk2(a[0], a[1]), qf::mk2(__frcp_rn(d[0]), __frcp_rn(d[1])), qf::mk2(-d[0], -d[1]))
                                   : qf::div2_1(qf::mk2(a[0], a[1]), qf::mk2(d[0], d[1]));
        const float got[2] = {q.x, q.y};
        for (int k = 0; k < 2; ++k) {
            const float want = __fdiv_rn(a[k], d[k]);
            const int32_t dist = (int32_t)__float_as_uint(got[k]) - (int32_t)__float_as_uint(want);
            if (dist != 0) atomicAdd(&r->bad, 1ull);
            if (dist > 1 || dist < -1) atomicAdd(&r->checked, 1ull);
            if (codes) {
                if (qf::search_m_lut(got[k], s.mlut, s.t.mm) != qf::search_m_lut(want, s.mlut, s.t.mm)) atomicAdd(&r->first_a, 1u);
                if (qf::search_v_closed(fabsf(got[k])) != qf::search_v_closed(fabsf(want))) atomicAdd(&r->first_b, 1u);
            }
        }
    }
}

// div2_prepared over every mantissa of the dividend (one binade, both signs folded into the index) against 64 divisors
// spread over a binade: all-zero and all-one mantissas, their neighbours, and an odd-strided walk in between.  The
// reciprocal comes from make_recip (what the kernels use for a block scale) when recip_mode is 0, from rcp.rn otherwise.
__global__ void k_div_all_mantissas(int a_exp, int d_exp, int recip_mode, Report* r) {
    const uint64_t total = (1ull << 23) * 64;
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x * 2) {
        float a[2], d[2];
        for (int k = 0; k < 2; ++k) {
            const uint64_t idx = i + (uint64_t)k * gridDim.x * blockDim.x;
            const uint32_t am = (uint32_t)(idx & 0x7fffffu), dk = (uint32_t)(idx >> 23) & 63u;
            uint32_t dm = dk < 4 ? dk : dk >= 60 ? 0x7fffffu - (63u - dk) : (dk * 0x20c49bu + 0x1357u) & 0x7fffffu;
            a[k] = __uint_as_float(((uint32_t)(a_exp + 127) << 23) | am);
            d[k] = __uint_as_float(((uint32_t)(d_exp + 127) << 23) | dm);
        }
        qf::f2 rr, nd = qf::mk2(-d[0], -d[1]);
        if (recip_mode == 0) {
            rr = qf::mk2(qf::make_recip(d[0]).r, qf::make_recip(d[1]).r);
        } else {
            rr = qf::mk2(__frcp_rn(d[0]), __frcp_rn(d[1]));
        }
        const qf::f2 q = qf::div2_prepared(qf::mk2(a[0], a[1]), rr, nd);
        if (__float_as_uint(q.x) != __float_as_uint(__fdiv_rn(a[0], d[0]))) note(r, __float_as_uint(a[0]), __float_as_uint(d[0]));
        if (i + (uint64_t)gridDim.x * blockDim.x < total && __float_as_uint(q.y) != __float_as_uint(__fdiv_rn(a[1], d[1])))
            note(r, __float_as_uint(a[1]), __float_as_uint(d[1]));
    }
}

// "round(a*b), then add c" written the way the kernels write it -- fma2(a, b, 0) followed by add2 -- must
// round twice like mul.rn + add.rn.
__global__ void k_nofuse(uint64_t seed, uint64_t per_thread, Report* r) {
    uint64_t st = seed ^ ((blockIdx.x * (uint64_t)blockDim.x + threadIdx.x) * 0x2545f4914f6cdd1dull);
    for (uint64_t i = 0; i < per_thread; ++i) {
        const float a0 = rnd_float(st, -8, 0, true, 0), a1 = rnd_float(st, -8, 0, true, 0);
        const float b0 = rnd_float(st, -1, 0, false, 0), b1 = rnd_float(st, -1, 0, false, 0);
        const float c0 = rnd_float(st, -12, -6, true, 0), c1 = rnd_float(st, -12, -6, true, 0);
        const qf::f2 d = qf::add2(qf::fma2(qf::mk2(a0, a1), qf::mk2(b0, b1), qf::bc2(0.0f)), qf::mk2(c0, c1));
        if (__float_as_uint(d.x) != __float_as_uint(__fadd_rn(__fmul_rn(a0, b0), c0))) note(r, __float_as_uint(a0), __float_as_uint(b0));
        if (__float_as_uint(d.y) != __float_as_uint(__fadd_rn(__fmul_rn(a1, b1), c1))) note(r, __float_as_uint(a1), __float_as_uint(b1));
    }
}

// Both searches against the 4-step binary search for every float bit pattern.
__global__ void k_search(Report* r) {
    __shared__ qf::Smem s;
    qf::load_smem(s);
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < (1ull << 32); i += (uint64_t)gridDim.x * blockDim.x) {
        const float x = __uint_as_float((uint32_t)i);
        if (x != x) continue;  // NaN is outside the contract of the fast searches
        if (qf::search_m_lut(x, s.mlut, s.t.mm) != qf::search16(x, s.t.mm)) note(r, (uint32_t)i, 0);
        if (qf::search_v_closed(x) != qf::search16(x, s.t.mv)) note(r, (uint32_t)i, 1);
    }
}

// Code -> value reconstruction of the fast dequantize: (2^23 + c) - (2^23 - 1) = c + 1 and (c + 1) * (s / 16)
// against qv[c] * s, for all 16 codes and `count` scale bit patterns from `lo` on.
__global__ void k_dequant_v(uint32_t lo, uint64_t count, Report* r) {
    __shared__ qf::Smem s;
    qf::load_smem(s);
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < count * 16; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t c = (uint32_t)(i & 15);
        const float sc = __uint_as_float(lo + (uint32_t)(i >> 4));
        if (!qf::scale_safe(sc)) continue;
        const float fast = __fmul_rn(__fadd_rn(qf::code_plus_2p23(c, 0), qf::kMagic), sc * 0.0625f);
        if (__float_as_uint(fast) != __float_as_uint(__fmul_rn(s.t.qv[c], sc))) note(r, c, __float_as_uint(sc));
    }
}

// ---- dispatch probe ------------------------------------------------------------------------------------------
// How many cycles an SM sub-partition needs per warp instruction of a class, alone and mixed 1 : 1 with packed FMAs:
// NF independent packed FMAs and NA independent instructions of class KIND (0 lop3, 1 prmt, 2 funnel shift, 3 integer
// multiply-add, 4 scalar fma) per group, four warps per sub-partition: the yardstick behind the statement that the step
// kernels are bound by instruction dispatch.
template <int NF, int NA, int KIND>
__global__ void __launch_bounds__(256) k_probe(float2* out, unsigned* iout, int iters, float2 a, float2 b, unsigned k) {
    float2 f[8];
    unsigned u[8];
    float s[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        f[i] = make_float2(threadIdx.x + i, i);
        u[i] = threadIdx.x * 7 + i;
        s[i] = i + threadIdx.x;
    }
    for (int it = 0; it < iters; ++it) {
#pragma unroll
        for (int rep = 0; rep < 4; ++rep) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                if (i < NF) f[i] = __ffma2_rn(f[i], a, b);
                if (i < NA) {
                    unsigned& x = u[i];
                    if (KIND == 0) asm volatile("lop3.b32 %0, %1, %2, %3, 0x6a;" : "=r"(x) : "r"(x), "r"(k), "r"(u[(i + 3) & 7]));
                    if (KIND == 1) asm volatile("prmt.b32 %0, %1, %2, 0x3021;" : "=r"(x) : "r"(x), "r"(k));
                    if (KIND == 2) x = __funnelshift_r(x, k, 3);
                    if (KIND == 3) asm volatile("mad.lo.u32 %0, %1, %2, %3;" : "=r"(x) : "r"(x), "r"(k), "r"(u[(i + 3) & 7]));
                    if (KIND == 4) s[i] = __fmaf_rn(s[i], a.x, b.x);
                }
            }
        }
    }
    float2 acc = make_float2(0, 0);
    unsigned ua = 0;
    for (int i = 0; i < 8; ++i) {
        acc.x += f[i].x + s[i];
        acc.y += f[i].y;
        ua += u[i];
    }
    out[blockIdx.x * blockDim.x + threadIdx.x] = acc;
    iout[blockIdx.x * blockDim.x + threadIdx.x] = ua;
}

template <int NF, int NA, int KIND>
double probe_ms(float2* out, unsigned* iout, int iters) {
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    const float2 a = make_float2(1.0001f, 0.9f), b = make_float2(0.5f, 0.25f);
    k_probe<NF, NA, KIND><<<148 * 2, 256>>>(out, iout, 50, a, b, 0x1234u);
    cudaEventRecord(e0);
    k_probe<NF, NA, KIND><<<148 * 2, 256>>>(out, iout, iters, a, b, 0x1234u);
    cudaEventRecord(e1);
    cudaDeviceSynchronize();
    float ms = 0;
    cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    return ms;
}

int finish(Report* d, unsigned long long* checked_bad, unsigned int* first) {
    Report h;
    cudaError_t e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = cudaMemcpy(&h, d, sizeof h, cudaMemcpyDeviceToHost);
    cudaFree(d);
    if (e != cudaSuccess) {
        fprintf(stderr, "math_check: %s\n", cudaGetErrorString(e));
        return 1;
    }
    checked_bad[0] = h.bad;
    first[0] = h.first_a;
    first[1] = h.first_b;
    return 0;
}

Report* fresh() {
    Report* d = nullptr;
    if (cudaMalloc(&d, sizeof(Report)) != cudaSuccess) return nullptr;
    cudaMemset(d, 0, sizeof(Report));
    return d;
}

}  // namespace

extern "C" {

int qfc_sqrt(uint32_t lo_bits, uint64_t count, unsigned long long* bad, unsigned int* first) {
    Report* d = fresh();
    if (!d) return 1;
    k_sqrt<<<148 * 8, 256>>>(lo_bits, count, d);
    return finish(d, bad, first);
}

int qfc_div(uint64_t seed, uint64_t per_thread, int mode, int a_emin, int a_emax, int d_emin, int d_emax, int mant_mode,
            unsigned long long* bad, unsigned int* first) {
    Report* d = fresh();
    if (!d) return 1;
    k_div<<<148 * 8, 256>>>(seed, per_thread, mode, a_emin, a_emax, d_emin, d_emax, mant_mode, d);
    return finish(d, bad, first);
}

// out[0] = quotients that differ from div.rn, out[1] = by more than one unit, out[2] / out[3] = differing first- /
// second-moment codes (only with codes != 0)
int qfc_div1(uint64_t seed, uint64_t per_thread, int mode, int a_emin, int a_emax, int d_emin, int d_emax, int mant_mode,
             int codes, unsigned long long* out) {
    Report* d = fresh();
    if (!d) return 1;
    k_div1<<<148 * 8, 256>>>(seed, per_thread, mode, a_emin, a_emax, d_emin, d_emax, mant_mode, codes, d);
    Report h;
    cudaError_t e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = cudaMemcpy(&h, d, sizeof h, cudaMemcpyDeviceToHost);
    cudaFree(d);
    if (e != cudaSuccess) {
        fprintf(stderr, "math_check: %s\n", cudaGetErrorString(e));
        return 1;
    }
    out[0] = h.bad;
    out[1] = h.checked;
    out[2] = h.first_a;
    out[3] = h.first_b;
    return 0;
}

int qfc_div_all_mantissas(int a_exp, int d_exp, int recip_mode, unsigned long long* bad, unsigned int* first) {
    Report* d = fresh();
    if (!d) return 1;
    k_div_all_mantissas<<<148 * 8, 256>>>(a_exp, d_exp, recip_mode, d);
    return finish(d, bad, first);
}

int qfc_nofuse(uint64_t seed, uint64_t per_thread, unsigned long long* bad, unsigned int* first) {
    Report* d = fresh();
    if (!d) return 1;
    k_nofuse<<<148 * 8, 256>>>(seed, per_thread, d);
    return finish(d, bad, first);
}

int qfc_search(unsigned long long* bad, unsigned int* first) {
    Report* d = fresh();
    if (!d) return 1;
    k_search<<<148 * 4, 256>>>(d);
    return finish(d, bad, first);
}

int qfc_dequant_v(uint32_t lo_bits, uint64_t count, unsigned long long* bad, unsigned int* first) {
    Report* d = fresh();
    if (!d) return 1;
    k_dequant_v<<<148 * 8, 256>>>(lo_bits, count, d);
    return finish(d, bad, first);
}

// out[0..10]: milliseconds of (packed FMA alone; lop3, prmt, shift, imad, scalar fma alone; each of those five mixed
// 1 : 1 with packed FMAs), 8 instructions of each class per group; out[11] = groups per warp.  Four warps per SM
// sub-partition, so cycles per group per sub-partition = ms * clock / (4 * groups).
int qfc_issue_probe(double* out) {
    float2* o = nullptr;
    unsigned* io = nullptr;
    if (cudaMalloc(&o, 148 * 2 * 256 * sizeof(float2)) != cudaSuccess || cudaMalloc(&io, 148 * 2 * 256 * 4) != cudaSuccess) return 1;
    const int iters = 5000;
    out[0] = probe_ms<8, 0, 0>(o, io, iters);
    out[1] = probe_ms<0, 8, 0>(o, io, iters);
    out[2] = probe_ms<0, 8, 1>(o, io, iters);
    out[3] = probe_ms<0, 8, 2>(o, io, iters);
    out[4] = probe_ms<0, 8, 3>(o, io, iters);
    out[5] = probe_ms<0, 8, 4>(o, io, iters);
    out[6] = probe_ms<8, 8, 0>(o, io, iters);
    out[7] = probe_ms<8, 8, 1>(o, io, iters);
    out[8] = probe_ms<8, 8, 2>(o, io, iters);
    out[9] = probe_ms<8, 8, 3>(o, io, iters);
    out[10] = probe_ms<8, 8, 4>(o, io, iters);
    out[11] = 4.0 * iters;
    const cudaError_t e = cudaDeviceSynchronize();
    cudaFree(o);
    cudaFree(io);
    return e == cudaSuccess ? 0 : 1;
}

int qfc_threads(void) { return 148 * 8 * 256; }

}  // extern "C"
