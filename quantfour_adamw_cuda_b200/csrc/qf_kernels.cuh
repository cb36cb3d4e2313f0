// Kernels of the fused 4-bit AdamW step for sm_100a.
//
// Work decomposition.  A warp is the unit of work: each lane owns 8 consecutive elements (one 128-bit
// load of bf16 parameters, one 32-bit word of codes), so a warp covers 256 consecutive elements = two
// 128-element quantization blocks, and a block's abs-max is a 4-step shuffle among 16 lanes with no
// shared memory and no CTA barrier.  A warp work item is
//   * for rank-1 tensors whose column count is a multiple of 256 ("panel" mapping): kRowsPerItem rows
//     of one 256-column panel.  A lane keeps the same 8 columns for the whole item, so the old and new
//     column maxima live in registers and the first pass reduces column maxima over the rows in
//     registers before touching global memory;
//   * otherwise ("flat" mapping): kRowsPerItem consecutive runs of 256 flattened elements.
// A multi-tensor launch numbers the work items of all tensors consecutively; a warp finds its tensor
// by binary search in the prefix-sum table.  CTAs hold 8 warps that take 8 consecutive items.
//
// Rank-1 second moments need the new row/column maxima of the whole tensor before any element can
// be requantized, hence two passes: `pre` recomputes v from (g, old codes) and accumulates the
// maxima with integer red.max on the bit patterns; `main` does the full update and recomputes the
// identical v (same instruction sequence) to quantize it against the finished maxima.
#pragma once

#include "qf_device.cuh"

namespace qf {

// Device-side tensor record (built by the host from QfTensorDesc).
struct DevTensor {
    char* p;
    const char* g;
    char* m;
    char* v;
    float* ms;
    float* vs;        // BLOCK: block scales; RANK1: row maxima
    float* vcol;
    float* vrow_new;
    float* vcol_new;
    int64_t numel;
    int32_t rows, cols;
    int32_t kind, dtype, hyper;
    int32_t flags;    // kFlagVec | kFlagPanel
    int32_t panels;   // panels per row band (cols / 256) for the panel mapping
    int32_t pad0;
    int64_t pad1[2];
};
static_assert(sizeof(DevTensor) == 128, "DevTensor must stay 128 bytes");

constexpr int kFlagVec = 1;    // every buffer is aligned for the vector path
constexpr int kFlagPanel = 2;  // rank-1 tensor uses the panel mapping

struct HyperPack {
    QfHyper h[QF_MAX_HYPERS];
};

// Largest t with base[t] <= item, base[0] = 0, base[n] = total.
__device__ __forceinline__ int find_tensor(const int64_t* __restrict__ base, int n, int64_t item) {
    int lo = 0, hi = n;  // invariant: base[lo] <= item < base[hi]
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (__ldg(base + mid) <= item)
            lo = mid;
        else
            hi = mid;
    }
    return lo;
}

// ---- quantize helpers on a lane's 8 values -------------------------------------------------------

__device__ __forceinline__ uint32_t quantize8(const float (&x)[8], float scale, const float* mid, int nv) {
    uint32_t w = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const uint32_t c = search16(scaled(x[k], scale), mid);
        w |= (k < nv ? c : 0u) << (4 * k);
    }
    return w;
}

__device__ __forceinline__ float absmax8_bits_to_block(const float (&x)[8]) {
    uint32_t a = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) a = max(a, absbits(x[k]));
    a = max(a, __shfl_xor_sync(kFull, a, 1));
    a = max(a, __shfl_xor_sync(kFull, a, 2));
    a = max(a, __shfl_xor_sync(kFull, a, 4));
    a = max(a, __shfl_xor_sync(kFull, a, 8));
    return __uint_as_float(a);
}

// =================================================================================================
// Panel mapping, rank-1 tensors
// =================================================================================================

template <typename T>
__device__ __forceinline__ void pre_panel(const DevTensor& t, int64_t li, const QfHyper& h, const Tables& s,
                                          uint32_t* status) {
    const int lane = threadIdx.x & 31;
    const int band = static_cast<int>(li / t.panels);
    const int panel = static_cast<int>(li - static_cast<int64_t>(band) * t.panels);
    const int r0 = band * kRowsPerItem;
    const int r1 = min(r0 + kRowsPerItem, t.rows);
    const int j0 = panel * kPanelCols + lane * 8;
    float col_old[8];
    load8f(t.vcol, j0, col_old);
    uint32_t cmax[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) cmax[k] = 0;
    const uint8_t* vc = reinterpret_cast<const uint8_t*>(t.v);
    for (int r = r0; r < r1; ++r) {
        const int64_t e = static_cast<int64_t>(r) * t.cols + j0;
        float g[8];
        Elem<T>::load8(t.g, e, g);
        const uint32_t wv = *reinterpret_cast<const uint32_t*>(vc + (e >> 1));
        const float row_old = __ldg(t.vs + r);
        uint32_t rmax = 0;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float v_old = __fmul_rn(s.qv[nib(wv, k)], fminf(row_old, col_old[k]));
            const uint32_t b = __float_as_uint(v_update(g[k], v_old, h));  // v >= 0: bits order like values
            rmax = max(rmax, b);
            cmax[k] = max(cmax[k], b);
        }
        rmax = __reduce_max_sync(kFull, rmax);
        if (lane == 0) {
            atomic_max_nonneg(t.vrow_new + r, rmax);
            if (rmax >= 0x7f800000u) atomicOr(status, QF_STATUS_NONFINITE);
        }
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) atomic_max_nonneg(t.vcol_new + j0 + k, cmax[k]);
}

template <typename T>
__device__ __forceinline__ void main_panel(const DevTensor& t, int64_t li, const QfHyper& h, const Tables& s,
                                           uint32_t* status) {
    const int lane = threadIdx.x & 31;
    const int band = static_cast<int>(li / t.panels);
    const int panel = static_cast<int>(li - static_cast<int64_t>(band) * t.panels);
    const int r0 = band * kRowsPerItem;
    const int r1 = min(r0 + kRowsPerItem, t.rows);
    const int j0 = panel * kPanelCols + lane * 8;
    float col_old[8], col_new[8];
    load8f(t.vcol, j0, col_old);
    load8f(t.vcol_new, j0, col_new);
    uint8_t* mc = reinterpret_cast<uint8_t*>(t.m);
    uint8_t* vc = reinterpret_cast<uint8_t*>(t.v);
    for (int r = r0; r < r1; ++r) {
        const int64_t e = static_cast<int64_t>(r) * t.cols + j0;
        float p[8], g[8], m[8], v[8];
        Elem<T>::load8(t.p, e, p);
        Elem<T>::load8(t.g, e, g);
        const uint32_t wm = *reinterpret_cast<const uint32_t*>(mc + (e >> 1));
        const uint32_t wv = *reinterpret_cast<const uint32_t*>(vc + (e >> 1));
        const float ms_old = __ldg(t.ms + (e >> 7));
        const float row_old = __ldg(t.vs + r);
        const float row_new = t.vrow_new[r];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            m[k] = __fmul_rn(s.qm[nib(wm, k)], ms_old);
            v[k] = __fmul_rn(s.qv[nib(wv, k)], fminf(row_old, col_old[k]));
            adamw_elem(p[k], g[k], m[k], v[k], h);
        }
        Elem<T>::store8(t.p, e, p);
        const float ms_new = absmax8_bits_to_block(m);
        *reinterpret_cast<uint32_t*>(mc + (e >> 1)) = quantize8(m, ms_new, s.mm, 8);
        if ((lane & 15) == 0) {
            t.ms[e >> 7] = ms_new;
            if (nonfinite(ms_new)) atomicOr(status, QF_STATUS_NONFINITE);
        }
        uint32_t w = 0;
#pragma unroll
        for (int k = 0; k < 8; ++k) w |= search16(scaled(v[k], fminf(row_new, col_new[k])), s.mv) << (4 * k);
        *reinterpret_cast<uint32_t*>(vc + (e >> 1)) = w;
    }
}

// =================================================================================================
// Flat mapping: fp32-state tensors, block-128 tensors, rank-1 tensors of any shape
// =================================================================================================

template <typename T>
__device__ __forceinline__ void load8_masked(const char* base, int64_t e, int nv, bool vec, float (&x)[8]) {
    if (vec && nv == 8) {
        Elem<T>::load8(base, e, x);
    } else {
#pragma unroll
        for (int k = 0; k < 8; ++k) x[k] = k < nv ? Elem<T>::load1(base, e + k) : 0.0f;
    }
}
template <typename T>
__device__ __forceinline__ void store8_masked(char* base, int64_t e, int nv, bool vec, const float (&x)[8]) {
    if (vec && nv == 8) {
        Elem<T>::store8(base, e, x);
    } else {
#pragma unroll
        for (int k = 0; k < 8; ++k)
            if (k < nv) Elem<T>::store1(base, e + k, x[k]);
    }
}
__device__ __forceinline__ uint32_t load_codes(const uint8_t* c, int64_t e, int nv, bool vec) {
    return (vec && nv == 8) ? *reinterpret_cast<const uint32_t*>(c + (e >> 1)) : load_codes_tail(c, e, nv);
}
__device__ __forceinline__ void store_codes(uint8_t* c, int64_t e, int nv, bool vec, uint32_t w) {
    if (vec && nv == 8)
        *reinterpret_cast<uint32_t*>(c + (e >> 1)) = w;
    else
        store_codes_tail(c, e, nv, w);
}

// Per-element rank-1 scale for the flat mapping: min(row[i], col[j]) for the 8 elements from e on.
__device__ __forceinline__ void rank1_scales(const float* row, const float* col, int64_t e, int nv, int cols,
                                             float (&sc)[8], int (&ri)[8], int (&ci)[8]) {
    int64_t r = e / cols;
    int c = static_cast<int>(e - r * cols);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        ri[k] = static_cast<int>(r);
        ci[k] = c;
        sc[k] = k < nv ? fminf(row[r], col[c]) : 0.0f;
        if (++c == cols) {
            c = 0;
            ++r;
        }
    }
}

template <typename T>
__device__ __forceinline__ void pre_flat_rank1(const DevTensor& t, int64_t li, const QfHyper& h, const Tables& s,
                                               uint32_t* status) {
    const int lane = threadIdx.x & 31;
    const bool vec = t.flags & kFlagVec;
    const int64_t start = li * (kPanelCols * kRowsPerItem);
    const uint8_t* vc = reinterpret_cast<const uint8_t*>(t.v);
    for (int it = 0; it < kRowsPerItem; ++it) {
        const int64_t wbase = start + static_cast<int64_t>(it) * kPanelCols;
        if (wbase >= t.numel) break;
        const int64_t e = wbase + lane * 8;
        const int nv = static_cast<int>(max(static_cast<int64_t>(0), min(static_cast<int64_t>(8), t.numel - e)));
        if (nv == 0) continue;
        float g[8], sc[8];
        int ri[8], ci[8];
        load8_masked<T>(t.g, e, nv, vec, g);
        const uint32_t wv = load_codes(vc, e, nv, vec);
        rank1_scales(t.vs, t.vcol, e, nv, t.cols, sc, ri, ci);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            if (k < nv) {
                const uint32_t b = __float_as_uint(v_update(g[k], __fmul_rn(s.qv[nib(wv, k)], sc[k]), h));
                atomic_max_nonneg(t.vrow_new + ri[k], b);
                atomic_max_nonneg(t.vcol_new + ci[k], b);
                if (b >= 0x7f800000u) atomicOr(status, QF_STATUS_NONFINITE);
            }
        }
    }
}

template <typename T, int KIND>
__device__ __forceinline__ void main_flat(const DevTensor& t, int64_t li, const QfHyper& h, const Tables& s,
                                          uint32_t* status) {
    const int lane = threadIdx.x & 31;
    const bool vec = t.flags & kFlagVec;
    const int64_t start = li * (kPanelCols * kRowsPerItem);
    uint8_t* mc = reinterpret_cast<uint8_t*>(t.m);
    uint8_t* vc = reinterpret_cast<uint8_t*>(t.v);
    for (int it = 0; it < kRowsPerItem; ++it) {
        const int64_t wbase = start + static_cast<int64_t>(it) * kPanelCols;
        if (wbase >= t.numel) break;  // warp-uniform
        const int64_t e = wbase + lane * 8;
        const int nv = static_cast<int>(max(static_cast<int64_t>(0), min(static_cast<int64_t>(8), t.numel - e)));
        float p[8], g[8], m[8], v[8];
        load8_masked<T>(t.p, e, nv, vec, p);
        load8_masked<T>(t.g, e, nv, vec, g);
        if (KIND == QF_KIND_FP32) {
            load8_masked<float>(t.m, e, nv, vec, m);
            load8_masked<float>(t.v, e, nv, vec, v);
#pragma unroll
            for (int k = 0; k < 8; ++k) adamw_elem(p[k], g[k], m[k], v[k], h);
            store8_masked<T>(t.p, e, nv, vec, p);
            store8_masked<float>(t.m, e, nv, vec, m);
            store8_masked<float>(t.v, e, nv, vec, v);
            continue;
        }
        const uint32_t wm = nv ? load_codes(mc, e, nv, vec) : 0u;
        const uint32_t wv = nv ? load_codes(vc, e, nv, vec) : 0u;
        const float ms_old = nv ? __ldg(t.ms + (e >> 7)) : 0.0f;
        float sc_old[8], sc_new[8];
        if (KIND == QF_KIND_BLOCK) {
            const float vs_old = nv ? __ldg(t.vs + (e >> 7)) : 0.0f;
#pragma unroll
            for (int k = 0; k < 8; ++k) sc_old[k] = vs_old;
        } else {
            int ri[8], ci[8];
            if (nv) {
                rank1_scales(t.vs, t.vcol, e, nv, t.cols, sc_old, ri, ci);
                rank1_scales(t.vrow_new, t.vcol_new, e, nv, t.cols, sc_new, ri, ci);
            }
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            m[k] = __fmul_rn(s.qm[nib(wm, k)], ms_old);
            v[k] = __fmul_rn(s.qv[nib(wv, k)], sc_old[k]);
            adamw_elem(p[k], g[k], m[k], v[k], h);
            if (k >= nv) {  // padding of the last block counts as zero
                m[k] = 0.0f;
                v[k] = 0.0f;
            }
        }
        store8_masked<T>(t.p, e, nv, vec, p);
        const float ms_new = absmax8_bits_to_block(m);  // all 32 lanes take part in the shuffles
        float vs_new = 0.0f;
        if (KIND == QF_KIND_BLOCK) vs_new = absmax8_bits_to_block(v);
        if (nv == 0) continue;
        store_codes(mc, e, nv, vec, quantize8(m, ms_new, s.mm, nv));
        uint32_t w = 0;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float sv = KIND == QF_KIND_BLOCK ? vs_new : sc_new[k];
            const uint32_t c = search16(scaled(v[k], sv), s.mv);
            w |= (k < nv ? c : 0u) << (4 * k);
        }
        store_codes(vc, e, nv, vec, w);
        if ((lane & 15) == 0) {
            t.ms[e >> 7] = ms_new;
            if (KIND == QF_KIND_BLOCK) t.vs[e >> 7] = vs_new;
            if (nonfinite(ms_new) || nonfinite(vs_new)) atomicOr(status, QF_STATUS_NONFINITE);
        }
    }
}

// =================================================================================================
// Multi-tensor kernels
// =================================================================================================

__global__ void __launch_bounds__(kThreads)
step_pre_kernel(const DevTensor* __restrict__ tensors, const int64_t* __restrict__ base, int n, HyperPack hp,
                uint32_t* status) {
    __shared__ Tables s;
    load_tables(s);
    const int64_t item = static_cast<int64_t>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
    if (item >= base[n]) return;
    const int ti = find_tensor(base, n, item);
    const DevTensor t = tensors[ti];
    const int64_t li = item - base[ti];
    const QfHyper& h = hp.h[t.hyper];
    if (t.flags & kFlagPanel) {
        if (t.dtype == QF_BF16)
            pre_panel<__nv_bfloat16>(t, li, h, s, status);
        else
            pre_panel<float>(t, li, h, s, status);
    } else {
        if (t.dtype == QF_BF16)
            pre_flat_rank1<__nv_bfloat16>(t, li, h, s, status);
        else
            pre_flat_rank1<float>(t, li, h, s, status);
    }
}

template <typename T>
__device__ __forceinline__ void main_dispatch(const DevTensor& t, int64_t li, const QfHyper& h, const Tables& s,
                                              uint32_t* status) {
    if (t.kind == QF_KIND_RANK1) {
        if (t.flags & kFlagPanel)
            main_panel<T>(t, li, h, s, status);
        else
            main_flat<T, QF_KIND_RANK1>(t, li, h, s, status);
    } else if (t.kind == QF_KIND_BLOCK) {
        main_flat<T, QF_KIND_BLOCK>(t, li, h, s, status);
    } else {
        main_flat<T, QF_KIND_FP32>(t, li, h, s, status);
    }
}

__global__ void __launch_bounds__(kThreads)
step_main_kernel(const DevTensor* __restrict__ tensors, const int64_t* __restrict__ base, int n, HyperPack hp,
                 uint32_t* status) {
    __shared__ Tables s;
    load_tables(s);
    const int64_t item = static_cast<int64_t>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
    if (item >= base[n]) return;
    const int ti = find_tensor(base, n, item);
    const DevTensor t = tensors[ti];
    const int64_t li = item - base[ti];
    const QfHyper& h = hp.h[t.hyper];
    if (t.dtype == QF_BF16)
        main_dispatch<__nv_bfloat16>(t, li, h, s, status);
    else
        main_dispatch<float>(t, li, h, s, status);
}

// One tensor passed by value (the single-tensor entry points that mirror the reference's per-tensor
// calls).  Block-128 and fp32-state kinds only; the non-finite flag goes to a word nobody reads.
__device__ uint32_t g_unread_status;
__global__ void __launch_bounds__(kThreads) single_tensor_kernel(DevTensor t, QfHyper h) {
    __shared__ Tables s;
    load_tables(s);
    const int64_t item = static_cast<int64_t>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
    if (item * (kPanelCols * kRowsPerItem) >= t.numel) return;
    if (t.dtype == QF_BF16)
        main_dispatch<__nv_bfloat16>(t, item, h, s, &g_unread_status);
    else
        main_dispatch<float>(t, item, h, s, &g_unread_status);
}

// mode 0: clear the scratch maxima of every rank-1 tensor; mode 1: copy them over the stored maxima.
// One CTA per (tensor, slice); tensors that are not rank-1 exit at once.
constexpr int kRollSlices = 4;
__global__ void __launch_bounds__(kThreads)
rank1_roll_kernel(const DevTensor* __restrict__ tensors, int n, int mode) {
    const int ti = blockIdx.x / kRollSlices;
    if (ti >= n) return;
    const DevTensor& t = tensors[ti];
    if (t.kind != QF_KIND_RANK1) return;
    const int total = t.rows + t.cols;
    for (int i = (blockIdx.x % kRollSlices) * kThreads + threadIdx.x; i < total; i += kRollSlices * kThreads) {
        float* nw = i < t.rows ? t.vrow_new + i : t.vcol_new + (i - t.rows);
        if (mode == 0) {
            *nw = 0.0f;
        } else {
            float* old = i < t.rows ? t.vs + i : t.vcol + (i - t.rows);
            *old = *nw;
        }
    }
}

// =================================================================================================
// Stand-alone quantize / dequantize kernels (fp32 in / out)
// =================================================================================================

// Block-128 quantize: one warp item = kRowsPerItem runs of 256 elements.
__global__ void __launch_bounds__(kThreads)
quantize_block_kernel(const float* __restrict__ x, int64_t numel, int map, uint8_t* __restrict__ codes,
                      float* __restrict__ scales, int vec) {
    __shared__ Tables s;
    load_tables(s);
    const float* mid = map ? s.mv : s.mm;
    const int lane = threadIdx.x & 31;
    const int64_t item = static_cast<int64_t>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
    const int64_t start = item * (kPanelCols * kRowsPerItem);
    for (int it = 0; it < kRowsPerItem; ++it) {
        const int64_t wbase = start + static_cast<int64_t>(it) * kPanelCols;
        if (wbase >= numel) break;
        const int64_t e = wbase + lane * 8;
        const int nv = static_cast<int>(max(static_cast<int64_t>(0), min(static_cast<int64_t>(8), numel - e)));
        float v[8];
        load8_masked<float>(reinterpret_cast<const char*>(x), e, nv, vec, v);
        const float sc = absmax8_bits_to_block(v);
        if (nv == 0) continue;
        store_codes(codes, e, nv, vec, quantize8(v, sc, mid, nv));
        if ((lane & 15) == 0) scales[e >> 7] = sc;
    }
}

__global__ void __launch_bounds__(kThreads)
dequantize_block_kernel(const uint8_t* __restrict__ codes, const float* __restrict__ scales, int64_t numel, int map,
                        float* __restrict__ out, int vec) {
    __shared__ Tables s;
    load_tables(s);
    const float* q = map ? s.qv : s.qm;
    const int lane = threadIdx.x & 31;
    const int64_t item = static_cast<int64_t>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
    const int64_t start = item * (kPanelCols * kRowsPerItem);
    for (int it = 0; it < kRowsPerItem; ++it) {
        const int64_t e = start + static_cast<int64_t>(it) * kPanelCols + lane * 8;
        if (e >= numel) break;
        const int nv = static_cast<int>(min(static_cast<int64_t>(8), numel - e));
        const uint32_t w = load_codes(codes, e, nv, vec);
        const float sc = __ldg(scales + (e >> 7));
        float v[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = __fmul_rn(q[nib(w, k)], sc);
        store8_masked<float>(reinterpret_cast<char*>(out), e, nv, vec, v);
    }
}

// Row / column maxima of |v| for an [R, C] fp32 matrix.  panel != 0: C is a multiple of 256 and the
// buffers are vector-aligned; otherwise one thread per element group with per-element atomics.
__global__ void __launch_bounds__(kThreads)
rank1_max_kernel(const float* __restrict__ v, int rows, int cols, float* __restrict__ row_max,
                 float* __restrict__ col_max, int panel) {
    const int lane = threadIdx.x & 31;
    const int64_t item = static_cast<int64_t>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
    if (panel) {
        const int panels = cols / kPanelCols;
        const int band = static_cast<int>(item / panels);
        const int r0 = band * kRowsPerItem;
        if (r0 >= rows) return;
        const int r1 = min(r0 + kRowsPerItem, rows);
        const int j0 = static_cast<int>(item - static_cast<int64_t>(band) * panels) * kPanelCols + lane * 8;
        uint32_t cmax[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) cmax[k] = 0;
        for (int r = r0; r < r1; ++r) {
            float x[8];
            load8f(v, static_cast<int64_t>(r) * cols + j0, x);
            uint32_t rmax = 0;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const uint32_t b = absbits(x[k]);
                rmax = max(rmax, b);
                cmax[k] = max(cmax[k], b);
            }
            rmax = __reduce_max_sync(kFull, rmax);
            if (lane == 0) atomic_max_nonneg(row_max + r, rmax);
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) atomic_max_nonneg(col_max + j0 + k, cmax[k]);
    } else {
        const int64_t numel = static_cast<int64_t>(rows) * cols;
        const int64_t start = item * (kPanelCols * kRowsPerItem);
        for (int it = 0; it < kRowsPerItem; ++it) {
            const int64_t e = start + static_cast<int64_t>(it) * kPanelCols + lane * 8;
            if (e >= numel) break;
            const int nv = static_cast<int>(min(static_cast<int64_t>(8), numel - e));
            int64_t r = e / cols;
            int c = static_cast<int>(e - r * cols);
            for (int k = 0; k < nv; ++k) {
                const uint32_t b = absbits(v[e + k]);
                atomic_max_nonneg(row_max + r, b);
                atomic_max_nonneg(col_max + c, b);
                if (++c == cols) {
                    c = 0;
                    ++r;
                }
            }
        }
    }
}

// Quantize / dequantize against finished row / column maxima; flat mapping over the matrix.
template <bool QUANT>
__global__ void __launch_bounds__(kThreads)
rank1_codec_kernel(const float* __restrict__ in, uint8_t* __restrict__ codes, const float* __restrict__ row_max,
                   const float* __restrict__ col_max, int rows, int cols, float* __restrict__ out, int vec) {
    __shared__ Tables s;
    load_tables(s);
    const int lane = threadIdx.x & 31;
    const int64_t numel = static_cast<int64_t>(rows) * cols;
    const int64_t item = static_cast<int64_t>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
    const int64_t start = item * (kPanelCols * kRowsPerItem);
    for (int it = 0; it < kRowsPerItem; ++it) {
        const int64_t e = start + static_cast<int64_t>(it) * kPanelCols + lane * 8;
        if (e >= numel) break;
        const int nv = static_cast<int>(min(static_cast<int64_t>(8), numel - e));
        float sc[8], x[8];
        int ri[8], ci[8];
        rank1_scales(row_max, col_max, e, nv, cols, sc, ri, ci);
        if (QUANT) {
            load8_masked<float>(reinterpret_cast<const char*>(in), e, nv, vec, x);
            uint32_t w = 0;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const uint32_t c = search16(scaled(x[k], sc[k]), s.mv);
                w |= (k < nv ? c : 0u) << (4 * k);
            }
            store_codes(codes, e, nv, vec, w);
        } else {
            const uint32_t w = load_codes(codes, e, nv, vec);
#pragma unroll
            for (int k = 0; k < 8; ++k) x[k] = __fmul_rn(s.qv[nib(w, k)], sc[k]);
            store8_masked<float>(reinterpret_cast<char*>(out), e, nv, vec, x);
        }
    }
}

}  // namespace qf
