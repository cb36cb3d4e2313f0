// Kernels of the fused 4-bit AdamW step for sm_100a.
//
// Work decomposition.  A warp is the unit of work: each lane owns 8 consecutive elements (one 128-bit
// load of bf16 parameters, one 32-bit word of codes), so a warp covers 256 consecutive elements = two
// 128-element quantization blocks, and a block's abs-max is a 4-step shuffle among 16 lanes with no
// shared memory and no CTA barrier.  A warp work item is
//   * for rank-1 tensors whose column count is a multiple of 256 ("panel" mapping): 64 rows of one
//     256-column panel.  A lane keeps the same 8 columns for the whole item, so everything that depends on
//     the column only (old and new column maxima, their reciprocals) is fetched once per item (registers in
//     the first pass, the warp's slice of shared memory in the main pass), and the first pass reduces column
//     maxima over the rows in registers before touching global memory;
//   * otherwise ("flat" mapping): kRowsPerItem (16) consecutive runs of 256 flattened elements.
// A multi-tensor launch numbers the work items of all tensors of one mapping consecutively; a warp finds
// its tensor by binary search in the prefix-sum table.  The step kernels are persistent: CTAs of 8 warps,
// every warp striding over the item list.
//
// Rank-1 second moments need the new row/column maxima of the whole tensor before any element can be
// requantized, hence two passes: `pre` recomputes v from (g, old codes) and accumulates the maxima with
// integer red.max on the bit patterns; `main` does the full update and recomputes the identical v to
// quantize it against the finished maxima.  A small kernel in between stores the reciprocals of the new
// maxima so that the main pass divides by multiplication plus exact residual correction.
//
// Arithmetic.  The path is instruction-issue bound on B200 if written with the general IEEE division and
// square-root expansions (about 135 instructions per element), so the hot loops use the packed-fp32
// sequences of qf_math.cuh (two elements per instruction, about 50 instructions per element) and take the
// plain IEEE intrinsics of qf_device.cuh only where an operand leaves the range those sequences are valid
// for.  Both give the same bits; the choice is warp-uniform.
#pragma once

#include <type_traits>

#include "qf_device.cuh"
#include "qf_math.cuh"

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
    float* vrow_new;  // [rows]: new row maxima
    float* vcol_new;  // [cols]: new column maxima
    float* vrow_rcp;  // [rows]: reciprocals of the new row maxima (NaN-tagged, see rank1_roll_kernel)
    float* vcol_rcp;  // [cols]: the same for the columns
    int64_t numel;    // elements this record covers
    int64_t flat_off; // RANK1, flat mapping: elements of the matrix that precede this record's first one
    int32_t rows, cols;
    int32_t kind, dtype, hyper;
    int32_t flags;    // kFlagVec | kFlagPanel
    int32_t panels;   // panels per row band (cols / 256) for the panel mapping
    int32_t main_rows;  // panel mapping: rows of one item of the second pass (kMainRowsPerItem, or fewer on small launches)
    int64_t pad1[3];
};
static_assert(sizeof(DevTensor) == 160, "DevTensor must stay 160 bytes");

constexpr int kFlagVec = 1;    // every buffer is aligned for the vector path
constexpr int kFlagPanel = 2;  // rank-1 tensor uses the panel mapping

// Hyper-parameters as the kernels take them: the public scalars plus what the fast path needs.
struct HyperDev {
    QfHyper h;
    float rb;    // RN(1 / bc2s)
    float nb;    // -bc2s
    int32_t fast;  // 0: the scalars are outside the ranges the fast sequences cover -> exact path only
    float gs;      // gradient scale (1 = none): g is replaced in place by RN(g * gs) in its own dtype before it is used
};

// x as a value of the parameter / gradient dtype (what a store followed by a load would give).
template <typename T>
__device__ __forceinline__ float round_as(float x);
template <>
__device__ __forceinline__ float round_as<float>(float x) { return x; }
template <>
__device__ __forceinline__ float round_as<__nv_bfloat16>(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
template <>
__device__ __forceinline__ float round_as<__half>(float x) { return __half2float(__float2half_rn(x)); }
struct HyperPack {
    HyperDev h[QF_MAX_HYPERS];
};

// The scalars as the kernels take them.  The packed sequences of the fast path need: finite scalars, an
// eps that absorbs the square root of a denormal second moment (>= 2^-40), a bias correction whose
// reciprocal is well defined, and a non-degenerate step size; anything else runs the exact path.
// Host and device give the same result: the one division is an IEEE double division on both.
__host__ __device__ inline HyperDev widen_hyper(const QfHyper& h) {
    HyperDev d;
    d.h = h;
    d.rb = static_cast<float>(1.0 / static_cast<double>(h.bc2s));  // double rounding is harmless for 1/x
    d.nb = -h.bc2s;
    d.gs = h.grad_scale == 0.0f ? 1.0f : h.grad_scale;
    const float all[] = {h.decay, h.w1, h.beta2, h.w2, h.eps, h.neg_step, h.bc2s};
    bool ok = true;
    for (float x : all) ok = ok && fabsf(x) <= 3.4028234663852886e38f;  // finite: false for NaN and infinities
    ok = ok && h.eps >= 0x1p-40f && h.eps <= 0x1p40f && h.bc2s >= 0x1p-30f && h.bc2s <= 2.0f;
    ok = ok && fabsf(h.neg_step) <= 0x1p40f && fabsf(h.decay) <= 0x1p40f && h.beta2 >= 0.0f && h.w2 >= 0.0f;
    d.fast = ok ? 1 : 0;
    return d;
}

// Hyper-parameters kept on the device, for a step that is recorded into a CUDA graph and replayed without the
// host: `table` holds `rows` rows of `n_hypers` sets (row r = the scalars of the r-th step after the table was
// written, derived on the host in doubles like every other set), counters[0] is the row the next step takes and
// counters[1] counts the steps done.  A step past the last row takes the last row again.
struct Sched {
    const QfHyper* table;
    const int32_t* counters;
    int32_t rows;
    int32_t n_hypers;
};
// The sets of the current row, widened, into shared memory; the caller's next __syncthreads() publishes them.
__device__ __forceinline__ void load_sched(HyperDev* sh, const Sched& sc) {
    if (threadIdx.x < sc.n_hypers) {
        const int32_t r = min(max(sc.counters[0], 0), sc.rows - 1);
        sh[threadIdx.x] = widen_hyper(sc.table[static_cast<int64_t>(r) * sc.n_hypers + threadIdx.x]);
    }
}

// Peer copies of the parameter buffer (sharded step): every updated parameter vector is stored at
// p + delta[k] as well, k < n, where delta[k] is the byte distance from this device's parameter buffer to
// the mapping of peer k's buffer.  The stores ride the peer links while the update computes.
struct PushPack {
    int32_t n;
    int32_t pad;
    int64_t delta[QF_MAX_PEERS];
};
template <typename T>
__device__ __forceinline__ void push_store8(char* base, int64_t e, const float (&x)[8], const PushPack* push) {
    const int n = push->n;
    for (int k = 0; k < n; ++k) Elem<T>::store8(base + push->delta[k], e, x);
}

// ---- first-moment search table ------------------------------------------------------------------------
// Index = sign, exponent and two mantissa bits of x (bits 31..21).  The floats that share an index form an
// interval that holds at most one of the 15 midpoints.  The table holds, per index, the number `base` of midpoints
// below the interval; code(x) = base + (mid[base] < x): mid[base] is the smallest midpoint that is not below the
// interval, i.e. the one inside it or one above it (then above x as well; mid[15] = +inf).  One byte per entry and the
// threshold from the 16-entry table, which cannot have a bank conflict, instead of (threshold, count) pairs of eight
// bytes: a warp's 32 look-ups then take about 3 shared-memory wavefronts instead of 5 (main pass -2.7 %, measured).
// Built at compile time from the midpoints' bit patterns.
struct Lut {
    alignas(16) uint8_t base[2048];
};
constexpr uint32_t kMidBits[15] = {0xbf466666u, 0xbf0ccccdu, 0xbea66666u, 0xbe147ae1u, 0xbd6147aeu,
                                   0xbc9ba5e3u, 0xbb343958u, 0x3b343958u, 0x3c9ba5e3u, 0x3d6147aeu,
                                   0x3e147ae1u, 0x3ea66666u, 0x3f0ccccdu, 0x3f466666u, 0x3f71999au};
constexpr Lut make_lut() {
    Lut t{};
    for (int idx = 0; idx < 2048; ++idx) {
        const uint32_t lo = static_cast<uint32_t>(idx & 1023) << 21, hi = lo | 0x1fffffu;  // magnitudes
        uint32_t base = 0;
        if (idx < 1024) {  // x >= 0: all seven negative midpoints are below
            base = 7;
            for (int k = 7; k < 15; ++k)
                if (kMidBits[k] < lo) ++base;
        } else {  // x < 0: a midpoint -a is below the interval [-hi, -lo] iff a > hi
            for (int k = 0; k < 7; ++k)
                if ((kMidBits[k] & 0x7fffffffu) > hi) ++base;
        }
        t.base[idx] = static_cast<uint8_t>(base);
    }
    return t;
}
__device__ const Lut g_mlut = make_lut();

// Shared memory of a CTA: the 16-entry tables (exact path), the first-moment search table, and two
// byte-indexed pair tables for the fast dequantize: a byte of packed codes (two elements) fetches the two
// map values of either moment with one 64-bit load.
// What the first pass needs of it.
struct SmemPre {
    Tables t;
    float2 qv2[256];
};
__device__ __forceinline__ void load_smem(SmemPre& s) {
    for (int i = threadIdx.x; i < 256; i += blockDim.x) s.qv2[i] = make_float2(c_qv[i & 15], c_qv[i >> 4]);
    load_tables(s.t);  // ends with __syncthreads()
}
struct Smem {
    Tables t;
    alignas(16) uint8_t mlut[2048];
    float2 qm2[256];   // (qm[b & 15], qm[b >> 4])
    float2 qv2[256];   // (qv[b & 15], qv[b >> 4])
};

__device__ __forceinline__ void load_smem(Smem& s) {
    for (int i = threadIdx.x; i < 512; i += blockDim.x)
        reinterpret_cast<uint32_t*>(s.mlut)[i] = reinterpret_cast<const uint32_t*>(g_mlut.base)[i];
    for (int i = threadIdx.x; i < 256; i += blockDim.x) {
        s.qm2[i] = make_float2(c_qm[i & 15], c_qm[i >> 4]);
        s.qv2[i] = make_float2(c_qv[i & 15], c_qv[i >> 4]);
    }
    load_tables(s.t);  // ends with __syncthreads()
}

// Entry of a pair table for byte j (elements 2j, 2j+1) of a word of eight codes.
__device__ __forceinline__ f2 pair_lookup(const float2* tab, uint32_t w, int j) {
    const uint32_t off = j == 0 ? (w << 3) & 0x7f8u : (w >> (8 * j - 3)) & 0x7f8u;
    return *reinterpret_cast<const float2*>(reinterpret_cast<const char*>(tab) + off);
}

// `mid`: the 15 midpoints in ascending order followed by +inf (Tables::mm).
__device__ __forceinline__ uint32_t search_m_lut(float x, const uint8_t* lut, const float* mid) {
    const uint32_t b = lut[__float_as_uint(x) >> 21];
    return b + (mid[b] < x ? 1u : 0u);
}

// Second-moment map: midpoints are (1.5 + k) / 16, so the count of midpoints below x is ceil(16 x - 1.5)
// clamped to 0..15; 16 x - 1.5 is exact wherever it is positive.
// CLAMP = false is for callers whose x cannot exceed 1 (the scale is a maximum over values that include the
// dividend, taken by the same kernel sequence): 16 x - 1.5 <= 14.5 then, and the code needs no upper clamp.
template <bool CLAMP = true>
__device__ __forceinline__ uint32_t code_from_y(float y) {
    uint32_t c;
    asm("cvt.rpi.u32.f32 %0, %1;" : "=r"(c) : "f"(y));  // saturating: negative and NaN -> 0
    return CLAMP ? min(c, 15u) : c;
}
__device__ __forceinline__ uint32_t search_v_closed(float x) { return code_from_y(__fmaf_rn(x, 16.0f, -1.5f)); }

// ---- integer helpers that compile to one instruction each --------------------------------------------------
// Two integers saturated to 0..15 become the low byte (hi in bits 7..4, lo in bits 3..0) of the result, above it
// the low 24 bits of c: four of these in a row pack eight codes, last byte first.  A negative input gives 0, so a
// code taken by rounding up 16 x - 1.5 needs no lower clamp.
__device__ __forceinline__ uint32_t pack_u4(int hi, int lo, uint32_t c) {
    uint32_t d;
    asm("cvt.pack.sat.u4.s32.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(hi), "r"(lo), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
// Byte j of w, zero-extended.
__device__ __forceinline__ uint32_t byte_of(uint32_t w, int j) {
    return j == 0 ? (w & 0xffu) : j == 3 ? (w >> 24) : prmt(w, 0u, 0x4440u + j);
}
// The two bf16 values of a word as floats (low half first): byte permutes, which keep the shift off the
// multiply-add pipe where the compiler would otherwise place it.
__device__ __forceinline__ f2 widen_bf16x2(uint32_t w) {
    return mk2(__uint_as_float(prmt(w, 0u, 0x1044u)), __uint_as_float(prmt(w, 0u, 0x3244u)));
}
// ceil(y) as a signed integer (saturating; NaN gives 0).
__device__ __forceinline__ int ceil_s32(float y) {
    int c;
    asm("cvt.rpi.s32.f32 %0, %1;" : "=r"(c) : "f"(y));
    return c;
}
// The pair table entry of byte j of a word of eight codes, and the first-moment code of x, both with the plain
// index (the scaling by the entry size folds into the shared-memory address).
__device__ __forceinline__ f2 pair_entry(const float2* tab, uint32_t w, int j) { return tab[byte_of(w, j)]; }

// A scale the fast division sequences may be used with.
__device__ __forceinline__ bool scale_safe(float s) { return s == 0.0f || (s >= 0x1p-90f && s <= 0x1p100f); }

// Largest t with base[t] <= item < base[t+1]; base[0] = 0, base[n] = total.
__device__ __forceinline__ int find_tensor(const int64_t* __restrict__ base, int n, int64_t item) {
    int lo = 0, hi = n;
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (__ldg(base + mid) <= item)
            lo = mid;
        else
            hi = mid;
    }
    return lo;
}

// ---- exact-path helpers on a lane's 8 values ------------------------------------------------------------

__device__ __forceinline__ uint32_t quantize8(const float (&x)[8], float scale, const float* mid, int nv) {
    uint32_t w = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const uint32_t c = search16(scaled(x[k], scale), mid);
        w |= (k < nv ? c : 0u) << (4 * k);
    }
    return w;
}

// Max of |x| over the 16 lanes that hold one 128-element block.  Works on bit patterns, so a NaN survives.
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

// ---- fast-path pieces -----------------------------------------------------------------------------------

struct Hyper2 {  // the scalars of one step, broadcast into both halves of a packed register
    f2 decay, w1, beta2, w2, eps, nstep, rb, nb;
};
__device__ __forceinline__ Hyper2 widen(const HyperDev& hd) {
    Hyper2 o;
    o.decay = bc2(hd.h.decay);
    o.w1 = bc2(hd.h.w1);
    o.beta2 = bc2(hd.h.beta2);
    o.w2 = bc2(hd.h.w2);
    o.eps = bc2(hd.h.eps);
    o.nstep = bc2(hd.h.neg_step);
    o.rb = bc2(hd.rb);
    o.nb = bc2(hd.nb);
    return o;
}

// The AdamW update of two elements; same roundings as adamw_elem.  V_FLOOR: the caller guarantees that the
// old second moment is at least 2^-94 (a stored scale of at least 2^-90 times the smallest map value), so
// the new one cannot fall below the range of the unchecked square root.
// BC1: sqrt(1 - beta2^t) has rounded to exactly 1 (from about step 17 000 on with beta2 = 0.999, i.e. for most
// of a long run), so the division by it is the identity and is left out.
template <bool V_FLOOR = false, bool BC1 = false>
__device__ __forceinline__ void adamw_pair(f2& p, f2 g, f2& m, f2& v, const Hyper2& h) {
    // p * decay as a fused multiply-add with a zero addend: same value, but unlike a packed multiply it
    // cannot be contracted with the add that consumes it further down (see qf_math.cuh).
    const f2 p1 = fma2(p, h.decay, bc2(0.0f));
    m = fma2(h.w1, fma2(m, bc2(-1.0f), g), m);            // m + w1 * (g - m)
    v = fma2(mul2(h.w2, g), g, mul2(h.beta2, v));          // beta2 * v + (w2 * g) * g
    const f2 s = sqrt2<!V_FLOOR>(v);
    const f2 den = add2(BC1 ? s : div2_prepared(s, h.rb, h.nb), h.eps);
    p = add2(p1, div2(mul2(h.nstep, m), den));
}
__device__ __forceinline__ f2 v_update2(f2 g, f2 v_old, const Hyper2& h) {
    return fma2(mul2(h.w2, g), g, mul2(h.beta2, v_old));
}

// Code k of a word as the float 2^23 + code (mantissa trick); subtracting 2^23 - 1 gives code + 1 exactly.
__device__ __forceinline__ float code_plus_2p23(uint32_t w, int k) {
    return __uint_as_float(((w >> (4 * k)) & 15u) | 0x4b000000u);
}
constexpr float kMagic = -8388607.0f;

// Exact quantization of four pairs, out of line: the rarely taken branch of the fast rows.
__device__ __noinline__ uint32_t quantize8_pairs_exact(f2 a, f2 b, f2 c, f2 d, float scale, const float* mid) {
    const float x[8] = {a.x, a.y, b.x, b.y, c.x, c.y, d.x, d.y};
    return quantize8(x, scale, mid, 8);
}

// First-moment codes of a lane's 8 values against the block scale; fast division when the scale allows.
__device__ __forceinline__ uint32_t quantize_m8(const f2 (&m)[4], float scale, const Smem& s) {
    if (!scale_safe(scale)) return quantize8_pairs_exact(m[0], m[1], m[2], m[3], scale, s.t.mm);
    const Recip rc = make_recip(scale);  // 0 for an all-zero block: every quotient is 0
    const f2 r2 = bc2(rc.r), ns2 = bc2(rc.nd);
    uint32_t w = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const f2 q = div2_prepared(m[j], r2, ns2);
        w += search_m_lut(q.x, s.mlut, s.t.mm) << (8 * j);  // disjoint nibbles: add == or, and folds into a shift-add
        w += search_m_lut(q.y, s.mlut, s.t.mm) << (8 * j + 4);
    }
    return w;
}

// Max of |x| over the 128-element block a lane's 8 values belong to (16 lanes), by redux instructions on the
// bit patterns (non-negative floats order like unsigned integers).  Two full-warp reductions, each over one half's
// values (the other half contributes 0): a reduction under a half-warp mask is compiled into a guarded collective
// with its own branches and warp syncs.
__device__ __forceinline__ float block_max_of_lane_max(uint32_t bits) {
    const bool hi = threadIdx.x & 16;
    const uint32_t lo_max = __reduce_max_sync(kFull, hi ? 0u : bits);
    const uint32_t hi_max = __reduce_max_sync(kFull, hi ? bits : 0u);
    return __uint_as_float(hi ? hi_max : lo_max);
}
// The lane's own maximum through fmaxf, which returns the other operand when one is a NaN: only for callers whose
// values cannot be NaN (the panel loop: a non-finite gradient or scale sends its row down the exact path first).
__device__ __forceinline__ float absmax_pairs_to_block(const f2 (&m)[4]) {
    float a = fmaxf(fmaxf(fabsf(m[0].x), fabsf(m[0].y)), fmaxf(fabsf(m[1].x), fabsf(m[1].y)));
    a = fmaxf(a, fmaxf(fmaxf(fabsf(m[2].x), fabsf(m[2].y)), fmaxf(fabsf(m[3].x), fabsf(m[3].y))));
    return block_max_of_lane_max(__float_as_uint(a));
}
// The same on bit patterns throughout: a NaN has the largest pattern and survives, as it does in the exact path
// (absmax8_bits_to_block) and in the reference's abs().max().
__device__ __forceinline__ float absmax_pairs_to_block_nan(const f2 (&m)[4]) {
    uint32_t a = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) a = max(a, max(absbits(m[j].x), absbits(m[j].y)));
    return block_max_of_lane_max(a);
}

// ---- cp.async helpers (per-lane asynchronous copies global -> shared) -------------------------------------
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<unsigned>(__cvta_generic_to_shared(smem))),
                 "l"(__cvta_generic_to_global(gmem))
                 : "memory");
}
__device__ __forceinline__ void cp_async4(void* smem, const void* gmem) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(static_cast<unsigned>(__cvta_generic_to_shared(smem))),
                 "l"(__cvta_generic_to_global(gmem))
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// A read-only scalar load the compiler may not sink below the following cp.async.wait_group (volatile asm
// statements keep their order): the loads for the next row have to be issued before this row's wait.
__device__ __forceinline__ float ldg_early(const float* p) {
    float v;
    asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(__cvta_generic_to_global(p)));
    return v;
}
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// =================================================================================================
// Panel mapping, rank-1 tensors
// =================================================================================================

// First pass over one item of a rank-1 panel.  This pass does little arithmetic per byte, so it needs many bytes in
// flight to cover HBM latency: each lane stages its own 16-byte piece of g and its code word of the next
// kPreStages - 1 rows into a per-warp ring with cp.async (a lane reads only what it copied, so no barrier), and the
// old row maxima of the item are fetched up front, two per lane, and handed out by shuffle.
constexpr int kPreStages = 8;
constexpr int pre_dyn_smem(bool any_f32) { return kWarpsPerCta * kPreStages * 32 * ((any_f32 ? 32 : 16) + 4); }

template <typename T, bool SCALE>
__device__ __forceinline__ void pre_panel(const DevTensor& t, int64_t li, const HyperDev& hd, const SmemPre& s,
                                          char* stage, uint32_t* status) {
    static_assert(kPreRowsPerItem == 64, "two old row maxima per lane");
    const int lane = threadIdx.x & 31;
    const int band = static_cast<int>(li / t.panels);
    const int panel = static_cast<int>(li - static_cast<int64_t>(band) * t.panels);
    const int r0 = band * kPreRowsPerItem;
    const int r1 = min(r0 + kPreRowsPerItem, t.rows);
    const int j0 = panel * kPanelCols + lane * 8;
    const uint8_t* vc = reinterpret_cast<const uint8_t*>(t.v);
    constexpr int NV = sizeof(T) / 2;
    constexpr int kRowBytes = 32 * (NV * 16 + 4);
    const uint32_t cols = static_cast<uint32_t>(t.cols);
    auto issue = [&](uint32_t e, int slot) {
        char* base = stage + slot * kRowBytes;
#pragma unroll
        for (int v = 0; v < NV; ++v) cp_async16(base + (v * 32 + lane) * 16, t.g + static_cast<size_t>(e) * sizeof(T) + v * 16);
        cp_async4(base + NV * 512 + lane * 4, vc + (e >> 1));
    };
    uint32_t e_issue = static_cast<uint32_t>(r0) * cols + j0;
    int r_issue = r0;
#pragma unroll
    for (int i = 0; i < kPreStages - 1; ++i) {
        if (r_issue < r1) issue(e_issue, i);
        cp_async_commit();
        e_issue += cols;
        ++r_issue;
    }
    const float rows_lo = __ldg(t.vs + min(r0 + lane, r1 - 1)), rows_hi = __ldg(t.vs + min(r0 + 32 + lane, r1 - 1));
    float col_old[8];
    load8f(t.vcol, j0, col_old);
    const Hyper2 h2 = widen(hd);
    uint32_t cmax[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) cmax[k] = 0;
    // Row maxima stay in registers until the item ends: lane k keeps the maxima of rows r0 + k and r0 + 32 + k,
    // which then go out as two warp-wide reductions instead of one single-lane atomic per row.
    uint32_t keep_lo = 0, keep_hi = 0;
    auto body = [&](int r, int slot) {  // `slot` is a compile-time constant in the unrolled groups below
        if (r_issue < r1) issue(e_issue, slot == 0 ? kPreStages - 1 : slot - 1);
        cp_async_commit();
        e_issue += cols;
        ++r_issue;
        cp_async_wait<kPreStages - 1>();
        const char* base = stage + slot * kRowBytes;
        Raw8<T> g_raw;
        g_raw.from_shared(base, lane);
        const uint32_t wv = *reinterpret_cast<const uint32_t*>(base + NV * 512 + lane * 4);
        const int k_row = r - r0;
        const float row_old = __shfl_sync(kFull, k_row < 32 ? rows_lo : rows_hi, k_row & 31);
        float g[8];
        g_raw.widen(g);
        if (SCALE) {  // the scaled gradient replaces the original: the main pass and the caller see it
#pragma unroll
            for (int k = 0; k < 8; ++k) g[k] = round_as<T>(__fmul_rn(g[k], hd.gs));
            Elem<T>::store8(const_cast<char*>(t.g), static_cast<int64_t>(static_cast<uint32_t>(r) * cols + j0), g);
        }
        uint32_t rmax = 0;
        if (hd.fast) {  // warp-uniform
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const f2 v_old = mul2(pair_lookup(s.qv2, wv, j),
                                      mk2(fminf(row_old, col_old[2 * j]), fminf(row_old, col_old[2 * j + 1])));
                const f2 v = v_update2(mk2(g[2 * j], g[2 * j + 1]), v_old, h2);
                const uint32_t b0 = __float_as_uint(v.x), b1 = __float_as_uint(v.y);  // v >= 0
                rmax = max(rmax, max(b0, b1));
                cmax[2 * j] = max(cmax[2 * j], b0);
                cmax[2 * j + 1] = max(cmax[2 * j + 1], b1);
            }
        } else {
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const float v_old = __fmul_rn(s.t.qv[nib(wv, k)], fminf(row_old, col_old[k]));
                const uint32_t b = __float_as_uint(v_update(g[k], v_old, hd.h));
                rmax = max(rmax, b);
                cmax[k] = max(cmax[k], b);
            }
        }
        rmax = __reduce_max_sync(kFull, rmax);
        const bool mine = (k_row & 31) == lane;
        keep_lo = mine && k_row < 32 ? rmax : keep_lo;
        keep_hi = mine && k_row >= 32 ? rmax : keep_hi;
    };
    int r = r0;
    for (; r + kPreStages <= r1; r += kPreStages) {  // whole turns of the ring: slots are constants
#pragma unroll
        for (int i = 0; i < kPreStages; ++i) body(r + i, i);
    }
    for (int i = 0; r < r1; ++r, ++i) body(r, i);    // fewer rows than one turn are left: the ring is at slot 0
    cp_async_wait<0>();
    if (r0 + lane < r1) atomic_max_nonneg(t.vrow_new + r0 + lane, keep_lo);
    if (r0 + 32 + lane < r1) atomic_max_nonneg(t.vrow_new + r0 + 32 + lane, keep_hi);
    if (__any_sync(kFull, max(keep_lo, keep_hi) >= 0x7f800000u) && lane == 0) atomicOr(status, QF_STATUS_NONFINITE);
#pragma unroll
    for (int k = 0; k < 8; ++k) atomic_max_nonneg(t.vcol_new + j0 + k, cmax[k]);
}

// One row of a panel, exact arithmetic (also the reference for what the fast row must produce).  Kept out
// of line and self-contained (it reloads its column maxima) so that it costs the hot loop no registers.
template <typename T>
__device__ __noinline__ void main_panel_row_exact(const DevTensor* tp, int64_t e, int r, int j0, const HyperDev& hd,
                                                  const Smem& s, uint32_t* status, const PushPack* push) {
    const DevTensor t = *tp;
    const int lane = threadIdx.x & 31;
    uint8_t* mc = reinterpret_cast<uint8_t*>(t.m);
    uint8_t* vc = reinterpret_cast<uint8_t*>(t.v);
    float p[8], g[8], m[8], v[8], col_old[8], col_new[8];
    load8f(t.vcol, j0, col_old);
    load8f(t.vcol_new, j0, col_new);
    Elem<T>::load8(t.p, e, p);
    Elem<T>::load8(t.g, e, g);
    const uint32_t wm = *reinterpret_cast<const uint32_t*>(mc + (e >> 1));
    const uint32_t wv = *reinterpret_cast<const uint32_t*>(vc + (e >> 1));
    const float ms_old = __ldg(t.ms + (e >> 7));
    const float row_old = __ldg(t.vs + r);
    const float row_new = t.vrow_new[r];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        m[k] = __fmul_rn(s.t.qm[nib(wm, k)], ms_old);
        v[k] = __fmul_rn(s.t.qv[nib(wv, k)], fminf(row_old, col_old[k]));
        adamw_elem(p[k], g[k], m[k], v[k], hd.h);
    }
    Elem<T>::store8(t.p, e, p);
    if (push) push_store8<T>(t.p, e, p, push);
    const float ms_new = absmax8_bits_to_block(m);
    *reinterpret_cast<uint32_t*>(mc + (e >> 1)) = quantize8(m, ms_new, s.t.mm, 8);
    if ((lane & 15) == 0) {
        t.ms[e >> 7] = ms_new;
        if (nonfinite(ms_new)) atomicOr(status, QF_STATUS_NONFINITE);
    }
    uint32_t w = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) w |= search16(scaled(v[k], fminf(row_new, col_new[k])), s.t.mv) << (4 * k);
    *reinterpret_cast<uint32_t*>(vc + (e >> 1)) = w;
}

// ---- asynchronous staging of the rows of a panel ---------------------------------------------------------
// Each lane copies its own 16-byte pieces of p and g and its two code words of the row ahead into one of two
// per-warp slots in shared memory with cp.async and reads them back when their row comes up.  A lane only
// ever reads what it copied itself, so the slots need no barrier: cp.async.wait_group orders a lane's
// copies with its own reads.  One row ahead per warp is enough at two CTAs per SM (a third slot measured
// slower, and so did bulk copies with an mbarrier per slot: four 128..512-byte requests per row and warp are too
// small for the copy engine).  The per-lane column maxima (old, new, reciprocal of new) sit in shared memory as
// well and are fetched pair by pair: registers are the scarce resource of this kernel (keeping them in registers
// measured 8 % slower at 128 registers per thread).
constexpr int kStages = 2;                             // this row and the next one
constexpr int kRowBytesBf16 = 32 * (2 * 16 + 8);       // staged bytes of one row of a panel, bf16 parameters
constexpr int kRowBytesF32 = 32 * (2 * 2 * 16 + 8);    // the same for fp32 parameters
constexpr int kColBytes = 3 * 4 * 32 * 8;              // per warp: old / new / reciprocal column maxima of its 256 columns
// Dynamic shared memory of the panel kernel: per warp the two slots plus the column block.  The host sizes the
// slots for fp32 rows only when the launch holds an fp32 panel tensor: less shared memory leaves more L1 to the
// CTA, which the measurements reward.
constexpr int main_dyn_smem(bool any_f32) { return kWarpsPerCta * (kStages * (any_f32 ? kRowBytesF32 : kRowBytesBf16) + kColBytes); }

// The AdamW update of two elements inside the panel loop (second moment at least 2^-94, see adamw_pair).  P1: the
// two divisions of the parameter update with one residual correction (div2_prepared1 says what that means); taken for
// bf16 parameters only.  BC1: sqrt(1 - beta2^t) has rounded to 1, the division by it is left out.
// RELAXED (with P1 only; an option the caller has to ask for): the square root and the two divisions of the parameter
// update are taken as v * rsqrt(v), a multiplication by RN(1 / bc2s) and a multiplication by the approximate reciprocal
// of the denominator, without corrections.  The update then carries a relative error of about 2^-21; the new bf16
// parameter differs from the exact one -- by one bf16 unit -- where the exact sum lies that close to a rounding
// boundary.  m and v, hence all codes and scales, do not depend on it and stay bit-identical.
template <bool P1, bool BC1, bool RELAXED = false>
__device__ __forceinline__ void adamw_pair_panel(f2& p, f2 g, f2& m, f2& v, const Hyper2& h) {
    const f2 p1 = fma2(p, h.decay, bc2(0.0f));            // not a packed multiply: see adamw_pair
    m = fma2(h.w1, add2(g, neg2(m)), m);                   // m + w1 * (g - m)
    v = fma2(mul2(h.w2, g), g, mul2(h.beta2, v));          // beta2 * v + (w2 * g) * g
    if (P1 && RELAXED) {
        const f2 s = mul2(v, mk2(rsqrt_approx(v.x), rsqrt_approx(v.y)));   // v > 0 on this path (old maxima above zero)
        const f2 den = BC1 ? add2(s, h.eps) : fma2(s, h.rb, h.eps);
        p = fma2(mul2(h.nstep, m), mk2(rcp_approx(den.x), rcp_approx(den.y)), p1);
        return;
    }
    const f2 s = sqrt2<false>(v);
    const f2 den = add2(BC1 ? s : div2_prepared_n<P1>(s, h.rb, h.nb), h.eps);
    const f2 a = mul2(h.nstep, m);
    p = add2(p1, P1 ? div2_1(a, den) : div2(a, den));
}

// Second pass over one item of a rank-1 panel: 64 rows of 256 columns.
//
// The hot loop holds no call and stores nothing of a row before it knows that the whole row could take the packed
// arithmetic: the row and column scalars inside the range of the division sequences (the pass that stored the
// reciprocals wrote NaN where an old or a new maximum is not), old maxima above zero (a zero one, as on the first
// step, lets the second moment fall below the range of the unchecked square root), the old block scale finite and
// the new one zero or inside the range.  A row that fails leaves the loop untouched and is redone by
// main_panel_row_exact from its unmodified inputs, after which the hot loop starts again behind it.  Rows go in
// pairs so that the two staging slots are compile-time offsets and the per-row scalars alternate between two sets of
// registers; an odd last row of an item takes the exact path as well.
template <typename T, bool PUSH, bool BC1, bool RELAXED = false>
__device__ __forceinline__ void main_panel(const DevTensor* tp, int64_t li, const HyperDev& hd, const Smem& s,
                                           char* stage, int ring_bytes, uint32_t* status, const PushPack* push) {
    constexpr bool BF16 = std::is_same<T, __nv_bfloat16>::value;
    const DevTensor t = *tp;
    const int lane = threadIdx.x & 31;
    const int band = static_cast<int>(li / t.panels);
    const int panel = static_cast<int>(li - static_cast<int64_t>(band) * t.panels);
    const int r0 = band * t.main_rows;
    const int r1 = min(r0 + t.main_rows, t.rows);
    const int j0 = panel * kPanelCols + lane * 8;
    uint8_t* mc = reinterpret_cast<uint8_t*>(t.m);
    uint8_t* vc = reinterpret_cast<uint8_t*>(t.v);

    constexpr int NV = sizeof(T) / 2;  // 16-byte vectors per lane and array: 1 (bf16) or 2 (fp32)
    constexpr int kArr = NV * 512;     // bytes of one staged array of one row
    constexpr int kRowBytes = 2 * kArr + 256;
    static_assert(kRowBytes == (NV == 1 ? kRowBytesBf16 : kRowBytesF32), "staged row size");
    static_assert(kStages == 2, "the loop below stages exactly one row ahead and alternates between two slots");
    // Element offsets inside the tensor fit 32 bits (the host gives larger tensors the flat mapping).
    const uint32_t cols = static_cast<uint32_t>(t.cols);
    char* const lane_vec = stage + lane * 16;             // this lane's 16-byte pieces of p (then g) in slot 0
    char* const lane_codes = stage + 2 * kArr + lane * 4;  // its first-moment (then second-moment) code word in slot 0
    auto issue = [&](uint32_t e, int slot_off) {
#pragma unroll
        for (int v = 0; v < NV; ++v) {
            cp_async16(lane_vec + slot_off + v * 512, t.p + static_cast<size_t>(e) * sizeof(T) + v * 16);
            cp_async16(lane_vec + slot_off + kArr + v * 512, t.g + static_cast<size_t>(e) * sizeof(T) + v * 16);
        }
        cp_async4(lane_codes + slot_off, mc + (e >> 1));
        cp_async4(lane_codes + slot_off + 128, vc + (e >> 1));
    };

    float4* colbuf = reinterpret_cast<float4*>(stage + ring_bytes) + lane;  // [old | -new | 1/new][half][lane]
    bool ok = hd.fast;
    {
        float col_old[8], col_new[8], rcol[8];
        load8f(t.vcol, j0, col_old);
        load8f(t.vcol_new, j0, col_new);
        load8f(t.vcol_rcp, j0, rcol);
#pragma unroll
        for (int k = 0; k < 8; ++k) ok &= rcol[k] == rcol[k] && col_old[k] > 0.0f;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            colbuf[(0 * 2 + j) * 32] = make_float4(col_old[4 * j], col_old[4 * j + 1], col_old[4 * j + 2], col_old[4 * j + 3]);
            colbuf[(1 * 2 + j) * 32] = make_float4(-col_new[4 * j], -col_new[4 * j + 1], -col_new[4 * j + 2], -col_new[4 * j + 3]);
            colbuf[(2 * 2 + j) * 32] = make_float4(rcol[4 * j], rcol[4 * j + 1], rcol[4 * j + 2], rcol[4 * j + 3]);
        }
    }
    const bool col_fast = __all_sync(kFull, ok);
    const Hyper2 h2 = widen(hd);

    struct RowScalars {
        float ms_old, row_old, row_new, rrow;
    };
    auto fetch_scalars = [&](int r, uint32_t e) {
        RowScalars o;
        o.ms_old = ldg_early(t.ms + (e >> 7));
        o.row_old = ldg_early(t.vs + r);
        o.row_new = ldg_early(t.vrow_new + r);
        o.rrow = ldg_early(t.vrow_rcp + r);
        return o;
    };

    // One row out of the staging slot at `slot_off`.  False: the row cannot take the packed arithmetic; nothing of
    // it has been stored.
    auto row = [&](const RowScalars& sc, uint32_t e, int slot_off) -> bool {
        // the staged row as it was copied: four words of two bf16 values, or eight floats, per array
        uint32_t pw[NV * 4], gw[NV * 4];
#pragma unroll
        for (int v = 0; v < NV; ++v) {
            const uint4 a = *reinterpret_cast<const uint4*>(lane_vec + slot_off + v * 512);
            const uint4 b = *reinterpret_cast<const uint4*>(lane_vec + slot_off + kArr + v * 512);
            pw[4 * v] = a.x; pw[4 * v + 1] = a.y; pw[4 * v + 2] = a.z; pw[4 * v + 3] = a.w;
            gw[4 * v] = b.x; gw[4 * v + 1] = b.y; gw[4 * v + 2] = b.z; gw[4 * v + 3] = b.w;
        }
        f2 pp[4];
        const uint32_t wm = *reinterpret_cast<const uint32_t*>(lane_codes + slot_off);
        const uint32_t wv = *reinterpret_cast<const uint32_t*>(lane_codes + slot_off + 128);
        const f2 ms_old = bc2(sc.ms_old);
        const float row_old = sc.row_old, nrow = -sc.row_new, rrow = sc.rrow;
        f2 m[4];
        int cv[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            pp[j] = BF16 ? widen_bf16x2(pw[j]) : mk2(__uint_as_float(pw[(2 * j) % (NV * 4)]), __uint_as_float(pw[(2 * j + 1) % (NV * 4)]));
            const f2 gg = BF16 ? widen_bf16x2(gw[j]) : mk2(__uint_as_float(gw[(2 * j) % (NV * 4)]), __uint_as_float(gw[(2 * j + 1) % (NV * 4)]));
            m[j] = mul2(pair_entry(s.qm2, wm, j), ms_old);
            const float4 a = colbuf[(0 * 2 + (j >> 1)) * 32], b = colbuf[(1 * 2 + (j >> 1)) * 32], c = colbuf[(2 * 2 + (j >> 1)) * 32];
            const f2 co = (j & 1) ? mk2(a.z, a.w) : mk2(a.x, a.y);
            const f2 ncn = (j & 1) ? mk2(b.z, b.w) : mk2(b.x, b.y);
            const f2 rcn = (j & 1) ? mk2(c.z, c.w) : mk2(c.x, c.y);
            f2 v = mul2(pair_entry(s.qv2, wv, j), mk2(fminf(row_old, co.x), fminf(row_old, co.y)));
            adamw_pair_panel<BF16, BC1, RELAXED>(pp[j], gg, m[j], v, h2);
            // requantize v: scale = min(row', col') -> -scale = max(-row', -col'), 1/scale = max(1/row', 1/col')
            const f2 nsv = mk2(fmaxf(nrow, ncn.x), fmaxf(nrow, ncn.y));
            const f2 rv = mk2(fmaxf(rrow, rcn.x), fmaxf(rrow, rcn.y));
            const f2 y = fma2(div2_prepared1(v, rv, nsv), bc2(16.0f), bc2(-1.5f));
            cv[2 * j] = ceil_s32(y.x);       // x <= 1 here (the scale is a maximum over values that include v): at most 15
            cv[2 * j + 1] = ceil_s32(y.y);
        }
        const float ms_new = absmax_pairs_to_block(m);
        const bool row_ok = sc.rrow == sc.rrow && sc.row_old > 0.0f && sc.ms_old < __builtin_huge_valf() && scale_safe(ms_new);
        if (!__all_sync(kFull, row_ok)) return false;     // the vote also tells the compiler that the branch is uniform
        uint32_t wmq;
        {
            const Recip rc = make_recip(ms_new);  // 0 for an all-zero block: every quotient is 0
            const f2 r2 = bc2(rc.r), ns2 = bc2(rc.nd);
            int c[8];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const f2 q = div2_prepared1(m[j], r2, ns2);
                c[2 * j] = search_m_lut(q.x, s.mlut, s.t.mm);
                c[2 * j + 1] = search_m_lut(q.y, s.mlut, s.t.mm);
            }
            wmq = pack_u4(c[1], c[0], pack_u4(c[3], c[2], pack_u4(c[5], c[4], pack_u4(c[7], c[6], 0u))));
        }
        const uint32_t wq = pack_u4(cv[1], cv[0], pack_u4(cv[3], cv[2], pack_u4(cv[5], cv[4], pack_u4(cv[7], cv[6], 0u))));
        if (BF16) {
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const __nv_bfloat162 h = __floats2bfloat162_rn(pp[j].x, pp[j].y);  // nearest even
                w[j] = *reinterpret_cast<const uint32_t*>(&h);
            }
            const uint4 out = make_uint4(w[0], w[1], w[2], w[3]);
            *reinterpret_cast<uint4*>(t.p + static_cast<size_t>(e) * 2) = out;
            if (PUSH) {
                const int n = push->n;
                for (int k = 0; k < n; ++k) *reinterpret_cast<uint4*>(t.p + push->delta[k] + static_cast<size_t>(e) * 2) = out;
            }
        } else {
            const float4 o0 = make_float4(pp[0].x, pp[0].y, pp[1].x, pp[1].y), o1 = make_float4(pp[2].x, pp[2].y, pp[3].x, pp[3].y);
            float4* dst = reinterpret_cast<float4*>(t.p + static_cast<size_t>(e) * 4);
            dst[0] = o0;
            dst[1] = o1;
            if (PUSH) {
                const int n = push->n;
                for (int k = 0; k < n; ++k) {
                    float4* pd = reinterpret_cast<float4*>(t.p + push->delta[k] + static_cast<size_t>(e) * 4);
                    pd[0] = o0;
                    pd[1] = o1;
                }
            }
        }
        *reinterpret_cast<uint32_t*>(vc + (e >> 1)) = wq;
        *reinterpret_cast<uint32_t*>(mc + (e >> 1)) = wmq;
        if ((lane & 15) == 0) t.ms[e >> 7] = ms_new;
        return true;
    };

    int r = r0;
    while (r < r1) {
        if (col_fast && r + 1 < r1) {
            uint32_t e = static_cast<uint32_t>(r) * cols + j0;
            issue(e, 0);
            cp_async_commit();
            RowScalars sa = fetch_scalars(r, e);
            // rows r (slot 0) and r + 1 (slot 1) per turn; row r is on its way when the turn starts
            for (; r + 1 < r1; r += 2, e += 2 * cols) {
                issue(e + cols, kRowBytes);
                cp_async_commit();
                const RowScalars sb = fetch_scalars(r + 1, e + cols);
                cp_async_wait<1>();  // everything but the newest group has landed
                if (!row(sa, e, 0)) break;
                // The row behind the pair goes into slot 0.  Past the end the last row is staged and its scalars are
                // fetched again (nobody reads them): cheaper than a branch around the copies.
                const bool more = r + 2 < r1;
                const uint32_t e2 = more ? e + 2 * cols : e + cols;
                issue(e2, 0);
                cp_async_commit();
                sa = fetch_scalars(more ? r + 2 : r + 1, e2);
                cp_async_wait<1>();
                if (!row(sb, e + cols, kRowBytes)) {
                    ++r;
                    break;
                }
            }
            cp_async_wait<0>();
        }
        if (r < r1) {  // cold: this row exactly, from its unmodified inputs
            main_panel_row_exact<T>(tp, static_cast<uint32_t>(r) * cols + j0, r, j0, hd, s, status, PUSH ? push : nullptr);
            ++r;
        }
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
template <typename T>
__device__ __forceinline__ void push_store8_masked(char* base, int64_t e, int nv, bool vec, const float (&x)[8],
                                                   const PushPack* push) {
    const int n = push->n;
    for (int k = 0; k < n; ++k) store8_masked<T>(base + push->delta[k], e, nv, vec, x);
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
__device__ __forceinline__ void pre_flat_rank1(const DevTensor& t, int64_t li, const HyperDev& hd, const SmemPre& s,
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
        if (hd.gs != 1.0f) {
#pragma unroll
            for (int k = 0; k < 8; ++k) g[k] = round_as<T>(__fmul_rn(g[k], hd.gs));
            store8_masked<T>(const_cast<char*>(t.g), e, nv, vec, g);
        }
        const uint32_t wv = load_codes(vc, e, nv, vec);
        rank1_scales(t.vs, t.vcol, e + t.flat_off, nv, t.cols, sc, ri, ci);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            if (k < nv) {
                const uint32_t b = __float_as_uint(v_update(g[k], __fmul_rn(s.t.qv[nib(wv, k)], sc[k]), hd.h));
                atomic_max_nonneg(t.vrow_new + ri[k], b);
                atomic_max_nonneg(t.vcol_new + ci[k], b);
                if (b >= 0x7f800000u) atomicOr(status, QF_STATUS_NONFINITE);
            }
        }
    }
}

// One run of 256 flattened elements, exact arithmetic, any tail, any alignment.
template <typename T, int KIND>
__device__ __noinline__ void main_flat_run_exact(const DevTensor* tp, int64_t wbase, const HyperDev& hd, const Smem& s,
                                                 uint32_t* status, const PushPack* push) {
    const DevTensor t = *tp;
    const int lane = threadIdx.x & 31;
    const bool vec = t.flags & kFlagVec;
    uint8_t* mc = reinterpret_cast<uint8_t*>(t.m);
    uint8_t* vc = reinterpret_cast<uint8_t*>(t.v);
    const int64_t e = wbase + lane * 8;
    const int nv = static_cast<int>(max(static_cast<int64_t>(0), min(static_cast<int64_t>(8), t.numel - e)));
    float p[8], g[8], m[8], v[8];
    load8_masked<T>(t.p, e, nv, vec, p);
    load8_masked<T>(t.g, e, nv, vec, g);
    if (KIND == QF_KIND_FP32) {
        load8_masked<float>(t.m, e, nv, vec, m);
        load8_masked<float>(t.v, e, nv, vec, v);
#pragma unroll
        for (int k = 0; k < 8; ++k) adamw_elem(p[k], g[k], m[k], v[k], hd.h);
        store8_masked<T>(t.p, e, nv, vec, p);
        if (push) push_store8_masked<T>(t.p, e, nv, vec, p, push);
        store8_masked<float>(t.m, e, nv, vec, m);
        store8_masked<float>(t.v, e, nv, vec, v);
        return;
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
#pragma unroll
        for (int k = 0; k < 8; ++k) sc_old[k] = sc_new[k] = 0.0f;
        if (nv) {
            rank1_scales(t.vs, t.vcol, e + t.flat_off, nv, t.cols, sc_old, ri, ci);
            rank1_scales(t.vrow_new, t.vcol_new, e + t.flat_off, nv, t.cols, sc_new, ri, ci);
        }
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        m[k] = __fmul_rn(s.t.qm[nib(wm, k)], ms_old);
        v[k] = __fmul_rn(s.t.qv[nib(wv, k)], sc_old[k]);
        adamw_elem(p[k], g[k], m[k], v[k], hd.h);
        if (k >= nv) {  // padding of the last block counts as zero
            m[k] = 0.0f;
            v[k] = 0.0f;
        }
    }
    store8_masked<T>(t.p, e, nv, vec, p);
    if (push) push_store8_masked<T>(t.p, e, nv, vec, p, push);
    const float ms_new = absmax8_bits_to_block(m);  // all 32 lanes take part in the shuffles
    float vs_new = 0.0f;
    if (KIND == QF_KIND_BLOCK) vs_new = absmax8_bits_to_block(v);
    if (nv == 0) return;
    store_codes(mc, e, nv, vec, quantize8(m, ms_new, s.t.mm, nv));
    uint32_t w = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const float sv = KIND == QF_KIND_BLOCK ? vs_new : sc_new[k];
        const uint32_t c = search16(scaled(v[k], sv), s.t.mv);
        w |= (k < nv ? c : 0u) << (4 * k);
    }
    store_codes(vc, e, nv, vec, w);
    if ((lane & 15) == 0) {
        t.ms[e >> 7] = ms_new;
        if (KIND == QF_KIND_BLOCK) t.vs[e >> 7] = vs_new;
        if (nonfinite(ms_new) || nonfinite(vs_new)) atomicOr(status, QF_STATUS_NONFINITE);
    }
}

// One full, vector-aligned run of 256 elements with the packed arithmetic (block-128 and fp32-state kinds).
template <typename T, int KIND>
__device__ __forceinline__ void main_flat_run_fast(const DevTensor& t, int64_t wbase, const Hyper2& h2, const Smem& s,
                                                   uint32_t* status, const PushPack* push) {
    const int lane = threadIdx.x & 31;
    const int64_t e = wbase + lane * 8;
    float p[8], g[8];
    Elem<T>::load8(t.p, e, p);
    Elem<T>::load8(t.g, e, g);
    if (KIND == QF_KIND_FP32) {
        float m[8], v[8];
        Elem<float>::load8(t.m, e, m);
        Elem<float>::load8(t.v, e, v);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            f2 pp = mk2(p[2 * j], p[2 * j + 1]), mm = mk2(m[2 * j], m[2 * j + 1]), vv = mk2(v[2 * j], v[2 * j + 1]);
            adamw_pair(pp, mk2(g[2 * j], g[2 * j + 1]), mm, vv, h2);
            p[2 * j] = pp.x; p[2 * j + 1] = pp.y;
            m[2 * j] = mm.x; m[2 * j + 1] = mm.y;
            v[2 * j] = vv.x; v[2 * j + 1] = vv.y;
        }
        Elem<T>::store8(t.p, e, p);
        if (push) push_store8<T>(t.p, e, p, push);
        Elem<float>::store8(t.m, e, m);
        Elem<float>::store8(t.v, e, v);
        return;
    }
    uint8_t* mc = reinterpret_cast<uint8_t*>(t.m);
    uint8_t* vc = reinterpret_cast<uint8_t*>(t.v);
    const uint32_t wm = *reinterpret_cast<const uint32_t*>(mc + (e >> 1));
    const uint32_t wv = *reinterpret_cast<const uint32_t*>(vc + (e >> 1));
    const f2 ms_old = bc2(__ldg(t.ms + (e >> 7)));
    const float vs_old = __ldg(t.vs + (e >> 7));
    const f2 vs2 = bc2(vs_old);
    f2 m[4], v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        f2 pp = mk2(p[2 * j], p[2 * j + 1]);
        m[j] = mul2(pair_lookup(s.qm2, wm, j), ms_old);
        v[j] = mul2(pair_lookup(s.qv2, wv, j), vs2);
        adamw_pair(pp, mk2(g[2 * j], g[2 * j + 1]), m[j], v[j], h2);
        p[2 * j] = pp.x;
        p[2 * j + 1] = pp.y;
    }
    Elem<T>::store8(t.p, e, p);
    if (push) push_store8<T>(t.p, e, p, push);
    const float ms_new = absmax_pairs_to_block_nan(m);   // no first pass vouches for these values: a NaN must survive
    const float vs_new = absmax_pairs_to_block_nan(v);
    *reinterpret_cast<uint32_t*>(mc + (e >> 1)) = quantize_m8(m, ms_new, s);
    uint32_t wq = 0;
    if (scale_safe(vs_new)) {
        const f2 r2 = bc2(vs_new == 0.0f ? 0.0f : __frcp_rn(vs_new)), ns2 = bc2(-vs_new);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const f2 y = fma2(div2_prepared(v[j], r2, ns2), bc2(16.0f), bc2(-1.5f));
            wq += code_from_y<false>(y.x) << (8 * j);
            wq += code_from_y<false>(y.y) << (8 * j + 4);
        }
    } else {
        wq = quantize8_pairs_exact(v[0], v[1], v[2], v[3], vs_new, s.t.mv);
    }
    *reinterpret_cast<uint32_t*>(vc + (e >> 1)) = wq;
    if ((lane & 15) == 0) {
        t.ms[e >> 7] = ms_new;
        t.vs[e >> 7] = vs_new;
        if (nonfinite(ms_new) || nonfinite(vs_new)) atomicOr(status, QF_STATUS_NONFINITE);
    }
}

template <typename T, int KIND>
__device__ __forceinline__ void main_flat(const DevTensor* tp, int64_t li, const HyperDev& hd, const Smem& s,
                                          uint32_t* status, const PushPack* push) {
    const DevTensor t = *tp;
    const bool vec = t.flags & kFlagVec;
    const int64_t start = li * (kPanelCols * kRowsPerItem);
    const Hyper2 h2 = widen(hd);
    for (int it = 0; it < kRowsPerItem; ++it) {
        const int64_t wbase = start + static_cast<int64_t>(it) * kPanelCols;
        if (wbase >= t.numel) break;  // warp-uniform
        if (KIND != QF_KIND_RANK1 && hd.gs != 1.0f) {  // no first pass for these kinds: the gradient is scaled here
            const int64_t e = wbase + (threadIdx.x & 31) * 8;
            const int nv = static_cast<int>(max(static_cast<int64_t>(0), min(static_cast<int64_t>(8), t.numel - e)));
            float g[8];
            load8_masked<T>(t.g, e, nv, vec, g);
#pragma unroll
            for (int k = 0; k < 8; ++k) g[k] = round_as<T>(__fmul_rn(g[k], hd.gs));
            store8_masked<T>(const_cast<char*>(t.g), e, nv, vec, g);
        }
        if (KIND != QF_KIND_RANK1 && hd.fast && vec && wbase + kPanelCols <= t.numel)
            main_flat_run_fast<T, KIND>(t, wbase, h2, s, status, push);
        else
            main_flat_run_exact<T, KIND>(tp, wbase, hd, s, status, push);
    }
}

// =================================================================================================
// Multi-tensor kernels.  `base` is the prefix-sum table of the mapping the kernel serves; tensors of
// the other mapping have zero items in it.
// =================================================================================================

// The multi-tensor kernels are persistent: the host launches about as many CTAs as fit on the device and every
// warp walks the item list with a fixed stride, so the shared-memory tables are filled once per CTA.
constexpr int kPreMinCtas = 3;   // CTAs per SM the first pass is compiled for (80 registers)
// SCALE (panel mapping): some hyper-parameter set of the launch carries a gradient scale other than 1.
// SCHED: the hyper-parameter sets come from the device-resident table `sc` instead of `hp`.
// (Forms of this kernel that carry one dtype's loop only, as step_main_kernel has them, measured 5 % slower.)
template <bool PANEL, bool SCALE = false, bool SCHED = false>
__global__ void __launch_bounds__(kThreads, kPreMinCtas)
step_pre_kernel(const DevTensor* __restrict__ tensors, const int64_t* __restrict__ base, int n,
                const __grid_constant__ HyperPack hp, int ring_bytes, uint32_t* status, const __grid_constant__ Sched sc) {
    __shared__ SmemPre s;
    __shared__ HyperDev sched_h[SCHED ? QF_MAX_HYPERS : 1];
    if (SCHED) load_sched(sched_h, sc);
    load_smem(s);
    extern __shared__ __align__(16) char staging[];  // panel kernel: one ring of rows per warp
    char* stage = staging + (threadIdx.x >> 5) * ring_bytes;
    const int64_t total = base[n], stride = static_cast<int64_t>(gridDim.x) * kWarpsPerCta;
    for (int64_t item = static_cast<int64_t>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5); item < total; item += stride) {
        const int ti = find_tensor(base, n, item);
        const DevTensor t = tensors[ti];
        const int64_t li = item - base[ti];
        const HyperDev& h = SCHED ? sched_h[t.hyper] : hp.h[t.hyper];
        if (PANEL) {
            if (t.dtype == QF_BF16)
                pre_panel<__nv_bfloat16, SCALE>(t, li, h, s, stage, status);
            else
                pre_panel<float, SCALE>(t, li, h, s, stage, status);
        } else {
            if (t.dtype == QF_BF16)
                pre_flat_rank1<__nv_bfloat16>(t, li, h, s, status);
            else if (t.dtype == QF_F16)
                pre_flat_rank1<__half>(t, li, h, s, status);
            else
                pre_flat_rank1<float>(t, li, h, s, status);
        }
    }
}

template <typename T>
__device__ __forceinline__ void main_flat_dispatch(const DevTensor* tp, int64_t li, const HyperDev& h, const Smem& s,
                                                   uint32_t* status, const PushPack* push) {
    const int kind = tp->kind;
    if (kind == QF_KIND_RANK1)
        main_flat<T, QF_KIND_RANK1>(tp, li, h, s, status, push);
    else if (kind == QF_KIND_BLOCK)
        main_flat<T, QF_KIND_BLOCK>(tp, li, h, s, status, push);
    else
        main_flat<T, QF_KIND_FP32>(tp, li, h, s, status, push);
}

constexpr int kMainMinCtas = 2;  // CTAs per SM the second pass is compiled for (128 registers)
// PUSH: the launch also stores every updated parameter vector into the peers' buffers named by `pp`.
// BC1 (panel mapping only): every hyper-parameter set of the launch has bc2s == 1.
// SCHED: the hyper-parameter sets come from the device-resident table `sc` instead of `hp`.
// RELAXED (panel mapping, bf16 tensors): the uncorrected parameter update of adamw_pair_panel.
// DT (panel mapping): 0 = tensors of both dtypes, 1 = the launch holds bf16 panel tensors only, 2 = fp32 only; a kernel
// that carries one dtype's loop is scheduled a little better than one that carries both.
template <bool PANEL, bool PUSH, bool BC1 = false, bool SCHED = false, bool RELAXED = false, int DT = 0>
__global__ void __launch_bounds__(kThreads, kMainMinCtas)
step_main_kernel(const DevTensor* __restrict__ tensors, const int64_t* __restrict__ base, int n,
                 const __grid_constant__ HyperPack hp, int ring_bytes, uint32_t* status,
                 const __grid_constant__ PushPack pp, const __grid_constant__ Sched sc) {
    const PushPack* push = PUSH ? &pp : nullptr;
    __shared__ Smem s;
    __shared__ HyperDev sched_h[SCHED ? QF_MAX_HYPERS : 1];
    if (SCHED) load_sched(sched_h, sc);
    load_smem(s);
    extern __shared__ __align__(16) char staging[];  // panel kernel: per warp a ring of rows plus the column block
    char* stage = staging + (threadIdx.x >> 5) * (ring_bytes + kColBytes);
    const int64_t total = base[n], stride = static_cast<int64_t>(gridDim.x) * kWarpsPerCta;
    for (int64_t item = static_cast<int64_t>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5); item < total; item += stride) {
        const int ti = find_tensor(base, n, item);
        const DevTensor* tp = tensors + ti;
        const int64_t li = item - base[ti];
        const HyperDev& h = SCHED ? sched_h[tp->hyper] : hp.h[tp->hyper];  // hp is a grid constant: its address is usable as it is
        if (PANEL) {
            if (DT == 1 || (DT == 0 && tp->dtype == QF_BF16))
                main_panel<__nv_bfloat16, PUSH, BC1, RELAXED>(tp, li, h, s, stage, ring_bytes, status, push);
            else
                main_panel<float, PUSH, BC1>(tp, li, h, s, stage, ring_bytes, status, push);
        } else {
            if (tp->dtype == QF_BF16)
                main_flat_dispatch<__nv_bfloat16>(tp, li, h, s, status, push);
            else if (tp->dtype == QF_F16)
                main_flat_dispatch<__half>(tp, li, h, s, status, push);
            else
                main_flat_dispatch<float>(tp, li, h, s, status, push);
        }
    }
}

// One tensor passed by value (the single-tensor entry points that mirror the reference's per-tensor
// calls).  Block-128 and fp32-state kinds only; the non-finite flag goes to a word nobody reads.
__device__ uint32_t g_unread_status;
__global__ void __launch_bounds__(kThreads)
single_tensor_kernel(const __grid_constant__ DevTensor t, const __grid_constant__ HyperDev h) {
    __shared__ Smem s;
    load_smem(s);
    const int64_t item = static_cast<int64_t>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
    if (item * (kPanelCols * kRowsPerItem) >= t.numel) return;
    if (t.dtype == QF_BF16)
        main_flat_dispatch<__nv_bfloat16>(&t, item, h, s, &g_unread_status, nullptr);
    else if (t.dtype == QF_F16)
        main_flat_dispatch<__half>(&t, item, h, s, &g_unread_status, nullptr);
    else
        main_flat_dispatch<float>(&t, item, h, s, &g_unread_status, nullptr);
}

// Mean of the copies of a gradient range that the devices of a node hold, taken by the device that owns the range (the
// gradient half of a sharded step): g[i] := RN((copy_0[i] + copy_1[i] + ...) * inv_count) in the gradient's dtype, the
// sum in fp32 in the order of `pp.delta` (byte distances from g to each copy; 0 = this device's own).  Every thread has
// one 16-byte load per copy in flight, so the peer links are busy from all warps at once; only this device's copy is
// written, and only inside the range, which no other device reads.
template <typename T>
__global__ void __launch_bounds__(kThreads)
grad_mean_peers_kernel(char* __restrict__ g, int64_t numel, const __grid_constant__ PushPack pp, float inv_count) {
    constexpr int64_t kVec = 8;
    const int64_t nvec = numel / kVec, npair = nvec / 2;
    const int n = pp.n;
    // two neighbouring vectors per thread and turn: all loads of a copy go out before the first sum needs one
    for (int64_t q = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; q < npair; q += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t e = q * 2 * kVec;
        float a0[8], a1[8], x0[8], x1[8];
        Elem<T>::load8(g + pp.delta[0], e, a0);
        Elem<T>::load8(g + pp.delta[0], e + kVec, a1);
        for (int k = 1; k < n; ++k) {
            Elem<T>::load8(g + pp.delta[k], e, x0);
            Elem<T>::load8(g + pp.delta[k], e + kVec, x1);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                a0[i] = __fadd_rn(a0[i], x0[i]);
                a1[i] = __fadd_rn(a1[i], x1[i]);
            }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            a0[i] = __fmul_rn(a0[i], inv_count);
            a1[i] = __fmul_rn(a1[i], inv_count);
        }
        Elem<T>::store8(g, e, a0);
        Elem<T>::store8(g, e + kVec, a1);
    }
    if (blockIdx.x == 0) {     // what two-vector turns leave over: at most 15 elements
        for (int64_t e = npair * 2 * kVec + threadIdx.x; e < numel; e += blockDim.x) {
            float a = Elem<T>::load1(g + pp.delta[0], e);
            for (int k = 1; k < n; ++k) a = __fadd_rn(a, Elem<T>::load1(g + pp.delta[k], e));
            Elem<T>::store1(g, e, __fmul_rn(a, inv_count));
        }
    }
}

// End of a step that took its hyper-parameters from a device-resident table: the next step takes the next row.
// counters[0] stops one past the last row; a step that ran there used the last row again, which is an error
// (reported in the status word) unless the caller said that the last row repeats for ever.
__global__ void sched_advance_kernel(int32_t* counters, int rows, int tail_repeats, uint32_t* status) {
    if (blockIdx.x != 0 || threadIdx.x != 0) return;
    const int32_t r = counters[0];
    if (r >= rows && !tail_repeats) atomicOr(status, QF_STATUS_SCHEDULE_END);
    counters[0] = r < rows ? r + 1 : rows;
    counters[1] += 1;
}

// Small passes over the row / column maxima of every rank-1 tensor.  One CTA per (tensor, slice).
//   kRollClear     new maxima := 0                       (before the first pass)
//   kRollRecip     reciprocals of the new maxima         (between the passes; 0 for a zero maximum, NaN
//                  where the old or the new maximum is outside the range of the fast division)
//   kRollCommit    stored maxima := new maxima           (after the second pass)
constexpr int kRollSlices = 4;
enum { kRollClear = 0, kRollRecip = 1, kRollCommit = 2 };
__global__ void __launch_bounds__(kThreads)
rank1_roll_kernel(const DevTensor* __restrict__ tensors, int n, int mode) {
    const int ti = blockIdx.x / kRollSlices;
    if (ti >= n) return;
    const DevTensor& t = tensors[ti];
    if (t.kind != QF_KIND_RANK1) return;
    const int total = t.rows + t.cols;
    for (int i = (blockIdx.x % kRollSlices) * kThreads + threadIdx.x; i < total; i += kRollSlices * kThreads) {
        const bool is_row = i < t.rows;
        const int k = is_row ? i : i - t.rows;
        float* nw = is_row ? t.vrow_new : t.vcol_new;
        float* rcp = is_row ? t.vrow_rcp : t.vcol_rcp;
        if (mode == kRollClear) {
            nw[k] = 0.0f;
        } else if (mode == kRollRecip) {
            const float x = nw[k], old = (is_row ? t.vs : t.vcol)[k];
            const float r = x == 0.0f ? 0.0f : __frcp_rn(x);
            rcp[k] = scale_safe(x) && scale_safe(old) ? r : __uint_as_float(0x7fc00000u);
        } else {
            (is_row ? t.vs : t.vcol)[k] = nw[k];
        }
    }
}

// =================================================================================================
// Stand-alone quantize / dequantize kernels (fp32 in / out)
// =================================================================================================

// Block-128 quantize: one warp item = kRowsPerItem runs of 256 elements.  MAP: 0 first-moment map (table search),
// 1 second-moment map (closed form).  Items that lie wholly inside a vector-aligned tensor take a loop without
// masks; the last item and unaligned tensors take the general one.
template <int MAP>
__global__ void __launch_bounds__(kThreads)
quantize_block_kernel(const float* __restrict__ x, int64_t numel, uint8_t* __restrict__ codes, float* __restrict__ scales,
                      int vec) {
    __shared__ Smem s;
    load_smem(s);
    const float* mid = MAP ? s.t.mv : s.t.mm;
    const int lane = threadIdx.x & 31;
    // warps stride over the items, so that a CTA fills its search table once for many items
    const int64_t per_item = static_cast<int64_t>(kPanelCols) * kRowsPerItem;
    const int64_t total = (numel + per_item - 1) / per_item, stride = static_cast<int64_t>(gridDim.x) * kWarpsPerCta;
    for (int64_t item = static_cast<int64_t>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5); item < total; item += stride) {
        const int64_t start = item * per_item;
        if (vec && start + per_item <= numel) {  // warp-uniform
            // Lane L takes elements 4L .. 4L+3 of the first and of the second 128-block of a run: each of its two
            // 128-bit loads is then one of 32 consecutive 16-byte pieces (a load instruction of the warp reads 512
            // contiguous bytes), and each block maximum is one reduction over the whole warp.
            const float4* src = reinterpret_cast<const float4*>(x + start) + lane;
            uint16_t* c16 = reinterpret_cast<uint16_t*>(codes + (start >> 1)) + lane;
            float* sc_out = scales + (start >> 7);
            float4 na = src[0], nb = src[32];  // the next run's input is requested before this run is worked on
            for (int it = 0; it < kRowsPerItem; ++it) {
                const f2 va[2] = {mk2(na.x, na.y), mk2(na.z, na.w)}, vb[2] = {mk2(nb.x, nb.y), mk2(nb.z, nb.w)};
                const int nx = it + 1 < kRowsPerItem ? it + 1 : it;  // past the end: read the last run again
                na = src[nx * 64];
                nb = src[nx * 64 + 32];
                // bit patterns, so that a NaN survives the maximum
                const uint32_t ma = max(max(absbits(va[0].x), absbits(va[0].y)), max(absbits(va[1].x), absbits(va[1].y)));
                const uint32_t mb = max(max(absbits(vb[0].x), absbits(vb[0].y)), max(absbits(vb[1].x), absbits(vb[1].y)));
                const float sa = __uint_as_float(__reduce_max_sync(kFull, ma)), sb = __uint_as_float(__reduce_max_sync(kFull, mb));
                uint32_t wa = 0, wb = 0;
                if (scale_safe(sa) && scale_safe(sb)) {   // warp-uniform: both are reduction results
                    const f2 ra = bc2(sa == 0.0f ? 0.0f : __frcp_rn(sa)), nsa = bc2(-sa);
                    const f2 rb = bc2(sb == 0.0f ? 0.0f : __frcp_rn(sb)), nsb = bc2(-sb);
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const f2 qa = div2_prepared(va[j], ra, nsa), qb = div2_prepared(vb[j], rb, nsb);
                        wa += (MAP ? search_v_closed(qa.x) : search_m_lut(qa.x, s.mlut, s.t.mm)) << (8 * j);
                        wa += (MAP ? search_v_closed(qa.y) : search_m_lut(qa.y, s.mlut, s.t.mm)) << (8 * j + 4);
                        wb += (MAP ? search_v_closed(qb.x) : search_m_lut(qb.x, s.mlut, s.t.mm)) << (8 * j);
                        wb += (MAP ? search_v_closed(qb.y) : search_m_lut(qb.y, s.mlut, s.t.mm)) << (8 * j + 4);
                    }
                } else {
                    const float xa[4] = {va[0].x, va[0].y, va[1].x, va[1].y}, xb[4] = {vb[0].x, vb[0].y, vb[1].x, vb[1].y};
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        wa |= search16(scaled(xa[k], sa), mid) << (4 * k);
                        wb |= search16(scaled(xb[k], sb), mid) << (4 * k);
                    }
                }
                c16[it * 64] = static_cast<uint16_t>(wa);
                c16[it * 64 + 32] = static_cast<uint16_t>(wb);
                if (lane == 0) {
                    sc_out[2 * it] = sa;
                    sc_out[2 * it + 1] = sb;
                }
            }
            continue;
        }
        for (int it = 0; it < kRowsPerItem; ++it) {
            const int64_t wbase = start + static_cast<int64_t>(it) * kPanelCols;
            if (wbase >= numel) break;
            const int64_t e = wbase + lane * 8;
            const int nv = static_cast<int>(max(static_cast<int64_t>(0), min(static_cast<int64_t>(8), numel - e)));
            float v[8];
            load8_masked<float>(reinterpret_cast<const char*>(x), e, nv, vec, v);
            const float sc = absmax8_bits_to_block(v);
            if (nv) store_codes(codes, e, nv, vec, quantize8(v, sc, mid, nv));
            if (nv && (lane & 15) == 0) scales[e >> 7] = sc;
        }
    }
}

// How the stand-alone dequantize kernels divide a run of 256 fp32 outputs (1 KB) among the lanes: lane L writes
// elements 4L .. 4L+3 and 128+4L .. 128+4L+3, so that each of its two 128-bit stores is one of 32 consecutive 16-byte
// pieces: a store instruction of the warp then covers 512 contiguous bytes.  With 8 consecutive elements per lane the
// two stores of a lane would sit 32 bytes apart and every instruction would write half of each 32-byte sector.
// The codes of a lane's two quads are two 16-bit loads (64 contiguous bytes per warp each).
__global__ void __launch_bounds__(kThreads)
dequantize_block_kernel(const uint8_t* __restrict__ codes, const float* __restrict__ scales, int64_t numel, int map,
                        float* __restrict__ out, int vec) {
    __shared__ Tables s;
    __shared__ float2 pair[256];   // (value of the low nibble, value of the high nibble) of a byte of codes
    for (int i = threadIdx.x; i < 256; i += blockDim.x)
        pair[i] = map ? make_float2(c_qv[i & 15], c_qv[i >> 4]) : make_float2(c_qm[i & 15], c_qm[i >> 4]);
    load_tables(s);  // ends with __syncthreads()
    const float* q = map ? s.qv : s.qm;
    const int lane = threadIdx.x & 31;
    const int64_t item = static_cast<int64_t>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
    const int64_t start = item * (kPanelCols * kRowsPerItem);
    if (vec && start + kPanelCols * kRowsPerItem <= numel) {  // warp-uniform: a whole item inside an aligned tensor
        const uint16_t* c16 = reinterpret_cast<const uint16_t*>(codes + (start >> 1)) + lane;
        const float* sc = scales + (start >> 7);
        float4* dst = reinterpret_cast<float4*>(out + start) + lane;
        // the code halves and scales of four runs are requested together, then expanded and stored
        for (int it0 = 0; it0 < kRowsPerItem; it0 += 4) {
            uint32_t wa[4], wb[4];
            float sa[4], sb[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                wa[i] = __ldg(c16 + (it0 + i) * 64);
                wb[i] = __ldg(c16 + (it0 + i) * 64 + 32);
                sa[i] = __ldg(sc + (it0 + i) * 2);
                sb[i] = __ldg(sc + (it0 + i) * 2 + 1);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const f2 a2 = bc2(sa[i]), b2 = bc2(sb[i]);
                const f2 a0 = mul2(pair[wa[i] & 0xffu], a2), a1 = mul2(pair[wa[i] >> 8], a2);
                const f2 b0 = mul2(pair[wb[i] & 0xffu], b2), b1 = mul2(pair[wb[i] >> 8], b2);
                dst[(it0 + i) * 64] = make_float4(a0.x, a0.y, a1.x, a1.y);
                dst[(it0 + i) * 64 + 32] = make_float4(b0.x, b0.y, b1.x, b1.y);
            }
        }
        return;
    }
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

// Rank-1 dequantize for matrices whose column count is a multiple of 256 (buffers vector-aligned), with the same
// division of a row's 256-column panel among the lanes: 512 contiguous bytes per store instruction.  A lane keeps
// the maxima of its 8 columns in registers; the next row's codes are requested before this row is worked on.
__global__ void __launch_bounds__(kThreads)
rank1_dequant_panel_kernel(const uint8_t* __restrict__ codes, const float* __restrict__ row_max, const float* __restrict__ col_max,
                           int rows, int cols, float* __restrict__ out) {
    __shared__ float2 pair[256];
    for (int i = threadIdx.x; i < 256; i += blockDim.x) pair[i] = make_float2(c_qv[i & 15], c_qv[i >> 4]);
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int panels = cols / kPanelCols;
    const int64_t total = static_cast<int64_t>((rows + kRowsPerItem - 1) / kRowsPerItem) * panels;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kWarpsPerCta;
    for (int64_t item = static_cast<int64_t>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5); item < total; item += stride) {
        const int band = static_cast<int>(item / panels);
        const int c0 = static_cast<int>(item - static_cast<int64_t>(band) * panels) * kPanelCols;   // first column of the panel
        const int r0 = band * kRowsPerItem, r1 = min(r0 + kRowsPerItem, rows);
        const float4 ca = __ldg(reinterpret_cast<const float4*>(col_max + c0) + lane);
        const float4 cb = __ldg(reinterpret_cast<const float4*>(col_max + c0 + 128) + lane);
        const uint16_t* c16 = reinterpret_cast<const uint16_t*>(codes) + lane;
        int64_t e = static_cast<int64_t>(r0) * cols + c0;      // first element of the panel's row
        uint32_t wa = __ldg(c16 + (e >> 2)), wb = __ldg(c16 + (e >> 2) + 32);
        float row = __ldg(row_max + r0);
        for (int r = r0; r < r1; ++r, e += cols) {
            const uint32_t xa = wa, xb = wb;
            const float rw = row;
            if (r + 1 < r1) {
                wa = __ldg(c16 + ((e + cols) >> 2));
                wb = __ldg(c16 + ((e + cols) >> 2) + 32);
                row = __ldg(row_max + r + 1);
            }
            const f2 a0 = mul2(pair[xa & 0xffu], mk2(fminf(rw, ca.x), fminf(rw, ca.y)));
            const f2 a1 = mul2(pair[xa >> 8], mk2(fminf(rw, ca.z), fminf(rw, ca.w)));
            const f2 b0 = mul2(pair[xb & 0xffu], mk2(fminf(rw, cb.x), fminf(rw, cb.y)));
            const f2 b1 = mul2(pair[xb >> 8], mk2(fminf(rw, cb.z), fminf(rw, cb.w)));
            float4* dst = reinterpret_cast<float4*>(out + e) + lane;
            dst[0] = make_float4(a0.x, a0.y, a1.x, a1.y);
            dst[32] = make_float4(b0.x, b0.y, b1.x, b1.y);
        }
    }
}

// Row / column maxima of |v| for an [R, C] fp32 matrix.  panel != 0: C is a multiple of 256 and the
// buffers are vector-aligned; otherwise per-element atomics.
__global__ void __launch_bounds__(kThreads)
rank1_max_kernel(const float* __restrict__ v, int rows, int cols, float* __restrict__ row_max,
                 float* __restrict__ col_max, int panel) {
    const int lane = threadIdx.x & 31;
    const int64_t item = static_cast<int64_t>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
    if (panel) {
        const int panels = cols / kPanelCols;
        const int band = static_cast<int>(item / panels);
        const int r0 = band * kPreRowsPerItem;  // tall items: one column atomic per 64 rows
        if (r0 >= rows) return;
        const int r1 = min(r0 + kPreRowsPerItem, rows);
        // lane L takes columns 4L .. 4L+3 and 128+4L .. 128+4L+3 of the panel: each of its two 128-bit loads is one of
        // 32 consecutive 16-byte pieces, a load instruction of the warp reads 512 contiguous bytes
        const int c0 = static_cast<int>(item - static_cast<int64_t>(band) * panels) * kPanelCols;
        uint32_t cmax[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) cmax[k] = 0;
        // four rows are requested together (4 KB per warp in flight): this pass does almost no arithmetic and
        // lives on memory-level parallelism.  Past the last row the last row is read again, which changes no maximum.
        for (int rb = r0; rb < r1; rb += 4) {
            float x[4][8];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float4* src = reinterpret_cast<const float4*>(v + static_cast<int64_t>(min(rb + i, r1 - 1)) * cols + c0) + lane;
                const float4 a = __ldg(src), b = __ldg(src + 32);
                x[i][0] = a.x; x[i][1] = a.y; x[i][2] = a.z; x[i][3] = a.w;
                x[i][4] = b.x; x[i][5] = b.y; x[i][6] = b.z; x[i][7] = b.w;
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                uint32_t rmax = 0;
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const uint32_t b = absbits(x[i][k]);
                    rmax = max(rmax, b);
                    cmax[k] = max(cmax[k], b);
                }
                rmax = __reduce_max_sync(kFull, rmax);
                if (lane == 0 && rb + i < r1) atomic_max_nonneg(row_max + rb + i, rmax);
            }
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) atomic_max_nonneg(col_max + c0 + (k < 4 ? 0 : 124) + lane * 4 + k, cmax[k]);
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

// Rank-1 quantize for matrices whose column count is a multiple of 256 and whose buffers are vector-aligned: panel
// mapping (a lane keeps its 8 column maxima in registers, the row maximum is one broadcast load per row), packed
// division and the closed-form search where the scales allow it.
__global__ void __launch_bounds__(kThreads)
rank1_quant_panel_kernel(const float* __restrict__ in, uint8_t* __restrict__ codes, const float* __restrict__ row_max,
                         const float* __restrict__ col_max, int rows, int cols) {
    __shared__ SmemPre s;
    load_smem(s);
    const int lane = threadIdx.x & 31;
    const int panels = cols / kPanelCols;
    const int64_t total = static_cast<int64_t>((rows + kRowsPerItem - 1) / kRowsPerItem) * panels;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kWarpsPerCta;
    for (int64_t item = static_cast<int64_t>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5); item < total; item += stride) {
        const int band = static_cast<int>(item / panels);
        // lane L takes columns 4L .. 4L+3 and 128+4L .. 128+4L+3 of the panel (512 contiguous bytes per load instruction)
        const int c0 = static_cast<int>(item - static_cast<int64_t>(band) * panels) * kPanelCols;
        const int r0 = band * kRowsPerItem, r1 = min(r0 + kRowsPerItem, rows);
        float col[8];
        {
            const float4 a = __ldg(reinterpret_cast<const float4*>(col_max + c0) + lane), b = __ldg(reinterpret_cast<const float4*>(col_max + c0 + 128) + lane);
            col[0] = a.x; col[1] = a.y; col[2] = a.z; col[3] = a.w;
            col[4] = b.x; col[5] = b.y; col[6] = b.z; col[7] = b.w;
        }
        bool ok = true;
#pragma unroll
        for (int k = 0; k < 8; ++k) ok &= scale_safe(col[k]) && col[k] > 0.0f;
        const bool col_fast = __all_sync(kFull, ok);
        // the next row's input is requested before this row is worked on: two rows per warp in flight
        int64_t e = static_cast<int64_t>(r0) * cols + c0;
        float4 na = __ldg(reinterpret_cast<const float4*>(in + e) + lane), nb = __ldg(reinterpret_cast<const float4*>(in + e) + lane + 32);
        float rown = __ldg(row_max + r0);
        for (int r = r0; r < r1; ++r, e += cols) {
            const float row = rown;
            const float x[8] = {na.x, na.y, na.z, na.w, nb.x, nb.y, nb.z, nb.w};
            if (r + 1 < r1) {
                rown = __ldg(row_max + r + 1);
                na = __ldg(reinterpret_cast<const float4*>(in + e + cols) + lane);
                nb = __ldg(reinterpret_cast<const float4*>(in + e + cols) + lane + 32);
            }
            uint32_t w = 0;   // codes of the first quad in bits 0..15, of the second in bits 16..31
            if (col_fast && scale_safe(row) && row > 0.0f) {  // warp-uniform
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const f2 sc = mk2(fminf(row, col[2 * j]), fminf(row, col[2 * j + 1]));
                    const f2 y = fma2(div2(mk2(x[2 * j], x[2 * j + 1]), sc), bc2(16.0f), bc2(-1.5f));
                    w += code_from_y(y.x) << (8 * j);
                    w += code_from_y(y.y) << (8 * j + 4);
                }
            } else {
#pragma unroll
                for (int k = 0; k < 8; ++k) w |= search16(scaled(x[k], fminf(row, col[k])), s.t.mv) << (4 * k);
            }
            uint16_t* c16 = reinterpret_cast<uint16_t*>(codes) + (e >> 2) + lane;
            c16[0] = static_cast<uint16_t>(w);
            c16[32] = static_cast<uint16_t>(w >> 16);
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
