// Host side of libquantfour_b200.so: argument validation, the device descriptor table and the
// launches.  The exported functions are declared and documented in include/quantfour_b200.h.
#include <algorithm>
#include <cmath>
#include <cstdarg>
#include <cstddef>
#include <cstdio>
#include <cstring>
#include <iterator>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "qf_kernels.cuh"

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
    return code;
}

#define QF_CUDA(call)                                                                          \
    do {                                                                                       \
        cudaError_t e_ = (call);                                                               \
        if (e_ != cudaSuccess) {                                                               \
            (void)cudaGetLastError(); /* a refused call must not leave its code for the host's next check */ \
            return fail(e_ == cudaErrorNoDevice || e_ == cudaErrorInsufficientDriver ? QF_ERR_NO_DEVICE : QF_ERR_CUDA, \
                        "%s failed: %s", #call, cudaGetErrorString(e_));                      \
        }                                                                                      \
    } while (0)

constexpr size_t kStatusBytes = 256;  // head of the workspace: status word, then padding

constexpr int kTables = 4;  // prefix sums: main/panel, main/flat, pre/panel, pre/flat
size_t table_bytes(int n) { return static_cast<size_t>(n) * sizeof(qf::DevTensor) + kTables * (static_cast<size_t>(n) + 1) * 8; }
size_t round_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }
bool valid_dtype(int dtype) { return dtype == QF_F32 || dtype == QF_BF16 || dtype == QF_F16; }
size_t elem_size(int dtype) { return dtype == QF_F32 ? 4 : 2; }

int64_t flat_items(int64_t numel) {
    const int64_t per = static_cast<int64_t>(qf::kPanelCols) * qf::kRowsPerItem;
    return (numel + per - 1) / per;
}

// What the library keeps per workspace: a pair of pinned staging buffers, so that the upload of the table
// only ever waits for the upload of the call before the previous one on the same workspace.  The table is uploaded on every call unless the caller says that it is in place
// (QF_RUN_TABLE_IN_PLACE): the library remembering "this table is already there" by itself would be wrong as soon as
// the caller recycles the memory (a freed workspace whose address comes back from the allocator zero-filled, with
// descriptors that happen to be identical).
struct WsCache {
    char* pinned[2] = {nullptr, nullptr};
    cudaEvent_t ev[2] = {nullptr, nullptr};
    size_t cap = 0;
    int cur = 0;
};
std::mutex g_mu;
std::unordered_map<uint64_t, WsCache> g_cache;
constexpr size_t kMaxCachedWorkspaces = 64;  // beyond this many, entries whose uploads have finished are dropped

uint64_t cache_key(int device, const void* workspace) {
    return (static_cast<uint64_t>(device) << 56) ^ reinterpret_cast<uint64_t>(workspace);
}
// Frees the staging buffers of one entry; waits for its uploads first when `wait`, else gives up (false) while one
// is still in flight.
bool drop_cache_entry(WsCache& c, bool wait) {
    for (int k = 0; k < 2; ++k) {
        if (!c.ev[k]) continue;
        if (wait)
            (void)cudaEventSynchronize(c.ev[k]);
        else if (cudaEventQuery(c.ev[k]) != cudaSuccess) {
            (void)cudaGetLastError();
            return false;
        }
    }
    for (int k = 0; k < 2; ++k) {
        if (c.pinned[k]) (void)cudaFreeHost(c.pinned[k]);
        if (c.ev[k]) (void)cudaEventDestroy(c.ev[k]);
        c.pinned[k] = nullptr;
        c.ev[k] = nullptr;
    }
    c.cap = 0;
    return true;
}

enum { kMainPanel = 0, kMainFlat = 1, kPrePanel = 2, kPreFlat = 3 };
struct Plan {
    int n = 0;                    // tensors in the table (zero-size tensors dropped)
    int64_t items[kTables] = {0, 0, 0, 0};
    int n_rank1 = 0;
    bool any_f32_panel = false;   // sizes the staging ring of the panel kernel
    bool any_bf16_panel = false;
    qf::DevTensor* d_tensors = nullptr;
    int64_t* d_base[kTables] = {nullptr, nullptr, nullptr, nullptr};
    uint32_t* d_status = nullptr;
};

// Rows per item of the second pass over rank-1 panels: the longest of 64 / 32 / 16 that still gives every warp slot
// of the device (two CTAs of eight warps per SM) an item; `bands64` = sum over the panel tensors of rows * panels / 64.
int sm_count();
int main_rows_for(int64_t items64) {
    const int64_t slots = static_cast<int64_t>(sm_count()) * qf::kMainMinCtas * qf::kWarpsPerCta;
    int rows = qf::kMainRowsPerItem;
    while (rows > 16 && items64 * (qf::kMainRowsPerItem / rows) < slots) rows /= 2;
    return rows;
}

int build_plan(const QfTensorDesc* descs, int n_tensors, int n_hypers, void* workspace, size_t workspace_bytes,
               int device, cudaStream_t stream, Plan* plan, bool upload = true) {
    if (n_tensors < 0) return fail(QF_ERR_BAD_ARG, "n_tensors is negative");
    if (n_tensors > 0 && !descs) return fail(QF_ERR_BAD_ARG, "descs is null");
    if (n_hypers < 1 || n_hypers > QF_MAX_HYPERS)
        return fail(QF_ERR_BAD_ARG, "n_hypers must be in 1..%d, got %d", QF_MAX_HYPERS, n_hypers);
    if (!workspace || workspace_bytes < qf_workspace_bytes(n_tensors))
        return fail(QF_ERR_WORKSPACE, "workspace of %zu bytes needed for %d tensors, got %zu", qf_workspace_bytes(n_tensors),
                    n_tensors, workspace_bytes);
    if (!aligned(workspace, 256)) return fail(QF_ERR_BAD_ARG, "workspace must be 256-byte aligned");

    std::vector<qf::DevTensor> tab;
    std::vector<int64_t> base[kTables];
    for (auto& b : base) b.push_back(0);
    tab.reserve(n_tensors);
    int n_rank1 = 0;
    for (int i = 0; i < n_tensors; ++i) {
        const QfTensorDesc& d = descs[i];
        if (d.numel < 0) return fail(QF_ERR_BAD_ARG, "tensor %d: negative numel", i);
        if (d.numel == 0) continue;
        if (!valid_dtype(d.dtype)) return fail(QF_ERR_BAD_ARG, "tensor %d: bad dtype %d", i, d.dtype);
        if (d.kind < QF_KIND_FP32 || d.kind > QF_KIND_RANK1) return fail(QF_ERR_BAD_ARG, "tensor %d: bad kind %d", i, d.kind);
        if (d.hyper < 0 || d.hyper >= n_hypers) return fail(QF_ERR_BAD_ARG, "tensor %d: hyper index %d out of range", i, d.hyper);
        if (!d.p || !d.g || !d.m || !d.v) return fail(QF_ERR_BAD_ARG, "tensor %d: null p/g/m/v pointer", i);
        const size_t esz = elem_size(d.dtype);
        if (!aligned(d.p, esz) || !aligned(d.g, esz)) return fail(QF_ERR_BAD_ARG, "tensor %d: p/g not element-aligned", i);
        qf::DevTensor t;
        memset(&t, 0, sizeof t);
        t.p = static_cast<char*>(d.p);
        t.g = static_cast<const char*>(d.g);
        t.m = static_cast<char*>(d.m);
        t.v = static_cast<char*>(d.v);
        t.numel = d.numel;
        t.kind = d.kind;
        t.dtype = d.dtype;
        t.hyper = d.hyper;
        bool vec = aligned(d.p, 16) && aligned(d.g, 16);
        if (d.kind == QF_KIND_FP32) {
            if (!aligned(d.m, 4) || !aligned(d.v, 4)) return fail(QF_ERR_BAD_ARG, "tensor %d: fp32 moments misaligned", i);
            vec = vec && aligned(d.m, 16) && aligned(d.v, 16);
        } else {
            if (!d.m_scale || !d.v_scale) return fail(QF_ERR_BAD_ARG, "tensor %d: null scale pointer", i);
            if (!aligned(d.m_scale, 4) || !aligned(d.v_scale, 4)) return fail(QF_ERR_BAD_ARG, "tensor %d: scales misaligned", i);
            vec = vec && aligned(d.m, 4) && aligned(d.v, 4);
            t.ms = d.m_scale;
            t.vs = d.v_scale;
        }
        int64_t items = flat_items(d.numel), pre_items = items;
        if (d.kind == QF_KIND_RANK1) {
            if (d.rows <= 0 || d.cols <= 0 || d.rows > INT32_MAX || d.cols > INT32_MAX || d.flat_offset < 0 ||
                d.flat_offset + d.numel > d.rows * d.cols || (d.flat_offset == 0 && !d.partial && d.rows * d.cols != d.numel))
                return fail(QF_ERR_BAD_ARG, "tensor %d: rows*cols must equal numel, or the record must be marked partial and lie inside the matrix (rows=%lld cols=%lld numel=%lld offset=%lld)",
                            i, (long long)d.rows, (long long)d.cols, (long long)d.numel, (long long)d.flat_offset);
            if (!d.v_col || !d.v_row_new || !d.v_col_new) return fail(QF_ERR_BAD_ARG, "tensor %d: null rank-1 buffer", i);
            if (!aligned(d.v_col, 4) || !aligned(d.v_row_new, 4) || !aligned(d.v_col_new, 4))
                return fail(QF_ERR_BAD_ARG, "tensor %d: rank-1 buffers misaligned", i);
            t.rows = static_cast<int32_t>(d.rows);
            t.cols = static_cast<int32_t>(d.cols);
            t.vcol = d.v_col;
            t.vrow_new = d.v_row_new;
            t.vcol_new = d.v_col_new;
            t.vrow_rcp = d.v_row_rcp ? d.v_row_rcp : d.v_row_new + d.rows;
            t.vcol_rcp = d.v_col_rcp ? d.v_col_rcp : d.v_col_new + d.cols;
            t.flat_off = d.flat_offset;
            if (!aligned(t.vrow_rcp, 4) || !aligned(t.vcol_rcp, 4)) return fail(QF_ERR_BAD_ARG, "tensor %d: rank-1 buffers misaligned", i);
            const bool whole = d.flat_offset == 0 && d.rows * d.cols == d.numel;
            const bool panel = whole && d.dtype != QF_F16 && d.numel < (1ll << 31) && vec && d.cols % qf::kPanelCols == 0 && aligned(d.v_col, 16) && aligned(d.v_col_new, 16) &&
                               aligned(t.vcol_rcp, 16);
            if (panel) {
                t.flags |= qf::kFlagPanel;
                t.panels = static_cast<int32_t>(d.cols / qf::kPanelCols);
                t.main_rows = qf::kMainRowsPerItem;
                items = (d.rows + qf::kMainRowsPerItem - 1) / qf::kMainRowsPerItem * t.panels;
                pre_items = (d.rows + qf::kPreRowsPerItem - 1) / qf::kPreRowsPerItem * t.panels;
                if (d.dtype == QF_F32) plan->any_f32_panel = true;
                if (d.dtype == QF_BF16) plan->any_bf16_panel = true;
            }
            ++n_rank1;
        }
        if (vec) t.flags |= qf::kFlagVec;
        const bool panel = t.flags & qf::kFlagPanel, rank1 = d.kind == QF_KIND_RANK1;
        base[kMainPanel].push_back(base[kMainPanel].back() + (panel ? items : 0));
        base[kMainFlat].push_back(base[kMainFlat].back() + (panel ? 0 : items));
        base[kPrePanel].push_back(base[kPrePanel].back() + (rank1 && panel ? pre_items : 0));
        base[kPreFlat].push_back(base[kPreFlat].back() + (rank1 && !panel ? pre_items : 0));
        tab.push_back(t);
    }
    const int n = static_cast<int>(tab.size());
    // a small launch: shorter items in the second pass, so that the whole device takes part
    const int main_rows = main_rows_for(base[kMainPanel].back());
    if (main_rows != qf::kMainRowsPerItem) {
        int64_t acc = 0;
        for (int i = 0; i < n; ++i) {
            if (tab[i].flags & qf::kFlagPanel) {
                tab[i].main_rows = main_rows;
                acc += (static_cast<int64_t>(tab[i].rows) + main_rows - 1) / main_rows * tab[i].panels;
            }
            base[kMainPanel][i + 1] = acc;
        }
    }
    plan->n = n;
    plan->n_rank1 = n_rank1;
    char* ws = static_cast<char*>(workspace);
    plan->d_status = reinterpret_cast<uint32_t*>(ws);
    plan->d_tensors = reinterpret_cast<qf::DevTensor*>(ws + kStatusBytes);
    const size_t tensors_bytes = static_cast<size_t>(n) * sizeof(qf::DevTensor);
    for (int k = 0; k < kTables; ++k) {
        plan->items[k] = base[k].back();
        plan->d_base[k] = reinterpret_cast<int64_t*>(ws + kStatusBytes + tensors_bytes) + static_cast<size_t>(k) * (n + 1);
    }
    if (n == 0 || !upload) return QF_OK;

    const size_t bytes = table_bytes(n);
    std::lock_guard<std::mutex> lock(g_mu);
    const uint64_t key = cache_key(device, workspace);
    if (g_cache.size() >= kMaxCachedWorkspaces && g_cache.find(key) == g_cache.end()) {
        // a host that keeps handing in new workspace addresses: forget the entries that are idle
        for (auto it = g_cache.begin(); it != g_cache.end();)
            it = drop_cache_entry(it->second, false) ? g_cache.erase(it) : std::next(it);
    }
    WsCache& c = g_cache[key];
    if (c.cap < bytes) {
        for (int k = 0; k < 2; ++k) {
            if (c.pinned[k]) cudaFreeHost(c.pinned[k]);
            c.pinned[k] = nullptr;
            QF_CUDA(cudaMallocHost(reinterpret_cast<void**>(&c.pinned[k]), round_up(bytes, 4096)));
            if (!c.ev[k]) QF_CUDA(cudaEventCreateWithFlags(&c.ev[k], cudaEventDisableTiming));
        }
        c.cap = round_up(bytes, 4096);
    }
    const int k = c.cur ^ 1;
    QF_CUDA(cudaEventSynchronize(c.ev[k]));  // the copy that last used this staging buffer has finished
    memcpy(c.pinned[k], tab.data(), tensors_bytes);
    for (int t = 0; t < kTables; ++t)
        memcpy(c.pinned[k] + tensors_bytes + static_cast<size_t>(t) * (n + 1) * 8, base[t].data(), (n + 1) * 8);
    QF_CUDA(cudaMemcpyAsync(ws + kStatusBytes, c.pinned[k], bytes, cudaMemcpyHostToDevice, stream));
    QF_CUDA(cudaEventRecord(c.ev[k], stream));
    c.cur = k;
    return QF_OK;
}

int grid_for(int64_t items, unsigned* grid) {
    const int64_t ctas = (items + qf::kWarpsPerCta - 1) / qf::kWarpsPerCta;
    if (ctas > 0x7fffffffLL) return fail(QF_ERR_BAD_ARG, "too many work items for one launch (%lld)", (long long)items);
    *grid = static_cast<unsigned>(ctas);
    return QF_OK;
}

// Grid of a multi-tensor kernel: kGridWaves waves of CTAs (16 measured best: CTAs live long enough to amortise
// their table set-up, yet the tail stays short), never more than there is work; warps stride over the items.
int sm_count() {
    static int cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (!cached[dev]) {
        int n = 0;
        cached[dev] = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0 ? n : 148;
    }
    return cached[dev];
}
constexpr int kGridWaves = 16;
unsigned persistent_grid(int64_t items, int per_sm, int waves = kGridWaves) {
    const int64_t ctas = (items + qf::kWarpsPerCta - 1) / qf::kWarpsPerCta;
    const int64_t cap = static_cast<int64_t>(sm_count()) * per_sm * waves;
    return static_cast<unsigned>(ctas < cap ? ctas : cap);
}

void roll(const Plan& pl, int mode, cudaStream_t stream) {
    qf::rank1_roll_kernel<<<pl.n * qf::kRollSlices, qf::kThreads, 0, stream>>>(pl.d_tensors, pl.n, mode);
}

qf::Sched no_sched() {
    qf::Sched sc;
    memset(&sc, 0, sizeof sc);
    return sc;
}

template <bool SCALE, bool SCHED>
int launch_pre_panel(const Plan& pl, const qf::HyperPack& hp, const qf::Sched& sc, cudaStream_t stream) {
    const int dyn = qf::pre_dyn_smem(pl.any_f32_panel);
    QF_CUDA(cudaFuncSetAttribute(qf::step_pre_kernel<true, SCALE, SCHED>, cudaFuncAttributeMaxDynamicSharedMemorySize, qf::pre_dyn_smem(true)));
    qf::step_pre_kernel<true, SCALE, SCHED><<<persistent_grid(pl.items[kPrePanel], qf::kPreMinCtas), qf::kThreads, dyn, stream>>>(
        pl.d_tensors, pl.d_base[kPrePanel], pl.n, hp, dyn / qf::kWarpsPerCta, pl.d_status, sc);
    return QF_OK;
}

// `sched`: null, or the device-resident hyper-parameter table the kernels read instead of `hp`; `scaled` then says
// whether some row of it carries a gradient scale (the host cannot look).
int launch_pre(const Plan& pl, const qf::HyperPack& hp, int n_hypers, cudaStream_t stream, const qf::Sched* sched = nullptr,
               bool scaled = false) {
    if (pl.n_rank1 == 0) return QF_OK;
    roll(pl, qf::kRollClear, stream);
    if (pl.items[kPrePanel]) {
        // the variant that rewrites the gradients runs only when some set asks for it
        if (!sched)
            for (int k = 0; k < n_hypers; ++k) scaled = scaled || hp.h[k].gs != 1.0f;
        int rc;
        if (sched)
            rc = scaled ? launch_pre_panel<true, true>(pl, hp, *sched, stream) : launch_pre_panel<false, true>(pl, hp, *sched, stream);
        else
            rc = scaled ? launch_pre_panel<true, false>(pl, hp, no_sched(), stream) : launch_pre_panel<false, false>(pl, hp, no_sched(), stream);
        if (rc) return rc;
    }
    if (pl.items[kPreFlat]) {
        const unsigned grid = persistent_grid(pl.items[kPreFlat], qf::kPreMinCtas);
        if (sched)
            qf::step_pre_kernel<false, false, true><<<grid, qf::kThreads, 0, stream>>>(pl.d_tensors, pl.d_base[kPreFlat], pl.n, hp, 0,
                                                                                     pl.d_status, *sched);
        else
            qf::step_pre_kernel<false><<<grid, qf::kThreads, 0, stream>>>(pl.d_tensors, pl.d_base[kPreFlat], pl.n, hp, 0, pl.d_status,
                                                                          no_sched());
    }
    QF_CUDA(cudaGetLastError());
    return QF_OK;
}

template <bool PUSH, bool BC1, bool SCHED, bool RELAXED, int DT>
int launch_main_panel_dt(const Plan& pl, const qf::HyperPack& hp, const qf::PushPack& pp, const qf::Sched& sc, cudaStream_t stream) {
    const int dyn = qf::main_dyn_smem(pl.any_f32_panel);
    const int ring = qf::kStages * (pl.any_f32_panel ? qf::kRowBytesF32 : qf::kRowBytesBf16);
    QF_CUDA(cudaFuncSetAttribute(qf::step_main_kernel<true, PUSH, BC1, SCHED, RELAXED, DT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 qf::main_dyn_smem(true)));
    qf::step_main_kernel<true, PUSH, BC1, SCHED, RELAXED, DT><<<persistent_grid(pl.items[kMainPanel], qf::kMainMinCtas), qf::kThreads, dyn, stream>>>(
        pl.d_tensors, pl.d_base[kMainPanel], pl.n, hp, ring, pl.d_status, pp, sc);
    return QF_OK;
}
// A launch whose panel tensors are all of one dtype takes the kernel that carries that dtype's loop only (the plain
// step, the common case; the rarer variants keep the two-dtype kernel): 1.4 % faster, measured.
template <bool PUSH, bool BC1, bool SCHED, bool RELAXED = false>
int launch_main_panel(const Plan& pl, const qf::HyperPack& hp, const qf::PushPack& pp, const qf::Sched& sc, cudaStream_t stream) {
    if (!PUSH && !SCHED && !RELAXED && !pl.any_f32_panel) return launch_main_panel_dt<false, BC1, false, false, 1>(pl, hp, pp, sc, stream);
    if (!PUSH && !SCHED && !RELAXED && !pl.any_bf16_panel) return launch_main_panel_dt<false, BC1, false, false, 2>(pl, hp, pp, sc, stream);
    return launch_main_panel_dt<PUSH, BC1, SCHED, RELAXED, 0>(pl, hp, pp, sc, stream);
}

// bc_one: every hyper-parameter set of the call has bc2s == 1 exactly (late in a run): the panel kernel then
// runs the variant without the division by it.
// relaxed (without peer stores only): the panel kernel whose bf16 parameter update is uncorrected.
template <bool PUSH>
int launch_main_kernels(const Plan& pl, const qf::HyperPack& hp, const qf::PushPack& pp, bool bc_one, cudaStream_t stream,
                        bool relaxed = false) {
    if (pl.items[kMainPanel]) {
        int rc;
        if (!PUSH && relaxed)
            rc = bc_one ? launch_main_panel<false, true, false, true>(pl, hp, pp, no_sched(), stream)
                        : launch_main_panel<false, false, false, true>(pl, hp, pp, no_sched(), stream);
        else
            rc = bc_one ? launch_main_panel<PUSH, true, false>(pl, hp, pp, no_sched(), stream)
                        : launch_main_panel<PUSH, false, false>(pl, hp, pp, no_sched(), stream);
        if (rc) return rc;
    }
    if (pl.items[kMainFlat])
        qf::step_main_kernel<false, PUSH><<<persistent_grid(pl.items[kMainFlat], qf::kMainMinCtas), qf::kThreads, 0, stream>>>(
            pl.d_tensors, pl.d_base[kMainFlat], pl.n, hp, 0, pl.d_status, pp, no_sched());
    return QF_OK;
}

// `push`: null, or the peer copies of the parameter buffer the kernels also store into.
// `sched`: null, or the device-resident hyper-parameter table the kernels read instead of `hp` (no peer stores then,
// and always the variant that divides by the bias correction: what the table holds is not known to the host).
int launch_main(const Plan& pl, const qf::HyperPack& hp, int n_hypers, cudaStream_t stream, const qf::PushPack* push = nullptr,
                const qf::Sched* sched = nullptr, bool relaxed = false) {
    if (pl.n == 0) return QF_OK;
    if (pl.n_rank1) roll(pl, qf::kRollRecip, stream);
    bool bc_one = true;
    for (int k = 0; k < n_hypers; ++k) bc_one = bc_one && hp.h[k].fast && hp.h[k].h.bc2s == 1.0f;
    qf::PushPack none;
    memset(&none, 0, sizeof none);
    if (sched) {
        if (pl.items[kMainPanel])
            if (int rc = launch_main_panel<false, false, true>(pl, hp, none, *sched, stream)) return rc;
        if (pl.items[kMainFlat])
            qf::step_main_kernel<false, false, false, true><<<persistent_grid(pl.items[kMainFlat], qf::kMainMinCtas), qf::kThreads, 0, stream>>>(
                pl.d_tensors, pl.d_base[kMainFlat], pl.n, hp, 0, pl.d_status, none, *sched);
    } else if (push && push->n > 0) {
        if (int rc = launch_main_kernels<true>(pl, hp, *push, bc_one, stream)) return rc;
    } else {
        if (int rc = launch_main_kernels<false>(pl, hp, none, bc_one, stream, relaxed)) return rc;
    }
    if (pl.n_rank1) roll(pl, qf::kRollCommit, stream);
    QF_CUDA(cudaGetLastError());
    return QF_OK;
}

using qf::widen_hyper;

int step_common(const QfTensorDesc* descs, int n_tensors, const QfHyper* hypers, int n_hypers, void* workspace,
                size_t workspace_bytes, int device, void* stream, bool pre, bool main_, const qf::PushPack* push = nullptr,
                bool relaxed = false, bool upload = true) {
    g_err[0] = 0;
    if (!hypers) return fail(QF_ERR_BAD_ARG, "hypers is null");
    QF_CUDA(cudaSetDevice(device));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    Plan pl;
    if (int rc = build_plan(descs, n_tensors, n_hypers, workspace, workspace_bytes, device, st, &pl, upload)) return rc;
    qf::HyperPack hp;
    memset(&hp, 0, sizeof hp);
    for (int k = 0; k < n_hypers; ++k) hp.h[k] = widen_hyper(hypers[k]);
    if (pre)
        if (int rc = launch_pre(pl, hp, n_hypers, st)) return rc;
    if (main_)
        if (int rc = launch_main(pl, hp, n_hypers, st, push, nullptr, relaxed)) return rc;
    return QF_OK;
}

int check_1d(const void* a, const void* b, int64_t numel, const char* what) {
    if (numel < 0) return fail(QF_ERR_BAD_ARG, "%s: negative numel", what);
    if (numel > 0 && (!a || !b)) return fail(QF_ERR_BAD_ARG, "%s: null pointer", what);
    return QF_OK;
}

unsigned flat_grid(int64_t numel) {
    return static_cast<unsigned>((flat_items(numel) + qf::kWarpsPerCta - 1) / qf::kWarpsPerCta);
}

}  // namespace

extern "C" {

int qf_abi_version(void) { return QF_ABI_VERSION; }

const char* qf_last_error(void) { return g_err; }

size_t qf_workspace_bytes(int n_tensors) {
    if (n_tensors < 0) n_tensors = 0;
    return round_up(kStatusBytes + table_bytes(n_tensors), 256);
}

void qf_make_hyper(double lr, double beta1, double beta2, double eps, double weight_decay, double step, QfHyper* out) {
    const double bc1 = 1.0 - std::pow(beta1, step);
    const double bc2 = 1.0 - std::pow(beta2, step);
    out->decay = static_cast<float>(1.0 - lr * weight_decay);
    out->w1 = static_cast<float>(1.0 - beta1);
    out->beta2 = static_cast<float>(beta2);
    out->w2 = static_cast<float>(1.0 - beta2);
    out->eps = static_cast<float>(eps);
    out->neg_step = static_cast<float>(-(lr / bc1));
    out->bc2s = static_cast<float>(std::sqrt(bc2));
    out->grad_scale = 0.0f;
}

int qf_step_multi(const QfTensorDesc* descs, int n_tensors, const QfHyper* hypers, int n_hypers, void* workspace,
                  size_t workspace_bytes, int device, void* stream) {
    return step_common(descs, n_tensors, hypers, n_hypers, workspace, workspace_bytes, device, stream, true, true);
}

int qf_step_pre(const QfTensorDesc* descs, int n_tensors, const QfHyper* hypers, int n_hypers, void* workspace,
                size_t workspace_bytes, int device, void* stream) {
    return step_common(descs, n_tensors, hypers, n_hypers, workspace, workspace_bytes, device, stream, true, false);
}

int qf_step_main(const QfTensorDesc* descs, int n_tensors, const QfHyper* hypers, int n_hypers, void* workspace,
                 size_t workspace_bytes, int device, void* stream) {
    return step_common(descs, n_tensors, hypers, n_hypers, workspace, workspace_bytes, device, stream, false, true);
}

int qf_step_prepare(const QfTensorDesc* descs, int n_tensors, int n_hypers, void* workspace, size_t workspace_bytes, int device,
                    void* stream) {
    g_err[0] = 0;
    QF_CUDA(cudaSetDevice(device));
    Plan pl;
    return build_plan(descs, n_tensors, n_hypers, workspace, workspace_bytes, device, static_cast<cudaStream_t>(stream), &pl);
}

int qf_step_scheduled(const QfTensorDesc* descs, int n_tensors, int n_hypers, void* workspace, size_t workspace_bytes, int device,
                      void* stream, const QfHyper* device_schedule, int schedule_rows, int32_t* device_counters, int flags) {
    g_err[0] = 0;
    if (!device_schedule || !device_counters) return fail(QF_ERR_BAD_ARG, "qf_step_scheduled: null schedule or counters");
    if (schedule_rows < 1) return fail(QF_ERR_BAD_ARG, "qf_step_scheduled: the schedule needs at least one row");
    if (!aligned(device_schedule, 4) || !aligned(device_counters, 4)) return fail(QF_ERR_BAD_ARG, "qf_step_scheduled: misaligned schedule or counters");
    if (flags & ~(QF_SCHED_TAIL_REPEATS | QF_SCHED_GRAD_SCALE)) return fail(QF_ERR_BAD_ARG, "qf_step_scheduled: unknown flag bits 0x%x", flags);
    QF_CUDA(cudaSetDevice(device));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    Plan pl;   // the host half of the plan only: the tables are in the workspace already
    if (int rc = build_plan(descs, n_tensors, n_hypers, workspace, workspace_bytes, device, st, &pl, false)) return rc;
    if (pl.n == 0) return QF_OK;
    qf::Sched sc;
    sc.table = device_schedule;
    sc.counters = device_counters;
    sc.rows = schedule_rows;
    sc.n_hypers = n_hypers;
    qf::HyperPack hp;
    memset(&hp, 0, sizeof hp);
    if (int rc = launch_pre(pl, hp, 0, st, &sc, (flags & QF_SCHED_GRAD_SCALE) != 0)) return rc;
    if (int rc = launch_main(pl, hp, 0, st, nullptr, &sc)) return rc;
    qf::sched_advance_kernel<<<1, 32, 0, st>>>(device_counters, schedule_rows, (flags & QF_SCHED_TAIL_REPEATS) != 0, pl.d_status);
    QF_CUDA(cudaGetLastError());
    return QF_OK;
}

int qf_step_run(const QfTensorDesc* descs, int n_tensors, const QfHyper* hypers, int n_hypers, void* workspace,
                size_t workspace_bytes, int device, void* stream, int what, const int64_t* peer_delta_bytes, int n_peers) {
    g_err[0] = 0;
    if (what & ~(QF_RUN_PRE | QF_RUN_MAIN | QF_RUN_TABLE_IN_PLACE | QF_RUN_RELAXED_UPDATE))
        return fail(QF_ERR_BAD_ARG, "qf_step_run: unknown bits in `what` (0x%x)", what);
    if (!(what & (QF_RUN_PRE | QF_RUN_MAIN))) return fail(QF_ERR_BAD_ARG, "qf_step_run: neither half of the step asked for");
    if (n_peers < 0 || n_peers > QF_MAX_PEERS) return fail(QF_ERR_BAD_ARG, "n_peers must be in 0..%d, got %d", QF_MAX_PEERS, n_peers);
    if (n_peers > 0 && !peer_delta_bytes) return fail(QF_ERR_BAD_ARG, "peer_delta_bytes is null");
    if (n_peers > 0 && !(what & QF_RUN_MAIN)) return fail(QF_ERR_BAD_ARG, "peer stores belong to the second half of the step");
    if (n_peers > 0 && (what & QF_RUN_RELAXED_UPDATE)) return fail(QF_ERR_BAD_ARG, "the relaxed update has no variant with peer stores");
    qf::PushPack pp;
    memset(&pp, 0, sizeof pp);
    pp.n = n_peers;
    for (int k = 0; k < n_peers; ++k) {
        // the vector path stores 16 bytes at p + delta whenever p itself is 16-byte aligned
        if (peer_delta_bytes[k] == 0 || peer_delta_bytes[k] % 16)
            return fail(QF_ERR_BAD_ARG, "peer %d: the distance to the peer buffer must be a non-zero multiple of 16 bytes", k);
        pp.delta[k] = peer_delta_bytes[k];
    }
    return step_common(descs, n_tensors, hypers, n_hypers, workspace, workspace_bytes, device, stream, (what & QF_RUN_PRE) != 0,
                       (what & QF_RUN_MAIN) != 0, n_peers > 0 ? &pp : nullptr, (what & QF_RUN_RELAXED_UPDATE) != 0,
                       !(what & QF_RUN_TABLE_IN_PLACE));
}

int qf_step_main_push(const QfTensorDesc* descs, int n_tensors, const QfHyper* hypers, int n_hypers, void* workspace,
                      size_t workspace_bytes, int device, void* stream, const int64_t* peer_delta_bytes, int n_peers) {
    return qf_step_run(descs, n_tensors, hypers, n_hypers, workspace, workspace_bytes, device, stream, QF_RUN_MAIN, peer_delta_bytes,
                       n_peers);
}

// ---- sharing the parameter buffer between the processes of a node --------------------------------------------
namespace {
// Base of the allocation that holds `ptr`, through the driver entry point (the library links the runtime only).
int allocation_base(const void* ptr, const void** base) {
    typedef int (*RangeFn)(unsigned long long*, size_t*, unsigned long long);
    static RangeFn fn = nullptr;
    if (!fn) {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult st;
        QF_CUDA(cudaGetDriverEntryPoint("cuMemGetAddressRange", &f, cudaEnableDefault, &st));
        if (!f || st != cudaDriverEntryPointSuccess) return fail(QF_ERR_CUDA, "driver entry point cuMemGetAddressRange not found");
        fn = reinterpret_cast<RangeFn>(f);
    }
    unsigned long long b = 0;
    size_t size = 0;
    const int rc = fn(&b, &size, static_cast<unsigned long long>(reinterpret_cast<uintptr_t>(ptr)));
    if (rc != 0) return fail(QF_ERR_BAD_ARG, "pointer is not inside a device allocation (driver error %d)", rc);
    *base = reinterpret_cast<const void*>(static_cast<uintptr_t>(b));
    return QF_OK;
}

// An allocation can be mapped only once per process: mappings are shared and counted.
struct PeerMapping {
    void* base;
    int refs;
};
std::mutex g_peer_mu;
std::unordered_map<std::string, PeerMapping> g_peer_maps;  // key: device byte + handle bytes
std::string peer_key(const unsigned char* handle, int device) {
    std::string k(1, static_cast<char>(device));
    k.append(reinterpret_cast<const char*>(handle), QF_PEER_HANDLE_BYTES);
    return k;
}
}  // namespace

int qf_peer_export(const void* ptr, int device, unsigned char* handle, int64_t* offset_bytes) {
    g_err[0] = 0;
    static_assert(sizeof(cudaIpcMemHandle_t) == QF_PEER_HANDLE_BYTES, "handle size");
    if (!ptr || !handle || !offset_bytes) return fail(QF_ERR_BAD_ARG, "qf_peer_export: null argument");
    QF_CUDA(cudaSetDevice(device));
    const void* base = nullptr;
    if (int rc = allocation_base(ptr, &base)) return rc;
    cudaIpcMemHandle_t h;
    QF_CUDA(cudaIpcGetMemHandle(&h, const_cast<void*>(base)));
    memcpy(handle, &h, sizeof h);
    *offset_bytes = static_cast<const char*>(ptr) - static_cast<const char*>(base);
    return QF_OK;
}

int qf_peer_open(const unsigned char* handle, int device, void** base) {
    g_err[0] = 0;
    if (!handle || !base) return fail(QF_ERR_BAD_ARG, "qf_peer_open: null argument");
    QF_CUDA(cudaSetDevice(device));
    std::lock_guard<std::mutex> lock(g_peer_mu);
    const std::string key = peer_key(handle, device);
    auto it = g_peer_maps.find(key);
    if (it != g_peer_maps.end()) {
        ++it->second.refs;
        *base = it->second.base;
        return QF_OK;
    }
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof h);
    QF_CUDA(cudaIpcOpenMemHandle(base, h, cudaIpcMemLazyEnablePeerAccess));
    g_peer_maps[key] = PeerMapping{*base, 1};
    return QF_OK;
}

int qf_peer_close(void* base, int device) {
    g_err[0] = 0;
    if (!base) return QF_OK;
    QF_CUDA(cudaSetDevice(device));
    std::lock_guard<std::mutex> lock(g_peer_mu);
    for (auto it = g_peer_maps.begin(); it != g_peer_maps.end(); ++it) {
        if (it->second.base != base || it->first[0] != static_cast<char>(device)) continue;
        if (--it->second.refs == 0) {
            g_peer_maps.erase(it);
            QF_CUDA(cudaIpcCloseMemHandle(base));
        }
        return QF_OK;
    }
    return fail(QF_ERR_BAD_ARG, "qf_peer_close: %p is not a mapping qf_peer_open returned", base);
}

int qf_peer_copy(void* dst, int dst_device, const void* src, size_t bytes, int device, void* stream) {
    g_err[0] = 0;
    if (bytes == 0) return QF_OK;
    if (!dst || !src) return fail(QF_ERR_BAD_ARG, "qf_peer_copy: null pointer");
    QF_CUDA(cudaSetDevice(device));
    if (dst_device >= 0)   // the explicit peer form: takes the direct device-to-device path also for mappings of another process's memory
        QF_CUDA(cudaMemcpyPeerAsync(dst, dst_device, src, device, bytes, static_cast<cudaStream_t>(stream)));
    else
        QF_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, static_cast<cudaStream_t>(stream)));
    return QF_OK;
}

int qf_grad_mean_peers(void* g, int64_t numel, int dtype, const int64_t* copy_delta_bytes, int n_copies, float inv_count,
                       int device, void* stream) {
    g_err[0] = 0;
    if (numel < 0) return fail(QF_ERR_BAD_ARG, "qf_grad_mean_peers: negative numel");
    if (numel == 0) return QF_OK;
    if (!g || !copy_delta_bytes) return fail(QF_ERR_BAD_ARG, "qf_grad_mean_peers: null pointer");
    if (!valid_dtype(dtype)) return fail(QF_ERR_BAD_ARG, "bad dtype %d", dtype);
    if (n_copies < 1 || n_copies > QF_MAX_PEERS)
        return fail(QF_ERR_BAD_ARG, "qf_grad_mean_peers: n_copies must be in 1..%d, got %d", QF_MAX_PEERS, n_copies);
    if (!aligned(g, 16)) return fail(QF_ERR_BAD_ARG, "qf_grad_mean_peers: the range must start on a 16-byte boundary");
    qf::PushPack pp;
    memset(&pp, 0, sizeof pp);
    pp.n = n_copies;
    for (int k = 0; k < n_copies; ++k) {
        if (copy_delta_bytes[k] % 16) return fail(QF_ERR_BAD_ARG, "copy %d: the distance to the copy must be a multiple of 16 bytes", k);
        pp.delta[k] = copy_delta_bytes[k];
    }
    QF_CUDA(cudaSetDevice(device));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int64_t turns = (numel + 15) / 16;     // a thread takes two 8-element vectors per turn
    const int64_t want = (turns + qf::kThreads - 1) / qf::kThreads;
    const unsigned grid = static_cast<unsigned>(std::min<int64_t>(want, static_cast<int64_t>(sm_count()) * 32));
    char* gp = static_cast<char*>(g);
    if (dtype == QF_BF16)
        qf::grad_mean_peers_kernel<__nv_bfloat16><<<grid, qf::kThreads, 0, st>>>(gp, numel, pp, inv_count);
    else if (dtype == QF_F16)
        qf::grad_mean_peers_kernel<__half><<<grid, qf::kThreads, 0, st>>>(gp, numel, pp, inv_count);
    else
        qf::grad_mean_peers_kernel<float><<<grid, qf::kThreads, 0, st>>>(gp, numel, pp, inv_count);
    QF_CUDA(cudaGetLastError());
    return QF_OK;
}

int qf_read_status(void* workspace, int device, void* stream, uint32_t* status) {
    g_err[0] = 0;
    if (!workspace || !status) return fail(QF_ERR_BAD_ARG, "null workspace or status pointer");
    QF_CUDA(cudaSetDevice(device));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    QF_CUDA(cudaMemcpyAsync(status, workspace, sizeof(uint32_t), cudaMemcpyDeviceToHost, st));
    QF_CUDA(cudaMemsetAsync(workspace, 0, sizeof(uint32_t), st));
    QF_CUDA(cudaStreamSynchronize(st));
    return QF_OK;
}

int qf_release_workspace(void* workspace, int device) {
    g_err[0] = 0;
    if (!workspace) return QF_OK;
    QF_CUDA(cudaSetDevice(device));
    std::lock_guard<std::mutex> lock(g_mu);
    auto it = g_cache.find(cache_key(device, workspace));
    if (it == g_cache.end()) return QF_OK;
    drop_cache_entry(it->second, true);
    g_cache.erase(it);
    return QF_OK;
}

int qf_fused_4bit(void* p, const void* g, void* exp, void* sq, float* exp_scale, float* sq_scale, int64_t numel,
                  int dtype, double beta1, double beta2, double lr, double weight_decay, double eps, double step,
                  int device, void* stream) {
    g_err[0] = 0;
    if (!valid_dtype(dtype)) return fail(QF_ERR_BAD_ARG, "bad dtype %d", dtype);
    if (numel < 0) return fail(QF_ERR_BAD_ARG, "negative numel");
    if (numel == 0) return QF_OK;
    if (!p || !g || !exp || !sq || !exp_scale || !sq_scale) return fail(QF_ERR_BAD_ARG, "null pointer");
    if (!aligned(p, elem_size(dtype)) || !aligned(g, elem_size(dtype)) || !aligned(exp_scale, 4) || !aligned(sq_scale, 4))
        return fail(QF_ERR_BAD_ARG, "qf_fused_4bit: p / g not element-aligned or scales not 4-byte aligned");
    QF_CUDA(cudaSetDevice(device));
    qf::DevTensor t;
    memset(&t, 0, sizeof t);
    t.p = static_cast<char*>(p);
    t.g = static_cast<const char*>(g);
    t.m = static_cast<char*>(exp);
    t.v = static_cast<char*>(sq);
    t.ms = exp_scale;
    t.vs = sq_scale;
    t.numel = numel;
    t.kind = QF_KIND_BLOCK;
    t.dtype = dtype;
    if (aligned(p, 16) && aligned(g, 16) && aligned(exp, 4) && aligned(sq, 4)) t.flags |= qf::kFlagVec;
    QfHyper h;
    qf_make_hyper(lr, beta1, beta2, eps, weight_decay, step, &h);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    qf::single_tensor_kernel<<<flat_grid(numel), qf::kThreads, 0, st>>>(t, widen_hyper(h));
    QF_CUDA(cudaGetLastError());
    return QF_OK;
}

int qf_fused_single_tensor(void* p, const void* g, float* exp_avg, float* exp_avg_sq, int64_t numel, int dtype,
                           double beta1, double beta2, double lr, double weight_decay, double eps, double step,
                           int device, void* stream) {
    g_err[0] = 0;
    if (!valid_dtype(dtype)) return fail(QF_ERR_BAD_ARG, "bad dtype %d", dtype);
    if (numel < 0) return fail(QF_ERR_BAD_ARG, "negative numel");
    if (numel == 0) return QF_OK;
    if (!p || !g || !exp_avg || !exp_avg_sq) return fail(QF_ERR_BAD_ARG, "null pointer");
    if (!aligned(p, elem_size(dtype)) || !aligned(g, elem_size(dtype)) || !aligned(exp_avg, 4) || !aligned(exp_avg_sq, 4))
        return fail(QF_ERR_BAD_ARG, "qf_fused_single_tensor: p / g not element-aligned or moments not 4-byte aligned");
    QF_CUDA(cudaSetDevice(device));
    qf::DevTensor t;
    memset(&t, 0, sizeof t);
    t.p = static_cast<char*>(p);
    t.g = static_cast<const char*>(g);
    t.m = reinterpret_cast<char*>(exp_avg);
    t.v = reinterpret_cast<char*>(exp_avg_sq);
    t.numel = numel;
    t.kind = QF_KIND_FP32;
    t.dtype = dtype;
    if (aligned(p, 16) && aligned(g, 16) && aligned(exp_avg, 16) && aligned(exp_avg_sq, 16)) t.flags |= qf::kFlagVec;
    QfHyper h;
    qf_make_hyper(lr, beta1, beta2, eps, weight_decay, step, &h);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    qf::single_tensor_kernel<<<flat_grid(numel), qf::kThreads, 0, st>>>(t, widen_hyper(h));
    QF_CUDA(cudaGetLastError());
    return QF_OK;
}

int qf_quantize_block(const float* x, int64_t numel, int map, uint8_t* codes, float* scales, int device, void* stream) {
    g_err[0] = 0;
    if (int rc = check_1d(x, codes, numel, "qf_quantize_block")) return rc;
    if (map != 0 && map != 1) return fail(QF_ERR_BAD_ARG, "map must be 0 or 1");
    if (numel == 0) return QF_OK;
    if (!scales) return fail(QF_ERR_BAD_ARG, "scales is null");
    if (!aligned(x, 4) || !aligned(scales, 4)) return fail(QF_ERR_BAD_ARG, "qf_quantize_block: x / scales not 4-byte aligned");
    QF_CUDA(cudaSetDevice(device));
    const int vec = aligned(x, 16) && aligned(codes, 4);
    const unsigned grid = persistent_grid(flat_items(numel), 8, 2);
    if (map)
        qf::quantize_block_kernel<1><<<grid, qf::kThreads, 0, static_cast<cudaStream_t>(stream)>>>(x, numel, codes, scales, vec);
    else
        qf::quantize_block_kernel<0><<<grid, qf::kThreads, 0, static_cast<cudaStream_t>(stream)>>>(x, numel, codes, scales, vec);
    QF_CUDA(cudaGetLastError());
    return QF_OK;
}

int qf_dequantize_block(const uint8_t* codes, const float* scales, int64_t numel, int map, float* out, int device,
                        void* stream) {
    g_err[0] = 0;
    if (int rc = check_1d(codes, out, numel, "qf_dequantize_block")) return rc;
    if (map != 0 && map != 1) return fail(QF_ERR_BAD_ARG, "map must be 0 or 1");
    if (numel == 0) return QF_OK;
    if (!scales) return fail(QF_ERR_BAD_ARG, "scales is null");
    if (!aligned(out, 4) || !aligned(scales, 4)) return fail(QF_ERR_BAD_ARG, "qf_dequantize_block: out / scales not 4-byte aligned");
    QF_CUDA(cudaSetDevice(device));
    const int vec = aligned(out, 16) && aligned(codes, 4);
    qf::dequantize_block_kernel<<<flat_grid(numel), qf::kThreads, 0, static_cast<cudaStream_t>(stream)>>>(codes, scales, numel,
                                                                                                        map, out, vec);
    QF_CUDA(cudaGetLastError());
    return QF_OK;
}

int qf_quantize_rank1(const float* v, int64_t rows, int64_t cols, uint8_t* codes, float* row_max, float* col_max,
                      int device, void* stream) {
    g_err[0] = 0;
    if (rows < 0 || cols < 0 || rows > INT32_MAX || cols > INT32_MAX) return fail(QF_ERR_BAD_ARG, "bad shape");
    const int64_t numel = rows * cols;
    if (numel == 0) return QF_OK;
    if (!v || !codes || !row_max || !col_max) return fail(QF_ERR_BAD_ARG, "null pointer");
    if (!aligned(v, 4) || !aligned(row_max, 4) || !aligned(col_max, 4))
        return fail(QF_ERR_BAD_ARG, "qf_quantize_rank1: v / row_max / col_max not 4-byte aligned");
    QF_CUDA(cudaSetDevice(device));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    QF_CUDA(cudaMemsetAsync(row_max, 0, sizeof(float) * rows, st));
    QF_CUDA(cudaMemsetAsync(col_max, 0, sizeof(float) * cols, st));
    const int vec = aligned(v, 16) && aligned(codes, 4);
    const int panel = vec && cols % qf::kPanelCols == 0;
    const int64_t items = panel ? (rows + qf::kRowsPerItem - 1) / qf::kRowsPerItem * (cols / qf::kPanelCols) : flat_items(numel);
    const int64_t max_items = panel ? (rows + qf::kPreRowsPerItem - 1) / qf::kPreRowsPerItem * (cols / qf::kPanelCols) : items;
    unsigned grid;
    if (int rc = grid_for(max_items, &grid)) return rc;
    qf::rank1_max_kernel<<<grid, qf::kThreads, 0, st>>>(v, static_cast<int>(rows), static_cast<int>(cols), row_max, col_max, panel);
    if (panel && aligned(col_max, 16))
        qf::rank1_quant_panel_kernel<<<persistent_grid(items, 8), qf::kThreads, 0, st>>>(v, codes, row_max, col_max, static_cast<int>(rows),
                                                                                      static_cast<int>(cols));
    else
        qf::rank1_codec_kernel<true><<<flat_grid(numel), qf::kThreads, 0, st>>>(v, codes, row_max, col_max, static_cast<int>(rows),
                                                                               static_cast<int>(cols), nullptr, vec);
    QF_CUDA(cudaGetLastError());
    return QF_OK;
}

int qf_dequantize_rank1(const uint8_t* codes, const float* row_max, const float* col_max, int64_t rows, int64_t cols,
                        float* out, int device, void* stream) {
    g_err[0] = 0;
    if (rows < 0 || cols < 0 || rows > INT32_MAX || cols > INT32_MAX) return fail(QF_ERR_BAD_ARG, "bad shape");
    const int64_t numel = rows * cols;
    if (numel == 0) return QF_OK;
    if (!codes || !row_max || !col_max || !out) return fail(QF_ERR_BAD_ARG, "null pointer");
    if (!aligned(out, 4) || !aligned(row_max, 4) || !aligned(col_max, 4))
        return fail(QF_ERR_BAD_ARG, "qf_dequantize_rank1: out / row_max / col_max not 4-byte aligned");
    QF_CUDA(cudaSetDevice(device));
    const int vec = aligned(out, 16) && aligned(codes, 4);
    if (vec && cols % qf::kPanelCols == 0 && aligned(col_max, 16)) {
        const int64_t items = (rows + qf::kRowsPerItem - 1) / qf::kRowsPerItem * (cols / qf::kPanelCols);
        qf::rank1_dequant_panel_kernel<<<persistent_grid(items, 8), qf::kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
            codes, row_max, col_max, static_cast<int>(rows), static_cast<int>(cols), out);
    } else {
        qf::rank1_codec_kernel<false><<<flat_grid(numel), qf::kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
            nullptr, const_cast<uint8_t*>(codes), row_max, col_max, static_cast<int>(rows), static_cast<int>(cols), out, vec);
    }
    QF_CUDA(cudaGetLastError());
    return QF_OK;
}

// ---- the step of one rank-1 tensor for callers that cannot allocate ------------------------------------
//
// Scratch of this entry point: a status word, the one-entry descriptor table and the new row / column
// maxima with their reciprocals.  It lives in this translation unit as a device array; each GPU that loads
// the library keeps its own copy of it for the life of the process.
constexpr size_t kNoAllocHeader = 1024;  // status word, tensor record, four two-entry prefix tables
constexpr size_t kNoAllocBytes = kNoAllocHeader + 8 * static_cast<size_t>(QF_NOALLOC_MAX_ROWS_PLUS_COLS);
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_noalloc_mu;
unsigned char* g_noalloc_ptr[kMaxDevices] = {};  // device address of g_noalloc_scratch, per device

// g_noalloc_scratch names the array in device code only.  Host code needs the address the device knows it
// by, asked for once per device while that device is current.
int noalloc_scratch(int device, unsigned char** out) {
    if (device < 0 || device >= kMaxDevices) return fail(QF_ERR_BAD_ARG, "device ordinal %d out of range", device);
    std::lock_guard<std::mutex> lock(g_noalloc_mu);
    if (!g_noalloc_ptr[device]) {
        void* ptr = nullptr;
        QF_CUDA(cudaGetSymbolAddress(&ptr, g_noalloc_scratch));
        g_noalloc_ptr[device] = static_cast<unsigned char*>(ptr);
    }
    *out = g_noalloc_ptr[device];
    return QF_OK;
}
}  // namespace

int qf_step_rank1_noalloc(void* p, const void* g, void* m_codes, void* v_codes, float* m_scale, float* v_row,
                          float* v_col, int64_t rows, int64_t cols, int dtype, const QfHyper* hyper, int device,
                          void* stream) {
    g_err[0] = 0;
    if (!hyper) return fail(QF_ERR_BAD_ARG, "hyper is null");
    if (!valid_dtype(dtype)) return fail(QF_ERR_BAD_ARG, "bad dtype %d", dtype);
    if (rows <= 0 || cols <= 0) return fail(QF_ERR_BAD_ARG, "rows and cols must be positive");
    if (rows + cols > QF_NOALLOC_MAX_ROWS_PLUS_COLS)
        return fail(QF_ERR_BAD_ARG, "rows + cols = %lld exceeds the built-in scratch (QF_NOALLOC_MAX_ROWS_PLUS_COLS = %d); use qf_step_multi with caller-owned scratch",
                    (long long)(rows + cols), QF_NOALLOC_MAX_ROWS_PLUS_COLS);
    if (!p || !g || !m_codes || !v_codes || !m_scale || !v_row || !v_col) return fail(QF_ERR_BAD_ARG, "null pointer");
    const size_t esz = elem_size(dtype);
    if (!aligned(p, esz) || !aligned(g, esz) || !aligned(m_scale, 4) || !aligned(v_row, 4) || !aligned(v_col, 4))
        return fail(QF_ERR_BAD_ARG, "buffer not element-aligned");
    QF_CUDA(cudaSetDevice(device));
    unsigned char* scratch = nullptr;
    if (int rc = noalloc_scratch(device, &scratch)) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);

    // layout: [status | tensor record | 4 prefix tables][row maxima, reciprocals][column maxima, reciprocals]
    float* row_new = reinterpret_cast<float*>(scratch + kNoAllocHeader);
    float* col_new = row_new + 2 * ((rows + 3) / 4 * 4);  // keeps the column part 16-byte aligned
    if (reinterpret_cast<unsigned char*>(col_new + 2 * cols) > scratch + kNoAllocBytes)
        return fail(QF_ERR_BAD_ARG, "rows + cols too large for the built-in scratch after alignment padding");

    qf::DevTensor t;
    memset(&t, 0, sizeof t);
    t.p = static_cast<char*>(p);
    t.g = static_cast<const char*>(g);
    t.m = static_cast<char*>(m_codes);
    t.v = static_cast<char*>(v_codes);
    t.ms = m_scale;
    t.vs = v_row;
    t.vcol = v_col;
    t.vrow_new = row_new;
    t.vcol_new = col_new;
    t.vrow_rcp = row_new + rows;
    t.vcol_rcp = col_new + cols;
    t.numel = rows * cols;
    t.rows = static_cast<int32_t>(rows);
    t.cols = static_cast<int32_t>(cols);
    t.kind = QF_KIND_RANK1;
    t.dtype = dtype;
    const bool vec = aligned(p, 16) && aligned(g, 16) && aligned(m_codes, 4) && aligned(v_codes, 4);
    if (vec) t.flags |= qf::kFlagVec;
    int64_t items = flat_items(t.numel), pre_items = items;
    if (vec && dtype != QF_F16 && t.numel < (1ll << 31) && cols % qf::kPanelCols == 0 && aligned(v_col, 16)) {
        t.flags |= qf::kFlagPanel;
        t.panels = static_cast<int32_t>(cols / qf::kPanelCols);
        t.main_rows = main_rows_for((rows + qf::kMainRowsPerItem - 1) / qf::kMainRowsPerItem * t.panels);
        items = (rows + t.main_rows - 1) / t.main_rows * t.panels;
        pre_items = (rows + qf::kPreRowsPerItem - 1) / qf::kPreRowsPerItem * t.panels;
    }
    const bool panel = t.flags & qf::kFlagPanel;

    struct Header {
        uint32_t status[64];
        qf::DevTensor t;
        int64_t base[kTables][2];
    } h;
    static_assert(sizeof(Header) <= kNoAllocHeader, "header must fit");
    memset(&h, 0, sizeof h);
    h.t = t;
    h.base[kMainPanel][1] = panel ? items : 0;
    h.base[kMainFlat][1] = panel ? 0 : items;
    h.base[kPrePanel][1] = panel ? pre_items : 0;
    h.base[kPreFlat][1] = panel ? 0 : pre_items;
    // The header goes up from this stack frame; a copy from pageable memory returns once the source has
    // been staged (for which the runtime may make the host wait for earlier work of the stream), so the frame
    // may die afterwards.  The status words ahead of the tensor record are not part of the copy: they
    // accumulate until qf_read_status_noalloc reads and clears them.
    QF_CUDA(cudaMemcpyAsync(scratch + offsetof(Header, t), reinterpret_cast<const char*>(&h) + offsetof(Header, t),
                            sizeof h - offsetof(Header, t), cudaMemcpyHostToDevice, st));

    Plan pl;
    pl.n = 1;
    pl.n_rank1 = 1;
    pl.any_f32_panel = panel && dtype == QF_F32;
    pl.any_bf16_panel = panel && dtype == QF_BF16;
    pl.d_status = reinterpret_cast<uint32_t*>(scratch);
    pl.d_tensors = reinterpret_cast<qf::DevTensor*>(scratch + offsetof(Header, t));
    for (int k = 0; k < kTables; ++k) {
        pl.items[k] = h.base[k][1];
        pl.d_base[k] = reinterpret_cast<int64_t*>(scratch + offsetof(Header, base)) + 2 * k;
    }
    qf::HyperPack hp;
    memset(&hp, 0, sizeof hp);
    hp.h[0] = widen_hyper(*hyper);
    if (int rc = launch_pre(pl, hp, 1, st)) return rc;   // clears the new maxima first: the array keeps the last call's
    return launch_main(pl, hp, 1, st);
}

int qf_read_status_noalloc(int device, void* stream, uint32_t* status) {
    g_err[0] = 0;
    if (!status) return fail(QF_ERR_BAD_ARG, "status is null");
    QF_CUDA(cudaSetDevice(device));
    unsigned char* scratch = nullptr;
    if (int rc = noalloc_scratch(device, &scratch)) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    QF_CUDA(cudaMemcpyAsync(status, scratch, sizeof(uint32_t), cudaMemcpyDeviceToHost, st));
    QF_CUDA(cudaMemsetAsync(scratch, 0, sizeof(uint32_t), st));
    QF_CUDA(cudaStreamSynchronize(st));
    return QF_OK;
}

}  // extern "C"
