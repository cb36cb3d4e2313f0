/*
 * quantfour_b200.h -- C ABI of libquantfour_b200.so: the fused 4-bit AdamW optimizer step for
 * NVIDIA B200 (sm_100a).
 *
 * This library stands where the reference project's pybind11 extension `quantfour_cuda` stands
 * (optim/cuda_fused_interface.cc:1-69, kernels in optim/cuda_adamw_kernels.cu).  It has no torch
 * or ATen type in any signature: device pointers, sizes, a device ordinal and a CUDA stream handle.
 * Every function returns a QfStatus; on failure qf_last_error() gives a message for the calling
 * thread.  All launches are asynchronous on the stream that is passed in; nothing synchronises the
 * device except qf_read_status(), qf_read_status_noalloc() and qf_release_workspace().  (A step call
 * uploads its descriptor table through one of two pinned host buffers kept per workspace; the host
 * waits only if the upload of the call before the previous one on that workspace is still in flight.)
 * The library allocates no device memory: the caller owns every buffer, the workspace included.
 *
 * Data layout (all buffers contiguous, in device memory):
 *   parameters / gradients ... fp32 or bf16, `numel` elements, 16-byte aligned
 *   4-bit codes .............. one byte per two elements, element 2j in bits 0-3 and element 2j+1
 *                              in bits 4-7 of byte j; ceil(numel/2) bytes, 4-byte aligned
 *   first-moment scales ...... fp32, one per 128 consecutive (flattened) elements
 *   second-moment scales ..... QF_KIND_BLOCK: fp32, one per 128 elements;
 *                              QF_KIND_RANK1: fp32 row maxima [rows] and column maxima [cols];
 *                              the scale of element (i, j) is min(row[i], col[j])
 *   QF_KIND_FP32 ............. both moments are plain fp32 arrays of `numel` elements
 */
#ifndef QUANTFOUR_B200_H
#define QUANTFOUR_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define QF_ABI_VERSION 5
#define QF_BLOCK 128        /* elements per quantization block (optim/cuda_adamw_kernels.cu:431) */
#define QF_MAX_HYPERS 16    /* hyper-parameter sets one launch can carry */
#define QF_MAX_PEERS 15     /* peer copies of the parameter buffer one launch can feed */
#define QF_PEER_HANDLE_BYTES 64

typedef enum QfStatus {
    QF_OK = 0,
    QF_ERR_BAD_ARG = 1,      /* null pointer, misaligned buffer, negative size, bad enum ... */
    QF_ERR_WORKSPACE = 2,    /* workspace missing or smaller than qf_workspace_bytes()      */
    QF_ERR_CUDA = 3,         /* a CUDA runtime call or a launch failed                      */
    QF_ERR_NO_DEVICE = 4     /* no usable CUDA device / driver                              */
} QfStatus;

/* QF_F16: IEEE half parameters and gradients (the reference's launcher dispatches half, optim/cuda_adamw_kernels.cu:443,
 * though its kernel only handles float): widened exactly, the step runs in fp32, the new parameter is rounded to nearest
 * even.  Tensors of this dtype take the flat mapping whatever their kind (correct, not tuned). */
typedef enum QfDtype { QF_F32 = 0, QF_BF16 = 1, QF_F16 = 2 } QfDtype;

typedef enum QfKind {
    QF_KIND_FP32 = 0,   /* moments kept in fp32 (tensors at or below the size threshold;
                           the reference's kernel_cuda_single_tensor, cuda_adamw_kernels.cu:100-133) */
    QF_KIND_BLOCK = 1,  /* both moments 4-bit with block-128 scales                               */
    QF_KIND_RANK1 = 2   /* first moment block-128, second moment rank-1 (2-D tensors)             */
} QfKind;

/* Bits of the device status word (see qf_read_status). */
#define QF_STATUS_NONFINITE 1u   /* a non-finite scale was produced (non-finite gradient or overflow) */
#define QF_STATUS_SCHEDULE_END 2u /* qf_step_scheduled ran past the last row of a schedule whose last row does not repeat */

/*
 * Scalars of one optimizer step, derived by the host in double precision and rounded once to fp32
 * (the reference derives them in fp32 inside its launcher, cuda_adamw_kernels.cu:435-440; its
 * PyTorch path uses Python doubles, adamw_fourbit_triton.py:458-465 -- the latter is followed).
 */
typedef struct QfHyper {
    float decay;     /* 1 - lr * weight_decay          */
    float w1;        /* 1 - beta1                      */
    float beta2;     /* beta2                          */
    float w2;        /* 1 - beta2                      */
    float eps;       /* eps                            */
    float neg_step;  /* -(lr / (1 - beta1^step))       */
    float bc2s;      /* sqrt(1 - beta2^step)           */
    float grad_scale; /* 0 or 1: gradients are used as they are.  Otherwise every gradient of the tensors that use
                         this set is replaced in place by RN(g * grad_scale), in g's own dtype, before the step uses
                         it (loss-scale removal or a clipping factor without a pass of its own).  No counterpart
                         in the reference.  With the split entry points, pass the same value to both halves.  */
} QfHyper;

/* One tensor of a multi-tensor step.  Replaces the per-tensor argument list of the reference's
 * fused_4bit(p, g, exp, sq, exp_scale, sq_scale, ...) (cuda_fused_interface.cc:19-25). */
typedef struct QfTensorDesc {
    void* p;              /* parameters, updated in place                                        */
    const void* g;        /* gradients, same dtype as p                                          */
    void* m;              /* first moment: codes (uint8) or, for QF_KIND_FP32, fp32 values       */
    void* v;              /* second moment: codes (uint8) or fp32 values                         */
    float* m_scale;       /* [ceil(numel/128)]; unused for QF_KIND_FP32                          */
    float* v_scale;       /* BLOCK: [ceil(numel/128)]; RANK1: row maxima [rows]; in/out          */
    float* v_col;         /* RANK1: column maxima [cols]; in/out                                 */
    float* v_row_new;     /* RANK1: scratch for the new row maxima: [2*rows] if v_row_rcp is null
                             (maxima, then their reciprocals), else [rows]                         */
    float* v_col_new;     /* RANK1: the same for the columns: [2*cols], or [cols] with v_col_rcp  */
    float* v_row_rcp;     /* RANK1, optional: separate scratch [rows] for the reciprocals          */
    float* v_col_rcp;     /* RANK1, optional: separate scratch [cols] for the reciprocals          */
    int64_t numel;        /* elements this record covers                                         */
    int64_t rows;         /* RANK1 only; rows * cols == numel unless the record is partial       */
    int64_t cols;
    int64_t flat_offset;  /* RANK1, partial records: elements of the rows x cols matrix that precede
                             the first element of this record; the row/column buffers then describe
                             the whole matrix while p, g, m, v, m_scale start at this record      */
    int32_t kind;         /* QfKind                                                              */
    int32_t dtype;        /* QfDtype of p and g                                                  */
    int32_t hyper;        /* index into the hyper-parameter array of the call                    */
    int32_t partial;      /* RANK1: non-zero if the record covers only part of the matrix (a shard);
                             flat_offset and numel must be multiples of 128 except at the matrix end */
} QfTensorDesc;

int qf_abi_version(void);

/* Message of the last failure on the calling thread ("" if none). */
const char* qf_last_error(void);

/* Bytes of device workspace a step over n_tensors tensors needs.  The workspace holds the device
 * copy of the descriptor table (rewritten by every call, on the call's stream) and the status word,
 * which accumulates between calls until qf_read_status clears it: hand in zero-filled memory. */
size_t qf_workspace_bytes(int n_tensors);

/*
 * One optimizer step over a ragged list of tensors: dequantize both moments, AdamW update with
 * decoupled weight decay, new scales, requantize, pack.  Replaces one call of the reference's
 * fused_4bit / fused_single_tensor per tensor (cuda_fused_interface.cc:19-64,
 * cuda_adamw_kernels.cu:136-164, :422-469; driver loop optim/fused_quantfour.py:171-292).
 *
 * `descs` and `hypers` are host arrays.  For RANK1 tensors the call (1) clears v_row_new/v_col_new,
 * (2) accumulates the new maxima, (3) stores their reciprocals in the second halves of the scratch
 * arrays, updates and requantizes using the old maxima for dequantize and the new ones for quantize,
 * (4) copies the new maxima into v_scale/v_col.
 */
int qf_step_multi(const QfTensorDesc* descs, int n_tensors, const QfHyper* hypers, int n_hypers,
                  void* workspace, size_t workspace_bytes, int device, void* stream);

/* The two halves of qf_step_multi, for callers that must combine the new column maxima of a tensor
 * split by rows across devices (element-wise max of v_col_new over the devices that share it)
 * between them.  qf_step_pre does (1)-(2), qf_step_main does (3)-(4). No counterpart in the
 * reference, which has no sharding. */
int qf_step_pre(const QfTensorDesc* descs, int n_tensors, const QfHyper* hypers, int n_hypers,
                void* workspace, size_t workspace_bytes, int device, void* stream);
int qf_step_main(const QfTensorDesc* descs, int n_tensors, const QfHyper* hypers, int n_hypers,
                 void* workspace, size_t workspace_bytes, int device, void* stream);

/*
 * The general form of the step calls above; they are shorthands for it.  `what` is a sum of:
 *   QF_RUN_PRE, QF_RUN_MAIN   which halves run (both = qf_step_multi);
 *   QF_RUN_TABLE_IN_PLACE     the workspace already holds the tensor table of exactly these `descs` (and n_hypers), written
 *                             by qf_step_prepare or by an earlier step call on this stream, and nothing has touched the
 *                             workspace since: the call then copies nothing from the host.  Every step call otherwise
 *                             begins with a copy of a few tens of kilobytes on `stream`; behind long host-to-device
 *                             copies already queued on other streams that copy, and the kernels after it, wait for them
 *                             (measured: a step meant to overlap the arrival of the next gradients did not start
 *                             until the last gradient had arrived);
 *   QF_RUN_RELAXED_UPDATE     bf16 tensors on the rank-1 panel mapping (whole 2-D tensors whose column count is a multiple
 *                             of 256) take a cheaper parameter update: the square root and the two divisions of
 *                             optim/adamw_fourbit_triton.py:467-473 as v * rsqrt(v) and multiplications by approximate
 *                             reciprocals, without corrections.  The update then carries a relative error of about 2^-21;
 *                             a new bf16 parameter differs from the exact one, by one bf16 unit, where the exact sum lies
 *                             that close to a rounding boundary (measured: 5 in 10^7 elements per step), and the
 *                             difference stays.  The moments do not depend on the parameter: every code and scale stays
 *                             bit-identical.  Measured gain: 4 % of a step.  Not with peer stores.
 * peer_delta_bytes / n_peers: as for qf_step_main_push (0 peers: none).  No counterpart in the reference.
 */
#define QF_RUN_PRE 1
#define QF_RUN_MAIN 2
#define QF_RUN_TABLE_IN_PLACE 4
#define QF_RUN_RELAXED_UPDATE 8
int qf_step_run(const QfTensorDesc* descs, int n_tensors, const QfHyper* hypers, int n_hypers, void* workspace,
                size_t workspace_bytes, int device, void* stream, int what, const int64_t* peer_delta_bytes,
                int n_peers);

/*
 * The step for CUDA graphs: nothing but kernel launches on `stream`, all per-step scalars resident on the device.
 * (Asked for as a "capturable" step: the reference reads the step count back to the host every step,
 * optim/adamw_fourbit_triton.py:458, and derives the bias corrections there; it has no counterpart of this.)
 *
 * qf_step_prepare writes the tensor table of `descs` into the workspace (a copy from the host: call it before the
 * capture begins, and again whenever a descriptor changes).  qf_step_scheduled is qf_step_multi for a workspace so
 * prepared, with the hyper-parameter sets read from device memory instead of the argument list:
 *   device_schedule   schedule_rows x n_hypers QfHyper records, row-major; row r holds the sets of the r-th step after
 *                     the table was written, each made by qf_make_hyper (doubles on the host: the kernels see the same
 *                     float32 scalars as through qf_step_multi, so results are bit-identical);
 *   device_counters   two int32: [0] the row the next step takes (the caller zeroes it when it writes the table),
 *                     [1] the number of steps done; the call's last kernel advances both.
 * A step past the last row takes the last row again; that is exact when the last row is stationary (constant
 * learning rate and both bias corrections rounded to 1, i.e. after a few thousand steps at beta2 = 0.999) and is then
 * announced with QF_SCHED_TAIL_REPEATS; without that flag such a step sets QF_STATUS_SCHEDULE_END in the status word.
 * QF_SCHED_GRAD_SCALE: some row carries a grad_scale other than 0 / 1 (selects the kernel variant that rewrites
 * the gradients).  The call itself may be captured into a graph: it enqueues kernels only, never copies, waits or
 * allocates; replaying the graph repeats the step with the next row.
 */
#define QF_SCHED_TAIL_REPEATS 1
#define QF_SCHED_GRAD_SCALE 2
int qf_step_prepare(const QfTensorDesc* descs, int n_tensors, int n_hypers, void* workspace, size_t workspace_bytes,
                    int device, void* stream);
int qf_step_scheduled(const QfTensorDesc* descs, int n_tensors, int n_hypers, void* workspace,
                      size_t workspace_bytes, int device, void* stream, const QfHyper* device_schedule,
                      int schedule_rows, int32_t* device_counters, int flags);

/*
 * qf_step_main that also stores every updated parameter into the same place of up to QF_MAX_PEERS
 * other devices' copies of the parameter buffer, from inside the update kernel: the all-gather of a
 * sharded step rides the peer links while the update computes instead of following it.
 * peer_delta_bytes[k] = (address at which peer k's buffer is mapped in this process) - (address of this
 * device's buffer); every desc's p must lie in this device's buffer, and the peers' buffers must have the
 * same layout.  The caller orders the launch after every peer's last read of its old parameters and
 * lets no peer read the new ones before every device's launch has completed (one small collective on
 * either side does both).  No counterpart in the reference, which has no sharding.
 */
int qf_step_main_push(const QfTensorDesc* descs, int n_tensors, const QfHyper* hypers, int n_hypers,
                      void* workspace, size_t workspace_bytes, int device, void* stream,
                      const int64_t* peer_delta_bytes, int n_peers);

/*
 * Sharing a device buffer between the processes of one node (one process per device), for
 * qf_step_main_push.  qf_peer_export writes an opaque handle of the allocation that holds `ptr` and the
 * offset of `ptr` inside it; the bytes travel to the other process by any host channel; there
 * qf_peer_open maps the allocation (enabling peer access) and returns its base, so the buffer is at
 * base + offset; qf_peer_close unmaps it.  Opening a handle that is already open in the process returns the
 * same mapping and counts it; the last qf_peer_close unmaps.  `ptr` must come from cudaMalloc (not from a
 * virtual-memory pool).  No counterpart in the reference.
 */
int qf_peer_export(const void* ptr, int device, unsigned char handle[QF_PEER_HANDLE_BYTES], int64_t* offset_bytes);
int qf_peer_open(const unsigned char handle[QF_PEER_HANDLE_BYTES], int device, void** base);
int qf_peer_close(void* base, int device);

/*
 * Copy `bytes` bytes from this device's memory to a buffer mapped with qf_peer_open, asynchronously on `stream`,
 * through the copy engines.  `dst_device` is the ordinal, in this process, of the device that holds `dst` (a negative
 * value lets the runtime work it out).  The other way to deliver a sharded step's new parameters: the rank updates
 * its range in pieces with qf_step_main and copies each finished piece to every peer on side streams while the next
 * piece computes.  Measured on 4 and 8 B200s (7B shape): with every GPU copying to all others at once, peers taken in
 * rotated order (rank+1, rank+2, ...), the copy engines move 770-800 GB/s per GPU, stores issued by a kernel
 * (qf_step_main_push) about 690; but in the pipelined step the engines serve the per-peer streams one after another
 * in an order the caller does not control, the ranks drift apart, several senders meet at one receiver, and the step
 * took 22-23 ms against 15.8 ms with qf_step_main_push, whose every warp spreads its stores evenly over all peers.
 * No counterpart in the reference.
 */
int qf_peer_copy(void* dst, int dst_device, const void* src, size_t bytes, int device, void* stream);

/*
 * The gradient half of a sharded step without a library collective: the device that owns a range of the flat gradient
 * buffer takes the mean of all devices' copies of that range through peer loads and writes it over its own copy:
 *     g[i] := RN((copy_0[i] + copy_1[i] + ... ) * inv_count)      sum in fp32, in the order given, rounded to `dtype`
 * copy_delta_bytes[k] = (address of copy k's range as mapped in this process, qf_peer_open) - g; 0 names this device's
 * own copy, which must be among them; at most QF_MAX_PEERS copies.  Only g[0 .. numel) is written, and nothing else
 * of any copy is read, so all devices can run their call at the same time as long as their ranges are disjoint.  The
 * caller makes sure that every device's gradients are complete before any call starts (one small collective) and that
 * no device overwrites its gradients before all calls have finished (any later collective of the step).  Measured on
 * two B200s, 13 G bf16 gradients: 21.0 ms (620 GB/s of peer loads per device) against 26.4 ms for NCCL's reduce-scatter
 * of the same bytes.  No counterpart in the reference (it has no sharding).
 */
int qf_grad_mean_peers(void* g, int64_t numel, int dtype, const int64_t* copy_delta_bytes, int n_copies,
                       float inv_count, int device, void* stream);

/* Synchronise `stream`, read the status word kept in `workspace` into *status (QF_STATUS_* bits)
 * and clear it. */
int qf_read_status(void* workspace, int device, void* stream, uint32_t* status);

/* Forget what the library keeps on the host for `workspace` (two pinned staging buffers and two events,
 * created by the first step call that saw this address): call it before the workspace memory is freed
 * for good.  Waits for uploads from those buffers that are still in flight.  A host that never calls it
 * loses nothing but host memory: beyond 64 workspaces the library drops idle entries by itself.  No
 * counterpart in the reference, whose extension keeps no state. */
int qf_release_workspace(void* workspace, int device);

/*
 * Single-tensor entry points with the reference's argument order
 * (fused_4bit: cuda_fused_interface.cc:19-25; fused_single_tensor: :49-60).  Scalars are doubles;
 * `step` is the step count after the increment.  In qf_fused_4bit both moments use block-128
 * scales (exp_scale, sq_scale: [ceil(numel/128)]), which is what the reference's signature can
 * express; rank-1 second moments go through qf_step_multi.  These two calls have no workspace and
 * therefore no status word: a non-finite gradient is not reported (it still propagates into the scales
 * and the parameters as the arithmetic dictates).  Callers that want the report use qf_step_multi.
 */
int qf_fused_4bit(void* p, const void* g, void* exp, void* sq, float* exp_scale, float* sq_scale,
                  int64_t numel, int dtype, double beta1, double beta2, double lr, double weight_decay,
                  double eps, double step, int device, void* stream);
int qf_fused_single_tensor(void* p, const void* g, float* exp_avg, float* exp_avg_sq, int64_t numel,
                           int dtype, double beta1, double beta2, double lr, double weight_decay,
                           double eps, double step, int device, void* stream);

/* Derive the scalars of a step the way the PyTorch path of the reference does
 * (adamw_fourbit_triton.py:415, :458-465). */
void qf_make_hyper(double lr, double beta1, double beta2, double eps, double weight_decay, double step,
                   QfHyper* out);

/*
 * Stand-alone quantize / dequantize (the pieces of the step; the reference describes them at
 * adamw_fourbit_triton.py:556-630, :801-863 and :497-546 but ships no kernel for them).
 * `map`: 0 = first-moment map (signed, dynamic exponent), 1 = second-moment map (unsigned,
 * linear, zero excluded).  Inputs / outputs are fp32.
 */
int qf_quantize_block(const float* x, int64_t numel, int map, uint8_t* codes, float* scales,
                      int device, void* stream);
int qf_dequantize_block(const uint8_t* codes, const float* scales, int64_t numel, int map, float* out,
                        int device, void* stream);
int qf_quantize_rank1(const float* v, int64_t rows, int64_t cols, uint8_t* codes, float* row_max,
                      float* col_max, int device, void* stream);
int qf_dequantize_rank1(const uint8_t* codes, const float* row_max, const float* col_max, int64_t rows,
                        int64_t cols, float* out, int device, void* stream);

/*
 * One optimizer step on one rank-1 (2-D) tensor without any caller-provided scratch and without any
 * allocation.  No counterpart in the reference.
 *
 * Who this is for: hosts that must not allocate while they step.  A training runtime that has handed all
 * device memory to its own pool cannot give this library a workspace it did not plan for, and a raw
 * allocation at that point would either fail or stall the device (device allocations synchronise);
 * plug-in hosts that only pass tensors through and own no allocator are in the same position.  For them
 * the scratch qf_step_multi asks for (descriptor table, status word, new row / column maxima and their
 * reciprocals) lives inside the library, in a device array of QF_NOALLOC_MAX_ROWS_PLUS_COLS * 8 + 1024
 * bytes (about 1 MiB) that every GPU which loads the library holds until the process ends.
 *
 * Limits and rules:
 *   - rows + cols <= QF_NOALLOC_MAX_ROWS_PLUS_COLS (a little less when rows is not a multiple of 4);
 *     larger tensors are refused with QF_ERR_BAD_ARG and a message, nothing is launched;
 *   - the first call on a device looks up the device address of the built-in array; make that first
 *     call before any stream capture begins;
 *   - all calls on a device share the one array.  Each call clears what it needs at zero (the status
 *     word excepted, which accumulates until qf_read_status_noalloc), so leftovers from the previous
 *     call do no harm, but two calls whose kernels overlap on the GPU (different
 *     streams, or different threads) race on it: keep calls on one device in one stream order;
 *   - the function calls no cudaMalloc / cudaFree / cudaMallocHost and nothing that does.  Its small
 *     descriptor goes up with cudaMemcpyAsync from pageable host memory, for which the CUDA runtime may
 *     make the calling thread wait until the stream has reached the copy;
 * Same arithmetic, same kernels and same in/out buffers as a QF_KIND_RANK1 tensor in qf_step_multi:
 * v_row [rows] and v_col [cols] hold the old maxima on entry and the new ones on return.
 */
#define QF_NOALLOC_MAX_ROWS_PLUS_COLS 131072
int qf_step_rank1_noalloc(void* p, const void* g, void* m_codes, void* v_codes, float* m_scale,
                          float* v_row, float* v_col, int64_t rows, int64_t cols, int dtype,
                          const QfHyper* hyper, int device, void* stream);

/* The status word of qf_step_rank1_noalloc on `device` (QF_STATUS_* bits accumulated over its calls since
 * the last read): synchronises `stream`, copies the word to *status and clears it.  Allocates nothing
 * either.  No counterpart in the reference. */
int qf_read_status_noalloc(int device, void* stream, uint32_t* status);

#ifdef __cplusplus
}
#endif
#endif /* QUANTFOUR_B200_H */
