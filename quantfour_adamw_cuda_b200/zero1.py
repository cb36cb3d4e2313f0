"""ShardedFourBitAdamW: the 4-bit AdamW step with the optimizer state sharded over data-parallel ranks.

The reference has no sharding or collectives (its only distributed call is an unused seed broadcast,
optim/adamw_fourbit_triton.py:163-165); this module adds the one place where the path shards naturally.

Layout.  All parameters (in optimizer order) are laid out in one flat buffer; every tensor starts at a
multiple of 128 elements so that its 128-element quantization blocks coincide with blocks of the flat
space.  The flat space is cut into `world` equal ranges of `shard` elements (a multiple of 128).  Rank r
owns the optimizer state of range r and updates the parameters in it; parameters and gradients stay
replicated.  After the step each rank's range is all-gathered in place into every rank's flat buffer
(`comm="nccl"`), or -- when the ranks are processes of one node whose devices reach one another's memory -- the
new parameters cross NVLink while the update still computes and no all-gather follows: the update kernel itself
stores each new parameter vector into every peer's flat buffer (`comm="p2p"`, qf_step_main_push; what `comm="auto"`
picks if the set-up succeeds on every rank), or the rank updates its range in pieces and the copy engines carry each
finished piece to every peer on side streams (`comm="ce"`: the copy engines alone move 10 % more bytes per second than
stores issued by a kernel, but the engines serve the per-peer streams in an order of their own, the ranks drift
apart and several senders meet at one receiver, so this form measured slower -- 22-23 against 15.8 ms per step on
4 GPUs, 7B shape -- and is kept as an option only).

A 2-D tensor cut by a range boundary keeps its rank-1 second-moment scales identical to the unsharded
optimizer: the new row / column maxima of such a tensor are combined with an element-wise max over the
ranks (one small all-reduce between the two halves of the step, qf_step_pre and qf_step_main).  Inside
one rank a cut tensor becomes up to three records: a partial first row, whole rows (fast panel mapping),
a partial last row.

The arithmetic runs in a backend: `CudaBackend` (the C ABI) is the only one shipped; it refuses CPU
tensors.  Tests inject a CPU backend to exercise partitioning, exchange and collectives with gloo.
"""
from __future__ import annotations

import ctypes as C
import math
import socket
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from . import _lib
from .optimizer import BLOCK, DEFAULT_THRESHOLD, make_hyper

__all__ = ["ShardedFourBitAdamW", "FlatLayout", "flat_layout", "rank_records", "Record", "CudaBackend",
           "assemble_full_state"]

FP32, BLOCKQ, RANK1 = _lib.QF_KIND_FP32, _lib.QF_KIND_BLOCK, _lib.QF_KIND_RANK1


def _round_up(x: int, a: int) -> int:
    return (x + a - 1) // a * a


@dataclass
class FlatLayout:
    shapes: List[Tuple[int, ...]]
    numels: List[int]
    offsets: List[int]   # start of each tensor in the flat space (multiples of 128)
    world: int
    shard: int           # elements per rank (multiple of 128)

    @property
    def total(self) -> int:
        return self.world * self.shard

    def range_of(self, rank: int) -> Tuple[int, int]:
        return rank * self.shard, (rank + 1) * self.shard

    def owners(self, t: int) -> List[int]:
        """Ranks whose range intersects tensor t."""
        lo, hi = self.offsets[t], self.offsets[t] + self.numels[t]
        return [r for r in range(self.world) if r * self.shard < hi and (r + 1) * self.shard > lo]


def flat_layout(shapes: Sequence[Sequence[int]], world: int) -> FlatLayout:
    shapes = [tuple(int(d) for d in s) for s in shapes]
    numels = [math.prod(s) if s else 1 for s in shapes]
    offsets, pos = [], 0
    for n in numels:
        offsets.append(pos)
        pos = _round_up(pos + n, BLOCK)
    shard = _round_up(-(-max(pos, 1) // world), BLOCK)
    return FlatLayout(shapes, numels, offsets, world, shard)


@dataclass
class Record:
    """One unit of work of a rank: a contiguous piece [a, b) of tensor `tensor` (tensor-relative elements)."""
    tensor: int
    kind: int
    a: int
    b: int
    rows: int = 0          # RANK1: rows / cols of what the row / column buffers of this record describe
    cols: int = 0
    row_lo: int = 0        # RANK1 whole-row records: first row of the piece inside the tensor
    flat_offset: int = 0   # RANK1 partial records: elements of the matrix before the piece
    partial: bool = False

    @property
    def numel(self) -> int:
        return self.b - self.a


def tensor_kind(shape: Tuple[int, ...], numel: int, threshold: int) -> int:
    if threshold and numel <= threshold:
        return FP32
    return RANK1 if len(shape) == 2 else BLOCKQ


def rank_records(layout: FlatLayout, rank: int, threshold: int = DEFAULT_THRESHOLD) -> List[Record]:
    lo, hi = layout.range_of(rank)
    out: List[Record] = []
    for t, (shape, n, off) in enumerate(zip(layout.shapes, layout.numels, layout.offsets)):
        a, b = max(lo, off) - off, min(hi, off + n) - off
        if a >= b:
            continue
        kind = tensor_kind(shape, n, threshold)
        if kind != RANK1:
            out.append(Record(t, kind, a, b))
            continue
        R, Cc = shape
        if a == 0 and b == n:
            out.append(Record(t, RANK1, 0, n, rows=R, cols=Cc))
            continue
        r_lo, r_hi = -(-a // Cc), b // Cc       # whole rows inside [a, b)
        if Cc % BLOCK or r_lo >= r_hi:
            # blocks straddle rows, or less than one whole row: one partial record
            out.append(Record(t, RANK1, a, b, rows=R, cols=Cc, flat_offset=a, partial=True))
            continue
        if a < r_lo * Cc:
            out.append(Record(t, RANK1, a, r_lo * Cc, rows=R, cols=Cc, flat_offset=a, partial=True))
        out.append(Record(t, RANK1, r_lo * Cc, r_hi * Cc, rows=r_hi - r_lo, cols=Cc, row_lo=r_lo))
        if r_hi * Cc < b:
            out.append(Record(t, RANK1, r_hi * Cc, b, rows=R, cols=Cc, flat_offset=r_hi * Cc, partial=True))
    return out


@dataclass
class RecordState:
    """Tensors of one record on its owner rank (views where they alias per-tensor buffers)."""
    rec: Record
    p: torch.Tensor                         # flat view of the parameters of the piece
    m: torch.Tensor                         # int8 codes or fp32 values
    v: torch.Tensor
    m_scale: Optional[torch.Tensor] = None
    v_scale: Optional[torch.Tensor] = None  # BLOCK: block scales; RANK1: old row maxima as this record sees them
    v_col: Optional[torch.Tensor] = None
    row_new: Optional[torch.Tensor] = None
    col_new: Optional[torch.Tensor] = None
    row_rcp: Optional[torch.Tensor] = None
    col_rcp: Optional[torch.Tensor] = None
    g: Optional[torch.Tensor] = None        # set per step: flat view of the gradient of the piece


def assemble_full_state(pieces: Sequence[Dict[str, Any]], shapes: Sequence[Tuple[int, ...]], step: int,
                        group: Dict[str, Any], threshold: int = DEFAULT_THRESHOLD) -> Dict[str, Any]:
    """Join the pieces of all ranks (ShardedFourBitAdamW.pieces) into a state dict with FourBitAdamW's layout
    (state keys step / exp_avg / exp_avg_sq / momentum_qstate / variance_qstate, fused_quantfour.py:61-70,
    :110-128): pieces start on 128-element boundaries, so codes join on byte boundaries and scales on blocks."""
    state: Dict[int, Dict[str, Any]] = {}
    for t, shape in enumerate(shapes):
        n = math.prod(shape) if shape else 1
        kind = tensor_kind(tuple(shape), n, threshold)
        q = kind != FP32
        f: Dict[str, Any] = {"step": torch.tensor(float(step)),
                             "momentum_qstate": {"enable": q, "overhead": {}, "qmap": None},
                             "variance_qstate": {"enable": q, "overhead": {}, "qmap": None}}
        mine = [e for e in pieces if e["tensor"] == t]
        covered = sorted((e["a"], e["b"]) for e in mine)
        if not covered or covered[0][0] != 0 or covered[-1][1] != n or any(x[1] != y[0] for x, y in zip(covered, covered[1:])):
            raise ValueError(f"the pieces of tensor {t} do not tile it: {covered}")
        if kind == FP32:
            m, v = torch.zeros(n), torch.zeros(n)
            for e in mine:
                m[e["a"]:e["b"]] = e["m"]
                v[e["a"]:e["b"]] = e["v"]
            f["exp_avg"], f["exp_avg_sq"] = m.view(shape), v.view(shape)
            state[t] = f
            continue
        nb, nblk = (n + 1) // 2, (n + BLOCK - 1) // BLOCK
        m, v = torch.zeros(nb, dtype=torch.int8), torch.zeros(nb, dtype=torch.int8)
        ms = torch.zeros(nblk)
        vs = torch.zeros(nblk) if kind == BLOCKQ else None
        rows = cols = None
        if kind == RANK1:
            rows, cols = torch.zeros(shape[0], 1), torch.zeros(1, shape[1])
        for e in mine:
            b0, b1, k0, k1 = e["a"] // 2, (e["b"] + 1) // 2, e["a"] // BLOCK, (e["b"] + BLOCK - 1) // BLOCK
            m[b0:b1], v[b0:b1], ms[k0:k1] = e["m"], e["v"], e["m_scale"]
            if kind == BLOCKQ:
                vs[k0:k1] = e["v_scale"]
            else:
                lo, hi, vals = e["rows"]
                rows[lo:hi, 0] = vals
                cols[0] = e["cols"]
        f["exp_avg"], f["exp_avg_sq"] = m, v
        f["momentum_qstate"]["overhead"]["max1"] = ms
        vo = f["variance_qstate"]["overhead"]
        vo["dim"] = len(shape)
        if kind == RANK1:
            vo["max_dims"], vo["max1"] = [rows, cols], None
        else:
            vo["max1"] = vs
        state[t] = f
    pg = {k: v for k, v in group.items() if k != "params"}
    pg["params"] = list(range(len(shapes)))
    return {"state": state, "param_groups": [pg]}


class CudaBackend:
    """Runs the two halves of the step through libquantfour_b200.so."""

    def __init__(self) -> None:
        self.L = _lib.lib()
        self.sig = None
        self.descs = None
        self.ws: Optional[torch.Tensor] = None
        self.generation = 0                      # counts the descriptor arrays built so far
        self.uploaded: Optional[tuple] = None    # (generation, stream) of the table that is in the workspace

    def _prepare(self, states: List[RecordState]) -> None:
        sig = tuple((s.p.data_ptr(), s.g.data_ptr(), s.m.data_ptr()) for s in states)
        if sig == self.sig:
            return
        dev = states[0].p.device
        if dev.type != "cuda":
            raise RuntimeError("ShardedFourBitAdamW needs CUDA parameters; there is no CPU path")
        dtype = {torch.bfloat16: _lib.QF_BF16, torch.float16: _lib.QF_F16}.get(states[0].p.dtype, _lib.QF_F32)
        descs = (_lib.QfTensorDesc * len(states))()
        for d, s in zip(descs, states):
            r = s.rec
            d.p, d.g, d.m, d.v = s.p.data_ptr(), s.g.data_ptr(), s.m.data_ptr(), s.v.data_ptr()
            d.numel, d.kind, d.dtype, d.hyper = r.numel, r.kind, dtype, 0
            if r.kind == FP32:
                continue
            d.m_scale, d.v_scale = s.m_scale.data_ptr(), s.v_scale.data_ptr()
            if r.kind == RANK1:
                d.rows, d.cols, d.flat_offset, d.partial = r.rows, r.cols, r.flat_offset, int(r.partial)
                d.v_col = s.v_col.data_ptr()
                d.v_row_new, d.v_col_new = s.row_new.data_ptr(), s.col_new.data_ptr()
                d.v_row_rcp, d.v_col_rcp = s.row_rcp.data_ptr(), s.col_rcp.data_ptr()
        need = self.L.qf_workspace_bytes(len(states))
        if self.ws is None or self.ws.numel() < need:
            self.ws = torch.zeros(need, dtype=torch.uint8, device=dev)
        self.descs, self.sig = descs, sig
        self.generation += 1

    def _call(self, what: int, states: List[RecordState], hyper: _lib.QfHyper, deltas: Sequence[int] = ()) -> None:
        if not states:
            return
        self._prepare(states)
        dev = states[0].p.device
        stream = torch.cuda.current_stream(dev).cuda_stream
        # the tensor table goes up with the first call after the descriptors changed (or on a new stream); later calls
        # say that it is in place and copy nothing
        if self.uploaded == (self.generation, stream):
            what |= _lib.QF_RUN_TABLE_IN_PLACE
        harr = (_lib.QfHyper * 1)(hyper)
        arr = (C.c_int64 * len(deltas))(*deltas) if deltas else None
        _lib.check(self.L.qf_step_run(self.descs, len(self.descs), harr, 1, self.ws.data_ptr(), self.ws.numel(), dev.index,
                                      C.c_void_p(stream), what, arr, len(deltas)), "sharded step")
        self.uploaded = (self.generation, stream)

    def pre(self, states: List[RecordState], hyper: _lib.QfHyper) -> None:
        self._call(_lib.QF_RUN_PRE, states, hyper)

    def main(self, states: List[RecordState], hyper: _lib.QfHyper) -> None:
        self._call(_lib.QF_RUN_MAIN, states, hyper)

    def main_push(self, states: List[RecordState], hyper: _lib.QfHyper, deltas: Sequence[int]) -> None:
        """`main` that also stores the new parameters at the same place of every peer's flat buffer."""
        self._call(_lib.QF_RUN_MAIN, states, hyper, deltas)

    def read_status(self) -> int:
        """Synchronise the current stream, return the status word of this backend's workspace and clear it."""
        if self.ws is None:
            return 0
        word = C.c_uint32(0)
        dev = self.ws.device
        _lib.check(self.L.qf_read_status(self.ws.data_ptr(), dev.index,
                                         C.c_void_p(torch.cuda.current_stream(dev).cuda_stream), C.byref(word)), "qf_read_status")
        return word.value

    # ---- the flat buffer in the other processes of the node -----------------------------------------

    def export_buffer(self, t: torch.Tensor) -> Tuple[bytes, int]:
        handle = C.create_string_buffer(_lib.QF_PEER_HANDLE_BYTES)
        off = C.c_int64(0)
        _lib.check(self.L.qf_peer_export(C.c_void_p(t.data_ptr()), t.device.index, handle, C.byref(off)), "qf_peer_export")
        return handle.raw, off.value

    def open_buffer(self, handle: bytes, offset: int, device: torch.device) -> Tuple[int, int]:
        """(base of the mapping, address of the peer's buffer in this process)."""
        base = C.c_void_p(0)
        _lib.check(self.L.qf_peer_open(handle, device.index, C.byref(base)), "qf_peer_open")
        return base.value, base.value + offset

    def close_buffer(self, base: int, device: torch.device) -> None:
        _lib.check(self.L.qf_peer_close(C.c_void_p(base), device.index), "qf_peer_close")


class ShardedFourBitAdamW(torch.optim.Optimizer):
    """FourBitAdamW with ZeRO-1 style sharding of the 4-bit state over the ranks of `process_group`.

    Same constructor arguments as FourBitAdamW.  All parameters must share one dtype (float32, bfloat16 or float16)
    and one device, and every parameter must have a gradient at each step.  The parameters are moved into
    one flat buffer and become views of it.

    `reduce_grads=True` adds the other half of ZeRO-1: the gradients live in a flat buffer of the same layout
    (every `p.grad` is a view of it, so backward accumulates in place), the ranks hold different gradients,
    and each step starts by leaving the mean over the ranks of this rank's range where the step reads it: inside a
    node through the library's own kernel (qf_grad_mean_peers: peer loads, fp32 sum in rank order, one rounding),
    otherwise through NCCL's reduce-scatter.  Without it (default) the caller has already made the gradients equal on all ranks.
    """

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2, *, fused: Optional[bool] = False,
                 quant_threshold: int = DEFAULT_THRESHOLD, process_group=None, backend=None,
                 rank: Optional[int] = None, world: Optional[int] = None, comm: str = "auto",
                 reduce_grads: bool = False):
        if not 0.0 < lr:
            raise ValueError(f"Invalid learning rate: {lr=}")
        if not 0.0 < eps:
            raise ValueError(f"Invalid eps value: {eps=}")
        if not 0.0 < betas[0] < 1.0:
            raise ValueError(f"Invalid Beta[0]: {betas[0]=}")
        if not 0.0 < betas[1] < 1.0:
            raise ValueError(f"Invalid Beta[1]: {betas[1]=}")
        if not 0.0 <= weight_decay:
            raise ValueError(f"Invalid weight_decay value: {weight_decay=}")
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, fused=fused))
        if len(self.param_groups) != 1:
            raise ValueError("ShardedFourBitAdamW takes one parameter group")
        self.param_quant_threshold = int(quant_threshold)
        self.group = process_group
        self.sharded = dist.is_available() and dist.is_initialized()
        self.world = dist.get_world_size(process_group) if self.sharded else 1
        self.rank = dist.get_rank(process_group) if self.sharded else 0
        if world is not None:
            # explicit placement without a process group: the caller moves the maxima and the parameter
            # ranges between the instances itself (step_pre / step_main); used to run several ranks in one process
            self.sharded, self.world, self.rank = False, int(world), int(rank or 0)
        self.backend = backend if backend is not None else CudaBackend()
        self.params: List[torch.Tensor] = list(self.param_groups[0]["params"])
        p0 = self.params[0]
        if any(p.dtype != p0.dtype or p.device != p0.device for p in self.params):
            raise ValueError("all parameters must share dtype and device")
        if p0.dtype not in (torch.float32, torch.bfloat16, torch.float16):
            raise TypeError(f"parameters must be float32, bfloat16 or float16, got {p0.dtype}")
        self.layout = flat_layout([p.shape for p in self.params], self.world)
        self.step_count = 0
        if comm not in ("auto", "nccl", "p2p", "ce"):
            raise ValueError(f"comm must be 'auto', 'nccl', 'p2p' or 'ce', got {comm!r}")
        self._flatten()
        self._build_state()
        self.reduce_grads = bool(reduce_grads)
        self.grad_deltas: List[int] = []      # byte distances to every rank's gradient buffer (peer mappings), or empty
        self.flat_grad: Optional[torch.Tensor] = None
        if self.reduce_grads:
            self.flat_grad = torch.zeros_like(self.flat)
            self._attach_grad_views()
        self.peer_deltas: List[int] = []
        self.peer_devices: List[int] = []
        self._peer_bases: List[int] = []
        self.comm = self._comm_selected = "nccl"
        if comm != "nccl" and self.sharded and self.world > 1 and self.flat.is_cuda:
            self._setup_p2p(required=comm in ("p2p", "ce"), mode="ce" if comm == "ce" else "p2p")

    # ---- set-up -----------------------------------------------------------------------------------

    def _flatten(self) -> None:
        p0 = self.params[0]
        self.flat = torch.zeros(self.layout.total, dtype=p0.dtype, device=p0.device)
        with torch.no_grad():
            for p, off, n in zip(self.params, self.layout.offsets, self.layout.numels):
                view = self.flat[off:off + n].view(p.shape)
                view.copy_(p)
                p.data = view

    def _attach_grad_views(self) -> None:
        """Make every p.grad the parameter's view of the flat gradient buffer (copying a gradient that was
        produced elsewhere, e.g. after zero_grad(set_to_none=True))."""
        for p, off, n in zip(self.params, self.layout.offsets, self.layout.numels):
            view = self.flat_grad[off:off + n].view(p.shape)
            if p.grad is not None and p.grad.data_ptr() != view.data_ptr():
                if p.grad.is_sparse:
                    raise RuntimeError("QuantFour AdamW does not support sparse gradients")
                view.copy_(p.grad)
            p.grad = view

    def zero_grad(self, set_to_none: bool = False) -> None:
        """With reduce_grads the gradients are zeroed in the flat buffer and stay attached whatever `set_to_none`
        says (a gradient set to None would be re-created outside the buffer by the next backward and have to be
        copied in); without it this is torch's zero_grad."""
        if not self.reduce_grads:
            return super().zero_grad(set_to_none=set_to_none)
        self.flat_grad.zero_()          # the views stay attached: backward keeps accumulating in place
        for p, off, n in zip(self.params, self.layout.offsets, self.layout.numels):
            if p.grad is None or p.grad.data_ptr() != self.flat_grad[off:off + n].data_ptr():
                p.grad = self.flat_grad[off:off + n].view(p.shape)

    def _reduce_gradients(self) -> None:
        """Mean of the ranks' gradients over this rank's range of the flat gradient buffer, in place."""
        if any(p.grad is None for p in self.params):
            raise RuntimeError("ShardedFourBitAdamW needs a gradient for every parameter at every step")
        self._attach_grad_views()
        if not (self.sharded and self.world > 1):
            return
        lo, hi = self.layout.range_of(self.rank)
        if self.grad_deltas:
            # this rank reads its range of every rank's gradients through peer loads and writes the mean over its own
            # copy (fp32 sum in rank order, one rounding).  The collective in front makes every rank's gradients
            # complete before anyone reads them; the next collective of the step (the exchange of maxima, the token
            # around the peer stores, the all-gather) keeps every rank from touching its gradients again before all
            # ranks' reads have finished.
            dist.all_reduce(self._token, op=dist.ReduceOp.MAX, group=self.group)
            dev = self.flat_grad.device
            arr = (C.c_int64 * len(self.grad_deltas))(*self.grad_deltas)
            dtype = {torch.bfloat16: _lib.QF_BF16, torch.float16: _lib.QF_F16}.get(self.flat_grad.dtype, _lib.QF_F32)
            _lib.check(_lib.lib().qf_grad_mean_peers(C.c_void_p(self.flat_grad[lo:hi].data_ptr()), hi - lo, dtype, arr, len(arr),
                                                     1.0 / self.world, dev.index,
                                                     C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)), "qf_grad_mean_peers")
        elif self.flat_grad.is_cuda:
            dist.reduce_scatter_tensor(self.flat_grad[lo:hi], self.flat_grad, op=dist.ReduceOp.AVG, group=self.group)
        else:  # CPU process groups (tests)
            dist.all_reduce(self.flat_grad, op=dist.ReduceOp.SUM, group=self.group)
            self.flat_grad.mul_(1.0 / self.world)

    def _build_state(self) -> None:
        dev = self.flat.device
        lay = self.layout
        self.records = rank_records(lay, self.rank, self.param_quant_threshold)
        # tensors cut by a range boundary: every rank keeps their full row/column buffers in one shared
        # allocation (same layout on all ranks) so that one all-reduce combines the new maxima
        self.split = [t for t in range(len(self.params))
                      if tensor_kind(lay.shapes[t], lay.numels[t], self.param_quant_threshold) == RANK1 and len(lay.owners(t)) > 1]
        f32 = dict(dtype=torch.float32, device=dev)
        # a tensor's buffer is [rows padded to a multiple of 4 | cols padded likewise]: keeps the column part
        # 16-byte aligned for the vector path
        def buf_len(t):
            return _round_up(lay.shapes[t][0], 4) + _round_up(lay.shapes[t][1], 4)
        sizes = {t: buf_len(t) for t in self.split}
        self.shared_new = torch.zeros(sum(sizes.values()), **f32)
        self.shared_pos, pos = {}, 0
        for t in self.split:
            self.shared_pos[t] = pos
            pos += sizes[t]
        # per-tensor rank-1 buffers: (old, new, rcp), each [R + C]; `new` of a split tensor aliases shared_new
        self.rank1_buf: Dict[int, Tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = {}
        self.states: List[RecordState] = []
        for rec in self.records:
            t, n = rec.tensor, rec.numel
            off = lay.offsets[t] + rec.a
            st = RecordState(rec, self.flat[off:off + n], None, None)
            if rec.kind == FP32:
                st.m, st.v = torch.zeros(n, **f32), torch.zeros(n, **f32)
            else:
                nb, nblk = (n + 1) // 2, (n + BLOCK - 1) // BLOCK
                st.m = torch.zeros(nb, dtype=torch.int8, device=dev)
                st.v = torch.zeros(nb, dtype=torch.int8, device=dev)
                st.m_scale = torch.zeros(nblk, **f32)
                if rec.kind == BLOCKQ:
                    st.v_scale = torch.zeros(nblk, **f32)
                else:
                    R, Cc = lay.shapes[t]
                    Rp = _round_up(R, 4)
                    if t not in self.rank1_buf:
                        new = (self.shared_new[self.shared_pos[t]:self.shared_pos[t] + buf_len(t)] if t in self.shared_pos
                               else torch.zeros(buf_len(t), **f32))
                        self.rank1_buf[t] = (torch.zeros(buf_len(t), **f32), new, torch.zeros(buf_len(t), **f32))
                    old, new, rcp = self.rank1_buf[t]
                    r0, r1 = (rec.row_lo, rec.row_lo + rec.rows) if not rec.partial else (0, R)
                    st.v_scale, st.row_new, st.row_rcp = old[r0:r1], new[r0:r1], rcp[r0:r1]
                    st.v_col, st.col_new, st.col_rcp = old[Rp:Rp + Cc], new[Rp:Rp + Cc], rcp[Rp:Rp + Cc]
            self.states.append(st)

    def _setup_p2p(self, required: bool, mode: str = "p2p") -> None:
        """Map every other rank's flat buffer into this process.  All ranks take the same decision: one
        failure anywhere (devices of different nodes, no peer access, a virtual-memory allocator) keeps the
        all-gather."""
        dev = self.flat.device
        self._token = torch.zeros(1, dtype=torch.float32, device=dev)
        err, mine = "", None
        try:
            mine = self.backend.export_buffer(self.flat) + (socket.gethostname(), str(torch.cuda.get_device_properties(dev).uuid))
            if self.reduce_grads:     # the gradient buffers are shared the same way: the reduction reads them through peer loads
                mine = mine + self.backend.export_buffer(self.flat_grad)
        except Exception as e:  # noqa: BLE001 - any failure means: no peer path
            err = f"{type(e).__name__}: {e}"
        everyone: List[Any] = [None] * self.world
        dist.all_gather_object(everyone, mine, group=self.group)
        if not err and any(x is not None and x[2] != everyone[self.rank][2] for x in everyone):
            err = "the ranks run on different hosts"     # a handle means nothing on another machine: do not try it
        if not err and all(x is not None for x in everyone) and self.world - 1 <= _lib.QF_MAX_PEERS:
            try:
                visible = {str(torch.cuda.get_device_properties(i).uuid): i for i in range(torch.cuda.device_count())}
                # peers in rotated order (rank + 1, rank + 2, ...): whatever walks the list -- the stores of a row, the
                # copies of a piece -- then targets a different GPU on every rank at any moment
                for k in range(1, self.world):
                    r = (self.rank + k) % self.world
                    handle, off, _, uuid = everyone[r][:4]
                    base, addr = self.backend.open_buffer(handle, off, dev)
                    self._peer_bases.append(base)
                    self.peer_deltas.append(addr - self.flat.data_ptr())
                    self.peer_devices.append(visible.get(uuid, -1))   # the peer's GPU as this process numbers it
                if self.reduce_grads:
                    # every rank's gradient buffer, in rank order (0 = this rank's own): the order of the sum
                    deltas = []
                    for r in range(self.world):
                        if r == self.rank:
                            deltas.append(0)
                            continue
                        base, addr = self.backend.open_buffer(everyone[r][4], everyone[r][5], dev)
                        self._peer_bases.append(base)
                        deltas.append(addr - self.flat_grad.data_ptr())
                    self.grad_deltas = deltas
            except Exception as e:  # noqa: BLE001
                err = f"{type(e).__name__}: {e}"
        elif not err:
            err = "a peer could not export its buffer"
        ok = torch.tensor([0.0 if err else 1.0], device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.group)
        if ok.item() == 1.0:
            self.comm = self._comm_selected = mode
            if mode == "ce":
                self._setup_chunks()
            return
        self.close()
        if required:
            raise RuntimeError(f"comm='p2p' is not available on rank {self.rank}: {err or 'another rank failed'}")

    def _setup_chunks(self, max_chunks: int = 8, min_bytes: int = 64 << 20) -> None:
        """Cut this rank's records into consecutive pieces of about equal size (all records of one tensor stay together:
        they share its row / column buffers) for the pipelined delivery: one update call and one copy per peer each."""
        esz = self.flat.element_size()
        total = sum(st.rec.numel for st in self.states)
        k = max(1, min(max_chunks, total * esz // min_bytes))
        target = -(-total // k)
        self.chunks: List[Tuple[List[RecordState], int, int]] = []
        cur: List[RecordState] = []
        acc = 0
        for i, st in enumerate(self.states):
            cur.append(st)
            acc += st.rec.numel
            last_of_tensor = i + 1 == len(self.states) or self.states[i + 1].rec.tensor != st.rec.tensor
            if last_of_tensor and (acc >= target or i + 1 == len(self.states)):
                lo = self.layout.offsets[cur[0].rec.tensor] + cur[0].rec.a
                hi = self.layout.offsets[cur[-1].rec.tensor] + cur[-1].rec.b
                self.chunks.append((cur, lo, hi))
                cur, acc = [], 0
        self._chunk_backends = [CudaBackend() for _ in self.chunks]
        dev = self.flat.device
        self._ce_streams = [torch.cuda.Stream(dev) for _ in self.peer_deltas]
        self._ce_events = [torch.cuda.Event() for _ in self.chunks]

    def _main_ce(self) -> None:
        """Second half of a step, delivery included: update piece k, then let the copy engines carry it to every
        peer on side streams while piece k + 1 is updated."""
        dev = self.flat.device
        cur = torch.cuda.current_stream(dev)
        base, esz, L = self.flat.data_ptr(), self.flat.element_size(), _lib.lib()
        for (states, lo, hi), backend, ev in zip(self.chunks, self._chunk_backends, self._ce_events):
            backend.main(states, self._hyper)
            ev.record(cur)
            for delta, pdev, stream in zip(self.peer_deltas, self.peer_devices, self._ce_streams):
                stream.wait_event(ev)
                _lib.check(L.qf_peer_copy(C.c_void_p(base + delta + lo * esz), pdev, C.c_void_p(base + lo * esz), (hi - lo) * esz,
                                          dev.index, C.c_void_p(stream.cuda_stream)), "qf_peer_copy")
        for stream in self._ce_streams:     # the next use of the stream (and of the flat buffer) comes after the copies
            cur.wait_stream(stream)

    def close(self) -> None:
        """Unmap the peers' buffers (the optimizer falls back to the all-gather afterwards)."""
        for base in self._peer_bases:
            try:
                self.backend.close_buffer(base, self.flat.device)
            except Exception:  # noqa: BLE001 - shutting down
                pass
        self._peer_bases, self.peer_deltas, self.peer_devices, self.comm = [], [], [], "nccl"
        self.grad_deltas = []

    def __del__(self):
        try:    # peer mappings must not outlive the optimizer; explicit close() stays the orderly way
            if getattr(self, "_peer_bases", None):
                self.close()
        except Exception:  # noqa: BLE001 - interpreter shutdown
            pass

    @property
    def comm_selected(self) -> str:
        """The way parameters were delivered before any close(): "p2p" or "nccl"."""
        return self._comm_selected

    # ---- step -------------------------------------------------------------------------------------

    @torch.no_grad()
    def step(self, closure=None, *, grad_scale: Optional[float] = None):
        """One step.  `grad_scale`: see FourBitAdamW.step (every rank passes the same value)."""
        self._grad_scale = 1.0 if grad_scale is None else float(grad_scale)
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        if self.reduce_grads:
            self._reduce_gradients()
        self.step_pre()
        multi = self.sharded and self.world > 1
        if multi and self.shared_new.numel():
            # element-wise max of the new row / column maxima of the tensors that are cut between ranks
            dist.all_reduce(self.shared_new, op=dist.ReduceOp.MAX, group=self.group)
        if multi and self.comm == "ce":
            if not self.shared_new.numel():
                dist.all_reduce(self._token, op=dist.ReduceOp.MAX, group=self.group)
            # same ordering argument as for the peer stores below: one collective on either side of the delivery
            self._main_ce()
            dist.all_reduce(self._token, op=dist.ReduceOp.MAX, group=self.group)
            return loss
        if multi and self.comm == "p2p":
            if not self.shared_new.numel():
                dist.all_reduce(self._token, op=dist.ReduceOp.MAX, group=self.group)
            # the collective above has put every rank's earlier work (its last reads of the old parameters)
            # before any rank's stores into it; the one below keeps every rank from reading the new
            # parameters before all ranks' kernels, and with them their stores, have completed
            self.backend.main_push(self.states, self._hyper, self.peer_deltas)
            dist.all_reduce(self._token, op=dist.ReduceOp.MAX, group=self.group)
            return loss
        self.step_main()
        if multi:
            self._all_gather()
        return loss

    def nonfinite_seen(self) -> bool:
        """Synchronise and report whether any step of this rank since the last call produced a non-finite scale
        (a non-finite gradient, or an overflow): the same question FourBitAdamW.nonfinite_seen answers."""
        word = 0
        for b in [self.backend] + list(getattr(self, "_chunk_backends", [])):
            read = getattr(b, "read_status", None)
            word |= read() if read else 0
        return bool(word & _lib.QF_STATUS_NONFINITE)

    @torch.no_grad()
    def step_pre(self) -> None:
        """First half of a step: new row / column maxima of this rank's pieces (into `shared_new` for the
        tensors that are cut between ranks)."""
        group = self.param_groups[0]
        flat_grads: List[torch.Tensor] = []
        for p in self.params:
            if p.grad is None:
                raise RuntimeError("ShardedFourBitAdamW needs a gradient for every parameter at every step")
            if p.grad.is_sparse:
                raise RuntimeError("QuantFour AdamW does not support sparse gradients")
            g = p.grad if p.grad.is_contiguous() else p.grad.contiguous()
            if g.dtype != p.dtype:
                raise RuntimeError("grad must match the parameter in dtype")
            flat_grads.append(g.reshape(-1))
        for st in self.states:
            st.g = flat_grads[st.rec.tensor][st.rec.a:st.rec.b]
        self.step_count += 1
        beta1, beta2 = group["betas"]
        self._hyper = make_hyper(group["lr"], beta1, beta2, group["eps"], group["weight_decay"], float(self.step_count),
                                 getattr(self, "_grad_scale", 1.0))
        if self.shared_new.numel():
            self.shared_new.zero_()
        self.backend.pre(self.states, self._hyper)

    @torch.no_grad()
    def step_main(self) -> None:
        """Second half of a step: update and requantize this rank's pieces (after the maxima were combined)."""
        self.backend.main(self.states, self._hyper)

    def _all_gather(self) -> None:
        """Every rank's range of the flat parameter buffer to every rank, in place."""
        lo, hi = self.layout.range_of(self.rank)
        if self.flat.is_cuda:
            dist.all_gather_into_tensor(self.flat, self.flat[lo:hi], group=self.group)
        else:  # CPU process groups (tests): list form, the input must not alias the outputs
            chunks = [self.flat[r * self.layout.shard:(r + 1) * self.layout.shard] for r in range(self.world)]
            dist.all_gather(chunks, self.flat[lo:hi].clone(), group=self.group)

    # ---- conversion between the sharded state and the per-parameter layout of FourBitAdamW --------------

    def pieces(self) -> List[Dict[str, Any]]:
        """This rank's records with their state on the CPU, in the form `assemble_full_state` takes."""
        out = []
        for st in self.states:
            r = st.rec
            e: Dict[str, Any] = {"tensor": r.tensor, "kind": r.kind, "a": r.a, "b": r.b,
                                 "m": st.m.detach().cpu().clone(), "v": st.v.detach().cpu().clone()}
            if r.kind != FP32:
                e["m_scale"] = st.m_scale.detach().cpu().clone()
            if r.kind == BLOCKQ:
                e["v_scale"] = st.v_scale.detach().cpu().clone()
            if r.kind == RANK1:
                R, Cc = self.layout.shapes[r.tensor]
                old = self.rank1_buf[r.tensor][0].detach().cpu()
                # the rows this piece touches are current on this rank; so are all columns
                lo, hi = r.a // Cc, (r.b - 1) // Cc + 1
                e["rows"] = (lo, hi, old[lo:hi].clone())
                e["cols"] = old[_round_up(R, 4):_round_up(R, 4) + Cc].clone()
            out.append(e)
        return out

    def full_state_dict(self) -> Dict[str, Any]:
        """The state of all ranks as one state dict in FourBitAdamW's layout (every rank returns it; a collective
        when the optimizer runs under a process group).  FourBitAdamW.load_state_dict reads it, and so does
        load_full_state_dict of a ShardedFourBitAdamW of any world size over the same parameter list."""
        mine = self.pieces()
        if self.sharded and self.world > 1:
            everyone: List[Any] = [None] * self.world
            dist.all_gather_object(everyone, mine, group=self.group)
            allp = [e for part in everyone for e in part]
        elif self.world > 1:
            raise RuntimeError("without a process group, collect pieces() of every instance and call assemble_full_state")
        else:
            allp = mine
        return assemble_full_state(allp, self.layout.shapes, self.step_count, self.param_groups[0], self.param_quant_threshold)

    def load_full_state_dict(self, sd: Dict[str, Any]) -> None:
        """Take this rank's part of a state dict in FourBitAdamW's layout (written by FourBitAdamW.state_dict or by
        full_state_dict under any world size).  All parameters must be at the same step."""
        ids = list(sd["param_groups"][0]["params"])
        if len(sd["param_groups"]) != 1 or len(ids) != len(self.params):
            raise ValueError("the state dict must hold one parameter group over the same parameter list")
        full = [sd["state"][i] for i in ids]
        steps = {float(f["step"]) for f in full}
        if len(steps) != 1:
            raise ValueError("ShardedFourBitAdamW keeps one step count; the state dict holds parameters at different steps")
        self.step_count = int(steps.pop())
        self.param_groups[0].update({k: v for k, v in sd["param_groups"][0].items() if k != "params"})
        lay = self.layout
        with torch.no_grad():
            for t, f in enumerate(full):
                kind = tensor_kind(lay.shapes[t], lay.numels[t], self.param_quant_threshold)
                if kind == RANK1 and t in self.rank1_buf:
                    R, Cc = lay.shapes[t]
                    row, col = f["variance_qstate"]["overhead"]["max_dims"]
                    old = self.rank1_buf[t][0]
                    old[:R].copy_(row.reshape(-1))
                    old[_round_up(R, 4):_round_up(R, 4) + Cc].copy_(col.reshape(-1))
            for st in self.states:
                r, f = st.rec, full[st.rec.tensor]
                if r.kind == FP32:
                    st.m.copy_(f["exp_avg"].reshape(-1)[r.a:r.b])
                    st.v.copy_(f["exp_avg_sq"].reshape(-1)[r.a:r.b])
                    continue
                b0, b1, k0, k1 = r.a // 2, (r.b + 1) // 2, r.a // BLOCK, (r.b + BLOCK - 1) // BLOCK
                st.m.copy_(f["exp_avg"][b0:b1])
                st.v.copy_(f["exp_avg_sq"][b0:b1])
                st.m_scale.copy_(f["momentum_qstate"]["overhead"]["max1"][k0:k1])
                if r.kind == BLOCKQ:
                    st.v_scale.copy_(f["variance_qstate"]["overhead"]["max1"][k0:k1])

    # ---- checkpoint ---------------------------------------------------------------------------------

    def state_dict(self) -> Dict[str, Any]:
        """This rank's shard: its records with their state tensors, plus the layout they belong to."""
        recs = []
        for st in self.states:
            r = st.rec
            entry = {"tensor": r.tensor, "kind": r.kind, "a": r.a, "b": r.b, "exp_avg": st.m, "exp_avg_sq": st.v}
            if r.kind != FP32:
                entry["max1"] = st.m_scale
            if r.kind == BLOCKQ:
                entry["sq_max1"] = st.v_scale
            recs.append(entry)
        rank1 = {t: old for t, (old, _, _) in self.rank1_buf.items()}
        return {"step": self.step_count, "rank": self.rank, "world": self.world, "shard": self.layout.shard,
                "shapes": self.layout.shapes, "records": recs, "rank1_maxima": rank1,
                "param_groups": [{k: v for k, v in self.param_groups[0].items() if k != "params"}]}

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        if sd["world"] != self.world or sd["rank"] != self.rank or list(map(tuple, sd["shapes"])) != self.layout.shapes:
            raise ValueError("sharded state was written for a different world size, rank or parameter list")
        self.step_count = int(sd["step"])
        self.param_groups[0].update(sd["param_groups"][0])
        by_key = {(e["tensor"], e["a"], e["b"]): e for e in sd["records"]}
        with torch.no_grad():
            for st in self.states:
                e = by_key[(st.rec.tensor, st.rec.a, st.rec.b)]
                st.m.copy_(e["exp_avg"])
                st.v.copy_(e["exp_avg_sq"])
                if st.rec.kind != FP32:
                    st.m_scale.copy_(e["max1"])
                if st.rec.kind == BLOCKQ:
                    st.v_scale.copy_(e["sq_max1"])
            for t, old in sd["rank1_maxima"].items():
                self.rank1_buf[t][0].copy_(old)
