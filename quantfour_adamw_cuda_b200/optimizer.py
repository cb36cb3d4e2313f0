"""FourBitAdamW: AdamW with 4-bit optimizer states, one fused multi-tensor CUDA launch per step.

Drop-in for the reference's optimizer classes ``AdamWFused_QuantFour`` (optim/fused_quantfour.py:25-313)
and ``AdamW_QuantFour`` (optim/adamw_fourbit_triton.py:137-382): same constructor arguments, defaults
and ValueError checks (fused_quantfour.py:28-58), same ``step(closure)`` contract (:131-138), same
per-parameter state keys (:61-70, :110-128).  Where the reference loops over parameters in Python and
launches one kernel plus one device synchronisation per tensor (:171-292), this class hands the whole
ragged parameter list to ``qf_step_run`` once per step and never synchronises.

State of a parameter ``p`` (what ``state_dict()`` carries):
  ``step``              0-dim float32 CPU tensor
  ``exp_avg``           int8 [ceil(numel/2)] packed 4-bit codes   (float32, shaped like p, if not quantized)
  ``exp_avg_sq``        int8 [ceil(numel/2)] packed 4-bit codes   (float32, shaped like p, if not quantized)
  ``momentum_qstate``   {"enable": bool, "overhead": {"max1": float32 [ceil(numel/128)]}, "qmap": None}
  ``variance_qstate``   {"enable": bool, "overhead": {...}, "qmap": None} where overhead is
                        2-D p:  {"max_dims": [float32 [R,1], float32 [1,C]], "max1": None, "dim": 2}
                        (with nd_rank1=True also p of 3 and more dimensions: one keep-dim vector per axis)
                        else:   {"max1": float32 [ceil(numel/128)], "dim": p.dim()}
Quantization is enabled iff ``numel > quant_threshold`` (fused_quantfour.py:18-22; threshold 4096 as in
adamw_fourbit_triton.py:118, :128).
"""
from __future__ import annotations

import ctypes as C
import math
from itertools import chain
from typing import Any, Dict, List, Optional, Tuple

import torch

from . import _lib
from .functional import _DTYPES, dequantize_m, dequantize_v, dequantize_v_block

__all__ = ["FourBitAdamW", "AdamWFused_QuantFour", "AdamW_Fused_QuantFour", "AdamW_QuantFour", "make_hyper",
           "enable_param_quantization"]

BLOCK = 128
DEFAULT_THRESHOLD = 4096


def enable_param_quantization(p, threshold) -> bool:
    """Only tensors with more than ``threshold`` elements are quantized (fused_quantfour.py:18-22)."""
    if threshold and p.numel() <= threshold:
        return False
    return True


def make_hyper(lr: float, beta1: float, beta2: float, eps: float, weight_decay: float, step: float,
               grad_scale: float = 1.0) -> _lib.QfHyper:
    """Scalars of one step, derived in Python doubles like the reference's PyTorch path
    (adamw_fourbit_triton.py:415, :458-465) and rounded once to float32 by ctypes.  `grad_scale` other than 1
    makes the step replace every gradient by g * grad_scale (rounded to g's dtype) before using it."""
    bc1 = 1 - beta1 ** step
    bc2 = 1 - beta2 ** step
    return _lib.QfHyper(1 - lr * weight_decay, 1 - beta1, beta2, 1 - beta2, eps, -(lr / bc1), math.sqrt(bc2),
                        0.0 if grad_scale == 1.0 else grad_scale)


def state_kind(p: torch.Tensor, threshold: int, nd_rank1: bool = False) -> int:
    if not enable_param_quantization(p, threshold):
        return _lib.QF_KIND_FP32
    return _lib.QF_KIND_RANK1 if p.dim() == 2 or (nd_rank1 and p.dim() > 2) else _lib.QF_KIND_BLOCK


class _DevicePlan:
    """Cached ctypes descriptor array + workspace for the tensors of one device."""

    def __init__(self) -> None:
        self.signature: Optional[tuple] = None
        self.descs = None
        self.workspace: Optional[torch.Tensor] = None
        self.keepalive: list = []
        self.nd: list = []      # (parameter, second-moment overhead) of the tensors of three and more dimensions with per-axis maxima


class FourBitAdamW(torch.optim.Optimizer):
    """AdamW with decoupled weight decay whose moments are stored in 4 bits.

    First moment: signed dynamic-exponent map, one abs-max scale per 128 elements.  Second moment:
    unsigned linear map without zero; for 2-D parameters the scale of element (i, j) is
    min(row_max[i], col_max[j]) (rank-1 normalisation), otherwise one scale per 128 elements.
    Parameters with at most ``quant_threshold`` elements keep float32 moments.  Parameters and
    gradients must be CUDA tensors of dtype float32 or bfloat16; float16 works as well, through the kernels' general
    (slower) element mapping.
    """

    def __init__(
        self,
        params,
        lr=1e-3,
        betas=(0.9, 0.999),
        eps=1e-8,
        weight_decay=1e-2,
        *,
        fused: Optional[bool] = False,
        quant_threshold: int = DEFAULT_THRESHOLD,
        capturable: bool = False,
        schedule_rows: int = 1 << 18,
        relaxed_update: bool = False,
        nd_rank1: bool = False,
    ):
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
        self.param_quant_threshold = int(quant_threshold)
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, fused=fused)
        super().__init__(params, defaults)
        self._scratch: Dict[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]] = {}
        self._plans: Dict[Tuple[int, int], _DevicePlan] = {}
        self._fast: Optional[dict] = None
        self.capturable = bool(capturable)
        self.schedule_rows = int(schedule_rows)
        # relaxed_update (not in the reference): bf16 matrices take the uncorrected parameter update (QF_RUN_RELAXED_UPDATE)
        # update -- new parameters within one bf16 unit of the exact ones, every code and scale unchanged
        self.relaxed_update = bool(relaxed_update)
        if self.relaxed_update and self.capturable:
            raise ValueError("relaxed_update and capturable cannot be combined")
        # nd_rank1 (the reference's scheme for every rank above one, adamw_fourbit_triton.py:841-856; off by default,
        # where tensors of three and more dimensions take block-128 scales like vectors): the second moment of such a
        # tensor is normalised by the smallest of its per-axis maxima.
        self.nd_rank1 = bool(nd_rank1)
        if self.nd_rank1 and self.capturable:
            raise ValueError("nd_rank1 and capturable cannot be combined")
        self._nd_rows: Dict[torch.Tensor, torch.Tensor] = {}
        self._cap: Optional[dict] = None
        self._status_bits = 0

    # ---- state ---------------------------------------------------------------------------------

    def init_qstate(self, p, state_name):
        """Create the ``{state_name}_qstate`` record of ``p`` (fused_quantfour.py:61-70)."""
        state = self.state[p]
        state[f"{state_name}_qstate"] = {
            "enable": enable_param_quantization(p, self.param_quant_threshold),
            "overhead": dict(),
            "qmap": None,
        }

    def _init_state(self, p: torch.Tensor) -> None:
        state = self.state[p]
        state["step"] = torch.tensor(0.0)
        self.init_qstate(p, "momentum")
        self.init_qstate(p, "variance")
        n, dev = p.numel(), p.device
        kind = state_kind(p, self.param_quant_threshold, self.nd_rank1)
        if kind == _lib.QF_KIND_FP32:
            state["exp_avg"] = torch.zeros_like(p, dtype=torch.float32, memory_format=torch.contiguous_format)
            state["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32, memory_format=torch.contiguous_format)
            return
        nb, nblk = (n + 1) // 2, (n + BLOCK - 1) // BLOCK
        state["exp_avg"] = torch.zeros(nb, dtype=torch.int8, device=dev)
        state["exp_avg_sq"] = torch.zeros(nb, dtype=torch.int8, device=dev)
        state["momentum_qstate"]["overhead"]["max1"] = torch.zeros(nblk, dtype=torch.float32, device=dev)
        vo = state["variance_qstate"]["overhead"]
        vo["dim"] = p.dim()
        if kind == _lib.QF_KIND_RANK1:
            # one vector of maxima per axis, shaped for broadcasting: [R,1], [1,C] for a matrix
            vo["max_dims"] = [torch.zeros([d if k == a else 1 for k in range(p.dim())], dtype=torch.float32, device=dev)
                              for a, d in enumerate(p.shape)]
            vo["max1"] = None
        else:
            vo["max1"] = torch.zeros(nblk, dtype=torch.float32, device=dev)

    def _scratch_for(self, p: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        s = self._scratch.get(p)
        if s is None or s[0].device != p.device:
            R, Cc = p.numel() // p.shape[-1], p.shape[-1]
            # new maxima followed by their reciprocals (the layout qf_step_multi expects)
            s = (torch.zeros(2 * R, dtype=torch.float32, device=p.device),
                 torch.zeros(2 * Cc, dtype=torch.float32, device=p.device))
            self._scratch[p] = s
        return s

    def __setstate__(self, state: Dict[str, Any]) -> None:
        super().__setstate__(state)
        for group in self.param_groups:
            group.setdefault("fused", None)
        self.__dict__.setdefault("param_quant_threshold", DEFAULT_THRESHOLD)
        self._scratch = {}
        self._plans = {}
        self._fast = None
        self._cap = None
        self.__dict__.setdefault("capturable", False)
        self.__dict__.setdefault("schedule_rows", 1 << 18)
        self.__dict__.setdefault("relaxed_update", False)
        self.__dict__.setdefault("nd_rank1", False)
        self._nd_rows = {}
        self.__dict__.setdefault("_status_bits", 0)
        state_values = list(self.state.values())
        step_is_tensor = len(state_values) != 0 and torch.is_tensor(state_values[0]["step"])
        if not step_is_tensor:
            for s in state_values:
                s["step"] = torch.tensor(float(s["step"]))

    def load_state_dict(self, state_dict: Dict[str, Any]) -> None:
        """Load a state dict written by ``state_dict()``.

        torch's loader casts every floating-point-parameter state tensor to the parameter's dtype,
        which would turn int8 code buffers and float32 scales into bfloat16 for bf16 parameters.
        After the base class has mapped ids and restored the groups, every state entry is therefore
        re-materialised from the saved value with its saved dtype, on the parameter's device.
        """
        self._cap = None
        super().load_state_dict(state_dict)
        saved_ids = chain.from_iterable(g["params"] for g in state_dict["param_groups"])
        params = chain.from_iterable(g["params"] for g in self.param_groups)
        id_map = dict(zip(saved_ids, params))

        def place(value, device, key=None):
            if torch.is_tensor(value):
                return value.detach().clone() if key == "step" else value.detach().to(device=device, copy=True)
            if isinstance(value, dict):
                return {k: place(v, device, k) for k, v in value.items()}
            if isinstance(value, (list, tuple)):
                return type(value)(place(v, device) for v in value)
            return value

        for pid, saved in state_dict["state"].items():
            if pid in id_map:
                p = id_map[pid]
                self.state[p] = place(saved, p.device)
        self._scratch = {}
        self._plans = {}
        self._fast = None
        self._nd_rows = {}

    def dequantized_state(self, p: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """(exp_avg, exp_avg_sq) of ``p`` as float32 tensors shaped like ``p`` (dequantized on the GPU)."""
        st = self.state[p]
        if not st["momentum_qstate"]["enable"]:
            return st["exp_avg"].clone(), st["exp_avg_sq"].clone()
        n = p.numel()
        m = dequantize_m(st["exp_avg"], st["momentum_qstate"]["overhead"]["max1"], n).view(p.shape)
        vo = st["variance_qstate"]["overhead"]
        if vo.get("max_dims") is not None:
            row, col = self._row_scale(p, vo), vo["max_dims"][-1]
            v = dequantize_v(st["exp_avg_sq"], row.reshape(-1), col.reshape(-1)).view(p.shape)
        else:
            v = dequantize_v_block(st["exp_avg_sq"], vo["max1"], n).view(p.shape)
        return m, v

    # ---- step ----------------------------------------------------------------------------------

    def _fill_desc(self, d: _lib.QfTensorDesc, p: torch.Tensor, g: torch.Tensor, st: Dict[str, Any], hyper: int) -> None:
        n = p.numel()
        d.p, d.g = p.data_ptr(), g.data_ptr()
        d.m, d.v = st["exp_avg"].data_ptr(), st["exp_avg_sq"].data_ptr()
        d.numel, d.dtype, d.hyper = n, _DTYPES[p.dtype], hyper
        if not st["momentum_qstate"]["enable"]:
            d.kind = _lib.QF_KIND_FP32
            return
        d.m_scale = st["momentum_qstate"]["overhead"]["max1"].data_ptr()
        vo = st["variance_qstate"]["overhead"]
        if vo.get("max_dims") is not None:
            row, col = self._row_scale(p, vo), vo["max_dims"][-1]
            nrow, ncol = self._scratch_for(p)
            d.kind = _lib.QF_KIND_RANK1
            d.rows, d.cols = p.numel() // p.shape[-1], p.shape[-1]
            d.v_scale, d.v_col = row.data_ptr(), col.data_ptr()
            d.v_row_new, d.v_col_new = nrow.data_ptr(), ncol.data_ptr()
        else:
            d.kind = _lib.QF_KIND_BLOCK
            d.v_scale = vo["max1"].data_ptr()

    # Tensors of three and more dimensions (nd_rank1=True) run through the kernels as matrices: the leading axes fold
    # into rows, the last axis gives the columns, and the row scale of row (i0, i1, ..) is the smallest of the leading
    # axes' maxima at i0, i1, ..: min(row scale, column maximum) is then the reference's per-axis scale.  The row scale
    # lives in a buffer of its own (the state keeps the per-axis vectors, as the reference does).
    def _row_scale(self, p: torch.Tensor, vo: Dict[str, Any]) -> torch.Tensor:
        dims = vo["max_dims"]
        if len(dims) == 2:
            return dims[0]
        r = self._nd_rows.get(p)
        if r is None or r.device != p.device:
            lead = dims[0]
            for mx in dims[1:-1]:
                lead = torch.minimum(lead, mx)
            r = self._nd_rows[p] = lead.expand(*p.shape[:-1], 1).reshape(-1).contiguous()
        return r

    def _fold_new_maxima(self, p: torch.Tensor, vo: Dict[str, Any]) -> None:
        """Between the two halves of a step: the first pass has left the new maximum of every row (a row = one index
        tuple of the leading axes) in the scratch; the new maxima of the leading axes follow from them, go into the
        state, and the smallest of them per row replaces the row maxima as the row scale the second pass divides by."""
        nrow, _ = self._scratch_for(p)
        rows = p.numel() // p.shape[-1]
        rm = nrow[:rows].view(p.shape[:-1])
        k = rm.dim()
        lead = None
        for a in range(k):
            others = [d for d in range(k) if d != a]
            mx = rm.amax(dim=others, keepdim=True) if others else rm
            vo["max_dims"][a].copy_(mx.unsqueeze(-1))
            lead = mx if lead is None else torch.minimum(lead, mx)
        rm.copy_(lead)

    @torch.no_grad()
    def step(self, closure=None, *, grad_scale: Optional[float] = None):
        """Perform a single optimization step (fused_quantfour.py:131-138); returns the closure's loss.

        `grad_scale` (not in the reference): a factor every gradient is multiplied by, in place and rounded to
        its own dtype, before the step uses it -- the inverse loss scale, a clipping coefficient.  For 2-D tensors
        the multiplication rides the pass that reads the gradients anyway, so it costs no pass of its own.  A
        gradient that had to be made contiguous is scaled in the copy only."""
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        self._grad_scale = 1.0 if grad_scale is None else float(grad_scale)

        if self.capturable:
            self._step_capturable()
            return loss
        if self._fast is not None and self._step_fast():
            return loss

        hypers: List[_lib.QfHyper] = []
        hyper_index: Dict[tuple, int] = {}
        work: Dict[torch.device, List[tuple]] = {}
        cacheable = True
        for group in self.param_groups:
            beta1, beta2 = group["betas"]
            gkey = (group["lr"], beta1, beta2, group["eps"], group["weight_decay"])
            for p in group["params"]:
                if p.grad is None:
                    continue
                if p.grad.is_sparse:
                    raise RuntimeError("QuantFour AdamW does not support sparse gradients")
                if not p.is_cuda:
                    raise RuntimeError("FourBitAdamW needs CUDA parameters; there is no CPU path")
                if not p.is_contiguous():
                    raise RuntimeError("param must be contiguous")
                if p.dtype not in _DTYPES:
                    raise TypeError(f"parameters must be float32, bfloat16 or float16, got {p.dtype}")
                g = p.grad
                if g.dtype != p.dtype or g.numel() != p.numel() or g.device != p.device:
                    raise RuntimeError("grad must match the parameter in dtype, numel and device")
                if not g.is_contiguous():
                    g = g.contiguous()
                    cacheable = False
                st = self.state[p]
                if len(st) == 0:
                    self._init_state(p)
                st["step"] += 1
                t = float(st["step"])
                key = gkey + (t,)
                hi = hyper_index.get(key)
                if hi is None:
                    hi = hyper_index[key] = len(hypers)
                    hypers.append(make_hyper(*gkey, t, self._grad_scale))
                work.setdefault(p.device, []).append((p, g, st, hi))

        for dev, entries in work.items():
            # a launch carries at most QF_MAX_HYPERS hyper-parameter sets: split by hyper index range
            lo = 0
            chunk = 0
            while lo < len(hypers):
                hi_end = lo + _lib.QF_MAX_HYPERS
                sel = [e for e in entries if lo <= e[3] < hi_end]
                if sel:
                    self._launch(dev, chunk, sel, hypers[lo:hi_end], lo)
                lo, chunk = hi_end, chunk + 1
        self._fast = None
        if cacheable and len(work) == 1 and len(hypers) <= _lib.QF_MAX_HYPERS:
            self._remember(next(iter(work.items())), hyper_index)
        return loss

    # ---- steady state: same tensors, same gradient buffers as the step before ---------------------------

    def _remember(self, dev_entries, hyper_index) -> None:
        """Record what the step just made so that the next one can skip rebuilding it: which gradient buffers
        were seen, which parameters had none, and the (group, step count) class behind every hyper index."""
        dev, entries = dev_entries
        group_of = {id(p): gi for gi, g in enumerate(self.param_groups) for p in g["params"]}
        seen = {id(e[0]) for e in entries}
        classes = [None] * len(hyper_index)
        for p, _, st, hi in entries:
            if classes[hi] is None:
                classes[hi] = [group_of[id(p)], float(st["step"]), st["step"]]
        # All step counters of the launch become views of one vector, so that the steady state advances them with a
        # single in-place add instead of one per parameter (a state dict still sees a 0-dim float32 tensor each).
        steps_vec = torch.stack([st["step"].reshape(()) for _, _, st, _ in entries])
        for i, (_, _, st, _) in enumerate(entries):
            st["step"] = steps_vec[i]
        for c in classes:
            c[2] = None
        for (_, _, st, hi) in entries:
            if classes[hi][2] is None:
                classes[hi][2] = st["step"]
        self._fast = {
            "dev": dev, "plan": self._plans[(dev.index, 0)], "checks": [(p, p.data_ptr(), g.data_ptr()) for p, g, _, _ in entries],
            "absent": [p for g in self.param_groups for p in g["params"] if id(p) not in seen],
            "steps_vec": steps_vec, "classes": classes, "stream": torch.cuda.current_stream(dev).cuda_stream,
            "n_params": sum(len(g["params"]) for g in self.param_groups),
        }

    def _step_fast(self) -> bool:
        f = self._fast
        if f["n_params"] != sum(len(g["params"]) for g in self.param_groups):
            return False
        plan = f["plan"]
        checks = f["checks"]
        moved = []
        for i, (p, pptr, gptr) in enumerate(checks):
            g = p.grad
            if g is None or p.data_ptr() != pptr:
                return False
            if g.data_ptr() != gptr:     # a new gradient buffer: only its address in the descriptor changes
                if not g.is_contiguous() or g.dtype != p.dtype or g.numel() != p.numel() or g.is_sparse:
                    return False
                moved.append((i, g))
        for p in f["absent"]:
            if p.grad is not None:
                return False
        for c in f["classes"]:
            if float(c[2]) != c[1]:      # somebody rewrote a step counter: rebuild the classes
                return False
        for i, g in moved:
            plan.descs[i].g = g.data_ptr()
            plan.keepalive[i] = g
            checks[i] = (checks[i][0], checks[i][1], g.data_ptr())
        if moved:
            plan.signature = None     # the slow path must not trust its cached signature any more
        f["steps_vec"].add_(1.0)
        hypers = []
        for c in f["classes"]:
            c[1] += 1.0
            group = self.param_groups[c[0]]
            beta1, beta2 = group["betas"]
            hypers.append(make_hyper(group["lr"], beta1, beta2, group["eps"], group["weight_decay"], c[1], self._grad_scale))
        dev = f["dev"]
        harr = (_lib.QfHyper * len(hypers))(*hypers)
        # the table of these descriptors is in the workspace since the last call, unless a gradient moved or the step
        # now runs on another stream than the one the table was copied on
        stream = torch.cuda.current_stream(dev).cuda_stream
        self._run(plan, harr, len(hypers), dev, table_in_place=not moved and f.get("stream") == stream)
        f["stream"] = stream
        return True

    def _run(self, plan, harr, n_hypers: int, dev: torch.device, table_in_place: bool) -> None:
        """Both halves of the step on `plan`; `table_in_place`: the workspace holds the table of plan.descs already."""
        flags = (_lib.QF_RUN_RELAXED_UPDATE if self.relaxed_update else 0) | (_lib.QF_RUN_TABLE_IN_PLACE if table_in_place else 0)
        L = _lib.lib()
        args = (plan.descs, len(plan.descs), harr, n_hypers, plan.workspace.data_ptr(), plan.workspace.numel(), dev.index,
                C.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
        if not plan.nd:
            _lib.check(L.qf_step_run(*args, _lib.QF_RUN_PRE | _lib.QF_RUN_MAIN | flags, None, 0), "qf_step_run")
            return
        _lib.check(L.qf_step_run(*args, _lib.QF_RUN_PRE | flags, None, 0), "qf_step_run")
        for p, vo in plan.nd:
            self._fold_new_maxima(p, vo)
        _lib.check(L.qf_step_run(*args, _lib.QF_RUN_MAIN | _lib.QF_RUN_TABLE_IN_PLACE | flags, None, 0), "qf_step_run")

    def _launch(self, dev: torch.device, chunk: int, entries: List[tuple], hypers: List[_lib.QfHyper], hyper_base: int) -> None:
        L = _lib.lib()
        plan = self._plans.setdefault((dev.index, chunk), _DevicePlan())
        signature = tuple((id(p), p.data_ptr(), g.data_ptr(), st["exp_avg"].data_ptr(), hi - hyper_base)
                          for p, g, st, hi in entries)
        if plan.signature != signature:
            n = len(entries)
            descs = (_lib.QfTensorDesc * n)()
            for d, (p, g, st, hi) in zip(descs, entries):
                self._fill_desc(d, p, g, st, hi - hyper_base)
            need = L.qf_workspace_bytes(n)
            if plan.workspace is None or plan.workspace.numel() < need or plan.workspace.device != dev:
                plan.workspace = torch.zeros(need, dtype=torch.uint8, device=dev)
            plan.descs, plan.signature = descs, signature
            plan.keepalive = [g for _, g, _, _ in entries]
            plan.nd = [(p, st["variance_qstate"]["overhead"]) for p, _, st, _ in entries
                       if st["momentum_qstate"]["enable"] and len(st["variance_qstate"]["overhead"].get("max_dims") or ()) > 2]
        harr = (_lib.QfHyper * len(hypers))(*hypers)
        self._run(plan, harr, len(hypers), dev, table_in_place=False)

    def _read_status(self) -> None:
        """Synchronise, fold the status word of every workspace into `_status_bits` and clear the words."""
        L = _lib.lib()
        for (dev_index, _), plan in self._plans.items():
            if plan.workspace is None:
                continue
            word = C.c_uint32(0)
            dev = torch.device("cuda", dev_index)
            _lib.check(L.qf_read_status(plan.workspace.data_ptr(), dev_index,
                                        C.c_void_p(torch.cuda.current_stream(dev).cuda_stream), C.byref(word)),
                       "qf_read_status")
            self._status_bits |= word.value

    def nonfinite_seen(self) -> bool:
        """Synchronise and report whether any step since the last call produced a non-finite scale."""
        self._read_status()
        seen = bool(self._status_bits & _lib.QF_STATUS_NONFINITE)
        self._status_bits &= ~_lib.QF_STATUS_NONFINITE
        return seen

    # ---- capturable=True: a step of kernel launches only, every per-step scalar resident on the device ----------
    #
    # The reference reads the step count back to the host every step (adamw_fourbit_triton.py:458) and derives the
    # bias corrections there, so its step cannot be recorded into a CUDA graph.  Here the scalars of the coming
    # steps are derived once, on the host and in doubles exactly as `make_hyper` derives them one step at a time,
    # into a table on the device; a device counter picks the row, the step's last kernel advances it.  The table
    # ends where a row equals the one before it (constant learning rate, both bias corrections rounded to 1: after
    # 17 000 steps at beta2 = 0.999), which then repeats for ever; with at most `schedule_rows` rows otherwise.
    #
    # Use: run one step() eagerly (it builds the tables), capture step() into a torch.cuda.CUDAGraph, replay.
    # Gradients must live in the same buffers at every replay.  After changing a group's lr (or any other
    # hyper-parameter) call refresh_schedule() between replays; the recorded graph stays valid.

    def _cap_entries(self):
        entries, classes, class_of = [], [], {}
        dev = None
        for gi, group in enumerate(self.param_groups):
            for p in group["params"]:
                if p.grad is None:
                    continue
                if p.grad.is_sparse:
                    raise RuntimeError("QuantFour AdamW does not support sparse gradients")
                if not p.is_cuda:
                    raise RuntimeError("FourBitAdamW needs CUDA parameters; there is no CPU path")
                if not p.is_contiguous():
                    raise RuntimeError("param must be contiguous")
                if p.dtype not in _DTYPES:
                    raise TypeError(f"parameters must be float32, bfloat16 or float16, got {p.dtype}")
                g = p.grad
                if g.dtype != p.dtype or g.numel() != p.numel() or g.device != p.device:
                    raise RuntimeError("grad must match the parameter in dtype, numel and device")
                if not g.is_contiguous():
                    raise RuntimeError("capturable=True needs contiguous gradients (they must stay where they are)")
                if dev is None:
                    dev = p.device
                elif p.device != dev:
                    raise RuntimeError("capturable=True needs all parameters on one device")
                st = self.state[p]
                if len(st) == 0:
                    self._init_state(p)
                key = (gi, float(st["step"]))
                ci = class_of.get(key)
                if ci is None:
                    ci = class_of[key] = len(classes)
                    classes.append(key)
                entries.append((p, g, st, ci))
        if len(classes) > _lib.QF_MAX_HYPERS:
            raise RuntimeError(f"capturable=True supports at most {_lib.QF_MAX_HYPERS} (param group, step count) classes")
        return dev, entries, classes

    @staticmethod
    def _group_key(group) -> tuple:
        return (group["lr"], group["betas"][0], group["betas"][1], group["eps"], group["weight_decay"])

    def _cap_sync_steps(self) -> None:
        """Bring every state["step"] up to the device's count (synchronises)."""
        cap = self._cap
        if cap is None:
            return
        done = int(cap["counters"][1].item())
        if done != cap["synced"]:
            for (_, _, st, ci) in cap["entries"]:
                st["step"] = torch.tensor(cap["classes"][ci][1] + done)
            cap["synced"] = done

    def _cap_write_schedule(self, cap) -> None:
        """Rows of the coming steps for every class, from the classes' current step counts; counters := [0, 0]."""
        import numpy as np
        classes = cap["classes"]
        nc = len(classes)
        keys = [self._group_key(self.param_groups[gi]) for gi, _ in classes]
        rows: List[List[_lib.QfHyper]] = []
        prev = None
        stationary = False
        while len(rows) < self.schedule_rows:
            r = len(rows) + 1
            row = [make_hyper(*keys[c], classes[c][1] + r) for c in range(nc)]
            sig = b"".join(bytes(h) for h in row)
            rows.append(row)
            if sig == prev:
                stationary = True
                break
            prev = sig
        flat = (_lib.QfHyper * (len(rows) * nc))(*[h for row in rows for h in row])
        host = torch.from_numpy(np.frombuffer(flat, dtype=np.uint8).copy())
        table = cap.get("table")
        if table is None or table.numel() < host.numel():
            if table is not None and cap.get("captured"):
                raise RuntimeError("the new schedule does not fit the table a recorded graph points at; capture again")
            table = torch.empty(max(host.numel(), 4096), dtype=torch.uint8, device=cap["dev"])
        table[:host.numel()].copy_(host)
        cap["table"], cap["rows"], cap["stationary"] = table, len(rows), stationary
        cap["counters"].zero_()
        cap["synced"] = 0
        cap["group_keys"] = [self._group_key(g) for g in self.param_groups]

    def refresh_schedule(self) -> None:
        """Rewrite the device-resident scalars after a hyper-parameter of a group changed (call between graph
        replays, not while capturing).  Synchronises once to read the step count."""
        if not self.capturable or self._cap is None:
            return
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("refresh_schedule() cannot run while a graph is being captured")
        cap = self._cap
        self._cap_sync_steps()
        cap["classes"] = [(gi, t + cap["synced"]) for gi, t in cap["classes"]]
        self._cap_write_schedule(cap)

    def _cap_build(self) -> dict:
        self._cap_sync_steps()
        old = self._cap
        dev, entries, classes = self._cap_entries()
        if not entries:
            return {"entries": [], "dev": None}
        L = _lib.lib()
        plan = self._plans.setdefault((dev.index, 0), _DevicePlan())
        n = len(entries)
        descs = (_lib.QfTensorDesc * n)()
        for d, (p, g, st, ci) in zip(descs, entries):
            self._fill_desc(d, p, g, st, ci)
        need = L.qf_workspace_bytes(n)
        if plan.workspace is None or plan.workspace.numel() < need or plan.workspace.device != dev:
            plan.workspace = torch.zeros(need, dtype=torch.uint8, device=dev)
        plan.descs, plan.signature, plan.keepalive = descs, None, [g for _, g, _, _ in entries]
        stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        _lib.check(L.qf_step_prepare(descs, n, len(classes), plan.workspace.data_ptr(), plan.workspace.numel(), dev.index, stream),
                   "qf_step_prepare")
        cap = {
            "dev": dev, "plan": plan, "entries": entries, "classes": classes, "captured": False,
            "checks": [(p, p.data_ptr(), g.data_ptr()) for p, g, _, _ in entries],
            "absent": [p for g in self.param_groups for p in g["params"] if p.grad is None],
            "n_params": sum(len(g["params"]) for g in self.param_groups),
            "counters": torch.zeros(2, dtype=torch.int32, device=dev),
        }
        if old is not None and old.get("table") is not None and old["dev"] == dev and not old.get("captured"):
            cap["table"] = old["table"]
        self._cap_write_schedule(cap)
        return cap

    def _cap_same_tensors(self, cap):
        """True: same parameters and gradient buffers as when the tables were built; a list of (index, gradient): the
        same except that these gradients live in new buffers; False: anything else."""
        if not cap["entries"]:
            return all(p.grad is None for g in self.param_groups for p in g["params"])
        if cap["n_params"] != sum(len(g["params"]) for g in self.param_groups):
            return False
        moved = []
        for i, (p, pptr, gptr) in enumerate(cap["checks"]):
            g = p.grad
            if g is None or p.data_ptr() != pptr:
                return False
            if g.data_ptr() != gptr:
                if not g.is_contiguous() or g.dtype != p.dtype or g.numel() != p.numel() or g.is_sparse or g.device != p.device:
                    return False
                moved.append((i, g))
        for p in cap["absent"]:
            if p.grad is not None:
                return False
        return moved or True

    def _cap_move_grads(self, cap, moved) -> None:
        """New gradient buffers, everything else as before: only their addresses in the tensor table change."""
        plan, dev = cap["plan"], cap["dev"]
        for i, g in moved:
            plan.descs[i].g = g.data_ptr()
            plan.keepalive[i] = g
            cap["checks"][i] = (cap["checks"][i][0], cap["checks"][i][1], g.data_ptr())
        _lib.check(_lib.lib().qf_step_prepare(plan.descs, len(plan.descs), len(cap["classes"]), plan.workspace.data_ptr(),
                                              plan.workspace.numel(), dev.index, C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)),
                   "qf_step_prepare")

    def _step_capturable(self) -> None:
        if self._grad_scale != 1.0:
            raise RuntimeError("capturable=True does not take a per-step grad_scale (the scalars of a step are fixed "
                               "when the schedule is written)")
        capturing = torch.cuda.is_current_stream_capturing()
        cap = self._cap
        same_tensors = cap is not None and self._cap_same_tensors(cap)
        same_keys = bool(same_tensors) and (not cap["entries"] or cap["group_keys"] == [self._group_key(g) for g in self.param_groups])
        if not (same_tensors is True and same_keys):
            if capturing:
                raise RuntimeError("run one step() before capturing: the first step with these parameters, gradient "
                                   "buffers and hyper-parameters builds tables on the host and copies them to the device")
            if not same_tensors:
                self._cap = self._cap_build()
            else:
                if same_tensors is not True:
                    self._cap_move_grads(cap, same_tensors)
                if not same_keys:
                    self.refresh_schedule()     # only a hyper-parameter changed: same tables, new rows
            cap = self._cap
        if not cap["entries"]:
            return
        if capturing:
            cap["captured"] = True
        plan, dev = cap["plan"], cap["dev"]
        flags = _lib.QF_SCHED_TAIL_REPEATS if cap["stationary"] else 0
        rc = _lib.lib().qf_step_scheduled(plan.descs, len(plan.descs), len(cap["classes"]), plan.workspace.data_ptr(),
                                          plan.workspace.numel(), dev.index, C.c_void_p(torch.cuda.current_stream(dev).cuda_stream),
                                          C.c_void_p(cap["table"].data_ptr()), cap["rows"], C.c_void_p(cap["counters"].data_ptr()), flags)
        _lib.check(rc, "qf_step_scheduled")

    def schedule_exhausted(self) -> bool:
        """capturable=True: synchronise and report whether a step ran past the last row of a schedule whose last row
        does not repeat (more than `schedule_rows` steps without refresh_schedule() while the scalars still change)."""
        self._read_status()
        seen = bool(self._status_bits & _lib.QF_STATUS_SCHEDULE_END)
        self._status_bits &= ~_lib.QF_STATUS_SCHEDULE_END
        return seen

    def state_dict(self):
        """As torch's; with capturable=True the step counts are first read back from the device (synchronises)."""
        if self.capturable:
            self._cap_sync_steps()
        return super().state_dict()


# The reference spells the class three ways (fused_quantfour.py:12, :25; adamw_fourbit_triton.py:137).
AdamWFused_QuantFour = FourBitAdamW
AdamW_Fused_QuantFour = FourBitAdamW
AdamW_QuantFour = FourBitAdamW
