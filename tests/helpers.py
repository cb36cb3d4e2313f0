"""Shared helpers of the GPU parity tests: device-side twins of the oracle's tensor state and a thin
driver that calls the C ABI (qf_step_multi) on lists of them."""
from __future__ import annotations

import ctypes as C
import math
from typing import List, Optional

import torch

from oracle import torch_oracle as TO
from quantfour_adamw_cuda_b200 import _lib
from quantfour_adamw_cuda_b200.optimizer import make_hyper

KIND = {"fp32": _lib.QF_KIND_FP32, "block": _lib.QF_KIND_BLOCK, "rank1": _lib.QF_KIND_RANK1}
DTYPE = {torch.float32: _lib.QF_F32, torch.bfloat16: _lib.QF_BF16, torch.float16: _lib.QF_F16}


class GpuState:
    """Device copy of an oracle TensorState (same fields, CUDA tensors)."""

    def __init__(self, st: TO.TensorState, device="cuda"):
        self.kind, self.shape, self.step = st.kind, st.shape, st.step
        self.device = torch.device(device)
        self.load(st)
        if self.kind == "rank1":
            self.row_new = torch.zeros(2 * self.shape[0], device=device)
            self.col_new = torch.zeros(2 * self.shape[1], device=device)

    def load(self, st: TO.TensorState) -> None:
        """Overwrite the device state with the oracle's (teacher forcing)."""
        d = self.device
        self.step = st.step
        if self.kind == "fp32":
            self.m, self.v = st.m.to(d), st.v.to(d)
            return
        self.m_codes, self.v_codes = st.m_codes.to(d), st.v_codes.to(d)
        self.m_scale = st.m_scale.to(d)
        if self.kind == "rank1":
            self.v_row, self.v_col = st.v_row.to(d), st.v_col.to(d)
        else:
            self.v_scale = st.v_scale.to(d)

    def desc(self, p: torch.Tensor, g: torch.Tensor, hyper: int) -> _lib.QfTensorDesc:
        d = _lib.QfTensorDesc()
        d.p, d.g, d.numel = p.data_ptr(), g.data_ptr(), p.numel()
        d.kind, d.dtype, d.hyper = KIND[self.kind], DTYPE[p.dtype], hyper
        if self.kind == "fp32":
            d.m, d.v = self.m.data_ptr(), self.v.data_ptr()
            return d
        d.m, d.v, d.m_scale = self.m_codes.data_ptr(), self.v_codes.data_ptr(), self.m_scale.data_ptr()
        if self.kind == "rank1":
            d.rows, d.cols = self.shape
            d.v_scale, d.v_col = self.v_row.data_ptr(), self.v_col.data_ptr()
            d.v_row_new, d.v_col_new = self.row_new.data_ptr(), self.col_new.data_ptr()
        else:
            d.v_scale = self.v_scale.data_ptr()
        return d

    def diff(self, st: TO.TensorState) -> dict:
        """Counts of differing entries per field against an oracle state."""
        out = {}
        if self.kind == "fp32":
            out["m"] = int((self.m.cpu() != st.m).sum())
            out["v"] = int((self.v.cpu() != st.v).sum())
            return out
        n = math.prod(self.shape)
        cm, cv = TO.unpack(self.m_codes.cpu(), n).int(), TO.unpack(self.v_codes.cpu(), n).int()
        om, ov = TO.unpack(st.m_codes, n).int(), TO.unpack(st.v_codes, n).int()
        out["m_codes"] = int((cm != om).sum())
        out["v_codes"] = int((cv != ov).sum())
        out["max_code_dist"] = int(max((cm - om).abs().max(), (cv - ov).abs().max()))
        out["packed_bytes"] = int((self.m_codes.cpu() != st.m_codes).sum() + (self.v_codes.cpu() != st.v_codes).sum())
        out["m_scale"] = int((self.m_scale.cpu() != st.m_scale).sum())
        if self.kind == "rank1":
            out["v_row"] = int((self.v_row.cpu() != st.v_row).sum())
            out["v_col"] = int((self.v_col.cpu() != st.v_col).sum())
        else:
            out["v_scale"] = int((self.v_scale.cpu() != st.v_scale).sum())
        return out


class AbiStepper:
    """Calls qf_step_multi on a fixed list of (param, state) pairs."""

    def __init__(self, params: List[torch.Tensor], states: List[GpuState], lr=1e-3, betas=(0.9, 0.999), eps=1e-8,
                 weight_decay=1e-2):
        self.params, self.states = params, states
        self.hp = (lr, betas[0], betas[1], eps, weight_decay)
        self.L = _lib.lib()
        need = self.L.qf_workspace_bytes(len(params))
        self.ws = torch.zeros(need, dtype=torch.uint8, device=params[0].device)

    def step(self, grads: List[Optional[torch.Tensor]], split: bool = False) -> None:
        descs, hypers, hidx = [], [], {}
        keep = []
        for p, g, st in zip(self.params, grads, self.states):
            if g is None:
                continue
            st.step += 1
            if st.step not in hidx:
                hidx[st.step] = len(hypers)
                hypers.append(make_hyper(*self.hp, float(st.step)))
            keep.append(g)
            descs.append(st.desc(p, g, hidx[st.step]))
        arr = (_lib.QfTensorDesc * len(descs))(*descs)
        harr = (_lib.QfHyper * len(hypers))(*hypers)
        dev = self.params[0].device
        stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        args = (arr, len(descs), harr, len(hypers), self.ws.data_ptr(), self.ws.numel(), dev.index, stream)
        if split:
            _lib.check(self.L.qf_step_pre(*args), "qf_step_pre")
            _lib.check(self.L.qf_step_main(*args), "qf_step_main")
        else:
            _lib.check(self.L.qf_step_multi(*args), "qf_step_multi")

    def status(self) -> int:
        word = C.c_uint32(0)
        dev = self.params[0].device
        _lib.check(self.L.qf_read_status(self.ws.data_ptr(), dev.index,
                                         C.c_void_p(torch.cuda.current_stream(dev).cuda_stream), C.byref(word)),
                   "qf_read_status")
        return word.value


def make_grad(shape, dtype, sigma=1e-3, outliers=True, gen=None) -> torch.Tensor:
    g = torch.randn(shape, generator=gen) * sigma
    if outliers and g.numel() >= 1000:
        mask = torch.rand(shape, generator=gen) < 1e-3
        g = torch.where(mask, g * 100, g)
    return g.to(dtype)
