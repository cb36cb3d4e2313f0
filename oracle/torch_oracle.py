"""CPU oracle, torch-ops form -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Restates the reference's pure-PyTorch 4-bit AdamW step with the same torch operators the
reference calls, vectorised (``torch.bucketize`` over the 15 midpoints in place of the
reference's per-element Python search).  Everything here runs on CPU tensors; the shipped
optimizer never imports this module.

Reference lines followed (paths inside the reference project):
  op order of one step ........ optim/adamw_fourbit_triton.py:412-473
  tables ...................... optim/adamw_fourbit_triton.py:16-97
  search, tie -> lower code ... optim/adamw_fourbit_triton.py:1020-1047
  block-128 abs-max scaling ... optim/adamw_fourbit_triton.py:618-630, grouping :633-649
  rank-1 scaling .............. optim/adamw_fourbit_triton.py:738-755, :834-863
  dequantize = qmap[c]*scale .. optim/adamw_fourbit_triton.py:515-528
  nibble order ................ optim/cuda_adamw_kernels.cu:295-296, :329, :358
  size threshold .............. optim/fused_quantfour.py:18-22, optim/adamw_fourbit_triton.py:118

Pinning: see the header of oracle/qf_oracle.c -- tables, search and the first step from zero
state are checked against the reference's own functions through tests/golden/.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional

import torch

BLOCK = 128
THRESHOLD = 4096

QM = torch.tensor([-0.8875, -0.6625, -0.4375, -0.2125, -0.0775, -0.0325, -0.0055, 0.0,
                   0.0055, 0.0325, 0.0775, 0.2125, 0.4375, 0.6625, 0.8875, 1.0], dtype=torch.float32)
MM = torch.tensor([-0.775, -0.55, -0.325, -0.145, -0.055, -0.019, -0.00275, 0.00275,
                   0.019, 0.055, 0.145, 0.325, 0.55, 0.775, 0.94375], dtype=torch.float32)
QV = torch.tensor([0.0625 * k for k in range(1, 17)], dtype=torch.float32)
MV = torch.tensor([0.09375 + 0.0625 * k for k in range(15)], dtype=torch.float32)


@dataclass
class Hyper:
    """Scalars of one step, derived in Python doubles (adamw_fourbit_triton.py:415, :458-465)."""
    decay: float
    w1: float
    beta2: float
    w2: float
    eps: float
    neg_step: float
    bc2s: float

    @staticmethod
    def make(lr: float, beta1: float, beta2: float, eps: float, weight_decay: float, step: int) -> "Hyper":
        bc1 = 1 - beta1 ** step
        bc2 = 1 - beta2 ** step
        return Hyper(decay=1 - lr * weight_decay, w1=1 - beta1, beta2=beta2, w2=1 - beta2, eps=eps,
                     neg_step=-(lr / bc1), bc2s=math.sqrt(bc2))


def codes_of(x: torch.Tensor, mid: torch.Tensor) -> torch.Tensor:
    """Number of midpoints strictly below x == the reference search incl. its end clamps."""
    return torch.bucketize(x, mid, right=False).to(torch.uint8)


def pack(codes: torch.Tensor) -> torch.Tensor:
    """Element 2j -> low nibble of byte j, element 2j+1 -> high nibble; odd tail nibble = 0."""
    c = codes.reshape(-1)
    if c.numel() % 2:
        c = torch.cat([c, torch.zeros(1, dtype=torch.uint8)])
    c = c.view(-1, 2)
    return (c[:, 0] | (c[:, 1] << 4)).contiguous()


def unpack(packed: torch.Tensor, numel: int) -> torch.Tensor:
    b = packed.view(torch.uint8).reshape(-1)
    out = torch.stack([b & 15, b >> 4], dim=1).reshape(-1)
    return out[:numel]


def group128(x: torch.Tensor) -> torch.Tensor:
    """Flatten, zero-pad to a multiple of 128, view as [-1, 128] (adamw_fourbit_triton.py:633-649)."""
    f = x.reshape(-1)
    pad = (-f.numel()) % BLOCK
    if pad:
        f = torch.cat([f, torch.zeros(pad, dtype=f.dtype)])
    return f.view(-1, BLOCK)


def _safe_div(x: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    """x.div(s) with the all-zero-group rule: a zero scale yields x = 0."""
    return torch.where(s == 0, torch.zeros((), dtype=x.dtype), x.div(s))


def quantize_block(x: torch.Tensor, mid: torch.Tensor):
    """Block-128 abs-max quantize (adamw_fourbit_triton.py:618-630). Returns (packed uint8, scales[nblk])."""
    n = x.numel()
    gx = group128(x.float())
    max1 = gx.abs().max(dim=1, keepdim=True).values
    codes = codes_of(_safe_div(gx, max1), mid).reshape(-1)[:n]
    return pack(codes), max1.reshape(-1).clone()


def dequantize_block(packed: torch.Tensor, scales: torch.Tensor, numel: int, qmap: torch.Tensor) -> torch.Tensor:
    c = unpack(packed, numel).long()
    s = scales.reshape(-1, 1).expand(-1, BLOCK).reshape(-1)[:numel]
    return qmap[c].mul(s)


def rank1_stats(v: torch.Tensor):
    """Per-axis maxima of |v| (adamw_fourbit_triton.py:738-746 with :1078-1087): row [R,1], col [1,C]."""
    a = v.abs()
    return a.max(dim=1, keepdim=True).values, a.max(dim=0, keepdim=True).values


def quantize_rank1(v: torch.Tensor):
    """Rank-1 quantize of a 2-D tensor (adamw_fourbit_triton.py:834-863). Returns (packed, row[R], col[C])."""
    row, col = rank1_stats(v)
    st = torch.min(row, col)
    codes = codes_of(_safe_div(v, st), MV)
    return pack(codes), row.reshape(-1).clone(), col.reshape(-1).clone()


def dequantize_rank1(packed: torch.Tensor, row: torch.Tensor, col: torch.Tensor, R: int, C: int) -> torch.Tensor:
    c = unpack(packed, R * C).long().view(R, C)
    return QV[c].mul(torch.min(row.view(R, 1), col.view(1, C)))


def axis_stats(v: torch.Tensor):
    """One vector of maxima of |v| per axis, each over all the other axes (adamw_fourbit_triton.py:738-746 with
    :1078-1087), shaped for broadcasting: [d0,1,..], [1,d1,1,..], ..."""
    a = v.abs()
    out = []
    for k in range(a.dim()):
        r = a
        for d in range(a.dim()):
            if d != k:
                r = r.max(dim=d, keepdim=True).values
        out.append(r)
    return out


def axis_scale(stats) -> torch.Tensor:
    """The scale of every element: the smallest of its axes' maxima (adamw_fourbit_triton.py:749-755, :540-546)."""
    st = stats[0].clone()
    for s in stats[1:]:
        st = torch.min(st, s)
    return st


def quantize_rank1_nd(v: torch.Tensor):
    """Rank-1 quantize of a tensor of any rank >= 2 (adamw_fourbit_triton.py:846-856). Returns (packed, [axis maxima])."""
    stats = axis_stats(v)
    codes = codes_of(_safe_div(v, axis_scale(stats)), MV)
    return pack(codes), [s.reshape(-1).clone() for s in stats]


def dequantize_rank1_nd(packed: torch.Tensor, axes, shape) -> torch.Tensor:
    n = math.prod(shape)
    c = unpack(packed, n).long().view(shape)
    stats = [a.view([-1 if d == k else 1 for d in range(len(shape))]) for k, a in enumerate(axes)]
    return QV[c].mul(axis_scale(stats))


def adamw_update_(p32: torch.Tensor, g32: torch.Tensor, m: torch.Tensor, v: torch.Tensor, h: Hyper) -> None:
    """The reference's update lines, operator for operator (adamw_fourbit_triton.py:415, :455-473)."""
    p32.mul_(h.decay)
    m.lerp_(g32, h.w1)
    v.mul_(h.beta2).addcmul_(g32, g32, value=h.w2)
    # IEEE square root.  torch's CPU float32 sqrt of a large contiguous tensor goes through a vendor
    # vector-math routine that is off by one ulp on ~0.7 % of inputs (measured on torch 2.11 + MKL); the
    # reference's own device computes a correctly rounded sqrt, so the oracle takes it through float64
    # (exact after rounding back: 53 >= 2*24 + 2).
    denom = (v.double().sqrt().float() / h.bc2s).add_(h.eps)
    p32.addcdiv_(m, denom, value=h.neg_step)


@dataclass
class TensorState:
    """Optimizer state of one tensor as the oracle keeps it."""
    kind: str                      # "rank1" | "rank1nd" (rank >= 3 with per-axis maxima: an option) | "block" | "fp32"
    shape: tuple
    step: int = 0
    m_codes: Optional[torch.Tensor] = None   # uint8 [ceil(n/2)]
    v_codes: Optional[torch.Tensor] = None
    m_scale: Optional[torch.Tensor] = None   # fp32 [ceil(n/128)]
    v_scale: Optional[torch.Tensor] = None   # block kind: fp32 [ceil(n/128)]
    v_row: Optional[torch.Tensor] = None     # rank1 kind: fp32 [R]
    v_col: Optional[torch.Tensor] = None     # rank1 kind: fp32 [C]
    v_axes: Optional[List[torch.Tensor]] = None   # rank1nd kind: one fp32 vector of maxima per axis
    m: Optional[torch.Tensor] = None         # fp32 kind
    v: Optional[torch.Tensor] = None

    @staticmethod
    def zeros(shape, threshold: int = THRESHOLD, nd_rank1: bool = False) -> "TensorState":
        shape = tuple(shape)
        n = math.prod(shape) if shape else 1
        if n <= threshold:      # optim/fused_quantfour.py:18-22
            return TensorState("fp32", shape, m=torch.zeros(n), v=torch.zeros(n))
        nb, nblk = (n + 1) // 2, (n + BLOCK - 1) // BLOCK
        kind = "rank1" if len(shape) == 2 else "rank1nd" if nd_rank1 and len(shape) > 2 else "block"
        st = TensorState(kind, shape,
                         m_codes=torch.zeros(nb, dtype=torch.uint8), v_codes=torch.zeros(nb, dtype=torch.uint8),
                         m_scale=torch.zeros(nblk))
        if st.kind == "rank1":
            st.v_row, st.v_col = torch.zeros(shape[0]), torch.zeros(shape[1])
        elif st.kind == "rank1nd":
            st.v_axes = [torch.zeros(d) for d in shape]
        else:
            st.v_scale = torch.zeros(nblk)
        return st

    def dequantized(self):
        """(m, v) as flat fp32 tensors."""
        n = math.prod(self.shape) if self.shape else 1
        if self.kind == "fp32":
            return self.m.clone(), self.v.clone()
        m = dequantize_block(self.m_codes, self.m_scale, n, QM)
        if self.kind == "rank1":
            v = dequantize_rank1(self.v_codes, self.v_row, self.v_col, *self.shape).reshape(-1)
        elif self.kind == "rank1nd":
            v = dequantize_rank1_nd(self.v_codes, self.v_axes, self.shape).reshape(-1)
        else:
            v = dequantize_block(self.v_codes, self.v_scale, n, QV)
        return m, v


def step_tensor(p: torch.Tensor, g: torch.Tensor, st: TensorState, lr: float, beta1: float, beta2: float, eps: float,
                weight_decay: float) -> None:
    """One optimizer step on one tensor, in place on ``p`` and ``st``.

    bf16 params/grads are widened to fp32 exactly, the step runs in fp32 and the new param is rounded
    to bf16 (nearest even); the states and scales are always fp32.
    """
    st.step += 1
    h = Hyper.make(lr, beta1, beta2, eps, weight_decay, st.step)
    n = p.numel()
    p32 = p.detach().float().reshape(-1).clone()
    g32 = g.detach().float().reshape(-1)
    m, v = st.dequantized()
    adamw_update_(p32, g32, m, v, h)
    p.detach().reshape(-1).copy_(p32)
    if st.kind == "fp32":
        st.m, st.v = m, v
        return
    st.m_codes, st.m_scale = quantize_block(m, MM)
    if st.kind == "rank1":
        st.v_codes, st.v_row, st.v_col = quantize_rank1(v.view(st.shape))
    elif st.kind == "rank1nd":
        st.v_codes, st.v_axes = quantize_rank1_nd(v.view(st.shape))
    else:
        st.v_codes, st.v_scale = quantize_block(v, MV)
    assert st.m_codes.numel() == (n + 1) // 2


@dataclass
class OracleAdamW:
    """Minimal multi-tensor driver around step_tensor with the reference constructor's hyper-parameters."""
    params: List[torch.Tensor]
    lr: float = 1e-3
    betas: tuple = (0.9, 0.999)
    eps: float = 1e-8
    weight_decay: float = 1e-2
    threshold: int = THRESHOLD
    states: List[TensorState] = field(default_factory=list)

    def __post_init__(self):
        self.states = [TensorState.zeros(p.shape, self.threshold) for p in self.params]

    def step(self, grads: List[Optional[torch.Tensor]]) -> None:
        for p, g, st in zip(self.params, grads, self.states):
            if g is None:
                continue
            step_tensor(p, g, st, self.lr, self.betas[0], self.betas[1], self.eps, self.weight_decay)
