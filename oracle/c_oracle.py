"""ctypes front-end of the C oracle (oracle/qf_oracle.c) -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Operates in place on contiguous CPU torch tensors.  The library is built on demand by
oracle/build_oracle.py.  It is the explicit-rounding twin of oracle/torch_oracle.py; the two are
required to agree bit for bit by the CPU test-suite, and it is what the benchmark times as the
CPU baseline (all host threads through OpenMP).
"""
from __future__ import annotations

import ctypes as C
import math

import torch

from . import build_oracle
from .torch_oracle import Hyper, TensorState

_lib = None


class _Hyper(C.Structure):
    _fields_ = [(n, C.c_float) for n in ("decay", "w1", "beta2", "w2", "eps", "neg_step", "bc2s", "pad")]


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(build_oracle.build())
        _lib.qfo_num_threads.restype = C.c_int
    return _lib


def _ptr(t: torch.Tensor):
    assert t.device.type == "cpu" and t.is_contiguous()
    return C.c_void_p(t.data_ptr())


def _dtype_code(t: torch.Tensor) -> int:
    return {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}[t.dtype]


def _h(h: Hyper) -> _Hyper:
    return _Hyper(h.decay, h.w1, h.beta2, h.w2, h.eps, h.neg_step, h.bc2s, 0.0)


def num_threads() -> int:
    return lib().qfo_num_threads()


def set_threads(n: int) -> None:
    lib().qfo_set_threads(C.c_int(n))


def tables():
    out = [torch.empty(16), torch.empty(15), torch.empty(16), torch.empty(15)]
    lib().qfo_tables(*[_ptr(t) for t in out])
    return out


def search(x: torch.Tensor, which: int, literal: bool = False) -> torch.Tensor:
    x = x.float().contiguous()
    out = torch.empty(x.numel(), dtype=torch.uint8)
    lib().qfo_search(_ptr(x), C.c_int64(x.numel()), C.c_int(which), C.c_int(int(literal)), _ptr(out))
    return out


def quantize_block(x: torch.Tensor, which: int):
    x = x.float().contiguous().reshape(-1)
    n = x.numel()
    packed = torch.empty((n + 1) // 2, dtype=torch.uint8)
    scales = torch.empty((n + 127) // 128)
    lib().qfo_quantize_block(_ptr(x), C.c_int64(n), C.c_int(which), _ptr(packed), _ptr(scales))
    return packed, scales


def dequantize_block(packed, scales, n: int, which: int):
    out = torch.empty(n)
    lib().qfo_dequantize_block(_ptr(packed), _ptr(scales), C.c_int64(n), C.c_int(which), _ptr(out))
    return out


def quantize_rank1(v: torch.Tensor):
    v = v.float().contiguous()
    R, Cc = v.shape
    packed = torch.empty((R * Cc + 1) // 2, dtype=torch.uint8)
    row, col = torch.empty(R), torch.empty(Cc)
    lib().qfo_quantize_rank1(_ptr(v), C.c_int64(R), C.c_int64(Cc), _ptr(packed), _ptr(row), _ptr(col))
    return packed, row, col


def dequantize_rank1(packed, row, col, R: int, Cc: int):
    out = torch.empty(R, Cc)
    lib().qfo_dequantize_rank1(_ptr(packed), _ptr(row), _ptr(col), C.c_int64(R), C.c_int64(Cc), _ptr(out))
    return out


def step_tensor(p: torch.Tensor, g: torch.Tensor, st: TensorState, lr, beta1, beta2, eps, weight_decay) -> None:
    """Same contract as torch_oracle.step_tensor, computed by the C library."""
    if st.kind == "rank1nd":     # per-axis maxima over more than two axes: the torch restatement only
        from . import torch_oracle as TO
        return TO.step_tensor(p, g, st, lr, beta1, beta2, eps, weight_decay)
    st.step += 1
    h = _h(Hyper.make(lr, beta1, beta2, eps, weight_decay, st.step))
    n = p.numel()
    g = g.contiguous()
    assert p.is_contiguous() and g.dtype == p.dtype
    dt = C.c_int(_dtype_code(p))
    L = lib()
    if st.kind == "fp32":
        L.qfo_step_fp32(_ptr(p), _ptr(g), dt, _ptr(st.m), _ptr(st.v), C.c_int64(n), C.byref(h))
    elif st.kind == "block":
        L.qfo_step_block(_ptr(p), _ptr(g), dt, _ptr(st.m_codes), _ptr(st.v_codes), _ptr(st.m_scale),
                         _ptr(st.v_scale), C.c_int64(n), C.byref(h))
    else:
        R, Cc = st.shape
        L.qfo_step_rank1(_ptr(p), _ptr(g), dt, _ptr(st.m_codes), _ptr(st.v_codes), _ptr(st.m_scale),
                         _ptr(st.v_row), _ptr(st.v_col), C.c_int64(R), C.c_int64(Cc), C.byref(h))
