"""ctypes binding of libquantfour_b200.so (declared in include/quantfour_b200.h).

There is no CPU or PyTorch fallback: if the shared library is missing or a call fails, an exception
is raised.  The library is built in-tree by ``python -m quantfour_adamw_cuda_b200.build``.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libquantfour_b200.so")

QF_ABI_VERSION = 5
QF_MAX_HYPERS = 16
QF_MAX_PEERS = 15
QF_PEER_HANDLE_BYTES = 64
QF_F32, QF_BF16, QF_F16 = 0, 1, 2
QF_KIND_FP32, QF_KIND_BLOCK, QF_KIND_RANK1 = 0, 1, 2
QF_STATUS_NONFINITE = 1
QF_STATUS_SCHEDULE_END = 2
QF_RUN_PRE, QF_RUN_MAIN, QF_RUN_TABLE_IN_PLACE, QF_RUN_RELAXED_UPDATE = 1, 2, 4, 8
QF_SCHED_TAIL_REPEATS = 1
QF_SCHED_GRAD_SCALE = 2
QF_NOALLOC_MAX_ROWS_PLUS_COLS = 131072


class QfHyper(C.Structure):
    _fields_ = [(n, C.c_float) for n in ("decay", "w1", "beta2", "w2", "eps", "neg_step", "bc2s", "grad_scale")]


class QfTensorDesc(C.Structure):
    _fields_ = [
        ("p", C.c_void_p), ("g", C.c_void_p), ("m", C.c_void_p), ("v", C.c_void_p),
        ("m_scale", C.c_void_p), ("v_scale", C.c_void_p), ("v_col", C.c_void_p),
        ("v_row_new", C.c_void_p), ("v_col_new", C.c_void_p), ("v_row_rcp", C.c_void_p), ("v_col_rcp", C.c_void_p),
        ("numel", C.c_int64), ("rows", C.c_int64), ("cols", C.c_int64), ("flat_offset", C.c_int64),
        ("kind", C.c_int32), ("dtype", C.c_int32), ("hyper", C.c_int32), ("partial", C.c_int32),
    ]


assert C.sizeof(QfTensorDesc) == 136 and C.sizeof(QfHyper) == 32

_STEP_ARGS = [C.POINTER(QfTensorDesc), C.c_int, C.POINTER(QfHyper), C.c_int, C.c_void_p, C.c_size_t, C.c_int, C.c_void_p]
_SCALARS = [C.c_double] * 6

_SIGNATURES = {
    "qf_abi_version": (C.c_int, []),
    "qf_last_error": (C.c_char_p, []),
    "qf_workspace_bytes": (C.c_size_t, [C.c_int]),
    "qf_step_multi": (C.c_int, _STEP_ARGS),
    "qf_step_run": (C.c_int, _STEP_ARGS + [C.c_int, C.POINTER(C.c_int64), C.c_int]),
    "qf_step_pre": (C.c_int, _STEP_ARGS),
    "qf_step_main": (C.c_int, _STEP_ARGS),
    "qf_step_prepare": (C.c_int, [C.POINTER(QfTensorDesc), C.c_int, C.c_int, C.c_void_p, C.c_size_t, C.c_int, C.c_void_p]),
    "qf_step_scheduled": (C.c_int, [C.POINTER(QfTensorDesc), C.c_int, C.c_int, C.c_void_p, C.c_size_t, C.c_int, C.c_void_p,
                                    C.c_void_p, C.c_int, C.c_void_p, C.c_int]),
    "qf_step_main_push": (C.c_int, _STEP_ARGS + [C.POINTER(C.c_int64), C.c_int]),
    "qf_peer_export": (C.c_int, [C.c_void_p, C.c_int, C.c_char_p, C.POINTER(C.c_int64)]),
    "qf_peer_open": (C.c_int, [C.c_char_p, C.c_int, C.POINTER(C.c_void_p)]),
    "qf_peer_close": (C.c_int, [C.c_void_p, C.c_int]),
    "qf_peer_copy": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_size_t, C.c_int, C.c_void_p]),
    "qf_grad_mean_peers": (C.c_int, [C.c_void_p, C.c_int64, C.c_int, C.POINTER(C.c_int64), C.c_int, C.c_float, C.c_int, C.c_void_p]),
    "qf_read_status": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.POINTER(C.c_uint32)]),
    "qf_release_workspace": (C.c_int, [C.c_void_p, C.c_int]),
    "qf_read_status_noalloc": (C.c_int, [C.c_int, C.c_void_p, C.POINTER(C.c_uint32)]),
    "qf_fused_4bit": (C.c_int, [C.c_void_p] * 6 + [C.c_int64, C.c_int] + _SCALARS + [C.c_int, C.c_void_p]),
    "qf_fused_single_tensor": (C.c_int, [C.c_void_p] * 4 + [C.c_int64, C.c_int] + _SCALARS + [C.c_int, C.c_void_p]),
    "qf_make_hyper": (None, _SCALARS + [C.POINTER(QfHyper)]),
    "qf_quantize_block": (C.c_int, [C.c_void_p, C.c_int64, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "qf_dequantize_block": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_void_p, C.c_int, C.c_void_p]),
    "qf_quantize_rank1": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "qf_step_rank1_noalloc": (C.c_int, [C.c_void_p] * 7 + [C.c_int64, C.c_int64, C.c_int, C.POINTER(QfHyper), C.c_int, C.c_void_p]),
    "qf_dequantize_rank1": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_int, C.c_void_p]),
}

EXPORTS = tuple(_SIGNATURES)

_lib = None


class QuantFourError(RuntimeError):
    """A call into libquantfour_b200.so failed."""


def lib() -> C.CDLL:
    """Load the shared library (once).  Raises if it has not been built: there is no fallback path."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise QuantFourError(
                f"{LIB_PATH} is missing: build it with `python -m quantfour_adamw_cuda_b200.build` "
                "(needs nvcc with sm_100a support). There is no CPU or PyTorch fallback.")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        if handle.qf_abi_version() != QF_ABI_VERSION:
            raise QuantFourError(f"ABI mismatch: library {handle.qf_abi_version()}, binding {QF_ABI_VERSION}")
        _lib = handle
    return _lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = lib().qf_last_error().decode(errors="replace")
        if rc == 1:
            raise ValueError(f"{what}: {msg}")
        raise QuantFourError(f"{what} failed with status {rc}: {msg}")
