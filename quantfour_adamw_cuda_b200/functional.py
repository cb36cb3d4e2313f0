"""Tensor-level entry points over the C ABI.

``fused_4bit`` and ``fused_single_tensor`` keep the positional signatures of the reference's
extension module ``quantfour_cuda`` (optim/cuda_fused_interface.cc:19-25, :49-60, bound at :66-69)
so that code which called the module directly keeps working.  The quantize / dequantize functions
expose the pieces of the step (the reference describes them at optim/adamw_fourbit_triton.py:556-630,
:801-863, :497-546 but has no kernel for them).

Everything here requires CUDA tensors and the built shared library; nothing falls back to PyTorch.
"""
from __future__ import annotations

import ctypes as C
from typing import Tuple

import torch

from . import _lib

BLOCK = 128

_DTYPES = {torch.float32: _lib.QF_F32, torch.bfloat16: _lib.QF_BF16, torch.float16: _lib.QF_F16}


def _dtype_code(t: torch.Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise TypeError(f"parameters must be float32, bfloat16 or float16, got {t.dtype}") from None


def _need_cuda(*tensors: torch.Tensor) -> torch.device:
    dev = tensors[0].device
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError("quantfour_adamw_cuda_b200 needs CUDA tensors; there is no CPU path")
        if t.device != dev:
            raise RuntimeError("all tensors of one call must live on the same device")
        if not t.is_contiguous():
            raise RuntimeError("tensors must be contiguous")
    return dev


def _stream(dev: torch.device) -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


def _step_scalar(step) -> float:
    return float(step.item()) if torch.is_tensor(step) else float(step)


def fused_4bit(p, g, exp, sq, exp_scale, sq_scale, beta1, beta2, lr, weight_decay, eps, step) -> None:
    """One 4-bit AdamW step on one tensor, both moments with block-128 scales, in place.

    Same argument order as the reference's ``quantfour_cuda.fused_4bit``.  ``exp`` / ``sq`` are packed
    code buffers of ceil(numel/2) bytes (int8 or uint8), ``exp_scale`` / ``sq_scale`` fp32 tensors of
    ceil(numel/128) entries, ``step`` the step count after the increment (number or 0-dim tensor).
    """
    dev = _need_cuda(p, g, exp, sq, exp_scale, sq_scale)
    n = p.numel()
    if g.numel() != n or g.dtype != p.dtype:
        raise ValueError("grad must match the parameter in numel and dtype")
    nb, nblk = (n + 1) // 2, (n + BLOCK - 1) // BLOCK
    if exp.numel() != nb or sq.numel() != nb or exp.element_size() != 1 or sq.element_size() != 1:
        raise ValueError(f"code buffers must hold ceil(numel/2) = {nb} bytes")
    if exp_scale.numel() != nblk or sq_scale.numel() != nblk or exp_scale.dtype != torch.float32 or sq_scale.dtype != torch.float32:
        raise ValueError(f"scale buffers must be float32 with ceil(numel/128) = {nblk} entries")
    L = _lib.lib()
    _lib.check(L.qf_fused_4bit(p.data_ptr(), g.data_ptr(), exp.data_ptr(), sq.data_ptr(), exp_scale.data_ptr(),
                               sq_scale.data_ptr(), n, _dtype_code(p), float(beta1), float(beta2), float(lr),
                               float(weight_decay), float(eps), _step_scalar(step), dev.index, _stream(dev)),
               "fused_4bit")


def fused_single_tensor(p, g, exp_avg, exp_avg_sq, beta1, beta2, lr, weight_decay, eps, step) -> None:
    """One AdamW step on one tensor with fp32 moments, in place (``quantfour_cuda.fused_single_tensor``)."""
    dev = _need_cuda(p, g, exp_avg, exp_avg_sq)
    n = p.numel()
    if g.numel() != n or g.dtype != p.dtype:
        raise ValueError("grad must match the parameter in numel and dtype")
    for t in (exp_avg, exp_avg_sq):
        if t.numel() != n or t.dtype != torch.float32:
            raise ValueError("moments must be float32 tensors with the parameter's numel")
    L = _lib.lib()
    _lib.check(L.qf_fused_single_tensor(p.data_ptr(), g.data_ptr(), exp_avg.data_ptr(), exp_avg_sq.data_ptr(), n,
                                        _dtype_code(p), float(beta1), float(beta2), float(lr), float(weight_decay),
                                        float(eps), _step_scalar(step), dev.index, _stream(dev)),
               "fused_single_tensor")


def _quantize_block(x: torch.Tensor, which: int) -> Tuple[torch.Tensor, torch.Tensor]:
    dev = _need_cuda(x)
    if x.dtype != torch.float32:
        raise TypeError("stand-alone quantize takes float32 input")
    n = x.numel()
    codes = torch.empty((n + 1) // 2, dtype=torch.int8, device=dev)
    scales = torch.empty((n + BLOCK - 1) // BLOCK, dtype=torch.float32, device=dev)
    _lib.check(_lib.lib().qf_quantize_block(x.data_ptr(), n, which, codes.data_ptr(), scales.data_ptr(), dev.index,
                                            _stream(dev)), "quantize_block")
    return codes, scales


def _dequantize_block(codes: torch.Tensor, scales: torch.Tensor, numel: int, which: int) -> torch.Tensor:
    dev = _need_cuda(codes, scales)
    if codes.numel() != (numel + 1) // 2 or scales.numel() != (numel + BLOCK - 1) // BLOCK or scales.dtype != torch.float32:
        raise ValueError("codes / scales do not match numel")
    out = torch.empty(numel, dtype=torch.float32, device=dev)
    _lib.check(_lib.lib().qf_dequantize_block(codes.data_ptr(), scales.data_ptr(), numel, which, out.data_ptr(),
                                              dev.index, _stream(dev)), "dequantize_block")
    return out


def quantize_m(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """First-moment quantize: signed dynamic-exponent map, block-128 abs-max scales -> (codes, scales)."""
    return _quantize_block(x, 0)


def dequantize_m(codes: torch.Tensor, scales: torch.Tensor, numel: int) -> torch.Tensor:
    return _dequantize_block(codes, scales, numel, 0)


def quantize_v_block(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Second-moment quantize with block-128 scales (tensors that are not 2-D)."""
    return _quantize_block(x, 1)


def dequantize_v_block(codes: torch.Tensor, scales: torch.Tensor, numel: int) -> torch.Tensor:
    return _dequantize_block(codes, scales, numel, 1)


def quantize_v(v: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Second-moment quantize of a 2-D tensor: unsigned linear map without zero, rank-1 scale
    min(row_max[i], col_max[j]) -> (codes, row_max [R], col_max [C])."""
    dev = _need_cuda(v)
    if v.dim() != 2 or v.dtype != torch.float32:
        raise TypeError("quantize_v takes a 2-D float32 tensor")
    R, Cc = v.shape
    codes = torch.empty((R * Cc + 1) // 2, dtype=torch.int8, device=dev)
    row = torch.empty(R, dtype=torch.float32, device=dev)
    col = torch.empty(Cc, dtype=torch.float32, device=dev)
    _lib.check(_lib.lib().qf_quantize_rank1(v.data_ptr(), R, Cc, codes.data_ptr(), row.data_ptr(), col.data_ptr(),
                                            dev.index, _stream(dev)), "quantize_rank1")
    return codes, row, col


def dequantize_v(codes: torch.Tensor, row: torch.Tensor, col: torch.Tensor) -> torch.Tensor:
    dev = _need_cuda(codes, row, col)
    R, Cc = row.numel(), col.numel()
    if codes.numel() != (R * Cc + 1) // 2 or row.dtype != torch.float32 or col.dtype != torch.float32:
        raise ValueError("codes / maxima do not match")
    out = torch.empty(R, Cc, dtype=torch.float32, device=dev)
    _lib.check(_lib.lib().qf_dequantize_rank1(codes.data_ptr(), row.data_ptr(), col.data_ptr(), R, Cc, out.data_ptr(),
                                              dev.index, _stream(dev)), "dequantize_rank1")
    return out
