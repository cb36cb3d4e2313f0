"""CPU stand-in for the two halves of the sharded step (test infrastructure).

Implements, with the oracle's torch operators, what qf_step_pre / qf_step_main do for one rank's records,
so that partitioning, the max exchange and the all-gather of ShardedFourBitAdamW can run as gloo ranks on
CPU.  The shipped optimizer never imports this file.
"""
from __future__ import annotations

import torch

from oracle import torch_oracle as TO
from quantfour_adamw_cuda_b200.zero1 import BLOCKQ, FP32, RANK1


def _hyper(h) -> TO.Hyper:
    return TO.Hyper(h.decay, h.w1, h.beta2, h.w2, h.eps, h.neg_step, h.bc2s)


def _index(st):
    """Row / column index of every element of a rank-1 record inside the buffers the record sees."""
    r = st.rec
    e = torch.arange(r.numel) + (r.flat_offset if r.partial else 0)
    return e // r.cols, e % r.cols


def _v_new(st, h):
    rows, cols = _index(st)
    n = st.rec.numel
    v_old = TO.QV[TO.unpack(st.v.view(torch.uint8), n).long()].mul(torch.min(st.v_scale[rows], st.v_col[cols]))
    g32 = st.g.float()
    return v_old.mul_(h.beta2).addcmul_(g32, g32, value=h.w2), rows, cols


class CpuBackend:
    def pre(self, states, hyper):
        h = _hyper(hyper)
        for st in states:
            if st.rec.kind != RANK1:
                continue
            st.row_new.zero_()
            st.col_new.zero_()
        for st in states:
            if st.rec.kind != RANK1:
                continue
            v, rows, cols = _v_new(st, h)
            st.row_new.index_reduce_(0, rows, v, "amax", include_self=True)
            st.col_new.index_reduce_(0, cols, v, "amax", include_self=True)

    def main(self, states, hyper):
        h = _hyper(hyper)
        for st in states:
            r, n = st.rec, st.rec.numel
            p32, g32 = st.p.float().clone(), st.g.float()
            if r.kind == FP32:
                TO.adamw_update_(p32, g32, st.m, st.v, h)
                st.p.copy_(p32)
                continue
            m = TO.dequantize_block(st.m.view(torch.uint8), st.m_scale, n, TO.QM)
            if r.kind == BLOCKQ:
                v = TO.dequantize_block(st.v.view(torch.uint8), st.v_scale, n, TO.QV)
            else:
                rows, cols = _index(st)
                v = TO.QV[TO.unpack(st.v.view(torch.uint8), n).long()].mul(torch.min(st.v_scale[rows], st.v_col[cols]))
            TO.adamw_update_(p32, g32, m, v, h)
            st.p.copy_(p32)
            mc, ms = TO.quantize_block(m, TO.MM)
            st.m.view(torch.uint8).copy_(mc)
            st.m_scale.copy_(ms)
            if r.kind == BLOCKQ:
                vc, vs = TO.quantize_block(v, TO.MV)
                st.v.view(torch.uint8).copy_(vc)
                st.v_scale.copy_(vs)
            else:
                scale = torch.min(st.row_new[rows], st.col_new[cols])
                st.v.view(torch.uint8).copy_(TO.pack(TO.codes_of(TO._safe_div(v, scale), TO.MV)))
        for st in states:            # commit the new maxima once every record of the rank has used the old ones
            if st.rec.kind == RANK1:
                st.v_scale.copy_(st.row_new)
                st.v_col.copy_(st.col_new)
