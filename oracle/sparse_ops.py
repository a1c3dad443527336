"""ORACLE (test infrastructure, never imported by the product path).

CPU restatement of the reference's batched sparse-dense products, written with
plain PyTorch tensor ops so that autograd supplies first and higher order
gradients for free.  Each function follows the semantics of the reference's own
CPU code:

* ``indexed_mul_scale_gather``     equitorch/ops/batched_sparse_dense_op.py:234-275
* ``indexed_outer_scale_gather``   :515-556
* ``indexed_inner_scale_gather``   :790-831
* ``indexed_vecmat_scale_gather``  :1461-1509
* ``indexed_vecsca_scale_gather``  :1752-1794
* ``indexed_scavec_scale_gather`` / ``indexed_mat_t_vec_scale_gather``: argument-swapping
  aliases, :994-1035 and :1200-1238
* ``indexed_scale_segment``        equitorch/ops/indexed_scale_segment_op.py:143-170

Common contract: operand rows are gathered with ``index1`` / ``index2`` (``None`` =
identity), combined per table entry, multiplied by ``scale``, optionally re-gathered
with ``gather_index``, summed over CSR segments ``seg``, optionally scattered to
``index_out`` rows of an ``out_size`` output, and summed over the batch when
``out_accumulated``.  An operand with one dimension fewer than its batched form is
shared by the whole batch.

Pinned against outputs of the reference itself (fixtures under tests/golden made by
tests/golden/make_golden.py).
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor


def _segment_sum(t: Tensor, seg: Tensor, dim: int) -> Tensor:
    """Sum consecutive slices ``[seg[i], seg[i+1])`` of ``t`` along ``dim``."""
    dim = dim % t.dim()
    counts = (seg[1:] - seg[:-1]).to(torch.long)
    owner = torch.repeat_interleave(torch.arange(counts.numel(), device=t.device), counts)
    shape = list(t.shape)
    shape[dim] = counts.numel()
    src = t.narrow(dim, int(seg[0]), int(seg[-1] - seg[0]))
    return t.new_zeros(shape).index_add(dim, owner, src)


def _finish(inter: Tensor, sparse_dim: int, scale, seg, gather_index, index_out, out_size, out_accumulated):
    sparse_dim = sparse_dim % inter.dim()
    if scale is not None:
        view = [1] * inter.dim()
        view[sparse_dim] = -1
        inter = inter * scale.view(view)
    if seg is not None:
        if gather_index is not None:
            inter = inter.index_select(sparse_dim, gather_index)
        inter = _segment_sum(inter, seg, sparse_dim)
    if index_out is not None:
        shape = list(inter.shape)
        shape[sparse_dim] = out_size
        inter = inter.new_zeros(shape).index_add(sparse_dim, index_out, inter)
    if out_accumulated:
        inter = inter.sum(dim=0)
    return inter


def _sel(t: Tensor, index: Optional[Tensor], dim: int) -> Tensor:
    return t if index is None else t.index_select(dim, index)


def indexed_mul_scale_gather(input1, input2, scale=None, index1=None, index2=None, seg=None,
                             gather_index=None, index_out=None, out=None, out_accumulated=False,
                             out_size=None, **_):
    inter = _sel(input1, index1, -2) * _sel(input2, index2, -2)
    return _finish(inter, -2, scale, seg, gather_index, index_out, out_size, out_accumulated)


def indexed_outer_scale_gather(input1, input2, scale=None, index1=None, index2=None, seg=None,
                               gather_index=None, index_out=None, out=None, out_accumulated=False,
                               out_size=None, **_):
    inter = _sel(input1, index1, -2).unsqueeze(-1) * _sel(input2, index2, -2).unsqueeze(-2)
    return _finish(inter, -3, scale, seg, gather_index, index_out, out_size, out_accumulated)


def indexed_inner_scale_gather(input1, input2, scale=None, index1=None, index2=None, seg=None,
                               gather_index=None, index_out=None, out=None, out_accumulated=False,
                               out_size=None, **_):
    inter = (_sel(input1, index1, -2) * _sel(input2, index2, -2)).sum(dim=-1)
    return _finish(inter, -1, scale, seg, gather_index, index_out, out_size, out_accumulated)


def indexed_vecmat_scale_gather(input1, input2, scale=None, index1=None, index2=None, seg=None,
                                gather_index=None, index_out=None, out=None, out_accumulated=False,
                                out_size=None, **_):
    inter = torch.einsum("...ti,...tij->...tj", _sel(input1, index1, -2), _sel(input2, index2, -3))
    return _finish(inter, -2, scale, seg, gather_index, index_out, out_size, out_accumulated)


def indexed_vecsca_scale_gather(input1, input2, scale=None, index1=None, index2=None, seg=None,
                                gather_index=None, index_out=None, out=None, out_accumulated=False,
                                out_size=None, **_):
    inter = _sel(input1, index1, -2) * _sel(input2, index2, -1).unsqueeze(-1)
    return _finish(inter, -2, scale, seg, gather_index, index_out, out_size, out_accumulated)


def indexed_scavec_scale_gather(input1, input2, scale=None, index1=None, index2=None, seg=None,
                                gather_index=None, index_out=None, out=None, out_accumulated=False,
                                out_size=None, **_):
    return indexed_vecsca_scale_gather(input2, input1, scale, index2, index1, seg, gather_index,
                                       index_out, out, out_accumulated, out_size)


def indexed_mat_t_vec_scale_gather(input1, input2, scale=None, index1=None, index2=None, seg=None,
                                   gather_index=None, index_out=None, out=None, out_accumulated=False,
                                   out_size=None, **_):
    return indexed_vecmat_scale_gather(input2, input1, scale, index2, index1, seg, gather_index,
                                       index_out, out, out_accumulated, out_size)


def indexed_scale_segment(input, scale, index, seg, out_size=None, out=None, **_):
    inter = _sel(input, index, -2)
    return _finish(inter, -2, scale, seg, None, None, out_size, False)
