"""Edge <-> node data movement around a layer: gather node rows by edge source, sum edge rows
into their destination node.  The reference leaves both to ``torch_geometric.utils.scatter``
and fancy indexing with ``edge_index`` (``equitorch/transforms/__init__.py:99-101``); here they
are two kernels that work on CSR-sorted edges and use no atomics."""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from .. import _lib


def _gather_rows_raw(x: Tensor, index: Tensor) -> Tensor:
    dev = _lib.require_cuda(x, index)
    x = x.contiguous()
    width = x[0].numel() if x.shape[0] else 0
    out = torch.empty(index.shape[0], *x.shape[1:], dtype=x.dtype, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().eqt_gather_rows(_lib.DTYPE_CODE[x.dtype], x.data_ptr(), index.contiguous().data_ptr(),
                                              out.data_ptr(), index.shape[0], width, _lib.stream_ptr(dev)),
                   "eqt_gather_rows")
    return out


def _segment_sum_raw(x: Tensor, ptr: Tensor, perm: Optional[Tensor] = None) -> Tensor:
    dev = _lib.require_cuda(x, ptr, perm)
    x = x.contiguous()
    width = x[0].numel() if x.shape[0] else int(torch.tensor(x.shape[1:]).prod())
    out = torch.empty(ptr.shape[0] - 1, *x.shape[1:], dtype=x.dtype, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().eqt_segment_sum(_lib.DTYPE_CODE[x.dtype], x.data_ptr(), ptr.contiguous().data_ptr(),
                                              None if perm is None else perm.contiguous().data_ptr(), out.data_ptr(),
                                              ptr.shape[0] - 1, width, _lib.stream_ptr(dev)), "eqt_segment_sum")
    return out


class _GatherRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, index):
        ctx.save_for_backward(index)
        ctx.rows = x.shape[0]
        return _gather_rows_raw(x, index)

    @staticmethod
    def backward(ctx, grad):
        (index,) = ctx.saved_tensors
        out = torch.zeros(ctx.rows, *grad.shape[1:], dtype=grad.dtype, device=grad.device)
        return out.index_add_(0, index, grad), None


class _SegmentSum(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, ptr, perm):
        ctx.save_for_backward(ptr, perm)
        ctx.rows = x.shape[0]
        return _segment_sum_raw(x, ptr, perm)

    @staticmethod
    def backward(ctx, grad):
        ptr, perm = ctx.saved_tensors
        # node of every summed position without a host round trip (the step stays capturable in a CUDA graph):
        # position e lies in segment d when ptr[d] <= e < ptr[d+1]; positions outside [ptr[0], ptr[-1]) get zero
        count = ctx.rows if perm is None else perm.shape[0]
        nodes = ptr.numel() - 1
        pos = torch.arange(count, device=ptr.device, dtype=ptr.dtype)
        node = torch.searchsorted(ptr.contiguous(), pos, right=True) - 1
        inside = (node >= 0) & (node < nodes)
        g = _gather_rows_raw(grad.contiguous(), node.clamp_(0, max(nodes - 1, 0)))      # gradient of the e-th summed row
        g = g * inside.view(-1, *([1] * (g.ndim - 1))).to(g.dtype)
        if perm is None:
            return g, None, None
        out = torch.zeros(ctx.rows, *g.shape[1:], dtype=g.dtype, device=g.device)
        return out.index_add_(0, perm, g), None, None


def gather_rows(x: Tensor, index: Tensor) -> Tensor:
    """``out[e] = x[index[e]]`` for ``x`` of shape (rows, ...); differentiable in ``x``."""
    return _GatherRows.apply(x, index)


def segment_sum(x: Tensor, ptr: Tensor, perm: Optional[Tensor] = None) -> Tensor:
    """``out[d] = sum_{e in [ptr[d], ptr[d+1])} x[perm[e] or e]`` (ascending e, no atomics, deterministic);
    differentiable in ``x``."""
    return _SegmentSum.apply(x, ptr, perm)
