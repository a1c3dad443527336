"""Edge <-> node data movement around a layer: gather node rows by edge source, sum edge rows
into their destination node.  The reference leaves both to ``torch_geometric.utils.scatter``
and fancy indexing with ``edge_index`` (``equitorch/transforms/__init__.py:99-101``); here they
are two kernels that work on CSR-sorted edges and use no atomics."""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from .. import _lib


def gather_rows(x: Tensor, index: Tensor) -> Tensor:
    """``out[e] = x[index[e]]`` for a contiguous ``x`` of shape (rows, ...)."""
    dev = _lib.require_cuda(x, index)
    x = x.contiguous()
    width = x[0].numel() if x.shape[0] else 0
    out = torch.empty(index.shape[0], *x.shape[1:], dtype=x.dtype, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().eqt_gather_rows(_lib.DTYPE_CODE[x.dtype], x.data_ptr(), index.contiguous().data_ptr(),
                                              out.data_ptr(), index.shape[0], width, _lib.stream_ptr(dev)),
                   "eqt_gather_rows")
    return out


def segment_sum(x: Tensor, ptr: Tensor, perm: Optional[Tensor] = None) -> Tensor:
    """``out[d] = sum_{e in [ptr[d], ptr[d+1])} x[perm[e] or e]`` (ascending e, deterministic)."""
    dev = _lib.require_cuda(x, ptr, perm)
    x = x.contiguous()
    width = x[0].numel() if x.shape[0] else int(torch.tensor(x.shape[1:]).prod())
    out = torch.empty(ptr.shape[0] - 1, *x.shape[1:], dtype=x.dtype, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().eqt_segment_sum(_lib.DTYPE_CODE[x.dtype], x.data_ptr(), ptr.contiguous().data_ptr(),
                                              None if perm is None else perm.contiguous().data_ptr(), out.data_ptr(),
                                              ptr.shape[0] - 1, width, _lib.stream_ptr(dev)), "eqt_segment_sum")
    return out
