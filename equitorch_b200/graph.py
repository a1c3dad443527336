"""Edge lists prepared for the fused graph kernels.

A layer of a message-passing network evaluates one tensor product per edge
``(source -> destination)`` and sums the results per destination node.  The fused kernels
walk the edges grouped by the node they reduce into, so they need the edges in CSR order by
destination (forward pass and the gradient of the edge attributes) and in CSR order by source
(gradient of the node features).  ``EdgeGraph`` computes both orders once; edge attributes
(vectors, spherical harmonics) always stay in the caller's order and are addressed through the
stored permutations.

Convention: ``edge_index[0]`` = source (row gathered from), ``edge_index[1]`` = destination
(row summed into), as in ``equitorch/transforms/__init__.py:99-101`` of the reference.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor


def _csr(sorted_ids: Tensor, n: int) -> Tensor:
    ptr = torch.zeros(n + 1, dtype=torch.int64, device=sorted_ids.device)
    if sorted_ids.numel():
        ptr[1:] = torch.cumsum(torch.bincount(sorted_ids, minlength=n), 0)
    return ptr


class EdgeGraph:
    """CSR-by-destination and CSR-by-source views of an edge list.

    Attributes (all int64 tensors on the edges' device):
      ``dst_ptr`` (num_dst + 1), ``dst_sorted`` (E), ``src_by_dst`` (E), ``dst_order`` (E) or ``None``
      when the edges already are sorted by destination; ``src_ptr`` (num_src + 1), ``dst_by_src`` (E),
      ``src_order`` (E): the same for the grouping by source.
    """

    def __init__(self, src: Tensor, dst: Tensor, num_src: int, num_dst: Optional[int] = None):
        assert src.dtype == torch.int64 and dst.dtype == torch.int64 and src.shape == dst.shape and src.ndim == 1
        self.num_src = int(num_src)
        self.num_dst = int(num_src if num_dst is None else num_dst)
        self.num_edges = src.numel()
        already = bool((dst[1:] >= dst[:-1]).all()) if dst.numel() > 1 else True
        if already:
            self.dst_order, self.dst_sorted, self.src_by_dst = None, dst.contiguous(), src.contiguous()
        else:
            self.dst_order = torch.argsort(dst, stable=True)
            self.dst_sorted, self.src_by_dst = dst[self.dst_order], src[self.dst_order]
        self.dst_ptr = _csr(self.dst_sorted, self.num_dst)
        self.src_order = torch.argsort(src, stable=True)
        self.dst_by_src = dst[self.src_order]
        self.src_ptr = _csr(src[self.src_order], self.num_src)

    @property
    def device(self):
        return self.dst_ptr.device

    def to(self, device) -> "EdgeGraph":
        out = object.__new__(EdgeGraph)
        for k, v in self.__dict__.items():
            setattr(out, k, v.to(device) if isinstance(v, Tensor) else v)
        return out

    @staticmethod
    def from_edge_index(edge_index: Tensor, num_nodes: int) -> "EdgeGraph":
        return EdgeGraph(edge_index[0], edge_index[1], num_nodes)
