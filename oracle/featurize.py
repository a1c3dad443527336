"""ORACLE (test infrastructure, never imported by the product path).

CPU restatement of the edge-featurisation chain of the reference's transforms
(equitorch/transforms/__init__.py:18-251):

* ``radius_graph``: all ordered pairs closer than ``r`` within a graph, no self loops unless asked, at most
  ``max_num_neighbors`` per target.  The reference delegates this search to ``torch_geometric.nn.radius_graph``
  (third party, absent here), so the search itself is **parity unpinned**; it is defined here by brute force with
  the neighbours of smallest index kept, edges sorted by (target, source), ``edge_index = [source, target]`` for the
  default flow (:99-101).
* ``edge_vec = pos[edge_index[1]] - pos[edge_index[0]]`` (:99-101), norm (:150), spherical harmonics of the edge
  vector (:203, via ``oracle.sphericals``), ``BesselBasis`` (equitorch/nn/radials.py:10-56) and the three cutoffs
  (equitorch/nn/functional/cutoffs.py) - these are pinned against reference outputs in tests/golden/radial.pt.gz.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
from torch import Tensor

from .sphericals import spherical_harmonics


def radius_graph(pos: Tensor, r: float, batch: Optional[Tensor] = None, loop: bool = False, max_num_neighbors: int = 32):
    n = pos.shape[0]
    d2 = ((pos[:, None, :] - pos[None, :, :]) ** 2).sum(-1)          # [target, source]
    ok = d2 < r * r
    if batch is not None:
        ok &= batch[:, None] == batch[None, :]
    if not loop:
        ok &= ~torch.eye(n, dtype=torch.bool)
    ok &= torch.cumsum(ok, dim=1) <= max_num_neighbors              # the neighbours of smallest index
    dst, src = ok.nonzero(as_tuple=True)
    return src, dst


def bessel_basis(x: Tensor, r_max: float, weights: Tensor) -> Tensor:
    return (2.0 / r_max) * (torch.sin(weights * x.unsqueeze(-1) / r_max) / x.unsqueeze(-1))


def cutoff(x: Tensor, kind: str, r_max: float, r_min: float = 0.0, p: float = 6.0, eps: float = 1e-7) -> Tensor:
    u = ((x - r_min) / (r_max - r_min)).clamp(0, 1)
    if kind == "polynomial":
        return 1.0 - ((p + 1.0) * (p + 2.0) / 2.0) * u ** p + p * (p + 2.0) * u ** (p + 1.0) - (p * (p + 1.0) / 2) * u ** (p + 2.0)
    if kind == "cosine":
        return 0.5 * (1.0 + torch.cos(math.pi * u))
    return torch.exp(1 - 1 / (1 - u ** 2 + eps))


def edge_features(pos: Tensor, src: Tensor, dst: Tensor, l_max: int, integral_normalize: bool = False):
    vec = pos[dst] - pos[src]
    length = vec.norm(dim=-1)
    sh = spherical_harmonics(torch.nn.functional.normalize(vec, dim=-1), l_max)
    if integral_normalize:
        sh = sh / (2 * math.sqrt(math.pi))
    return vec, length, sh
