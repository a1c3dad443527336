"""Radius graph and fused edge features (operator layer over ``eqt_radius_count`` / ``eqt_radius_edges``)."""
from __future__ import annotations

import ctypes as C
import math
from typing import NamedTuple, Optional

import torch
from torch import Tensor

from .. import _lib

CUTOFF_KINDS = {"polynomial": 0, "cosine": 1, "mollifier": 2}
_status = {}


def _flag(dev) -> Tensor:
    if dev not in _status:
        _status[dev] = torch.zeros(1, dtype=torch.int32, device=dev)
    return _status[dev]


class CellList(NamedTuple):
    struct: "_lib.RadiusGridStruct"
    keep: tuple          # tensors the struct points at


def build_cell_list(pos: Tensor, r: float, batch: Optional[Tensor] = None) -> CellList:
    """Bin ``pos`` (N, 3) into cubic cells of side ``r`` (slightly more), one slab of cells per graph."""
    n = pos.shape[0]
    dev = pos.device
    cell_size = float(r) * (1.0 + 1e-5)
    lo = pos.min(dim=0).values
    extent = (pos.max(dim=0).values - lo).tolist()                      # one host synchronisation
    dims = [max(1, int(math.floor(e / cell_size)) + 1) for e in extent]
    per_graph = dims[0] * dims[1] * dims[2]
    graphs = 1 if batch is None else int(batch.max()) + 1
    if graphs * per_graph >= 2 ** 31:
        raise ValueError("cell grid too large; the positions are too spread out for this cutoff")
    c = ((pos - lo) / cell_size).floor().long()
    for k in range(3):
        c[:, k].clamp_(0, dims[k] - 1)
    cell = (c[:, 2] * dims[1] + c[:, 1]) * dims[0] + c[:, 0]
    if batch is not None:
        cell = cell + batch.long() * per_graph
    order = torch.argsort(cell, stable=True)
    cell_start = torch.searchsorted(cell[order], torch.arange(graphs * per_graph + 1, device=dev)).int()
    point_cell, sorted_index = cell.int().contiguous(), order.int().contiguous()
    struct = _lib.RadiusGridStruct(cell_start.data_ptr(), sorted_index.data_ptr(), point_cell.data_ptr(), cell_size,
                                   (C.c_int32 * 3)(*dims))
    return CellList(struct, (cell_start, sorted_index, point_cell))


class EdgeFeatures(NamedTuple):
    src: Tensor                       # (E,) int64, ascending within a target
    dst: Tensor                       # (E,) int64, ascending
    ptr: Tensor                       # (N + 1,) int64 CSR by target
    vec: Optional[Tensor]             # (E, 3) pos[dst] - pos[src]
    length: Optional[Tensor]          # (E,)
    sh: Optional[Tensor]              # (E, (l_max + 1)^2)
    bessel: Optional[Tensor]          # (E, num_basis)
    cutoff: Optional[Tensor]          # (E,)


def radius_graph_features(pos: Tensor, r: float, batch: Optional[Tensor] = None, loop: bool = False,
                          max_num_neighbors: int = 32, with_vec: bool = True, with_length: bool = False,
                          l_max: Optional[int] = None, integral_normalize: bool = False,
                          bessel_weights: Optional[Tensor] = None, bessel_r_max: Optional[float] = None,
                          cutoff: Optional[str] = None, cutoff_r_max: Optional[float] = None, cutoff_r_min: float = 0.0,
                          cutoff_p: float = 6.0, cutoff_eps: float = 1e-7) -> EdgeFeatures:
    """Edges ``j -> i`` for ``|pos_i - pos_j| < r`` (same graph, at most ``max_num_neighbors`` per target, those of
    smallest index) sorted by (target, source), and the requested per-edge features, in two kernel passes."""
    dev = _lib.require_cuda(pos, batch, bessel_weights)
    if pos.dtype != torch.float32 or pos.ndim != 2 or pos.shape[1] != 3:
        raise TypeError("pos must be a float32 (N, 3) tensor")
    pos = pos.detach().contiguous()
    n = pos.shape[0]
    if n == 0:
        z = torch.zeros(0, dtype=torch.long, device=dev)
        return EdgeFeatures(z, z, torch.zeros(1, dtype=torch.long, device=dev), None, None, None, None, None)
    if l_max is not None and not 0 <= l_max <= 4:
        raise ValueError("the fused kernel takes l_max <= 4; use SphericalHarmonics on edge_vec for higher degrees")
    cells = build_cell_list(pos, r, batch)
    degree = torch.empty(n, dtype=torch.int32, device=dev)
    flag = _flag(dev)
    lib = _lib.lib()
    with torch.cuda.device(dev):
        _lib.check(lib.eqt_radius_count(C.byref(cells.struct), pos.data_ptr(), _lib.ptr(batch), n, float(r), int(loop),
                                        int(max_num_neighbors), degree.data_ptr(), flag.data_ptr(), _lib.stream_ptr(dev)),
                   "eqt_radius_count")
    ptr = torch.zeros(n + 1, dtype=torch.long, device=dev)
    torch.cumsum(degree, 0, out=ptr[1:])
    e = int(ptr[-1])                                                     # host synchronisation: the output size
    if int(flag.item()) != 0:
        flag.zero_()
        raise _lib.EqtError("a node has more than 512 candidate neighbours; lower the cutoff")
    src = torch.empty(e, dtype=torch.long, device=dev)
    dst = torch.empty(e, dtype=torch.long, device=dev)
    f32 = dict(dtype=torch.float32, device=dev)
    vec = torch.empty(e, 3, **f32) if with_vec else None
    length = torch.empty(e, **f32) if with_length else None
    sh = torch.empty(e, (l_max + 1) ** 2, **f32) if l_max is not None else None
    bw = None if bessel_weights is None else bessel_weights.detach().to(**f32).contiguous()
    bes = torch.empty(e, bw.numel(), **f32) if bw is not None else None
    cut = torch.empty(e, **f32) if cutoff is not None else None
    if bw is not None and bessel_r_max is None:
        raise ValueError("bessel_r_max is required with bessel_weights")
    if cutoff is not None and cutoff_r_max is None:
        raise ValueError("cutoff_r_max is required with cutoff")
    feats = _lib.EdgeFeaturesStruct(_lib.ptr(vec), _lib.ptr(length), _lib.ptr(sh), _lib.ptr(bes), _lib.ptr(cut), _lib.ptr(bw),
                                    l_max or 0, int(integral_normalize), 0 if bw is None else bw.numel(),
                                    CUTOFF_KINDS[cutoff] if cutoff is not None else 0, float(bessel_r_max or 1.0),
                                    float(cutoff_r_min), float(cutoff_r_max or 1.0), float(cutoff_p), float(cutoff_eps))
    with torch.cuda.device(dev):
        _lib.check(lib.eqt_radius_edges(C.byref(cells.struct), pos.data_ptr(), _lib.ptr(batch), n, float(r), int(loop),
                                        int(max_num_neighbors), ptr.data_ptr(), src.data_ptr(), dst.data_ptr(), C.byref(feats),
                                        flag.data_ptr(), _lib.stream_ptr(dev)), "eqt_radius_edges")
    return EdgeFeatures(src, dst, ptr, vec, length, sh, bes, cut)
