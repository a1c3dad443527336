"""Seeded synthetic inputs with the shapes, sizes and value distributions of the benchmark
configurations (no dataset is involved anywhere: every tensor is generated here).

* ``random_graph``: uniformly random sources, destinations sorted (the single-GPU microbenchmark:
  200k edges over 10k nodes).
* ``radius_graph``: random geometric graph - points uniform in a cube, directed edges between
  points closer than a cutoff, node ids in Morton (Z-curve) order of the cell they fall in so that
  a contiguous id range is a compact region of space (the multi-GPU scaling graph: 100k nodes,
  about 2M edges, average degree 20).

Everything is generated on the CPU from ``numpy.random.default_rng(seed)`` so that every rank
of a multi-process run and the CPU oracle see identical data.
"""
from __future__ import annotations

from typing import NamedTuple, Tuple

import numpy as np
import torch


class SyntheticGraph(NamedTuple):
    num_nodes: int
    src: torch.Tensor        # (E,) int64
    dst: torch.Tensor        # (E,) int64, ascending
    edge_vec: torch.Tensor   # (E, 3) float32, position[dst] - position[src] (or random directions)


def random_graph(num_nodes: int, num_edges: int, seed: int = 0) -> SyntheticGraph:
    rng = np.random.default_rng(seed)
    src = rng.integers(0, num_nodes, num_edges, dtype=np.int64)
    dst = np.sort(rng.integers(0, num_nodes, num_edges, dtype=np.int64))
    vec = rng.standard_normal((num_edges, 3)).astype(np.float32)
    return SyntheticGraph(num_nodes, torch.from_numpy(src), torch.from_numpy(dst), torch.from_numpy(vec))


def _morton(ix: np.ndarray, iy: np.ndarray, iz: np.ndarray) -> np.ndarray:
    def spread(v):
        v = v.astype(np.uint64) & np.uint64(0x1FFFFF)
        v = (v | (v << np.uint64(32))) & np.uint64(0x1F00000000FFFF)
        v = (v | (v << np.uint64(16))) & np.uint64(0x1F0000FF0000FF)
        v = (v | (v << np.uint64(8))) & np.uint64(0x100F00F00F00F00F)
        v = (v | (v << np.uint64(4))) & np.uint64(0x10C30C30C30C30C3)
        v = (v | (v << np.uint64(2))) & np.uint64(0x1249249249249249)
        return v
    return spread(ix) | (spread(iy) << np.uint64(1)) | (spread(iz) << np.uint64(2))


def _pairs_within(pos: np.ndarray, box: float, cutoff: float) -> Tuple[np.ndarray, np.ndarray]:
    """All ordered pairs (i, j), i != j, with |pos_i - pos_j| < cutoff, via a cell list."""
    ncell = max(1, int(np.floor(box / cutoff)))
    cell = np.minimum((pos / (box / ncell)).astype(np.int64), ncell - 1)
    lin = (cell[:, 0] * ncell + cell[:, 1]) * ncell + cell[:, 2]
    order = np.argsort(lin, kind="stable")
    lin_sorted = lin[order]
    starts = np.searchsorted(lin_sorted, np.arange(ncell ** 3 + 1))
    src_all, dst_all = [], []
    n = pos.shape[0]
    idx = np.arange(n)
    for dx in (-1, 0, 1):
        for dy in (-1, 0, 1):
            for dz in (-1, 0, 1):
                nb = cell + np.array([dx, dy, dz])
                ok = np.all((nb >= 0) & (nb < ncell), axis=1)
                nlin = (nb[:, 0] * ncell + nb[:, 1]) * ncell + nb[:, 2]
                lo = np.where(ok, starts[np.clip(nlin, 0, ncell ** 3 - 1)], 0)
                hi = np.where(ok, starts[np.clip(nlin, 0, ncell ** 3 - 1) + 1], 0)
                cnt = hi - lo
                i = np.repeat(idx, cnt)
                off = np.arange(cnt.sum()) - np.repeat(np.cumsum(cnt) - cnt, cnt)
                j = order[np.repeat(lo, cnt) + off]
                d2 = ((pos[i] - pos[j]) ** 2).sum(1)
                keep = (d2 < cutoff * cutoff) & (i != j)
                src_all.append(j[keep]); dst_all.append(i[keep])
    return np.concatenate(src_all), np.concatenate(dst_all)


def radius_graph(num_nodes: int = 100_000, target_edges: int = 2_000_000, cutoff: float = 1.0,
                 seed: int = 0, tolerance: float = 0.02) -> Tuple[SyntheticGraph, torch.Tensor]:
    """Random geometric graph with about ``target_edges`` directed edges; returns the graph and the
    (Morton ordered) positions.  The cube side is chosen for the target degree in the bulk and the
    cutoff is rescaled once to absorb the deficit of the points near the faces."""
    rng = np.random.default_rng(seed)
    degree = target_edges / num_nodes
    box = (num_nodes * 4.0 / 3.0 * np.pi * cutoff ** 3 / degree) ** (1.0 / 3.0)
    pos = rng.random((num_nodes, 3)) * box
    ncell = max(1, int(np.floor(box / cutoff)))
    c = np.minimum((pos / (box / ncell)).astype(np.int64), ncell - 1)
    pos = pos[np.argsort(_morton(c[:, 0], c[:, 1], c[:, 2]), kind="stable")]
    src, dst = _pairs_within(pos, box, cutoff)
    if abs(len(src) - target_edges) > tolerance * target_edges:
        cutoff = cutoff * (target_edges / len(src)) ** (1.0 / 3.0)
        src, dst = _pairs_within(pos, box, cutoff)
    assert abs(len(src) - target_edges) <= tolerance * target_edges, (len(src), target_edges)
    order = np.lexsort((src, dst))
    src, dst = src[order], dst[order]
    vec = (pos[dst] - pos[src]).astype(np.float32)
    g = SyntheticGraph(num_nodes, torch.from_numpy(src.astype(np.int64)), torch.from_numpy(dst.astype(np.int64)),
                       torch.from_numpy(vec))
    return g, torch.from_numpy(pos.astype(np.float32))


def node_features(num_nodes: int, dim: int, channels: int, seed: int = 1, dtype=torch.float32) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return torch.randn(num_nodes, dim, channels, generator=g, dtype=dtype)
