"""Graph transforms (``equitorch/transforms/__init__.py:18-251``): ``RadiusGraph``, ``AddVectorNorm``,
``AddSphericalHarmonics``, ``AddVectorLengthEmbedding`` with the reference's constructor arguments and attribute
names, on any object that carries tensors as attributes (``torch_geometric.data.Data``, a ``SimpleNamespace``).

``RadiusGraph`` runs the cell-list kernels of ``ops.featurize_op`` on CUDA positions (the reference delegates the
search to a third-party package); ``EdgeFeaturizer`` is the fused form of the whole chain - edges, vectors,
harmonics, Bessel basis and cutoff written in one pass - for pipelines that do not differentiate through positions.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
from torch import Tensor

from .nn.cutoffs import CosineCutoff, MollifierCutoff, PolynomialCutoff
from .nn.radials import BesselBasis
from .nn.sphericals import SphericalHarmonics
from .ops.featurize_op import EdgeFeatures, radius_graph_features


class RadiusGraph:
    def __init__(self, r: float, loop: bool = False, max_num_neighbors: int = 32, flow: str = "source_to_target",
                 pos_attr: str = "pos", edge_index_attr: str = "edge_index", edge_vector_attr: str = "edge_vec",
                 num_workers: int = 1) -> None:
        assert flow in ("source_to_target", "target_to_source")
        self.r, self.loop, self.max_num_neighbors, self.flow, self.num_workers = r, loop, max_num_neighbors, flow, num_workers
        self.pos_attr, self.edge_index_attr, self.edge_vector_attr = pos_attr, edge_index_attr, edge_vector_attr

    def forward(self, data):
        pos = getattr(data, self.pos_attr)
        f = radius_graph_features(pos, self.r, getattr(data, "batch", None), self.loop, self.max_num_neighbors, with_vec=False)
        row, col = (f.src, f.dst) if self.flow == "source_to_target" else (f.dst, f.src)
        edge_index = torch.stack([row, col])
        setattr(data, self.edge_index_attr, edge_index)
        setattr(data, self.edge_vector_attr, pos[edge_index[1]] - pos[edge_index[0]])      # differentiable in pos
        return data

    __call__ = forward

    def __repr__(self) -> str:
        return f"{self.__class__.__name__}(r={self.r})"


class AddVectorNorm:
    def __init__(self, vector_attr: str = "edge_vec", norm_attr: str = "edge_norm") -> None:
        self.vector_attr, self.norm_attr = vector_attr, norm_attr

    def forward(self, data):
        setattr(data, self.norm_attr, getattr(data, self.vector_attr).norm(dim=-1))
        return data

    __call__ = forward


class AddSphericalHarmonics:
    def __init__(self, l_max: int, vector_attr: str = "edge_vec", sh_attr: str = "edge_sh", integral_normalize: bool = False) -> None:
        self.l_max, self.vector_attr, self.sh_attr, self.integral_normalize = l_max, vector_attr, sh_attr, integral_normalize
        self._sh = SphericalHarmonics(l_max, integral_normalize=integral_normalize)

    def forward(self, data):
        setattr(data, self.sh_attr, self._sh(getattr(data, self.vector_attr)))
        return data

    __call__ = forward


class AddVectorLengthEmbedding:
    def __init__(self, emb: Callable[[Tensor], Tensor], vector_attr: str = "edge_vec", embedding_attr: str = "edge_emb") -> None:
        self.emb, self.vector_attr, self.embedding_attr = emb, vector_attr, embedding_attr

    def forward(self, data):
        setattr(data, self.embedding_attr, self.emb(getattr(data, self.vector_attr).norm(dim=-1)))
        return data

    __call__ = forward


class EdgeFeaturizer:
    """``RadiusGraph(r) -> AddSphericalHarmonics(l_max) -> AddVectorLengthEmbedding(BesselBasis) -> cutoff`` as two
    kernel passes; sets ``edge_index``, ``edge_vec``, ``edge_sh``, ``edge_emb``, ``edge_cutoff`` and ``edge_ptr`` (CSR
    by target).  No gradient flows to the positions."""

    def __init__(self, r: float, l_max: Optional[int] = None, basis: Optional[BesselBasis] = None, cutoff=None,
                 loop: bool = False, max_num_neighbors: int = 32, integral_normalize: bool = False, pos_attr: str = "pos"):
        self.r, self.l_max, self.basis, self.cutoff = r, l_max, basis, cutoff
        self.loop, self.max_num_neighbors, self.integral_normalize, self.pos_attr = loop, max_num_neighbors, integral_normalize, pos_attr

    def features(self, pos: Tensor, batch: Optional[Tensor] = None) -> EdgeFeatures:
        kw = {}
        if self.basis is not None:
            kw.update(bessel_weights=self.basis.bessel_weights, bessel_r_max=self.basis.r_max)
        if isinstance(self.cutoff, PolynomialCutoff):
            kw.update(cutoff="polynomial", cutoff_r_max=self.cutoff.r_max, cutoff_r_min=self.cutoff.r_min, cutoff_p=self.cutoff.p)
        elif isinstance(self.cutoff, CosineCutoff):
            kw.update(cutoff="cosine", cutoff_r_max=self.cutoff.r_max, cutoff_r_min=self.cutoff.r_min)
        elif isinstance(self.cutoff, MollifierCutoff):
            kw.update(cutoff="mollifier", cutoff_r_max=self.cutoff.r_max, cutoff_r_min=self.cutoff.r_min, cutoff_eps=self.cutoff.eps)
        elif self.cutoff is not None:
            raise TypeError("cutoff must be a PolynomialCutoff, CosineCutoff or MollifierCutoff")
        return radius_graph_features(pos, self.r, batch, self.loop, self.max_num_neighbors, with_vec=True, with_length=True,
                                     l_max=self.l_max, integral_normalize=self.integral_normalize, **kw)

    def forward(self, data):
        f = self.features(getattr(data, self.pos_attr), getattr(data, "batch", None))
        data.edge_index, data.edge_vec, data.edge_norm, data.edge_ptr = torch.stack([f.src, f.dst]), f.vec, f.length, f.ptr
        if f.sh is not None:
            data.edge_sh = f.sh
        if f.bessel is not None:
            data.edge_emb = f.bessel
        if f.cutoff is not None:
            data.edge_cutoff = f.cutoff
        return data

    __call__ = forward


__all__ = ["RadiusGraph", "AddSphericalHarmonics", "AddVectorNorm", "AddVectorLengthEmbedding", "EdgeFeaturizer"]
