"""Equivariant gating (mirrors ``equitorch/nn/functional/activations.py:9-36``)."""
from __future__ import annotations

from torch import Tensor

from ...structs import IrrepsInfo, SparseProductInfo
from .sparse_product import sparse_mul


def irrep_scale_infos(irreps_info: IrrepsInfo):
    """Tables of ``out[.., i, c] = x[.., i, c] * s[.., irrep(i), c]`` and of its two gradients."""
    return (SparseProductInfo(index2=irreps_info.irrep_index), SparseProductInfo(index1=irreps_info.irrep_index),
            SparseProductInfo(seg_out=irreps_info.irrep_seg))


def gating(input: Tensor, gates: Tensor, irreps_info: IrrepsInfo) -> Tensor:
    """``out[n, i, c] = input[n, i, c] * gates[(n,) irrep(i), c]``; one fused pass forward, one per gradient."""
    fwd, bwd1, bwd2 = irrep_scale_infos(irreps_info)
    return sparse_mul(input, gates, fwd, bwd1, bwd2)
