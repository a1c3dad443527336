"""Equivariant gating (mirrors ``equitorch/nn/functional/activations.py:9-36``)."""
from __future__ import annotations

from torch import Tensor

from ...ops.irrep_ops import PER_SAMPLE_CHANNEL, SHARED
from ...structs import IrrepsInfo
from ._irrep import irrep_scale


def gating(input: Tensor, gates: Tensor, irreps_info: IrrepsInfo) -> Tensor:
    """``out[n, i, c] = input[n, i, c] * gates[(n,) irrep(i), c]``; ``gates`` is (N, num_irreps, C) or, shared
    by the batch, (num_irreps, C).  One streaming pass forward, one per gradient."""
    lead = input.shape[:-2]
    x = input.reshape(-1, *input.shape[-2:])
    if gates.ndim == 2:
        out = irrep_scale(x, gates, irreps_info, SHARED)
    else:
        out = irrep_scale(x, gates.reshape(-1, *gates.shape[-2:]), irreps_info, PER_SAMPLE_CHANNEL)
    return out.reshape(*lead, *out.shape[-2:])
