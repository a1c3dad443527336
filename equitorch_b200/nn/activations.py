"""``Gate`` (same constructor, argument meaning and checks as ``equitorch/nn/activations.py:13-175``)."""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor, nn

from ..irreps import check_irreps
from ..tables import irreps_info
from .functional.activations import gating


class _IrrepsModule(nn.Module):
    """Keeps ``irreps_info`` (a plain attribute, as in the reference) on the module's device."""

    def _apply(self, fn, *args, **kwargs):
        module = super()._apply(fn, *args, **kwargs)
        module.irreps_info = self.irreps_info._apply(fn)
        return module


class Gate(_IrrepsModule):
    """Element-wise gates on equivariant features: one gate scalar per irrep and channel
    (``irrep_wise``) or one per channel, given separately or concatenated after the features."""

    def __init__(self, irreps, activation: Optional[nn.Module] = None, irrep_wise: bool = True):
        super().__init__()
        self.irreps = check_irreps(irreps)
        self.irreps_dim = self.irreps.dim
        self.activation = activation
        self.irrep_wise = irrep_wise
        self.num_gates = len(self.irreps)
        self.irreps_info = irreps_info(self.irreps)

    def forward(self, input: Tensor, gate: Optional[Tensor] = None) -> Tensor:
        channels = input.shape[-1]
        if gate is None:
            total = self.irreps_dim + self.num_gates
            assert input.shape[-2] == total, \
                f"Input spherical dim mismatch (concatenated mode): expected {total} (irreps.dim + num_gates), got {input.shape[-2]}"
            features, gate = torch.split(input, [self.irreps_dim, self.num_gates], dim=-2)
        else:
            features = input
            assert features.shape[-2] == self.irreps_dim, \
                f"Input feature spherical dim mismatch: expected {self.irreps_dim}, got {features.shape[-2]}"
            per_sample = channels * input.shape[0]
            if self.irrep_wise:
                assert gate.numel() in (self.num_gates * channels, self.num_gates * per_sample), \
                    f"Gate numel mismatch (irrep_wise): expected {self.num_gates * channels} or {self.num_gates * per_sample}, got {gate.numel()}"
            else:
                assert gate.numel() in (channels, per_sample), \
                    f"Gate numel mismatch (global): expected {channels} or {per_sample}, got {gate.numel()}"
        if not self.irrep_wise:
            gate = gate.reshape(-1, 1, channels)
            return features * (self.activation(gate) if self.activation is not None else gate)
        gate = gate.reshape(-1, self.num_gates, channels) if gate.numel() > self.num_gates * channels \
            else gate.reshape(self.num_gates, channels)
        if self.activation is not None:
            gate = self.activation(gate)
        return gating(features.contiguous(), gate.contiguous(), self.irreps_info)

    def __repr__(self):
        return (f"{self.__class__.__name__}(irreps={self.irreps.short_repr()}, activation={self.activation}, "
                f"irrep_wise={self.irrep_wise}, num_gates={self.num_gates})")
