"""Radial basis (``equitorch/nn/radials.py:10-56``)."""
import math

import torch
from torch import Tensor, nn


class BesselBasis(nn.Module):
    r"""``(2 / r_max) sin(w_n x / r_max) / x`` with ``w_n = n pi`` (trainable by default), n = 1..num_basis."""

    def __init__(self, r_max, num_basis=8, trainable=True):
        super().__init__()
        self.trainable, self.num_basis = trainable, num_basis
        self.r_max = float(r_max)
        self.prefactor = 2.0 / self.r_max
        w = torch.linspace(start=1.0, end=num_basis, steps=num_basis) * math.pi
        if trainable:
            self.bessel_weights = nn.Parameter(w)
        else:
            self.register_buffer("bessel_weights", w)

    def forward(self, x: Tensor) -> Tensor:
        numerator = torch.sin(self.bessel_weights * x.unsqueeze(-1) / self.r_max)
        return self.prefactor * (numerator / x.unsqueeze(-1))
