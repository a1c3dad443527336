"""Cutoff envelopes (``equitorch/nn/cutoffs.py:7-140``, ``equitorch/nn/functional/cutoffs.py``)."""
import torch
from torch import Tensor, nn


def radial_standarize(input: Tensor, range: float, r_min: float) -> Tensor:
    """``clamp((r - r_min) / range, 0, 1)`` (the reference's spelling of the name is kept)."""
    if r_min != 0:
        input = input - r_min
    return (input / range).clamp(0, 1)


def polynomial_cutoff(input: Tensor, p: float = 6.0) -> Tensor:
    out = 1.0 - (((p + 1.0) * (p + 2.0) / 2.0) * torch.pow(input, p))
    out = out + (p * (p + 2.0) * torch.pow(input, p + 1.0))
    return out - ((p * (p + 1.0) / 2) * torch.pow(input, p + 2.0))


def cosine_cutoff(input: Tensor) -> Tensor:
    return 0.5 * (1.0 + torch.cos(torch.pi * input))


def mollifier_cutoff(input: Tensor, eps: float = 1e-12) -> Tensor:
    return torch.exp(1 - 1 / (1 - input ** 2 + eps))


class PolynomialCutoff(nn.Module):
    def __init__(self, r_max: float, r_min: float = 0.0, p: float = 6):
        super().__init__()
        assert r_max >= r_min
        assert p >= 2.0
        self.p, self.r_max, self.r_min, self.range = float(p), r_max, r_min, float(r_max - r_min)

    def forward(self, input: Tensor) -> Tensor:
        return polynomial_cutoff(radial_standarize(input, self.range, self.r_min), p=self.p)


class CosineCutoff(nn.Module):
    def __init__(self, r_max: float, r_min: float = 0):
        super().__init__()
        assert r_min < r_max
        self.r_max, self.r_min, self.range = r_max, r_min, float(r_max - r_min)

    def forward(self, input: Tensor) -> Tensor:
        return cosine_cutoff(radial_standarize(input, self.range, self.r_min))


class MollifierCutoff(nn.Module):
    def __init__(self, r_max: float, r_min: float = 0, eps: float = 1e-7):
        super().__init__()
        assert r_min < r_max
        self.r_max, self.r_min, self.range, self.eps = r_max, r_min, float(r_max - r_min), eps

    def forward(self, input: Tensor) -> Tensor:
        return mollifier_cutoff(radial_standarize(input, self.range, self.r_min), eps=self.eps)
