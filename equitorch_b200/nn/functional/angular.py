"""Packed sines and cosines of integer multiples of an angle
(``equitorch/nn/functional/angular.py:4-35``): ``[1, sin a, cos a, sin 2a, cos 2a, ...]``."""
import torch
from torch import Tensor


def sincos(angle: Tensor, max_m: int, with_ones: bool = True, component_normalize: bool = False) -> Tensor:
    if max_m == 0:
        return torch.ones_like(angle).unsqueeze(-1)
    m = torch.arange(1, max_m + 1, dtype=angle.dtype, device=angle.device)
    ma = angle.unsqueeze(-1) * m
    pair = torch.stack([torch.sin(ma), torch.cos(ma)], dim=-1)
    if component_normalize:
        pair = pair * (2 ** 0.5)
    pair = pair.flatten(-2, -1)
    if not with_ones:
        return pair
    return torch.cat([torch.ones_like(angle).unsqueeze(-1), pair], dim=-1)
