"""``SinCos`` module (``equitorch/nn/angular.py``)."""
from torch import Tensor, nn

from .functional.angular import sincos


class SinCos(nn.Module):
    """``angle (...,) -> [1, sin a, cos a, ..., sin(max_m a), cos(max_m a)]``."""

    def __init__(self, max_m: int, with_ones: bool = True, component_normalize: bool = False):
        super().__init__()
        self.max_m, self.with_ones, self.component_normalize = max_m, with_ones, component_normalize

    def forward(self, angle: Tensor) -> Tensor:
        return sincos(angle, self.max_m, self.with_ones, self.component_normalize)

    def extra_repr(self) -> str:
        return f"max_m={self.max_m}, with_ones={self.with_ones}, component_normalize={self.component_normalize}"
