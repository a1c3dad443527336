"""``SphericalHarmonics`` module (``equitorch/nn/sphericals.py:8-35``)."""
import math

from torch import Tensor, nn

from ..ops.spherical_harmonics import spherical_harmonics_fused


class SphericalHarmonics(nn.Module):
    """Real spherical harmonics up to ``l_max`` of vectors ``(..., 3)`` -> ``(..., (l_max+1)^2)``.
    Normalisation of the input, the harmonics and the optional ``1/sqrt(4 pi)`` factor run in one
    kernel (the reference chains ``F.normalize`` and dozens of elementwise kernels)."""

    def __init__(self, l_max: int, normalize_input: bool = True, integral_normalize: bool = False):
        super().__init__()
        self.l_max, self.normalize_input, self.integral_normalize = l_max, normalize_input, integral_normalize

    def forward(self, input: Tensor) -> Tensor:
        scale = 1.0 / (2.0 * math.sqrt(math.pi)) if self.integral_normalize else 1.0
        return spherical_harmonics_fused(input, self.l_max, normalize=self.normalize_input, out_scale=scale)

    def extra_repr(self) -> str:
        return f"l_max={self.l_max}, normalize_input={self.normalize_input}, integral_normalize={self.integral_normalize}"
