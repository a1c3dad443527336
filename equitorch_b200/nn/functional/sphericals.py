"""Spherical harmonics (functional form, ``equitorch/nn/functional/sphericals.py:9-14``)."""
import math

from torch import Tensor

from ...ops.spherical_harmonics import spherical_harmonics as _spherical_harmonics
from ...ops.spherical_harmonics import spherical_harmonics_fused


def spherical_harmonics(input: Tensor, l_max: int, dim: int = -1, integral_normalize: bool = False) -> Tensor:
    """Component-normalised real harmonics of ``input`` (xyz along ``dim``); with
    ``integral_normalize`` everything is divided by ``sqrt(4 pi)``."""
    if dim in (-1, input.ndim - 1):
        scale = 1.0 / (2.0 * math.sqrt(math.pi)) if integral_normalize else 1.0
        return spherical_harmonics_fused(input, l_max, normalize=False, out_scale=scale)
    sh = _spherical_harmonics(input, l_max, dim)
    return sh * (1.0 / (2.0 * math.sqrt(math.pi))) if integral_normalize else sh
