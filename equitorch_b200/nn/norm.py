"""Per-irrep norm modules (same API as ``equitorch/nn/norm.py:12-187``)."""
from __future__ import annotations

from torch import Tensor

from ..irreps import check_irreps
from ..tables import irreps_info
from .activations import _IrrepsModule
from .functional.norm import batch_mean_squared_norm, channel_mean_squared_norm, norm, squared_norm


class _NormBase(_IrrepsModule):
    def __init__(self, irreps, scaled: bool = True):
        super().__init__()
        self.irreps = check_irreps(irreps)
        self.scaled = scaled
        self.irreps_dim = self.irreps.dim
        self.irreps_info = irreps_info(self.irreps)

    def _check(self, input_tensor: Tensor) -> None:
        if input_tensor.shape[-2] != self.irreps_dim:
            raise ValueError(f"Input tensor's irreps dimension ({input_tensor.shape[-2]}) "
                             f"does not match expected irreps dimension ({self.irreps_dim})")

    def extra_repr(self) -> str:
        return f"irreps={self.irreps.short_repr()}, scaled={self.scaled}"


class SquaredNorm(_NormBase):
    """(..., irreps.dim, C) -> (..., len(irreps), C): squared L2 norm of every irrep block."""

    def forward(self, input_tensor: Tensor) -> Tensor:
        self._check(input_tensor)
        return squared_norm(input_tensor, self.irreps_info, self.scaled)


class Norm(_NormBase):
    """(..., irreps.dim, C) -> (..., len(irreps), C): L2 norm of every irrep block (zero gradient at zero)."""

    def forward(self, input_tensor: Tensor) -> Tensor:
        self._check(input_tensor)
        return norm(input_tensor, self.irreps_info, self.scaled)


class MeanSquaredNorm(_NormBase):
    """Squared norms averaged over the batch (``dim=0`` -> (len(irreps), C)) or over the channels
    (``dim=-1`` or ``2`` -> (N, len(irreps)))."""

    def __init__(self, irreps, scaled: bool = True, dim: int = -1):
        super().__init__(irreps, scaled)
        if dim not in (0, -1, 2):
            raise ValueError(f"Unsupported dim value: {dim}. Allowed values are 0, -1, 2.")
        self.dim = -1 if dim == 2 else dim

    def forward(self, input_tensor: Tensor) -> Tensor:
        self._check(input_tensor)
        if self.dim == 0:
            return batch_mean_squared_norm(input_tensor, self.irreps_info, self.scaled)
        return channel_mean_squared_norm(input_tensor, self.irreps_info, self.scaled)
