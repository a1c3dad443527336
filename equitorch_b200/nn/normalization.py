"""RMS normalisation layers (same API, parameters and buffers as ``equitorch/nn/normalization.py:9-238``)."""
from __future__ import annotations

import torch
from torch import Tensor, nn

from ..irreps import check_irreps
from ..tables import irreps_info
from .activations import _IrrepsModule
from .functional.normalization import batch_rms_norm, layer_rms_norm


class _RMSBase(_IrrepsModule):
    def __init__(self, irreps, channels: int, eps: float, affine: bool, scaled: bool):
        super().__init__()
        self.irreps = check_irreps(irreps)
        self.channels, self.eps, self.affine, self.scaled = channels, eps, affine, scaled
        self.irreps_dim = self.irreps.dim
        self.num_irreps = len(self.irreps)
        self.irreps_info = irreps_info(self.irreps)
        if affine:
            self.weight = nn.Parameter(torch.ones(self.num_irreps, channels))
        else:
            self.register_parameter("weight", None)

    def _check(self, x: Tensor) -> None:
        if x.ndim != 3:
            raise ValueError(f"Input tensor must be 3D (N, irreps_dim, C), got {x.ndim}D. Shape: {x.shape}")
        if x.shape[-2] != self.irreps_dim:
            raise ValueError(f"Input tensor's irreps dimension ({x.shape[-2]}) "
                             f"does not match expected irreps dimension ({self.irreps_dim})")
        if x.shape[-1] != self.channels:
            raise ValueError(f"Input tensor's channel dimension ({x.shape[-1]}) "
                             f"does not match expected channels ({self.channels})")

    def extra_repr(self) -> str:
        return (f"irreps={self.irreps.short_repr()}, channels={self.channels}, eps={self.eps}, "
                f"affine={self.affine}, scaled={self.scaled}")


class BatchRMSNorm(_RMSBase):
    """Divides every irrep block and channel by the root of its mean squared norm over the batch (running
    average ``running_squared_norm`` in evaluation mode), optional learnable scale per irrep and channel."""

    def __init__(self, irreps, channels: int, eps: float = 1e-5, momentum: float = 0.1, affine: bool = True,
                 scaled: bool = True):
        super().__init__(irreps, channels, eps, affine, scaled)
        self.momentum = momentum
        self.register_buffer("running_squared_norm", torch.ones(self.num_irreps, channels))

    def reset_running_stats(self) -> None:
        self.running_squared_norm.fill_(1.0)

    def reset_parameters(self) -> None:
        self.reset_running_stats()
        if self.weight is not None:
            nn.init.ones_(self.weight)

    def forward(self, input_tensor: Tensor) -> Tensor:
        self._check(input_tensor)
        return batch_rms_norm(input_tensor, self.running_squared_norm, self.irreps_info, self.weight, scaled=self.scaled,
                              training=self.training, momentum=self.momentum, eps=self.eps)


class LayerRMSNorm(_RMSBase):
    """Divides every irrep block of every sample by the root of its squared norm averaged over the channels."""

    def __init__(self, irreps, channels: int, eps: float = 1e-5, affine: bool = True, scaled: bool = True):
        super().__init__(irreps, channels, eps, affine, scaled)

    def reset_parameters(self) -> None:
        if self.weight is not None:
            nn.init.ones_(self.weight)

    def forward(self, input_tensor: Tensor) -> Tensor:
        self._check(input_tensor)
        return layer_rms_norm(input_tensor, self.irreps_info, self.weight, scaled=self.scaled, eps=self.eps)
