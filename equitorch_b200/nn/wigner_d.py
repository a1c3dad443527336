"""Wigner-D modules (``equitorch/nn/wigner_d.py:15-189``)."""
from typing import Optional

import torch
from torch import Tensor, nn

from ..irreps import Irreps, check_irreps
from ..tables import wigner_d_info
from .functional.wigner_d import dense_wigner_rotation, sparse_wigner_rotation, wigner_d_matrix


class _WithRotationInfo(nn.Module):
    def _apply(self, fn, *args, **kwargs):
        module = super()._apply(fn, *args, **kwargs)
        module.info = self.info._apply(fn)
        return module


class SparseWignerRotation(_WithRotationInfo):
    """Rotate ``(N, irreps.dim, C)`` features by per-sample ZYZ Euler angles given as packed sin/cos
    rows, without forming the dense D-matrix."""

    def __init__(self, irreps: Irreps):
        super().__init__()
        self.irreps = check_irreps(irreps)
        self.info = wigner_d_info(self.irreps)
        self.max_m = max(ir.l for ir in self.irreps)

    def forward(self, input: Tensor, sincos_alpha: Optional[Tensor], sincos_beta: Optional[Tensor],
                sincos_gamma: Optional[Tensor]) -> Tensor:
        return sparse_wigner_rotation(input, sincos_alpha, sincos_beta, sincos_gamma, self.info)

    def extra_repr(self) -> str:
        return f"irreps={self.irreps}, max_m={self.max_m}"


class DenseWignerRotation(nn.Module):
    """``wigner_d (N, dim, dim) @ input (N, dim, C)``.

    A Wigner D-matrix is block diagonal over the irreps (455 of 2401 entries for l = 0..6).  With ``block_diagonal``
    (the default) the CUDA kernels read and multiply only those blocks and return a ``wigner_d`` gradient that is zero
    outside them; pass ``block_diagonal=False`` to multiply by arbitrary dense matrices."""

    def __init__(self, irreps: Irreps, block_diagonal: bool = True):
        super().__init__()
        self.irreps = check_irreps(irreps)
        self.block_diagonal = block_diagonal

    def forward(self, input: Tensor, wigner_d: Tensor) -> Tensor:
        row_range = None
        if self.block_diagonal and input.is_cuda and wigner_d.shape[-1] == self.irreps.dim:
            from ..ops.wigner_op import block_row_range
            row_range = block_row_range(self.irreps, input.device)
        return dense_wigner_rotation(input, wigner_d, row_range)

    def extra_repr(self) -> str:
        return f"irreps={self.irreps}, block_diagonal={self.block_diagonal}"


class WignerD(_WithRotationInfo):
    """Dense ``D(alpha, beta, gamma) = Dz(alpha) Dy(beta) Dz(gamma)`` of shape ``(N, dim, dim)``."""

    def __init__(self, irreps: Irreps):
        super().__init__()
        self.irreps = check_irreps(irreps)
        self.max_m = max((ir.l for ir in self.irreps), default=0)
        self.info = wigner_d_info(self.irreps)
        self.register_buffer("identity", torch.eye(self.irreps.dim))

    def forward(self, alpha: Optional[Tensor] = None, beta: Optional[Tensor] = None, gamma: Optional[Tensor] = None,
                sincos_alpha: Optional[Tensor] = None, sincos_beta: Optional[Tensor] = None,
                sincos_gamma: Optional[Tensor] = None) -> Tensor:
        return wigner_d_matrix(self.identity, alpha, beta, gamma, sincos_alpha, sincos_beta, sincos_gamma, self.info,
                               irreps=self.irreps)

    def extra_repr(self) -> str:
        return f"irreps={self.irreps}"
