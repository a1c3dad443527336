"""Wigner-D rotations from sparse z-rotations and the J matrix
(``equitorch/nn/functional/wigner_d.py:14-139``): ``D(a, b, c) = Dz(a) J Dz(b) J Dz(c)``."""
from typing import Optional

import torch
from torch import Tensor

from ...structs import WignerRotationInfo
from .angular import sincos
from .sparse_product import sparse_vecsca
from .sparse_scale import sparse_scale


def sparse_wigner_rotation(input: Tensor, sincos_alpha: Optional[Tensor], sincos_beta: Optional[Tensor],
                           sincos_gamma: Optional[Tensor], info: WignerRotationInfo) -> Tensor:
    """Rotate features ``(N, dim, C)`` (or a shared ``(dim, C)``) by per-sample Euler angles given as
    packed sin/cos rows; ``None`` skips that factor."""
    z = (info.rotate_z_info_fwd, info.rotate_z_info_bwd_input, info.rotate_z_info_bwd_cs)
    x = input
    if sincos_gamma is not None:
        x = sparse_vecsca(x, sincos_gamma, *z)
    if sincos_beta is not None:
        x = sparse_scale(x, info.j_matrix_info, info.j_matrix_info)
        x = sparse_vecsca(x, sincos_beta, *z)
        x = sparse_scale(x, info.j_matrix_info, info.j_matrix_info)
    if sincos_alpha is not None:
        x = sparse_vecsca(x, sincos_alpha, *z)
    return x


def dense_wigner_rotation(input: Tensor, wigner_d: Tensor) -> Tensor:
    """``wigner_d (N, dim, dim) @ input (N, dim, C)``."""
    return wigner_d @ input


def wigner_d_matrix(eye: Tensor, alpha: Optional[Tensor] = None, beta: Optional[Tensor] = None,
                    gamma: Optional[Tensor] = None, sincos_alpha: Optional[Tensor] = None,
                    sincos_beta: Optional[Tensor] = None, sincos_gamma: Optional[Tensor] = None,
                    info: Optional[WignerRotationInfo] = None) -> Tensor:
    """Dense D-matrices obtained by rotating the columns of the identity."""
    assert info is not None
    if sincos_alpha is None and alpha is not None:
        sincos_alpha = sincos(alpha, info.max_m)
    if sincos_beta is None and beta is not None:
        sincos_beta = sincos(beta, info.max_m)
    if sincos_gamma is None and gamma is not None:
        sincos_gamma = sincos(gamma, info.max_m)
    given = [t for t in (sincos_alpha, sincos_beta, sincos_gamma) if t is not None]
    if eye.shape[0] == 0:
        return torch.empty((given[0].shape[0] if given else 1, 0, 0), device=eye.device, dtype=eye.dtype)
    rotated = sparse_wigner_rotation(eye, sincos_alpha, sincos_beta, sincos_gamma, info)
    batched = any(t.ndim > 1 and t.shape[0] > 1 for t in given)
    if not batched and rotated.ndim == 3 and rotated.shape[0] == 1:
        return rotated.squeeze(0)
    return rotated
