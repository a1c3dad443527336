"""Wigner-D rotations from sparse z-rotations and the J matrix
(``equitorch/nn/functional/wigner_d.py:14-139``): ``D(a, b, c) = Dz(a) J Dz(b) J Dz(c)``."""
from typing import Optional

import torch
from torch import Tensor

from ...ops import wigner_op as _wop
from ...structs import WignerRotationInfo
from .angular import sincos
from .sparse_product import sparse_vecsca
from .sparse_scale import sparse_scale


#: set to True to build D through the sparse z-rotation passes (twice differentiable) instead of the fused kernel
FORCE_SPARSE = False


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


class _DenseRotation(torch.autograd.Function):
    """``matrix (N, D, D) @ x (N, D, C)`` (``transposed``: ``matrix^T @ x``) on the shared-memory kernels.
    ``row_range``: the matrices are block diagonal (see ``ops.wigner_op.block_row_range``)."""

    @staticmethod
    def forward(ctx, x: Tensor, matrix: Tensor, transposed: bool, row_range):
        ctx.save_for_backward(x if matrix.requires_grad else None, matrix if x.requires_grad else None)
        ctx.transposed, ctx.row_range = transposed, row_range
        return _wop.dense_rotation(matrix, x, transposed, row_range)

    @staticmethod
    def backward(ctx, grad: Tensor):
        x, matrix = ctx.saved_tensors
        grad = grad.contiguous()
        gx = gm = None
        if ctx.needs_input_grad[0]:
            gx = _DenseRotation.apply(grad, matrix, not ctx.transposed, ctx.row_range)
        if ctx.needs_input_grad[1]:
            # d/dM of M x is g x^T; of M^T x it is x g^T
            gm = (_RotationGradMatrix.apply(x, grad, ctx.row_range) if ctx.transposed
                  else _RotationGradMatrix.apply(grad, x, ctx.row_range))
        return gx, gm, None, None


class _RotationGradMatrix(torch.autograd.Function):
    """``a (N, D, C), b (N, D, C) -> a @ b^T (N, D, D)`` (restricted to the diagonal blocks with ``row_range``)."""

    @staticmethod
    def forward(ctx, a: Tensor, b: Tensor, row_range):
        ctx.save_for_backward(a if b.requires_grad else None, b if a.requires_grad else None)
        ctx.row_range = row_range
        return _wop.dense_rotation_grad_matrix(a.contiguous(), b.contiguous(), row_range)

    @staticmethod
    def backward(ctx, grad: Tensor):
        a, b = ctx.saved_tensors
        grad = grad.contiguous()
        ga = _DenseRotation.apply(b, grad, False, ctx.row_range) if ctx.needs_input_grad[0] else None      # g b
        gb = _DenseRotation.apply(a, grad, True, ctx.row_range) if ctx.needs_input_grad[1] else None       # g^T a
        return ga, gb, None


def dense_wigner_rotation(input: Tensor, wigner_d: Tensor, row_range: Optional[Tensor] = None) -> Tensor:
    """``wigner_d (N, dim, dim) @ input (N, dim, C)``.  A ``wigner_d`` that is the transposed view of a contiguous
    tensor (``d.transpose(-1, -2)``, the inverse rotation) is applied without materialising the transpose.
    ``row_range`` declares the matrices block diagonal over the irreps: only the blocks are read and multiplied, and
    the gradient with respect to ``wigner_d`` is zero outside them."""
    if wigner_d.ndim == 3 and input.ndim == 3:
        if wigner_d.is_contiguous() and _wop.rotation_supported(wigner_d, input):
            return _DenseRotation.apply(input.contiguous(), wigner_d, False, row_range)
        base = wigner_d.transpose(-1, -2)
        if base.is_contiguous() and _wop.rotation_supported(base, input):
            return _DenseRotation.apply(input.contiguous(), base, True, row_range)
    return wigner_d @ input


class _WignerDFromAngles(torch.autograd.Function):
    """Dense block-diagonal D (N, dim, dim) from the three angle vectors in one kernel; the backward pass turns
    grad_D into the three angle gradients in one kernel."""

    @staticmethod
    def forward(ctx, alpha: Tensor, beta: Tensor, gamma: Tensor, table):
        ctx.save_for_backward(alpha, beta, gamma)
        ctx.table = table
        return _wop.wigner_d_forward(table, alpha, beta, gamma)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, grad: Tensor):
        alpha, beta, gamma = ctx.saved_tensors
        ga, gb, gc = _wop.wigner_d_backward(ctx.table, alpha, beta, gamma, grad)
        return ga, gb, gc, None


def wigner_d_from_angles(alpha: Tensor, beta: Tensor, gamma: Tensor, irreps) -> Tensor:
    """``D(alpha, beta, gamma) = Dz(alpha) J Dz(beta) J Dz(gamma)`` for CUDA angle vectors (float32 / float64)."""
    table = _wop.wigner_table(irreps, alpha.device, alpha.dtype)
    return _WignerDFromAngles.apply(alpha, beta, gamma, table)


def wigner_d_matrix(eye: Tensor, alpha: Optional[Tensor] = None, beta: Optional[Tensor] = None,
                    gamma: Optional[Tensor] = None, sincos_alpha: Optional[Tensor] = None,
                    sincos_beta: Optional[Tensor] = None, sincos_gamma: Optional[Tensor] = None,
                    info: Optional[WignerRotationInfo] = None, irreps=None) -> Tensor:
    """Dense D-matrices.  With all three angles given as CUDA vectors (and ``irreps`` known) one kernel writes D
    from the angles; otherwise (packed sin/cos inputs, missing factors, higher-order derivatives with
    ``FORCE_SPARSE = True``) D is obtained by rotating the columns of the identity with the sparse z-rotations."""
    assert info is not None
    if (irreps is not None and not FORCE_SPARSE and alpha is not None and beta is not None and gamma is not None
            and sincos_alpha is None and sincos_beta is None and sincos_gamma is None
            and _wop.supported(irreps, alpha, beta, gamma) and alpha.shape[0] > 0):
        return wigner_d_from_angles(alpha, beta, gamma, irreps)
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
