"""Per-irrep norms (mirrors ``equitorch/nn/functional/norm.py:14-276``).

The reduction over the components of an irrep is the segmented form of the sparse ``mul`` kernel
(``x * x`` summed over ``irrep_seg``): one pass over the features, no ``x**2`` intermediate.  Its adjoint
is the indexed form of the same kernel, which the autograd rule of ``sparse_mul`` supplies.
"""
from __future__ import annotations

import torch
from torch import Tensor
from torch.autograd import Function

from ...structs import IrrepsInfo, SparseProductInfo
from .sparse_product import sparse_mul


def _reduce_infos(irreps_info: IrrepsInfo):
    return (SparseProductInfo(seg_out=irreps_info.irrep_seg), SparseProductInfo(index2=irreps_info.irrep_index),
            SparseProductInfo(index1=irreps_info.irrep_index))


def _as3d(x: Tensor):
    """(..., D, C) -> (N, D, C) and the leading shape."""
    return x.reshape(-1, x.shape[-2], x.shape[-1]), x.shape[:-2]


def _sum_squares(x: Tensor, irreps_info: IrrepsInfo) -> Tensor:
    x3, lead = _as3d(x)
    fwd, bwd1, bwd2 = _reduce_infos(irreps_info)
    out = sparse_mul(x3, x3, fwd, bwd1, bwd2)
    return out.reshape(*lead, out.shape[-2], out.shape[-1])


def squared_norm(input_tensor: Tensor, irreps_info: IrrepsInfo, scaled: bool = True) -> Tensor:
    """``out[.., k, c] = sum_{i in irrep k} x[.., i, c]^2``, divided by the irrep's dimension if ``scaled``."""
    out = _sum_squares(input_tensor, irreps_info)
    return out * irreps_info.rdims.unsqueeze(-1) if scaled else out


class _Sqrt0(Function):
    """sqrt with derivative 0 at 0 (the norm of a zero vector has zero gradient, as in the reference)."""

    @staticmethod
    def forward(ctx, s: Tensor) -> Tensor:
        y = torch.sqrt(s)
        ctx.save_for_backward(y)
        return y

    @staticmethod
    def backward(ctx, grad: Tensor):
        (y,) = ctx.saved_tensors
        return grad * torch.reciprocal(2 * y).nan_to_num(posinf=0.0, neginf=0.0)


def norm(input_tensor: Tensor, irreps_info: IrrepsInfo, scaled: bool = True) -> Tensor:
    """L2 norm of every irrep block, times ``dim^-1/2`` if ``scaled``."""
    out = _Sqrt0.apply(_sum_squares(input_tensor, irreps_info))
    return out * irreps_info.rsqrt_dims.unsqueeze(-1) if scaled else out


def channel_mean_squared_norm(input_tensor: Tensor, irreps_info: IrrepsInfo, scaled: bool = True) -> Tensor:
    """Mean over channels of the squared norms: (.., D, C) -> (.., num_irreps)."""
    out = _sum_squares(input_tensor, irreps_info).mean(dim=-1)
    return out * irreps_info.rdims if scaled else out


def batch_mean_squared_norm(input_tensor: Tensor, irreps_info: IrrepsInfo, scaled: bool = True) -> Tensor:
    """Mean over the batch of the squared norms: (N, D, C) -> (num_irreps, C).

    The batch sum is taken inside the kernel (``out_accumulated``), so the (N, num_irreps, C) intermediate
    is never written.
    """
    if input_tensor.ndim != 3:
        return squared_norm(input_tensor, irreps_info, scaled).mean(dim=0)
    fwd, bwd1, bwd2 = _reduce_infos(irreps_info)
    out = sparse_mul(input_tensor, input_tensor, fwd, bwd1, bwd2, True) / input_tensor.shape[0]
    return out * irreps_info.rdims.unsqueeze(-1) if scaled else out
