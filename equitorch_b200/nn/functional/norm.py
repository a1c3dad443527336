"""Per-irrep norms (mirrors ``equitorch/nn/functional/norm.py:14-276``).

The reduction over the components of an irrep is one streaming pass (``irrep_dot`` of the features with
themselves, no ``x**2`` intermediate); its adjoint is ``irrep_scale``.
"""
from __future__ import annotations

import torch
from torch import Tensor
from torch.autograd import Function

from ...structs import IrrepsInfo
from ._irrep import irrep_dot


def _sum_squares(x: Tensor, irreps_info: IrrepsInfo) -> Tensor:
    x3 = x.reshape(-1, x.shape[-2], x.shape[-1])
    out = irrep_dot(x3, x3, irreps_info)
    return out.reshape(*x.shape[:-2], out.shape[-2], out.shape[-1])


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
    """Mean over the batch of the squared norms: (N, D, C) -> (num_irreps, C)."""
    return squared_norm(input_tensor, irreps_info, scaled).mean(dim=0)
