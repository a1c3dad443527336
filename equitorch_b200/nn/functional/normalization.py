"""RMS normalisation of equivariant features (mirrors ``equitorch/nn/functional/normalization.py:8-160``)."""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from torch.autograd import Function
from torch.autograd.function import once_differentiable

from ...ops import irrep_ops as _iops
from ...ops.irrep_ops import PER_SAMPLE, SHARED
from ...structs import IrrepsInfo
from ._irrep import irrep_scale
from .norm import batch_mean_squared_norm, channel_mean_squared_norm


def batch_rms_norm(input: Tensor, running_squared_norm: Tensor, irreps_info: IrrepsInfo, weight: Optional[Tensor] = None,
                   scaled: bool = True, training: bool = False, momentum: float = 0.1, eps: float = 1e-05) -> Tensor:
    """``out[n, i, c] = x[n, i, c] * weight[k, c] / sqrt(stat[k, c] + eps)``, ``k = irrep(i)``; ``stat`` is the
    batch mean of the (scaled) squared norms when training (``running_squared_norm`` is updated in place),
    else ``running_squared_norm``."""
    if training:
        stat = batch_mean_squared_norm(input, irreps_info, scaled)
        running_squared_norm.data.lerp_(stat.detach().to(running_squared_norm.dtype), momentum)
    else:
        stat = running_squared_norm
    scale = torch.rsqrt(stat + eps)
    if weight is not None:
        scale = weight * scale
    return irrep_scale(input, scale.to(input.dtype), irreps_info, SHARED)


#: use the fused one-pass LayerRMSNorm kernels when the input allows it (first derivatives only; set to False
#: for higher-order derivatives, which the composition of per-irrep operators below provides)
FUSED_LAYER_RMS = True


class _LayerRMSNormFused(Function):
    @staticmethod
    def forward(ctx, x: Tensor, weight: Optional[Tensor], info: IrrepsInfo, scaled: bool, eps: float) -> Tensor:
        out, rsigma = _iops.layer_rms_forward(x, weight, info.irrep_seg, scaled, eps)
        ctx.save_for_backward(x, weight, rsigma)
        ctx.info, ctx.scaled = info, scaled
        return out

    @staticmethod
    @once_differentiable
    def backward(ctx, grad: Tensor):
        x, weight, rsigma = ctx.saved_tensors
        need_w = weight is not None and ctx.needs_input_grad[1]
        gx, gw = _iops.layer_rms_backward(x, grad, weight, rsigma, ctx.info.irrep_seg, ctx.scaled, need_w)
        return gx, (gw.to(weight.dtype) if gw is not None else None), None, None, None


def layer_rms_norm(input_tensor: Tensor, irreps_info: IrrepsInfo, weight: Optional[Tensor] = None, scaled: bool = True,
                   eps: float = 1e-05) -> Tensor:
    """``out[n, i, c] = x[n, i, c] * weight[k, c] / sqrt(mean_c |x[n, irrep k]|^2 (/ dim_k) + eps)``."""
    if FUSED_LAYER_RMS and _iops.layer_rms_supported(input_tensor, irreps_info.num_irreps):
        return _LayerRMSNormFused.apply(input_tensor, weight, irreps_info, scaled, eps)
    rsigma = torch.rsqrt(channel_mean_squared_norm(input_tensor, irreps_info, scaled) + eps)      # (N, K)
    out = irrep_scale(input_tensor, rsigma, irreps_info, PER_SAMPLE)
    if weight is not None:
        out = irrep_scale(out, weight.to(out.dtype), irreps_info, SHARED)
    return out
