"""Differentiable per-irrep scale and dot (autograd layer over ``ops.irrep_ops``).

Each gradient is again one of the two operators, so derivatives of any order are available:

    scale(x, s)  ->  grad x = scale(g, s) ;  grad s = dot(g, x) reduced to the shape of s
    dot(a, b)    ->  grad a = scale(b, g) ;  grad b = scale(a, g)
"""
from __future__ import annotations

from torch import Tensor
from torch.autograd import Function

from ...ops import irrep_ops as _ops
from ...structs import IrrepsInfo


class IrrepScale(Function):
    @staticmethod
    def forward(ctx, x: Tensor, s: Tensor, info: IrrepsInfo, mode: int) -> Tensor:
        ctx.save_for_backward(x if s.requires_grad else None, s if x.requires_grad else None)
        ctx.info, ctx.mode = info, mode
        return _ops.irrep_scale(x, s, info.irrep_index, mode)

    @staticmethod
    def backward(ctx, grad: Tensor):
        x, s = ctx.saved_tensors
        gx = gs = None
        if ctx.needs_input_grad[0]:
            gx = IrrepScale.apply(grad, s, ctx.info, ctx.mode)
        if ctx.needs_input_grad[1]:
            gs = IrrepDot.apply(grad, x, ctx.info)                      # (N, K, C)
            if ctx.mode == _ops.SHARED:
                gs = gs.sum(dim=0)
            elif ctx.mode == _ops.PER_SAMPLE:
                gs = gs.sum(dim=-1)
        return gx, gs, None, None


class IrrepDot(Function):
    @staticmethod
    def forward(ctx, a: Tensor, b: Tensor, info: IrrepsInfo) -> Tensor:
        ctx.save_for_backward(a if b.requires_grad else None, b if a.requires_grad else None)
        ctx.info = info
        return _ops.irrep_dot(a, b, info.irrep_seg)

    @staticmethod
    def backward(ctx, grad: Tensor):
        a, b = ctx.saved_tensors
        ga = gb = None
        if ctx.needs_input_grad[0]:
            ga = IrrepScale.apply(b, grad, ctx.info, _ops.PER_SAMPLE_CHANNEL)
        if ctx.needs_input_grad[1]:
            gb = IrrepScale.apply(a, grad, ctx.info, _ops.PER_SAMPLE_CHANNEL)
        return ga, gb, None


def irrep_scale(x: Tensor, s: Tensor, info: IrrepsInfo, mode: int) -> Tensor:
    return IrrepScale.apply(x, s, info, mode)


def irrep_dot(a: Tensor, b: Tensor, info: IrrepsInfo) -> Tensor:
    return IrrepDot.apply(a, b, info)
