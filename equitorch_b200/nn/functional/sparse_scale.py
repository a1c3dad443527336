"""Differentiable sparse row mixing ``z[M] = sum_t scale[t] x[index[t]]``
(``equitorch/nn/functional/sparse_scale.py:14-47``); the gradient is the same operation on the
transposed table ``info_bwd``."""
from typing import Optional

from torch import Tensor
from torch.autograd import Function

from ...ops.indexed_scale_segment_op import indexed_scale_segment
from ...structs import SparseScaleInfo


class SparseScale(Function):
    @staticmethod
    def forward(ctx, input: Tensor, info_fwd: SparseScaleInfo, info_bwd: Optional[SparseScaleInfo]):
        ctx.infos = (info_fwd, info_bwd)
        return indexed_scale_segment(input, info_fwd.scale, info_fwd.index, info_fwd.seg_out, info_fwd.out_size)

    @staticmethod
    def backward(ctx, grad: Tensor):
        info_fwd, info_bwd = ctx.infos
        if not ctx.needs_input_grad[0]:
            return None, None, None
        if info_bwd is None:
            raise RuntimeError("sparse_scale: info_bwd is required to differentiate the input")
        return SparseScale.apply(grad, info_bwd, info_fwd), None, None


def sparse_scale(input: Tensor, info_fwd: SparseScaleInfo, info_bwd: Optional[SparseScaleInfo] = None) -> Tensor:
    return SparseScale.apply(input, info_fwd, info_bwd)
