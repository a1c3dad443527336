"""Tensor products of two channelled operands (``TensorProduct``) and the irrep-wise dot
product.  Names follow ``equitorch/nn/functional/tensor_products.py``:
``tensor_product_uuu`` :9-90, ``tensor_product_uvw`` :92-172, ``tensor_dot_uu`` :173-223.

Both products are their own adjoint family: the gradient with respect to either input is the
same kind of product on role-rotated tables (for ``uvw`` with the weight axes permuted so that
the differentiated operand's channel axis comes last).
"""
from __future__ import annotations

import torch
from torch import Tensor
from torch.autograd import Function

from ...structs import IrrepsInfo, SparseProductInfo, TensorProductInfo
from ._irrep import irrep_dot
from ._tp_common import add, expand_like_inter, save_for_tp_backward
from .linears import _m, _mij, _rot
from .sparse_product import sparse_mat_t_vec, sparse_mul, sparse_outer, sparse_vecmat


class TensorProductUUUDummy(Function):
    """x1 (N, D1, C), x2 (N, D2, C), weight (P, C) | (N, P, C) -> (N, Dout, C)."""

    @staticmethod
    def forward(ctx, input1, input2, weight, tp_info_forward, tp_info_backward1, tp_info_backward2):
        inter = sparse_mul(input1, input2, tp_info_forward.info_Mij_fwd)
        ret = sparse_mul(inter, weight, tp_info_forward.info_M_fwd)
        save_for_tp_backward(ctx, input1, input2, weight, inter,
                             (tp_info_forward, tp_info_backward1, tp_info_backward2))
        return ret, inter

    @staticmethod
    def backward(ctx, grad, grad_inter):
        input1, input2, weight, inter = ctx.saved_tensors
        f = ctx.tp_info[0]
        r1, r2 = _rot(ctx.tp_info)
        grad_inter = expand_like_inter(ctx, grad_inter)
        g1 = g2 = gw = None
        if ctx.needs_input_grad[0]:
            if grad is not None:
                g1 = tensor_product_uuu(input2, grad, weight, *r1)
            if grad_inter is not None:
                g1 = add(g1, sparse_mul(input2, grad_inter, *_mij(f, 1)))
        if ctx.needs_input_grad[1]:
            if grad is not None:
                g2 = tensor_product_uuu(grad, input1, weight, *r2)
            if grad_inter is not None:
                g2 = add(g2, sparse_mul(grad_inter, input1, *_mij(f, 2)))
        if ctx.needs_input_grad[2] and grad is not None:
            gw = sparse_mul(grad, inter, *_m(f, 2), out_accumulated=ctx.weight_ndim == 2)
        return g1, g2, gw, None, None, None


def tensor_product_uuu(input1, input2, weight, tp_info_forward, tp_info_backward1=None, tp_info_backward2=None):
    return TensorProductUUUDummy.apply(input1, input2, weight, tp_info_forward, tp_info_backward1, tp_info_backward2)[0]


class TensorProductUVWDummy(Function):
    """x1 (N, D1, C1), x2 (N, D2, C2), weight (P, C1, C2, Cout) | (N, P, C1, C2, Cout) -> (N, Dout, Cout)."""

    @staticmethod
    def forward(ctx, input1, input2, weight, tp_info_forward, tp_info_backward1, tp_info_backward2):
        inter = sparse_outer(input1, input2, tp_info_forward.info_Mij_fwd)
        ret = sparse_vecmat(inter.flatten(-2), weight.flatten(-3, -2), tp_info_forward.info_M_fwd)
        save_for_tp_backward(ctx, input1, input2, weight, inter,
                             (tp_info_forward, tp_info_backward1, tp_info_backward2))
        return ret, inter

    @staticmethod
    def backward(ctx, grad, grad_inter):
        input1, input2, weight, inter = ctx.saved_tensors
        f = ctx.tp_info[0]
        r1, r2 = _rot(ctx.tp_info)
        grad_inter = expand_like_inter(ctx, grad_inter)
        g1 = g2 = gw = None
        if ctx.needs_input_grad[0]:
            if grad is not None:
                lead = tuple(range(weight.ndim - 3))
                w1 = weight.permute(*lead, -2, -1, -3).contiguous()       # (.., C2, Cout, C1)
                g1 = tensor_product_uvw(input2, grad, w1, *r1)
            if grad_inter is not None:
                g1 = add(g1, sparse_vecmat(input2, grad_inter.transpose(-1, -2).contiguous(), *_mij(f, 1)))
        if ctx.needs_input_grad[1]:
            if grad is not None:
                lead = tuple(range(weight.ndim - 3))
                w2 = weight.permute(*lead, -1, -3, -2).contiguous()       # (.., Cout, C1, C2)
                g2 = tensor_product_uvw(grad, input1, w2, *r2)
            if grad_inter is not None:
                g2 = add(g2, sparse_mat_t_vec(grad_inter, input1, *_mij(f, 2)))
        if ctx.needs_input_grad[2] and grad is not None:
            gw = sparse_outer(grad, inter.flatten(-2), *_m(f, 2), out_accumulated=ctx.weight_ndim == 4)
            gw = gw.transpose(-1, -2).contiguous().unflatten(-2, inter.shape[-2:])
        return g1, g2, gw, None, None, None


#: largest per-call intermediate (N, num_Mij, C1, C2) of the 'uvw' product in bytes; larger batches are processed in
#: slices of samples whose intermediate stays below it
UVW_INTERMEDIATE_LIMIT = 1 << 30


class TensorProductUVWChunked(Function):
    """'uvw' product with weights shared by the batch, evaluated slice by slice over the samples.

    The two-step chain materialises ``(N, num_Mij, C1, C2)`` - 1.6 MB per sample at l_max 3 and 64 channels - and
    keeps it for the backward pass.  Here the forward pass runs the chain on slices of the batch and keeps
    nothing but the inputs; the backward pass recomputes the intermediate of a slice, differentiates the slice
    and adds up the weight gradient.  Memory is bounded by ``UVW_INTERMEDIATE_LIMIT`` whatever the batch size;
    within a slice the contraction with the weights (K = C1 * C2 per path) and the weight gradient run on the
    tensor-core paths of the indexed products."""

    @staticmethod
    def forward(ctx, input1, input2, weight, tp_info_forward, tp_info_backward1, tp_info_backward2, chunk):
        infos = (tp_info_forward, tp_info_backward1, tp_info_backward2)
        with torch.no_grad():
            outs = [TensorProductUVWDummy.apply(input1[s:s + chunk], input2[s:s + chunk], weight, *infos)[0]
                    for s in range(0, input1.shape[0], chunk)]
        ctx.save_for_backward(input1, input2, weight)
        ctx.infos, ctx.chunk = infos, chunk
        return torch.cat(outs, dim=0)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, grad):
        input1, input2, weight = ctx.saved_tensors
        need = ctx.needs_input_grad[:3]
        g1 = torch.empty_like(input1) if need[0] else None
        g2 = torch.empty_like(input2) if need[1] else None
        gw = torch.zeros_like(weight) if need[2] else None
        for s in range(0, input1.shape[0], ctx.chunk):
            sl = slice(s, s + ctx.chunk)
            with torch.enable_grad():
                a = input1[sl].detach().requires_grad_(need[0])
                b = input2[sl].detach().requires_grad_(need[1])
                # the reference's backward needs a weight that requires grad (it saves the intermediate only then)
                w = weight.detach().requires_grad_(True)
                out = TensorProductUVWDummy.apply(a, b, w, *ctx.infos)[0]
                wanted = [t for t, n in zip((a, b, w), need) if n]
                got = iter(torch.autograd.grad(out, wanted, grad[sl]))
            if need[0]:
                g1[sl] = next(got)
            if need[1]:
                g2[sl] = next(got)
            if need[2]:
                gw += next(got)
        return g1, g2, gw, None, None, None, None


def tensor_product_uvw(input1, input2, weight, tp_info_forward, tp_info_backward1=None, tp_info_backward2=None):
    if weight.ndim == 4 and input1.ndim == 3 and input2.ndim == 3 and input1.shape[0] == input2.shape[0]:
        per_sample = (tp_info_forward.info_Mij_fwd.out_size * input1.shape[-1] * input2.shape[-1] * input1.element_size())
        if per_sample * input1.shape[0] > UVW_INTERMEDIATE_LIMIT:
            chunk = max(1, UVW_INTERMEDIATE_LIMIT // per_sample)
            if chunk >= 512:
                chunk = chunk // 512 * 512           # whole tiles for the tensor-core paths
            return TensorProductUVWChunked.apply(input1, input2, weight, tp_info_forward, tp_info_backward1,
                                                 tp_info_backward2, chunk)
    return TensorProductUVWDummy.apply(input1, input2, weight, tp_info_forward, tp_info_backward1, tp_info_backward2)[0]


class TensorDotUU(Function):
    """Per-irrep dot product on the table-driven sparse products (operands of different shape, e.g. one of them
    shared by the batch)."""

    @staticmethod
    def forward(ctx, input1: Tensor, input2: Tensor, irreps_info: IrrepsInfo, scaled: bool = True):
        infos = (SparseProductInfo(seg_out=irreps_info.irrep_seg),
                 SparseProductInfo(index2=irreps_info.irrep_index),
                 SparseProductInfo(index1=irreps_info.irrep_index))
        ret = sparse_mul(input1, input2, *infos)
        if scaled:
            ret = ret * irreps_info.rsqrt_dims.to(ret.dtype).unsqueeze(-1)
        ctx.save_for_backward(input1 if input2.requires_grad else None, input2 if input1.requires_grad else None)
        ctx.infos, ctx.irreps_info, ctx.scaled = infos, irreps_info, scaled
        return ret

    @staticmethod
    def backward(ctx, grad):
        input1, input2 = ctx.saved_tensors
        fwd, bwd1, bwd2 = ctx.infos
        if ctx.scaled:
            grad = grad * ctx.irreps_info.rsqrt_dims.to(grad.dtype).unsqueeze(-1)
        g1 = sparse_mul(input2, grad, bwd1, bwd2, fwd) if ctx.needs_input_grad[0] else None
        g2 = sparse_mul(grad, input1, bwd2, fwd, bwd1) if ctx.needs_input_grad[1] else None
        return g1, g2, None, None


def tensor_dot_uu(input1: Tensor, input2: Tensor, irreps_info: IrrepsInfo, scaled: bool = True) -> Tensor:
    """Per-irrep dot product over the components, (N, D, C) x (N, D, C) -> (N, num_irreps, C), divided by
    sqrt(2l + 1) when ``scaled`` (``TensorDotUU``, equitorch/nn/functional/tensor_products.py:173-223).  Operands of
    equal shape and dtype take one pass of the streaming per-irrep dot kernel, whose gradients are the per-irrep
    scale kernel (``_irrep.IrrepDot``)."""
    if input1.shape != input2.shape or input1.dtype != input2.dtype or input1.ndim != 3:
        return TensorDotUU.apply(input1, input2, irreps_info, scaled)
    ret = irrep_dot(input1, input2, irreps_info)
    if scaled:
        ret = ret * irreps_info.rsqrt_dims.to(ret.dtype).unsqueeze(-1)
    return ret


def tensor_dot_uv(input1, input2, irreps_info, scaled=True):
    """Channel-cartesian irrep-wise dot product; not implemented by the reference either
    (``equitorch/nn/functional/tensor_products.py:225-235``)."""
    raise NotImplementedError("tensor_dot_uv")
