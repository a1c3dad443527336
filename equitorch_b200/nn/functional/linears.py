"""Tensor products whose second operand has no channel axis (``SO3Linear``), their adjoints,
and the per-irrep channel mixing layers.

Function names and argument order follow ``equitorch/nn/functional/linears.py``:
``tensor_product_u1u`` (= ``so3_linear_uu``) :16-93, ``_1uu`` :98-173, ``_uu1`` :175-252,
``_u1v`` (= ``so3_linear_uv``) :254-336, ``_1vu`` :339-414, ``_vu1`` :415-492,
``irrep_wise_linear`` :494-530, ``irreps_linear`` :532-574, ``so2_linear_uu/uv`` :576-577.

The letter pattern reads (input1, input2, output): ``u``/``v`` = channelled operand,
``1`` = channel-less operand.  The three members of a family are each other's adjoints: the
gradient of ``u1u`` with respect to its first input is a ``1uu`` product on the tables with
roles rotated once (``tp_info_backward1``), with respect to its second input a ``uu1`` product
on the tables rotated twice (``tp_info_backward2``), and so on cyclically.
"""
from __future__ import annotations

import torch
from torch import Tensor
from torch.autograd import Function

from ...ops.graph_ops import segment_sum  # noqa: F401  (re-exported for users of the functional API)
from ...ops.indexed_product_scale_segment_op import indexed_vecmat_scale_segment
from ...ops.indexed_product_segment_op import indexed_outer_segment
from ...structs import IrrepsInfo, IrrepsLinearInfo, SparseProductInfo, TensorProductInfo
from ._tp_common import add, expand_like_inter, save_for_tp_backward
from .sparse_product import (sparse_inner, sparse_mat_t_vec, sparse_mul, sparse_outer, sparse_scavec,
                             sparse_vecmat, sparse_vecsca)
from .sparse_scale import sparse_scale


def _rot(infos):
    """(fwd, bwd1, bwd2) -> the two cyclic rotations used by the adjoint products."""
    f, b1, b2 = infos
    return (b1, b2, f), (b2, f, b1)


def _mij(info: TensorProductInfo, which: int):
    """Tables of the CG step with roles rotated ``which`` times."""
    t = (info.info_Mij_fwd, info.info_Mij_bwd1, info.info_Mij_bwd2)
    return t[which % 3], t[(which + 1) % 3], t[(which + 2) % 3]


def _m(info: TensorProductInfo, which: int):
    t = (info.info_M_fwd, info.info_M_bwd1, info.info_M_bwd2)
    return t[which % 3], t[(which + 1) % 3], t[(which + 2) % 3]


# ------------------------------------------------------------------------------------------
# uu family: weights (P, C) or (N, P, C), channel-wise
# ------------------------------------------------------------------------------------------
class TensorProductU1UDummy(Function):
    """x (N, D1, C), y (N, D2) -> (N, Dout, C)."""

    @staticmethod
    def forward(ctx, input1, input2, weight, tp_info_forward, tp_info_backward1, tp_info_backward2):
        inter = sparse_vecsca(input1, input2, tp_info_forward.info_Mij_fwd)
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
                g1 = tensor_product_1uu(input2, grad, weight, *r1)
            if grad_inter is not None:
                g1 = add(g1, sparse_scavec(input2, grad_inter, *_mij(f, 1)))
        if ctx.needs_input_grad[1]:
            if grad is not None:
                g2 = tensor_product_uu1(grad, input1, weight, *r2)
            if grad_inter is not None:
                g2 = add(g2, sparse_inner(grad_inter, input1, *_mij(f, 2)))
        if ctx.needs_input_grad[2] and grad is not None:
            gw = sparse_mul(grad, inter, *_m(f, 2), out_accumulated=ctx.weight_ndim == 2)
        return g1, g2, gw, None, None, None


class TensorProduct1UUDummy(Function):
    """y (N, D1), x (N, D2, C) -> (N, Dout, C)."""

    @staticmethod
    def forward(ctx, input1, input2, weight, tp_info_forward, tp_info_backward1, tp_info_backward2):
        inter = sparse_scavec(input1, input2, tp_info_forward.info_Mij_fwd)
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
                g1 = tensor_product_uu1(input2, grad, weight, *r1)
            if grad_inter is not None:
                g1 = add(g1, sparse_inner(input2, grad_inter, *_mij(f, 1)))
        if ctx.needs_input_grad[1]:
            if grad is not None:
                g2 = tensor_product_u1u(grad, input1, weight, *r2)
            if grad_inter is not None:
                g2 = add(g2, sparse_vecsca(grad_inter, input1, *_mij(f, 2)))
        if ctx.needs_input_grad[2] and grad is not None:
            gw = sparse_mul(grad, inter, *_m(f, 2), out_accumulated=ctx.weight_ndim == 2)
        return g1, g2, gw, None, None, None


class TensorProductUU1Dummy(Function):
    """x1 (N, D1, C), x2 (N, D2, C) -> (N, Dout): channels are contracted with the weight."""

    @staticmethod
    def forward(ctx, input1, input2, weight, tp_info_forward, tp_info_backward1, tp_info_backward2):
        inter = sparse_mul(input1, input2, tp_info_forward.info_Mij_fwd)
        ret = sparse_inner(inter, weight, tp_info_forward.info_M_fwd)
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
                g1 = tensor_product_u1u(input2, grad, weight, *r1)
            if grad_inter is not None:
                g1 = add(g1, sparse_mul(input2, grad_inter, *_mij(f, 1)))
        if ctx.needs_input_grad[1]:
            if grad is not None:
                g2 = tensor_product_1uu(grad, input1, weight, *r2)
            if grad_inter is not None:
                g2 = add(g2, sparse_mul(grad_inter, input1, *_mij(f, 2)))
        if ctx.needs_input_grad[2] and grad is not None:
            gw = sparse_scavec(grad, inter, *_m(f, 2), out_accumulated=ctx.weight_ndim == 2)
        return g1, g2, gw, None, None, None


def tensor_product_u1u(input1, input2, weight, tp_info_forward, tp_info_backward1=None, tp_info_backward2=None):
    return TensorProductU1UDummy.apply(input1, input2, weight, tp_info_forward, tp_info_backward1, tp_info_backward2)[0]


def tensor_product_1uu(input1, input2, weight, tp_info_forward, tp_info_backward1=None, tp_info_backward2=None):
    return TensorProduct1UUDummy.apply(input1, input2, weight, tp_info_forward, tp_info_backward1, tp_info_backward2)[0]


def tensor_product_uu1(input1, input2, weight, tp_info_forward, tp_info_backward1=None, tp_info_backward2=None):
    return TensorProductUU1Dummy.apply(input1, input2, weight, tp_info_forward, tp_info_backward1, tp_info_backward2)[0]


so3_linear_uu = tensor_product_u1u


# ------------------------------------------------------------------------------------------
# uv family: weights (P, Cin, Cout) or (N, P, Cin, Cout), full channel mixing
# ------------------------------------------------------------------------------------------
class TensorProductU1VDummy(Function):
    """x (N, D1, Cin), y (N, D2) -> (N, Dout, Cout)."""

    @staticmethod
    def forward(ctx, input1, input2, weight, tp_info_forward, tp_info_backward1, tp_info_backward2):
        inter = sparse_vecsca(input1, input2, tp_info_forward.info_Mij_fwd)
        ret = sparse_vecmat(inter, weight, tp_info_forward.info_M_fwd)
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
        wt = weight.transpose(-1, -2).contiguous() if weight is not None and grad is not None else None
        if ctx.needs_input_grad[0]:
            if grad is not None:
                g1 = tensor_product_1vu(input2, grad, wt, *r1)
            if grad_inter is not None:
                g1 = add(g1, sparse_scavec(input2, grad_inter, *_mij(f, 1)))
        if ctx.needs_input_grad[1]:
            if grad is not None:
                g2 = tensor_product_vu1(grad, input1, wt, *r2)
            if grad_inter is not None:
                g2 = add(g2, sparse_inner(grad_inter, input1, *_mij(f, 2)))
        if ctx.needs_input_grad[2] and grad is not None:
            gw = sparse_outer(grad, inter, *_m(f, 2), out_accumulated=ctx.weight_ndim == 3)
            gw = gw.transpose(-1, -2).contiguous()
        return g1, g2, gw, None, None, None


class TensorProduct1VUDummy(Function):
    """y (N, D1), x (N, D2, Cin) -> (N, Dout, Cout)."""

    @staticmethod
    def forward(ctx, input1, input2, weight, tp_info_forward, tp_info_backward1, tp_info_backward2):
        inter = sparse_scavec(input1, input2, tp_info_forward.info_Mij_fwd)
        ret = sparse_vecmat(inter, weight, tp_info_forward.info_M_fwd)
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
                g1 = tensor_product_vu1(input2, grad, weight, *r1)
            if grad_inter is not None:
                g1 = add(g1, sparse_inner(input2, grad_inter, *_mij(f, 1)))
        if ctx.needs_input_grad[1]:
            if grad is not None:
                g2 = tensor_product_u1v(grad, input1, weight.transpose(-1, -2).contiguous(), *r2)
            if grad_inter is not None:
                g2 = add(g2, sparse_vecsca(grad_inter, input1, *_mij(f, 2)))
        if ctx.needs_input_grad[2] and grad is not None:
            gw = sparse_outer(grad, inter, *_m(f, 2), out_accumulated=ctx.weight_ndim == 3)
            gw = gw.transpose(-1, -2).contiguous()
        return g1, g2, gw, None, None, None


class TensorProductVU1Dummy(Function):
    """g (N, D1, Cout), x (N, D2, Cin), weight (.., P, Cout, Cin) -> (N, Dout).

    Weights first: u = g W per (path, component of input1), v = <u, x> per CG entry, then the
    CG-scaled sum of v into the channel-less output.  No intermediate is exposed.
    """

    @staticmethod
    def forward(ctx, input1, input2, weight, tp_info_forward, tp_info_backward1, tp_info_backward2):
        f = tp_info_forward
        u = sparse_vecmat(input1, weight, f.info_kM1j_fwd)
        v = sparse_inner(u, input2, f.info_kM1M2_fwd)
        ret = sparse_scale(v.unsqueeze(-1), f.info_M_kM1M2_fwd).squeeze(-1)
        g1, g2 = input1.requires_grad, input2.requires_grad
        ctx.save_for_backward(input1 if (g2 or weight.requires_grad) else None, input2 if (g1 or weight.requires_grad) else None,
                              weight if (g1 or g2) else None)
        ctx.tp_info = (tp_info_forward, tp_info_backward1, tp_info_backward2)
        ctx.set_materialize_grads(False)
        return ret, None

    @staticmethod
    def backward(ctx, grad, _unused):
        input1, input2, weight = ctx.saved_tensors
        f = ctx.tp_info[0]
        r1, r2 = _rot(ctx.tp_info)
        g1 = g2 = gw = None
        if grad is None:
            return None, None, None, None, None, None
        if ctx.needs_input_grad[0]:
            g1 = tensor_product_u1v(input2, grad, weight.transpose(-1, -2).contiguous(), *r1)
        if ctx.needs_input_grad[1]:
            g2 = tensor_product_1vu(grad, input1, weight, *r2)
        if ctx.needs_input_grad[2]:
            gv = sparse_scale(grad.unsqueeze(-1), f.info_M_kM1M2_bwd, f.info_M_kM1M2_fwd).squeeze(-1)
            gu = sparse_vecsca(input2, gv, f.info_kM1M2_bwd1, f.info_kM1M2_bwd2, f.info_kM1M2_fwd)
            gw = sparse_outer(gu, input1, f.info_kM1j_bwd2, f.info_kM1j_fwd, f.info_kM1j_bwd1,
                              out_accumulated=weight is not None and weight.ndim == 3)
            gw = gw.transpose(-1, -2).contiguous()
        return g1, g2, gw, None, None, None


def tensor_product_u1v(input1, input2, weight, tp_info_forward, tp_info_backward1=None, tp_info_backward2=None):
    return TensorProductU1VDummy.apply(input1, input2, weight, tp_info_forward, tp_info_backward1, tp_info_backward2)[0]


def tensor_product_1vu(input1, input2, weight, tp_info_forward, tp_info_backward1=None, tp_info_backward2=None):
    return TensorProduct1VUDummy.apply(input1, input2, weight, tp_info_forward, tp_info_backward1, tp_info_backward2)[0]


def tensor_product_vu1(input1, input2, weight, tp_info_forward, tp_info_backward1=None, tp_info_backward2=None):
    return TensorProductVU1Dummy.apply(input1, input2, weight, tp_info_forward, tp_info_backward1, tp_info_backward2)[0]


so3_linear_uv = tensor_product_u1v


# ------------------------------------------------------------------------------------------
# per-irrep channel mixing
# ------------------------------------------------------------------------------------------
class IrrepWiseLinear(Function):
    """``out[n, M, :] = x[n, M, :] @ W[irrep(M)]`` with W (num_irreps, Cin, Cout) or per sample."""

    @staticmethod
    def forward(ctx, input: Tensor, weight: Tensor, irreps_info: IrrepsInfo):
        infos = (SparseProductInfo(index2=irreps_info.irrep_index),
                 SparseProductInfo(index1=irreps_info.irrep_index),
                 SparseProductInfo(seg_out=irreps_info.irrep_seg))
        ctx.save_for_backward(input, weight)
        ctx.infos = infos
        return sparse_vecmat(input, weight, infos[0])

    @staticmethod
    def backward(ctx, grad):
        input, weight = ctx.saved_tensors
        fwd, bwd1, bwd2 = ctx.infos
        gx = gw = None
        if ctx.needs_input_grad[0]:
            gx = sparse_mat_t_vec(weight.transpose(-1, -2), grad, bwd1, bwd2, fwd)
        if ctx.needs_input_grad[1]:
            gw = sparse_outer(grad, input, bwd2, fwd, bwd1, weight.ndim == 3).transpose(-1, -2).contiguous()
        return gx, gw, None


irrep_wise_linear = IrrepWiseLinear.apply


class IrrepsLinear(Function):
    """Channel mixing between every pair of equal irreps of the input and the output
    (``equitorch/nn/functional/linears.py:532-574``).  The reference scatters the per-row results
    to their output components with a third-party ``scatter``; the rows are already unique and
    sorted, so here ``M_out`` is handed to the kernel as its output-row table."""

    @staticmethod
    def forward(ctx, input: Tensor, weight: Tensor, info_forward: IrrepsLinearInfo, info_backward: IrrepsLinearInfo):
        from ...ops.batched_sparse_dense_op import indexed_vecmat_scale_gather
        f = info_forward
        out = indexed_vecmat_scale_gather(input, weight, scale=f.scale_MM0, index1=f.M0_MM0, index2=f.ii0_MM0,
                                          seg=f.M_seg_MM0, index_out=f.M_out, out_size=f.out_size)
        ctx.save_for_backward(input, weight)
        ctx.infos = (info_forward, info_backward)
        return out

    @staticmethod
    def backward(ctx, grad):
        input, weight = ctx.saved_tensors
        f, b = ctx.infos
        gx = gw = None
        if ctx.needs_input_grad[0]:
            gx = IrrepsLinear.apply(grad, weight.transpose(-1, -2), b, f)
        if ctx.needs_input_grad[1]:
            gw = indexed_outer_segment(input, grad, index1=f.M0_ii0MM0, index2=f.M_ii0MM0, seg=f.ii0_seg_ii0MM0,
                                       accumulated=weight.ndim == 3)
            gw = gw * f.scales_ii0.to(gw.dtype).unsqueeze(-1).unsqueeze(-1)
        return gx, gw, None, None


irreps_linear = IrrepsLinear.apply

so2_linear_uu = sparse_mul
so2_linear_uv = sparse_vecmat

__all__ = ["tensor_product_u1u", "tensor_product_1uu", "tensor_product_uu1", "tensor_product_u1v",
           "tensor_product_1vu", "tensor_product_vu1", "so3_linear_uu", "so3_linear_uv", "irrep_wise_linear",
           "irreps_linear", "so2_linear_uu", "so2_linear_uv", "indexed_vecmat_scale_segment"]
