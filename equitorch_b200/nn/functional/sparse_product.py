"""Differentiable sparse products (autograd layer over ``equitorch_b200.ops``).

Seven ``torch.autograd.Function``s with the names and call signature of
``equitorch/nn/functional/sparse_product.py:20-500``:

    sparse_<op>(input1, input2, info_fwd, info_bwd1=None, info_bwd2=None, out_accumulated=False)

``info_bwd1`` / ``info_bwd2`` are the role-rotated tables of ``info_fwd`` (as returned by
``sparse_product_infos``): the gradient with respect to an operand is again a sparse product,
of the other operand and the incoming gradient, run on the rotated table, and summed over the
batch when that operand was shared.  Because every backward is expressed with these same
Functions, gradients of any order are available.

Dual products (gradient of input1, gradient of input2):

    mul        -> mul(in2, g)              , mul(g, in1)
    outer      -> vecmat(in2, g^T)         , mat_t_vec(g, in1)
    inner      -> vecsca(in2, g)           , scavec(g, in1)
    vecmat     -> mat_t_vec(in2^T, g)      , outer(g, in1)^T
    vecsca     -> scavec(in2, g)           , inner(g, in1)
    scavec     -> inner(in2, g)            , vecsca(g, in1)
    mat_t_vec  -> outer(in2, g)            , vecmat(g, in1^T)
"""
from __future__ import annotations

from typing import Callable, Dict, Optional

from torch import Tensor
from torch.autograd import Function

from ...ops import batched_sparse_dense_op as _ops
from ...structs import SparseProductInfo


def _t(m: Tensor) -> Tensor:
    return m.transpose(-1, -2).contiguous()


# name -> (operator, batched ndim of input1, batched ndim of input2,
#          dual for grad1 as (name, f(in2, g)), dual for grad2 as (name, f(g, in1)), post-process of grad2)
_SPEC = {
    "mul": (_ops.indexed_mul_scale_gather, 3, 3, ("mul", lambda b, g: (b, g)), ("mul", lambda g, a: (g, a)), None),
    "outer": (_ops.indexed_outer_scale_gather, 3, 3, ("vecmat", lambda b, g: (b, _t(g))),
              ("mat_t_vec", lambda g, a: (g, a)), None),
    "inner": (_ops.indexed_inner_scale_gather, 3, 3, ("vecsca", lambda b, g: (b, g)),
              ("scavec", lambda g, a: (g, a)), None),
    "vecmat": (_ops.indexed_vecmat_scale_gather, 3, 4, ("mat_t_vec", lambda b, g: (_t(b), g)),
               ("outer", lambda g, a: (g, a)), _t),
    "vecsca": (_ops.indexed_vecsca_scale_gather, 3, 2, ("scavec", lambda b, g: (b, g)),
               ("inner", lambda g, a: (g, a)), None),
    "scavec": (_ops.indexed_scavec_scale_gather, 2, 3, ("inner", lambda b, g: (b, g)),
               ("vecsca", lambda g, a: (g, a)), None),
    "mat_t_vec": (_ops.indexed_mat_t_vec_scale_gather, 4, 3, ("outer", lambda b, g: (b, g)),
                  ("vecmat", lambda g, a: (g, _t(a))), None),
}
_FUNCTIONS: Dict[str, type] = {}


def _build(name: str) -> type:
    op, nd1, nd2, dual1, dual2, post2 = _SPEC[name]

    class _Product(Function):
        @staticmethod
        def forward(ctx, input1: Tensor, input2: Tensor, info_fwd: SparseProductInfo,
                    info_bwd1: Optional[SparseProductInfo] = None, info_bwd2: Optional[SparseProductInfo] = None,
                    out_accumulated: bool = False) -> Tensor:
            out = op(input1, input2, info_fwd.scale, info_fwd.index1, info_fwd.index2, info_fwd.seg_out,
                     info_fwd.gather_index, info_fwd.index_out, out_accumulated=out_accumulated,
                     out_size=info_fwd.out_size)
            ctx.save_for_backward(input1 if input2.requires_grad else None,
                                  input2 if input1.requires_grad else None)
            ctx.infos = (info_fwd, info_bwd1, info_bwd2)
            ctx.shared = (input1.ndim < nd1, input2.ndim < nd2)
            return out

        @staticmethod
        def backward(ctx, grad: Tensor):
            input1, input2 = ctx.saved_tensors
            fwd, bwd1, bwd2 = ctx.infos
            grad1 = grad2 = None
            if ctx.needs_input_grad[0]:
                if bwd1 is None:
                    raise RuntimeError(f"sparse_{name}: info_bwd1 is required to differentiate input1")
                a, b = dual1[1](input2, grad)
                grad1 = _FUNCTIONS[dual1[0]].apply(a, b, bwd1, bwd2, fwd, ctx.shared[0])
            if ctx.needs_input_grad[1]:
                if bwd2 is None:
                    raise RuntimeError(f"sparse_{name}: info_bwd2 is required to differentiate input2")
                a, b = dual2[1](grad, input1)
                grad2 = _FUNCTIONS[dual2[0]].apply(a, b, bwd2, fwd, bwd1, ctx.shared[1])
                if post2 is not None:
                    grad2 = post2(grad2)
            return grad1, grad2, None, None, None, None

    _Product.__name__ = _Product.__qualname__ = "Sparse" + "".join(p.capitalize() for p in name.split("_"))
    return _Product


for _name in _SPEC:
    _FUNCTIONS[_name] = _build(_name)

SparseMul, SparseOuter, SparseInner = _FUNCTIONS["mul"], _FUNCTIONS["outer"], _FUNCTIONS["inner"]
SparseVecMat, SparseVecSca, SparseScaVec = _FUNCTIONS["vecmat"], _FUNCTIONS["vecsca"], _FUNCTIONS["scavec"]
SparseMatTVec = _FUNCTIONS["mat_t_vec"]


def _public(name: str) -> Callable:
    fn = _FUNCTIONS[name]

    def product(input1: Tensor, input2: Tensor, info_fwd: SparseProductInfo,
                info_bwd1: Optional[SparseProductInfo] = None, info_bwd2: Optional[SparseProductInfo] = None,
                out_accumulated: bool = False) -> Tensor:
        return fn.apply(input1, input2, info_fwd, info_bwd1, info_bwd2, out_accumulated)

    product.__name__ = f"sparse_{name}"
    product.__doc__ = f"Differentiable ``indexed_{name}_scale_gather`` driven by ``info_fwd`` (see module docstring)."
    return product


sparse_mul = _public("mul")
sparse_outer = _public("outer")
sparse_inner = _public("inner")
sparse_vecmat = _public("vecmat")
sparse_vecsca = _public("vecsca")
sparse_scavec = _public("scavec")
sparse_mat_t_vec = _public("mat_t_vec")
