"""Batched sparse-dense products on the GPU (operator layer).

Same names, argument order and semantics as ``equitorch/ops/batched_sparse_dense_op.py``
of the reference (``indexed_mul_scale_gather`` :277, ``indexed_outer_scale_gather`` :557,
``indexed_inner_scale_gather`` :833, ``indexed_scavec_scale_gather`` :994,
``indexed_mat_t_vec_scale_gather`` :1200, ``indexed_vecmat_scale_gather`` :1511,
``indexed_vecsca_scale_gather`` :1796); each call is one launch of
``eqt_sparse_product`` from ``libeqt_b200.so`` on the current CUDA stream.

Contract kept from the reference:

* an operand with one dimension fewer than its batched form is shared by the batch
  (vector ``(M, C)``, scalar ``(M,)``, matrix ``(M, Cin, Cout)``);
* ``N = max`` of the batch sizes, output ``(N, out_size, ...)`` or ``(out_size, ...)`` when
  ``out_accumulated``; the output dtype is ``torch.result_type(input1, input2)``;
* ``index*``/``seg``/``gather_index`` are int64 tensors on the operands' device, ``None``
  means identity; rows ``[0, num_segments)`` are always written, an empty segment gives zeros;
* tile-size keywords (``block_size_*``, ``num_stages``, ``loop_unroll_factor``) are accepted
  and ignored: tiling is fixed inside the kernels.

Differences: sums are carried in float32 for bfloat16 operands (the reference accumulates
in bfloat16); tensors must be CUDA tensors - there is no CPU implementation here.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch
from torch import Tensor

from .. import _lib
from . import indexed_tc_op as _tc

_ARITH = {torch.float32: torch.float32, torch.bfloat16: torch.float32, torch.float64: torch.float64}

# op -> (batched ndim of input2, position of its sparse dimension counted from the end)
_IN2_LAYOUT = {
    _lib.OP_MUL: (3, 2), _lib.OP_OUTER: (3, 2), _lib.OP_INNER: (3, 2),
    _lib.OP_VECSCA: (2, 1), _lib.OP_VECMAT: (4, 3),
}


def _index(t: Optional[Tensor], name: str, device) -> Optional[Tensor]:
    if t is None:
        return None
    if t.dtype != torch.int64:
        raise TypeError(f"{name} must be an int64 tensor, got {t.dtype}")
    if t.device != device:
        raise _lib.EqtError(f"{name} is on {t.device}, operands are on {device}")
    return t.contiguous()


def sparse_product(op: int, input1: Tensor, input2: Optional[Tensor], scale=None, index1=None, index2=None,
                   seg=None, gather_index=None, index_out=None, out=None, out_accumulated=False,
                   out_size=None) -> Tensor:
    """Shared driver of all products; see the module docstring for the contract."""
    dev = _lib.require_cuda(input1, input2)
    rt = input1.dtype if input2 is None else torch.result_type(input1, input2)
    if rt not in _lib.DTYPE_CODE:
        raise TypeError(f"unsupported dtype {rt}; use float32, float64 or bfloat16")
    arith = _ARITH[rt]
    x = input1.to(rt).contiguous()
    shared1 = x.ndim == 2
    if x.ndim not in (2, 3):
        raise ValueError(f"input1 must be (N, M, C) or (M, C), got {tuple(x.shape)}")
    rows1, c1 = x.shape[-2], x.shape[-1]
    n1 = None if shared1 else x.shape[0]

    if op == _lib.OP_SCALE:
        y, shared2, rows2, c2, n2 = None, True, 0, 0, None
    else:
        y = input2.to(rt).contiguous()
        nd, sparse_pos = _IN2_LAYOUT[op]
        if y.ndim not in (nd - 1, nd):
            raise ValueError(f"input2 has {y.ndim} dims, expected {nd - 1} (shared) or {nd}")
        shared2 = y.ndim == nd - 1
        rows2 = y.shape[-sparse_pos]
        n2 = None if shared2 else y.shape[0]
        c2 = y.shape[-1] if op in (_lib.OP_OUTER, _lib.OP_VECMAT) else 0
        if op in (_lib.OP_MUL, _lib.OP_INNER) and y.shape[-1] != c1:
            raise ValueError(f"channel mismatch: {c1} vs {y.shape[-1]}")
        if op == _lib.OP_VECMAT and y.shape[-2] != c1:
            raise ValueError(f"vector has {c1} channels, matrix expects {y.shape[-2]}")
    if n1 is not None and n2 is not None and n1 != n2:
        # N = max of the two batch sizes as in the reference (:189); the only well-defined unequal case is a
        # batch of one, which is the shared operand with an explicit leading 1
        if n1 == 1:
            x, shared1, n1 = x[0], True, None
        elif n2 == 1:
            y, shared2, n2 = y[0], True, None
        else:
            raise ValueError(f"batch sizes differ: {n1} vs {n2}")
    n = max((v for v in (n1, n2) if v is not None), default=1)

    index1 = _index(index1, "index1", dev)
    index2 = _index(index2, "index2", dev)
    seg = _index(seg, "seg", dev)
    gather_index = _index(gather_index, "gather_index", dev)
    index_out = _index(index_out, "index_out", dev)
    if scale is not None:
        scale = scale.to(device=dev, dtype=arith).contiguous()

    if seg is not None:
        num_out = seg.shape[0] - 1
    elif index1 is not None:
        num_out = index1.shape[0]
    elif index2 is not None:
        num_out = index2.shape[0]
    else:
        num_out = rows1
    if out_size is None:
        out_size = num_out

    # GEMM-shaped cases with an operand shared by the batch go to the tensor cores (float32, channels % 32 == 0)
    if out is None and op == _lib.OP_VECMAT and not shared1 and shared2 \
            and _tc.vecmat_supported(x, y, gather_index, index_out, out_accumulated, out_size, num_out):
        return _tc.vecmat_tc(x, y, scale, index1, index2, seg, num_out)
    elif out is None and op == _lib.OP_OUTER and not shared1 and not shared2 \
            and _tc.outer_supported(x, y, gather_index, index_out, out_accumulated, out_size, num_out):
        return _tc.outer_tc(x, y, scale, index1, index2, seg, num_out)
    elif out is None and op == _lib.OP_OUTER and not shared1 and not shared2 \
            and _tc.outer_supported(y, x, gather_index, index_out, out_accumulated, out_size, num_out):
        # second operand wider than one tile (e.g. a flattened C1 * C2 intermediate): swap the roles, transpose back
        return _tc.outer_tc(y, x, scale, index2, index1, seg, num_out).transpose(-1, -2).contiguous()

    tail = {_lib.OP_OUTER: (c1, c2), _lib.OP_INNER: (), _lib.OP_VECMAT: (c2,)}.get(op, (c1,))
    lead = (out_size,) if out_accumulated else (n, out_size)
    work_dtype = arith if out_accumulated else rt
    must_zero = out_accumulated or index_out is not None or out_size != num_out
    if out is not None:
        # the reference writes into `out`; a buffer the kernels cannot write into is an error, not a silent copy
        if tuple(out.shape) != (*lead, *tail) or out.dtype != rt or out.device != dev or not out.is_contiguous():
            raise ValueError(f"out must be a contiguous {rt} tensor of shape {(*lead, *tail)} on {dev}, got "
                             f"{out.dtype} {tuple(out.shape)} on {out.device} (contiguous: {out.is_contiguous()})")
    if out is not None and out.dtype == work_dtype:
        buf = out          # accumulated / indexed outputs add into the caller's values, as in the reference
    else:
        buf = (torch.zeros if must_zero else torch.empty)((*lead, *tail), dtype=work_dtype, device=dev)
        if out is not None and must_zero:
            buf.copy_(out)     # bfloat16 `out` summed in float32: start from the caller's values

    args = _lib.ProductArgs(
        op=op, dtype=_lib.DTYPE_CODE[rt], shared1=int(shared1), shared2=int(shared2),
        accumulated=int(bool(out_accumulated)), reserved=0,
        in1=x.data_ptr(), in2=_lib.ptr(y), out=buf.data_ptr(), scale=_lib.ptr(scale),
        index1=_lib.ptr(index1), index2=_lib.ptr(index2), seg=_lib.ptr(seg),
        gather_index=_lib.ptr(gather_index), index_out=_lib.ptr(index_out),
        n=n, rows1=rows1, rows2=rows2, num_out=num_out, out_size=out_size, c1=c1, c2=c2)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().eqt_sparse_product(C.byref(args), _lib.stream_ptr(dev)), "eqt_sparse_product")
    if out is not None and buf is not out:
        out.copy_(buf)
        return out
    return buf if buf.dtype == rt else buf.to(rt)


def indexed_mul_scale_gather(input1, input2, scale=None, index1=None, index2=None, seg=None,
                             gather_index=None, index_out=None, out=None, out_accumulated=False,
                             out_size=None, block_size_n=64, block_size_c=64, num_stages=2):
    r"""``out[n, M, c] = \sum_{t \in seg[M]} s_t\, x[n, i1_t, c]\, y[n, i2_t, c]``."""
    return sparse_product(_lib.OP_MUL, input1, input2, scale, index1, index2, seg, gather_index,
                          index_out, out, out_accumulated, out_size)


def indexed_outer_scale_gather(input1, input2, scale=None, index1=None, index2=None, seg=None,
                               gather_index=None, index_out=None, out=None, out_accumulated=False,
                               out_size=None, block_size_n=8, block_size_c1=32, block_size_c2=32, num_stages=2):
    r"""``out[n, M, a, b] = \sum_t s_t\, x[n, i1_t, a]\, y[n, i2_t, b]``."""
    return sparse_product(_lib.OP_OUTER, input1, input2, scale, index1, index2, seg, gather_index,
                          index_out, out, out_accumulated, out_size)


def indexed_inner_scale_gather(input1, input2, scale=None, index1=None, index2=None, seg=None,
                               gather_index=None, index_out=None, out=None, out_accumulated=False,
                               out_size=None, block_size_n=32, block_size_c=32, num_stages=2,
                               loop_unroll_factor=4):
    r"""``out[n, M] = \sum_t s_t \sum_c x[n, i1_t, c]\, y[n, i2_t, c]``."""
    return sparse_product(_lib.OP_INNER, input1, input2, scale, index1, index2, seg, gather_index,
                          index_out, out, out_accumulated, out_size)


def indexed_vecmat_scale_gather(input1, input2, scale=None, index1=None, index2=None, seg=None,
                                gather_index=None, index_out=None, out=None, out_accumulated=False,
                                out_size=None, block_size_n=8, block_size_c_out=32, block_size_c_in=32,
                                num_stages=1, loop_unroll_factor=4):
    r"""``out[n, M, o] = \sum_t s_t \sum_i x[n, i1_t, i]\, W[n, i2_t, i, o]``."""
    return sparse_product(_lib.OP_VECMAT, input1, input2, scale, index1, index2, seg, gather_index,
                          index_out, out, out_accumulated, out_size)


def indexed_vecsca_scale_gather(input1, input2, scale=None, index1=None, index2=None, seg=None,
                                gather_index=None, index_out=None, out=None, out_accumulated=False,
                                out_size=None, block_size_n=64, block_size_c=64, num_stages=2):
    r"""``out[n, M, c] = \sum_t s_t\, x[n, i1_t, c]\, y[n, i2_t]`` (``y`` has no channel axis)."""
    return sparse_product(_lib.OP_VECSCA, input1, input2, scale, index1, index2, seg, gather_index,
                          index_out, out, out_accumulated, out_size)


def indexed_scavec_scale_gather(input1, input2, scale=None, index1=None, index2=None, seg=None,
                                gather_index=None, index_out=None, out=None, out_accumulated=False,
                                out_size=None, block_size_n=64, block_size_c=64, num_stages=2):
    """Scalar (input1) times vector (input2): the vector-scalar product with operands swapped."""
    return sparse_product(_lib.OP_VECSCA, input2, input1, scale, index2, index1, seg, gather_index,
                          index_out, out, out_accumulated, out_size)


def indexed_mat_t_vec_scale_gather(input1, input2, scale=None, index1=None, index2=None, seg=None,
                                   gather_index=None, index_out=None, out=None, out_accumulated=False,
                                   out_size=None, block_size_n=8, block_size_c_in=32, block_size_c_out=32,
                                   num_stages=1, loop_unroll_factor=4):
    """Matrix (input1, ``(.., Cin, Cout)``) applied to vector (input2): vec @ mat with operands swapped."""
    return sparse_product(_lib.OP_VECMAT, input2, input1, scale, index2, index1, seg, gather_index,
                          index_out, out, out_accumulated, out_size)
