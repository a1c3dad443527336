"""Indexed products summed over CSR segments, no scaling.  Presets as in
``equitorch/ops/indexed_product_segment_op.py:11-146`` (only the outer product takes
``accumulated`` there, and so it does here)."""
from .batched_sparse_dense_op import (indexed_inner_scale_gather, indexed_mul_scale_gather,
                                      indexed_outer_scale_gather, indexed_vecmat_scale_gather,
                                      indexed_vecsca_scale_gather)

_MSG_SEG = "seg cannot be None for segment operations"
_MSG_IDX = "At least one of index1 or index2 must be provided"


def _preset(fn, with_accumulated=False):
    if with_accumulated:
        def op(input1, input2, index1=None, index2=None, seg=None, out=None, accumulated=False, **tile_kwargs):
            assert seg is not None, _MSG_SEG
            assert index1 is not None or index2 is not None, _MSG_IDX
            return fn(input1, input2, index1=index1, index2=index2, seg=seg, out=out, out_accumulated=accumulated)
    else:
        def op(input1, input2, index1=None, index2=None, seg=None, out=None, **tile_kwargs):
            assert seg is not None, _MSG_SEG
            assert index1 is not None or index2 is not None, _MSG_IDX
            return fn(input1, input2, index1=index1, index2=index2, seg=seg, out=out)
    op.__name__ = fn.__name__.replace("_scale_gather", "_segment")
    return op


indexed_mul_segment = _preset(indexed_mul_scale_gather)
indexed_outer_segment = _preset(indexed_outer_scale_gather, with_accumulated=True)
indexed_inner_segment = _preset(indexed_inner_scale_gather)
indexed_vecmat_segment = _preset(indexed_vecmat_scale_gather)
indexed_vecsca_segment = _preset(indexed_vecsca_scale_gather)
