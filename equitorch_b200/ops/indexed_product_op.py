"""Indexed products without scaling or segment reduction (one table entry per output row).
Keyword presets over the generic products, as in ``equitorch/ops/indexed_product_op.py:11-119``."""
from .batched_sparse_dense_op import (indexed_inner_scale_gather, indexed_mul_scale_gather,
                                      indexed_outer_scale_gather, indexed_vecmat_scale_gather,
                                      indexed_vecsca_scale_gather)


def _preset(fn):
    def op(input1, input2, index1=None, index2=None, out=None, **tile_kwargs):
        assert index1 is not None or index2 is not None
        return fn(input1, input2, index1=index1, index2=index2, out=out)
    op.__name__ = fn.__name__.replace("_scale_gather", "")
    op.__doc__ = f"``{fn.__name__}`` with only ``index1``/``index2``."
    return op


indexed_mul = _preset(indexed_mul_scale_gather)
indexed_outer = _preset(indexed_outer_scale_gather)
indexed_inner = _preset(indexed_inner_scale_gather)
indexed_vecmat = _preset(indexed_vecmat_scale_gather)
indexed_vecsca = _preset(indexed_vecsca_scale_gather)
