"""Products of un-indexed operands summed over CSR segments.  Presets as in
``equitorch/ops/product_segment_op.py:11-124``.  In the reference three of the five forward
an unknown keyword and raise; here all five work."""
from .batched_sparse_dense_op import (indexed_inner_scale_gather, indexed_mul_scale_gather,
                                      indexed_outer_scale_gather, indexed_vecmat_scale_gather,
                                      indexed_vecsca_scale_gather)


def _preset(fn):
    def op(input1, input2, seg, out=None, accumulated=False, **tile_kwargs):
        return fn(input1, input2, seg=seg, out=out, out_accumulated=accumulated)
    op.__name__ = fn.__name__.replace("indexed_", "").replace("_scale_gather", "_segment")
    return op


mul_segment = _preset(indexed_mul_scale_gather)
outer_segment = _preset(indexed_outer_scale_gather)
inner_segment = _preset(indexed_inner_scale_gather)
vecmat_segment = _preset(indexed_vecmat_scale_gather)
vecsca_segment = _preset(indexed_vecsca_scale_gather)
