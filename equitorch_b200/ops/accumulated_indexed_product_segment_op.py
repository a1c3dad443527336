"""Indexed products summed over CSR segments **and** over the batch (shared-operand
gradients).  Presets as in ``equitorch/ops/accumulated_indexed_product_segment_op.py:9-150``."""
from .batched_sparse_dense_op import (indexed_inner_scale_gather, indexed_mul_scale_gather,
                                      indexed_outer_scale_gather, indexed_vecmat_scale_gather,
                                      indexed_vecsca_scale_gather)


def _preset(fn):
    def op(input1, input2, index1=None, index2=None, seg=None, out=None, **tile_kwargs):
        assert seg is not None, "seg cannot be None for segment operations"
        assert index1 is not None or index2 is not None, "At least one of index1 or index2 must be provided"
        return fn(input1, input2, index1=index1, index2=index2, seg=seg, out=out, out_accumulated=True)
    op.__name__ = "accumulated_" + fn.__name__.replace("_scale_gather", "_segment")
    return op


accumulated_indexed_mul_segment = _preset(indexed_mul_scale_gather)
accumulated_indexed_outer_segment = _preset(indexed_outer_scale_gather)
accumulated_indexed_inner_segment = _preset(indexed_inner_scale_gather)
accumulated_indexed_vecmat_segment = _preset(indexed_vecmat_scale_gather)
accumulated_indexed_vecsca_segment = _preset(indexed_vecsca_scale_gather)
