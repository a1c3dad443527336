"""``out[n, M, c] = sum_{t in seg[M]} scale[t] * x[n, index[t], c]`` (a sparse matrix applied
along the second-to-last axis).  Mirrors ``equitorch/ops/indexed_scale_segment_op.py:172-181``."""
from .. import _lib
from .batched_sparse_dense_op import sparse_product


def indexed_scale_segment(input, scale, index, seg, out_size=None, out=None, block_size_n=64, block_size_c=64):
    if input.ndim != 3:
        raise ValueError(f"input must be (N, M, C), got {tuple(input.shape)}")
    if seg is None and index is None and out_size is not None and out_size != input.shape[-2]:
        raise ValueError("without seg and index the output has as many rows as the input")
    return sparse_product(_lib.OP_SCALE, input, None, scale, index, None, seg, None, None, out, False, out_size)
