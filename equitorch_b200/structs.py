"""Index-table containers consumed by the sparse kernels.

Field names, order and defaults follow ``equitorch/structs/__init__.py:50-139``
of the reference, because the autograd Functions pass these tuples around
positionally and the ``None``-ness of a field selects a kernel code path
(``index1 is None`` means "identity gather", ``seg_out is None`` means "one
table entry per output row").

Every container can be moved like a tensor (``.to()``, ``.cuda()``, ``.cpu()``,
``._apply(fn)``); ``.to(dtype)`` only converts floating-point fields, integer
index fields keep int64.
"""
from __future__ import annotations

from typing import NamedTuple, Optional

import torch
from torch import Tensor


def _map_fields(tup, fn):
    moved = []
    for value in tup:
        if isinstance(value, Tensor):
            moved.append(fn(value))
        elif hasattr(value, "_apply") and isinstance(value, tuple):
            moved.append(value._apply(fn))
        else:
            moved.append(value)
    return type(tup)(*moved)


def _movable(cls):
    """Give a NamedTuple class tensor-like device/dtype movement."""

    def _apply(self, fn, *_, **__):
        return _map_fields(self, fn)

    def to(self, *args, **kwargs):
        device, dtype, non_blocking, _ = torch._C._nn._parse_to(*args, **kwargs)

        def move(t: Tensor) -> Tensor:
            return t.to(device=device, dtype=dtype if t.is_floating_point() else None,
                        non_blocking=non_blocking)

        return _map_fields(self, move)

    cls._apply = _apply
    cls.to = to
    cls.cuda = lambda self, *a, **k: _map_fields(self, lambda t: t.cuda(*a, **k))
    cls.cpu = lambda self, *a, **k: _map_fields(self, lambda t: t.cpu(*a, **k))
    return cls


@_movable
class SparseScaleInfo(NamedTuple):
    """``z[M] = sum_{t in seg_out[M]} scale[t] * x[index[t]]``."""
    scale: Optional[Tensor] = None      # (T,) float
    index: Optional[Tensor] = None      # (T,) int64 into the input rows
    seg_out: Optional[Tensor] = None    # (num_out+1,) int64 CSR pointer into t
    index_out: Optional[Tensor] = None  # (num_out,) int64 output row ids
    out_size: Optional[int] = None


@_movable
class SparseProductInfo(NamedTuple):
    """``z[M] = sum_{t in seg_out[M]} scale[t] * x[index1[t]] (*) y[index2[t]]``."""
    scale: Optional[Tensor] = None
    index1: Optional[Tensor] = None
    index2: Optional[Tensor] = None
    seg_out: Optional[Tensor] = None
    gather_index: Optional[Tensor] = None
    index_out: Optional[Tensor] = None
    out_size: Optional[int] = None


@_movable
class TensorProductInfo(NamedTuple):
    info_Mij_fwd: SparseProductInfo
    info_Mij_bwd1: SparseProductInfo
    info_Mij_bwd2: SparseProductInfo

    info_M_fwd: SparseProductInfo
    info_M_bwd1: SparseProductInfo
    info_M_bwd2: SparseProductInfo

    info_kM1j_fwd: SparseProductInfo
    info_kM1j_bwd1: SparseProductInfo
    info_kM1j_bwd2: SparseProductInfo
    info_kM1M2_fwd: SparseProductInfo
    info_kM1M2_bwd1: SparseProductInfo
    info_kM1M2_bwd2: SparseProductInfo
    info_M_kM1M2_fwd: SparseScaleInfo
    info_M_kM1M2_bwd: SparseScaleInfo
    out_size: int


@_movable
class IrrepsInfo(NamedTuple):
    rsqrt_dims: Tensor
    rdims: Tensor
    irrep_index: Tensor
    irrep_seg: Tensor
    num_irreps: int


@_movable
class IrrepsLinearInfo(NamedTuple):
    scale_MM0: Tensor
    M_seg_MM0: Tensor
    ii0_MM0: Tensor
    M0_MM0: Tensor
    M_MM0: Tensor
    M_out: Tensor
    # weight-gradient view
    ii0_seg_ii0MM0: Tensor
    M_ii0MM0: Tensor
    M0_ii0MM0: Tensor
    scales_ii0: Tensor
    out_size: int


@_movable
class WignerRotationInfo(NamedTuple):
    j_matrix_info: SparseScaleInfo
    rotate_z_info_fwd: SparseProductInfo
    rotate_z_info_bwd_input: Optional[SparseProductInfo] = None
    rotate_z_info_bwd_cs: Optional[SparseProductInfo] = None
    sign: Optional[Tensor] = None
    max_m: Optional[int] = None
