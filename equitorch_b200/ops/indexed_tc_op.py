"""Tensor-core paths of the indexed products with an operand shared by the batch.

``indexed_vecmat_scale_gather`` with a 3-D matrix operand and ``indexed_outer_scale_gather`` with
``out_accumulated=True`` are GEMMs over the batch; for float32 operands with channel counts that are multiples of 32
they run on tcgen05 (``eqt_vecmat_tc`` / ``eqt_outer_tc``) instead of the table-driven CUDA-core kernels.  What the
kernels need besides the operands depends on the index tables only (k-block columns, packing of entries into
128-row slices, reduction lists) and is built once per table and device and cached.
"""
from __future__ import annotations

import ctypes as C
from collections import OrderedDict
from typing import Dict, Optional

import numpy as np
import torch
from torch import Tensor

from .. import _lib
from .mix_tc_op import status_flag

MIN_BATCH = 512          # below this the table-driven kernels are as fast and have no set-up cost
MAX_PLANS = 256
_plans: "OrderedDict[tuple, tuple]" = OrderedDict()
_scratch: Dict[torch.device, Tensor] = {}


def _cached(kind, dev, tensors, extra, build):
    """Plan for these index tensors.  A plan is keyed by the identity and version of the tensors it was built from
    and keeps them alive, so that neither a recycled address nor an in-place update can alias another table; the
    tables of a module are persistent buffers, so layers hit the cache on every call after the first."""
    key = (kind, dev, tuple(None if t is None else (id(t), t._version) for t in tensors)) + tuple(extra)
    hit = _plans.get(key)
    if hit is not None:
        _plans.move_to_end(key)
        return hit[0]
    plan = build()
    _plans[key] = (plan, tensors)
    if len(_plans) > MAX_PLANS:
        _plans.popitem(last=False)
    return plan


def _host(t: Optional[Tensor], default: np.ndarray) -> np.ndarray:
    return default if t is None else t.detach().cpu().numpy()


def _buffer(dev, floats: int) -> Tensor:
    buf = _scratch.get(dev)
    if buf is None or buf.numel() < floats:
        buf = torch.empty(max(floats, 1), dtype=torch.float32, device=dev)
        _scratch[dev] = buf
    return buf


class VecmatPlan:
    def __init__(self, index1, seg, entries: int, num_out: int, cin: int, dev):
        chunks = cin // 32
        i1 = _host(index1, np.arange(entries, dtype=np.int64))
        sg = _host(seg, np.arange(num_out + 1, dtype=np.int64))
        a_col = (i1[:, None] * cin + np.arange(chunks)[None, :] * 32).reshape(-1)
        self.kb_begin = torch.from_numpy((sg * chunks).astype(np.int32)).to(dev)
        self.a_col = torch.from_numpy(a_col.astype(np.int32)).to(dev)
        if self.a_col.numel() == 0:
            self.a_col = torch.zeros(1, dtype=torch.int32, device=dev)


def vecmat_supported(x: Tensor, w: Tensor, gather_index, index_out, out_accumulated, out_size, num_out) -> bool:
    return (x.is_cuda and x.dtype == torch.float32 and w.dtype == torch.float32 and x.ndim == 3 and w.ndim == 3
            and gather_index is None and index_out is None and not out_accumulated and out_size == num_out
            and x.shape[0] >= MIN_BATCH and x.shape[2] % 32 == 0 and w.shape[2] % 16 == 0 and w.shape[2] <= 128
            and x.data_ptr() % 16 == 0)


def vecmat_tc(x: Tensor, w: Tensor, scale, index1, index2, seg, num_out: int) -> Tensor:
    """``out[i, M, :] = sum_{t in seg[M]} scale[t] x[i, index1[t], :] @ w[index2[t]]`` on tensor cores."""
    dev = x.device
    n, rows1, cin = x.shape
    cout = w.shape[2]
    entries = (index1.shape[0] if index1 is not None else index2.shape[0] if index2 is not None
               else int(seg[-1]) if seg is not None else rows1)
    plan = _cached("vecmat", dev, (index1, seg), (entries, num_out, cin),
                   lambda: VecmatPlan(index1, seg, entries, num_out, cin, dev))
    packed = torch.empty(2, max(entries, 1) * cin * cout, dtype=torch.float32, device=dev)
    out = torch.empty(n, num_out, cout, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().eqt_vecmat_tc(x.data_ptr(), w.data_ptr(), _lib.ptr(index2), _lib.ptr(scale), packed[0].data_ptr(),
                                            packed[1].data_ptr(), out.data_ptr(), n, rows1, cin, cout, num_out, entries,
                                            plan.kb_begin.data_ptr(), plan.a_col.data_ptr(), status_flag(dev).data_ptr(),
                                            _lib.stream_ptr(dev)), "eqt_vecmat_tc")
    return out


class OuterPlan:
    """Packing of the entries of an accumulated outer product into 128-row slices (see ``eqt_outer_tc``)."""

    def __init__(self, scale, index1, index2, seg, entries: int, num_w: int, c1: int, c2: int, dev):
        chunks = c1 // 32
        i1 = _host(index1, np.arange(entries, dtype=np.int64))
        i2 = _host(index2, np.arange(entries, dtype=np.int64))
        sg = _host(seg, np.arange(num_w + 1, dtype=np.int64))
        sc = _host(scale, np.ones(entries, dtype=np.float32)).astype(np.float32)
        w_of = np.repeat(np.arange(num_w), np.diff(sg))
        a_cols, b_cols, units = [], [], []            # units: (weight, chunk, slot, scale)
        for row2 in np.unique(i2):
            ts = np.nonzero(i2 == row2)[0]
            slots = [(t, ch) for t in ts for ch in range(chunks)]
            for s0 in range(0, len(slots), 4):
                group = slots[s0:s0 + 4]
                tile = len(b_cols)
                b_cols.append(int(row2) * c2)
                for q in range(4):
                    if q < len(group):
                        t, ch = group[q]
                        a_cols.append(int(i1[t]) * c1 + ch * 32)
                        units.append((int(w_of[t]), ch, tile * 4 + q, float(sc[t])))
                    else:
                        a_cols.append(0)
        self.m_tiles = len(b_cols)
        units.sort(key=lambda u: (u[0], u[1], u[2]))
        keys = np.array([u[0] * chunks + u[1] for u in units], dtype=np.int64)
        red_ptr = np.searchsorted(keys, np.arange(num_w * chunks + 1)).astype(np.int32)

        def dev_i32(v):
            return torch.tensor(v if len(v) else [0], dtype=torch.int32, device=dev)
        self.a_cols, self.b_cols = dev_i32(a_cols), dev_i32(b_cols)
        self.red_ptr = torch.from_numpy(red_ptr).to(dev)
        self.red_slot = dev_i32([u[2] for u in units])
        self.red_scale = torch.tensor([u[3] for u in units] or [0.0], dtype=torch.float32, device=dev)


def outer_supported(a: Tensor, b: Tensor, gather_index, index_out, out_accumulated, out_size, num_out) -> bool:
    return (a.is_cuda and a.dtype == torch.float32 and b.dtype == torch.float32 and a.ndim == 3 and b.ndim == 3
            and out_accumulated and gather_index is None and index_out is None and out_size == num_out
            and a.shape[0] == b.shape[0] and a.shape[0] >= MIN_BATCH and a.shape[2] % 32 == 0 and b.shape[2] % 32 == 0
            and b.shape[2] <= 128 and a.data_ptr() % 16 == 0 and b.data_ptr() % 16 == 0)


def outer_tc(a: Tensor, b: Tensor, scale, index1, index2, seg, num_w: int) -> Tensor:
    """``out[w] = sum_i sum_{t in seg[w]} scale[t] a[i, index1[t], :, None] b[i, index2[t], None, :]`` on tensor cores."""
    dev = a.device
    n, rows1, c1 = a.shape
    rows2, c2 = b.shape[1], b.shape[2]
    entries = (index1.shape[0] if index1 is not None else index2.shape[0] if index2 is not None
               else int(seg[-1]) if seg is not None else rows1)
    plan = _cached("outer", dev, (scale, index1, index2, seg), (entries, num_w, c1, c2),
                   lambda: OuterPlan(scale, index1, index2, seg, entries, num_w, c1, c2, dev))
    out = torch.empty(num_w, c1, c2, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        need = int(_lib.lib().eqt_outer_tc_scratch_floats(n, c2, max(plan.m_tiles, 1)))
        scratch = _buffer(dev, max(need, 1))
        _lib.check(_lib.lib().eqt_outer_tc(a.data_ptr(), b.data_ptr(), out.data_ptr(), scratch.data_ptr(), scratch.numel(), n,
                                           rows1, c1, rows2, c2, plan.a_cols.data_ptr(), plan.b_cols.data_ptr(), plan.m_tiles,
                                           plan.red_ptr.data_ptr(), plan.red_slot.data_ptr(), plan.red_scale.data_ptr(), num_w,
                                           status_flag(dev).data_ptr(), _lib.stream_ptr(dev)), "eqt_outer_tc")
    return out
