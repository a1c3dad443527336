"""Fused gather + Clebsch-Gordan + segment-sum kernels (operator layer, float32).

``TpTable`` packs the CG step of one role assignment of a layer (the ``info_Mij_fwd`` table of a
``TensorProductInfo``) for ``eqt_tp_cg_segment_sum`` / ``eqt_tp_cg_inner``; its ``structure_key``
selects the kernels unrolled at build time when the index structure is one of the registered ones.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, Optional

import numpy as np
import torch
from torch import Tensor

from .. import _lib
from ..csrc.gen_tp_specs import outer_order, structure_from_info, structure_key
from ..structs import SparseProductInfo

_status: Dict[torch.device, Tensor] = {}


def status_flag(device: torch.device) -> Tensor:
    """Per-device int32 flag the kernels raise when a bounded wait gives up."""
    if device not in _status:
        _status[device] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status[device]


def check_status(device=None) -> None:
    """Synchronise and raise if any fused kernel reported a timed-out wait since the last check."""
    for dev, flag in _status.items():
        if device is None or dev == torch.device(device):
            if int(flag.item()) != 0:
                flag.zero_()
                raise _lib.EqtError(f"a fused tensor-product kernel on {dev} gave up waiting for an asynchronous copy")


class TpTable:
    """Device copy of one CG table plus the C struct that points at it."""

    def __init__(self, info: SparseProductInfo, feat_is_input1: bool, d_feat: int, d_y: int, device):
        s = structure_from_info(info, feat_is_input1, d_feat, d_y)
        rowptr = np.searchsorted(s.row, np.arange(s.num_rows + 1)).astype(np.int64)
        self.key = structure_key(s)
        self.scale = info.scale.detach().to(device=device, dtype=torch.float32).contiguous()
        self.m_feat = torch.from_numpy(s.mf.copy()).to(device)
        self.m_y = torch.from_numpy(s.my.copy()).to(device)
        self.row_ptr = torch.from_numpy(rowptr).to(device)
        self.num_entries, self.num_rows, self.d_feat, self.d_y = len(s.mf), s.num_rows, d_feat, d_y
        self.device = torch.device(device)
        order = torch.from_numpy(outer_order(s)).to(device)
        self.scale_o = torch.where(order >= 0, self.scale[order.clamp_min(0)], self.scale.new_zeros(())).contiguous()
        self.struct = _lib.TpTableStruct(self.scale.data_ptr(), self.m_feat.data_ptr(), self.m_y.data_ptr(),
                                         self.row_ptr.data_ptr(), self.num_entries, self.num_rows, d_feat, d_y, self.key,
                                         self.scale_o.data_ptr())


def _f32(t: Tensor, what: str) -> Tensor:
    if t.dtype != torch.float32:
        raise TypeError(f"{what} must be float32 for the fused kernels, got {t.dtype}")
    return t.contiguous()


def cg_segment_sum(table: TpTable, feat: Tensor, y: Tensor, feat_index: Optional[Tensor], y_index: Optional[Tensor],
                   seg_ptr: Optional[Tensor], num_out: int) -> Tensor:
    """``out[d, r, :] = sum_{e in seg[d]} sum_{t in r} scale[t] y[y_index[e], m_y[t]] feat[feat_index[e], m_feat[t], :]``."""
    dev = _lib.require_cuda(feat, y, feat_index, y_index, seg_ptr)
    feat, y = _f32(feat, "feat"), _f32(y, "y")
    assert feat.ndim == 3 and feat.shape[1] == table.d_feat and y.shape[-1] == table.d_y
    c = feat.shape[2]
    n_edges = feat_index.numel() if feat_index is not None else feat.shape[0]
    if seg_ptr is None:
        num_out = n_edges
    out = torch.empty(num_out, table.num_rows, c, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().eqt_tp_cg_segment_sum(
            C.byref(table.struct), feat.data_ptr(), _lib.ptr(feat_index), y.data_ptr(), _lib.ptr(y_index),
            _lib.ptr(seg_ptr), out.data_ptr(), num_out, n_edges, c, status_flag(dev).data_ptr(),
            _lib.stream_ptr(dev)), "eqt_tp_cg_segment_sum")
    return out


def cg_inner(table: TpTable, feat: Tensor, g: Tensor, feat_index: Optional[Tensor], seg_ptr: Tensor,
             edge_node: Tensor, y_index: Optional[Tensor], num_y_rows: int) -> Tensor:
    """``grad_y[y_index[e], k] = sum_{t: m_y[t]=k} scale[t] <feat[feat_index[e], m_feat[t]], g[node(e), row(t)]>``."""
    dev = _lib.require_cuda(feat, g, feat_index, seg_ptr, edge_node, y_index)
    feat, g = _f32(feat, "feat"), _f32(g, "g")
    assert g.ndim == 3 and g.shape[1] == table.num_rows and g.shape[2] == feat.shape[2]
    n_edges = edge_node.numel()
    out = (torch.empty if num_y_rows == n_edges else torch.zeros)(num_y_rows, table.d_y, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().eqt_tp_cg_inner(
            C.byref(table.struct), feat.data_ptr(), _lib.ptr(feat_index), g.data_ptr(), seg_ptr.data_ptr(),
            edge_node.data_ptr(), _lib.ptr(y_index), out.data_ptr(), g.shape[0], n_edges, feat.shape[2],
            status_flag(dev).data_ptr(), _lib.stream_ptr(dev)), "eqt_tp_cg_inner")
    return out
