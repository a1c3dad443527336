"""Weight step (channel mixing with shared weights) on tcgen05 tensor cores: operator layer.

``MixPlan`` analyses the weight-step table of a layer (``info_M_fwd``: one table entry per intermediate
row, entries of an output component contiguous, ``index2`` = path of the row) and, when it has the
regular block structure the GEMM formulation needs - every component of an output irrep receives the
same paths in the same order - records one ``eqt_mix_block`` per irrep.  ``mix_tc`` packs and splits
the weights (a few small elementwise kernels on at most a few hundred KB) and calls ``eqt_mix_tc``.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence

import numpy as np
import torch
from torch import Tensor

from .. import _lib
from ..structs import SparseProductInfo
from .fused_tp_op import status_flag


class MixPlan:
    """Block structure of a weight-step table, or ``regular = False`` if it has none."""

    def __init__(self, info: SparseProductInfo, out_dims: Sequence[int], device):
        self.regular = False
        self.device = torch.device(device)
        if info.index1 is not None or info.scale is not None or info.index2 is None or info.gather_index is not None:
            return
        w = info.index2.cpu().numpy()
        n_out = info.out_size
        seg = info.seg_out.cpu().numpy() if info.seg_out is not None else np.arange(n_out + 1)
        if len(seg) != n_out + 1 or sum(out_dims) != n_out or seg[-1] != len(w):
            return
        blocks, gather, comp = [], [], 0
        for dim in out_dims:
            lists = [tuple(w[seg[comp + m]:seg[comp + m + 1]]) for m in range(dim)]
            if len(set(lists)) != 1:
                return
            paths = len(lists[0])
            if paths:
                blocks.append((int(seg[comp]), comp, dim, paths, len(gather)))
                gather += list(lists[0])
            comp += dim
        self.blocks_host = blocks                  # (in_row0, out_row0, dim, paths, first packed path)
        self.rows = int(len(w))
        self.comps = n_out
        self.path_gather = torch.tensor(gather, dtype=torch.long, device=device)
        self.paths_in_order = list(gather) == list(range(len(gather)))   # packed path p is weight path p
        self.regular = len(blocks) > 0 and comp == n_out
        self._struct_cache = {}

    def structs(self, cin: int, cout: int):
        key = (cin, cout)
        if key not in self._struct_cache:
            arr = (_lib.MixBlockStruct * len(self.blocks_host))()
            for k, (in0, out0, dim, paths, first) in enumerate(self.blocks_host):
                arr[k] = _lib.MixBlockStruct(in0, out0, dim, paths, first * cin * cout)
            self._struct_cache[key] = arr
        return self._struct_cache[key]

    def pack(self, weight: Tensor, k_major: bool = True):
        """Gather the blocks' paths from ``weight`` (P, cin, cout), lay them out for the GEMM (per block
        (cout, paths*cin) when ``k_major`` else stacked (paths*cin, cout)) and split into big + small."""
        w = weight.detach().contiguous()
        cin, cout = w.shape[-2:]
        n = self.path_gather.numel() * cin * cout
        big = torch.empty(n, dtype=torch.float32, device=w.device)
        small = torch.empty(n, dtype=torch.float32, device=w.device)
        blocks = self.structs(cin, cout)
        with torch.cuda.device(w.device):
            _lib.check(_lib.lib().eqt_pack_weights(w.data_ptr(), self.path_gather.data_ptr(), cin, cout, blocks,
                                                   len(blocks), int(k_major), big.data_ptr(), small.data_ptr(),
                                                   _lib.stream_ptr(w.device)), "eqt_pack_weights")
        return big, small


def mix_tc_transposed(g: Tensor, weight: Tensor, plan: MixPlan) -> Tensor:
    """Gradient of :func:`mix_tc` w.r.t. its first argument: ``g_inter[n, r, :] = g[n, M(r), :] @ weight[path(r)]^T``."""
    dev = _lib.require_cuda(g, weight)
    assert g.dtype == torch.float32 and weight.dtype == torch.float32 and plan.regular
    g = g.contiguous()
    n, comps, cout = g.shape
    cin = weight.shape[-2]
    assert comps == plan.comps and weight.shape[-1] == cout
    big, small = plan.pack(weight, k_major=False)
    out = torch.empty(n, plan.rows, cin, dtype=torch.float32, device=dev)
    blocks = plan.structs(cin, cout)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().eqt_mix_tc_transposed(g.data_ptr(), big.data_ptr(), small.data_ptr(), out.data_ptr(), n,
                                                    plan.rows, comps, cin, cout, blocks, len(blocks),
                                                    status_flag(dev).data_ptr(), _lib.stream_ptr(dev)),
                   "eqt_mix_tc_transposed")
    return out


_scratch = {}


def wgrad_scratch(device, cout: int, need: int = 0) -> Tensor:
    """Per-device scratch for the split reduction of :func:`wgrad_tc` (at least 128 * cout floats per SM)."""
    device = torch.device(device)
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    need = max(need, 128 * cout * sms)
    buf = _scratch.get(device)
    if buf is None or buf.numel() < need:
        buf = torch.empty(need, dtype=torch.float32, device=device)
        _scratch[device] = buf
    return buf


def wgrad_tc(s: Tensor, g: Tensor, plan: MixPlan, num_paths: int) -> Tensor:
    """``gw[p] = sum_n sum_{rows r of path p} s[n, r, :]^T g[n, M(r), :]`` -> (num_paths, cin, cout), deterministic."""
    dev = _lib.require_cuda(s, g)
    assert s.dtype == torch.float32 and g.dtype == torch.float32 and plan.regular
    s, g = s.contiguous(), g.contiguous()
    n, rows, cin = s.shape
    cout = g.shape[-1]
    packed = torch.empty(plan.path_gather.numel(), cin, cout, dtype=torch.float32, device=dev)
    blocks = plan.structs(cin, cout)
    with torch.cuda.device(dev):
        need = int(_lib.lib().eqt_wgrad_tc_scratch_floats(n, cin, cout, blocks, len(blocks)))
        if need < 0:
            raise _lib.EqtError("eqt_wgrad_tc refuses these blocks")
        scratch = wgrad_scratch(dev, cout, need)
        _lib.check(_lib.lib().eqt_wgrad_tc(s.data_ptr(), g.data_ptr(), packed.data_ptr(), scratch.data_ptr(),
                                           scratch.numel(), n, rows, plan.comps, cin, cout, blocks, len(blocks),
                                           status_flag(dev).data_ptr(), _lib.stream_ptr(dev)), "eqt_wgrad_tc")
    if plan.paths_in_order and plan.path_gather.numel() == num_paths:
        return packed
    return torch.zeros(num_paths, cin, cout, dtype=torch.float32, device=dev).index_add_(0, plan.path_gather, packed)


def supported_wgrad(cin: int, cout: int) -> bool:
    return cin % 32 == 0 and cout % 32 == 0 and cout <= 128


def supported_transposed(cin: int, cout: int) -> bool:
    return cout % 32 == 0 and cin % 16 == 0 and cin <= 256


def supported(cin: int, cout: int) -> bool:
    return cin % 32 == 0 and cout % 16 == 0 and cout <= 256


def mix_tc(s: Tensor, weight: Tensor, plan: MixPlan) -> Tensor:
    """``out[n, M, :] = sum_{rows r of M} s[n, r, :] @ weight[path(r)]`` with float32 accuracy."""
    dev = _lib.require_cuda(s, weight)
    assert s.dtype == torch.float32 and weight.dtype == torch.float32 and plan.regular
    s = s.contiguous()
    n, rows, cin = s.shape
    cout = weight.shape[-1]
    assert rows == plan.rows and weight.shape[-2] == cin
    big, small = plan.pack(weight)
    out = torch.zeros(n, plan.comps, cout, dtype=torch.float32, device=dev) if _has_empty(plan) else \
        torch.empty(n, plan.comps, cout, dtype=torch.float32, device=dev)
    blocks = plan.structs(cin, cout)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().eqt_mix_tc(s.data_ptr(), big.data_ptr(), small.data_ptr(), out.data_ptr(), n, rows,
                                         plan.comps, cin, cout, blocks, len(blocks), status_flag(dev).data_ptr(),
                                         _lib.stream_ptr(dev)), "eqt_mix_tc")
    return out


def _has_empty(plan: MixPlan) -> bool:
    return sum(b[2] for b in plan.blocks_host) != plan.comps
