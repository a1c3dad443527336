"""Wigner-D generation and dense rotation (operator layer over ``eqt_wigner_d_*`` / ``eqt_dense_rotation*``)."""
from __future__ import annotations

import ctypes as C
from typing import Dict, Tuple

import numpy as np
import torch
from torch import Tensor

from .. import _lib
from ..constants import j_matrix
from ..irreps import Irreps

MAX_L = 7


def _block_coefficients(l: int) -> np.ndarray:
    """(l + 1, n, n, 2) coefficients [k][a][b][A, B] of ``J Z(beta) J = sum_k A_k cos(k beta) + B_k sin(k beta)``."""
    n = 2 * l + 1
    J = j_matrix(l)
    out = np.zeros((l + 1, n, n, 2), dtype=np.float64)
    out[0, :, :, 0] = np.outer(J[:, l], J[l, :])
    for k in range(1, l + 1):
        out[k, :, :, 0] = np.outer(J[:, l + k], J[l + k, :]) + np.outer(J[:, l - k], J[l - k, :])
        out[k, :, :, 1] = -np.outer(J[:, l + k], J[l - k, :]) + np.outer(J[:, l - k], J[l + k, :])
    return out


class WignerTable:
    """Device tables of one irreps list for the Wigner-D kernels (coefficients in float32 or float64)."""

    def __init__(self, irreps: Irreps, device, dtype: torch.dtype):
        ls = [ir.l for ir in irreps]
        if not ls or max(ls) > MAX_L:
            raise ValueError(f"the Wigner-D kernels take 1 or more irreps of degree <= {MAX_L}")
        offsets: Dict[int, int] = {}
        chunks, total = [], 0
        for l in sorted(set(ls)):
            c = _block_coefficients(l).reshape(-1)
            offsets[l] = total
            chunks.append(c)
            total += c.size
        comp, blocks, start = [], [], 0
        for l in ls:
            blocks.append((start, l, offsets[l]))
            comp += [(start, l, offsets[l], m) for m in range(-l, l + 1)]
            start += 2 * l + 1
        self.dim, self.max_l, self.dtype = start, max(ls), dtype
        self.coef = torch.from_numpy(np.concatenate(chunks)).to(device=device, dtype=dtype).contiguous()
        self.comp = torch.tensor(comp, dtype=torch.int32, device=device).contiguous()
        self.blocks = torch.tensor(blocks, dtype=torch.int32, device=device).contiguous()
        self.struct = _lib.WignerTableStruct(self.coef.data_ptr(), self.comp.data_ptr(), self.blocks.data_ptr(), self.dim,
                                             len(blocks), self.max_l, total)


_tables: Dict[Tuple, WignerTable] = {}


def wigner_table(irreps: Irreps, device, dtype: torch.dtype) -> WignerTable:
    key = (tuple((ir.l, ir.p) for ir in irreps), torch.device(device), dtype)
    if key not in _tables:
        _tables[key] = WignerTable(irreps, device, dtype)
    return _tables[key]


def supported(irreps: Irreps, *angles) -> bool:
    """Whether the kernels take these irreps and angle tensors (1-D, equal length, float32 / float64, CUDA)."""
    if len(irreps) == 0 or max(ir.l for ir in irreps) > MAX_L:
        return False
    a0 = angles[0]
    return all(torch.is_tensor(a) and a.is_cuda and a.ndim == 1 and a.shape == a0.shape and a.dtype == a0.dtype
               and a.dtype in (torch.float32, torch.float64) for a in angles)


def wigner_d_forward(table: WignerTable, alpha: Tensor, beta: Tensor, gamma: Tensor) -> Tensor:
    dev = _lib.require_cuda(alpha, beta, gamma)
    alpha, beta, gamma = alpha.contiguous(), beta.contiguous(), gamma.contiguous()
    n = alpha.shape[0]
    out = torch.empty(n, table.dim, table.dim, dtype=alpha.dtype, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().eqt_wigner_d_forward(C.byref(table.struct), alpha.data_ptr(), beta.data_ptr(), gamma.data_ptr(),
                                                   out.data_ptr(), n, _lib.DTYPE_CODE[alpha.dtype], _lib.stream_ptr(dev)),
                   "eqt_wigner_d_forward")
    return out


def wigner_d_backward(table: WignerTable, alpha: Tensor, beta: Tensor, gamma: Tensor, grad_d: Tensor):
    dev = _lib.require_cuda(alpha, beta, gamma, grad_d)
    alpha, beta, gamma, grad_d = alpha.contiguous(), beta.contiguous(), gamma.contiguous(), grad_d.contiguous()
    n = alpha.shape[0]
    grads = torch.empty(3, n, dtype=alpha.dtype, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().eqt_wigner_d_backward(C.byref(table.struct), alpha.data_ptr(), beta.data_ptr(), gamma.data_ptr(),
                                                    grad_d.data_ptr(), grads[0].data_ptr(), grads[1].data_ptr(),
                                                    grads[2].data_ptr(), n, _lib.DTYPE_CODE[alpha.dtype], _lib.stream_ptr(dev)),
                   "eqt_wigner_d_backward")
    return grads[0], grads[1], grads[2]


_row_ranges: Dict[Tuple, Tensor] = {}


def block_row_range(irreps: Irreps, device) -> Tensor:
    """(dim, 2) int32: for every row of a matrix that is block diagonal over ``irreps`` the column range of its block."""
    key = (tuple(ir.dim for ir in irreps), torch.device(device))
    if key not in _row_ranges:
        rows, start = [], 0
        for ir in irreps:
            rows += [(start, start + ir.dim)] * ir.dim
            start += ir.dim
        _row_ranges[key] = torch.tensor(rows, dtype=torch.int32, device=device).contiguous()
    return _row_ranges[key]


def dense_rotation(matrix: Tensor, x: Tensor, transposed: bool = False, row_range: Tensor = None) -> Tensor:
    """``out[n] = matrix[n] @ x[n]`` (or ``matrix[n].T @ x[n]``); matrix (N, D, D), x (N, D, C), contiguous.
    ``row_range`` (see :func:`block_row_range`): the matrices are block diagonal, entries outside the blocks are
    neither read nor multiplied."""
    dev = _lib.require_cuda(matrix, x)
    n, d, c = x.shape
    out = torch.empty_like(x)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().eqt_dense_rotation(matrix.data_ptr(), x.data_ptr(), out.data_ptr(), n, d, c, int(transposed),
                                                 _lib.ptr(row_range), _lib.DTYPE_CODE[x.dtype], _lib.stream_ptr(dev)),
                   "eqt_dense_rotation")
    return out


def dense_rotation_grad_matrix(grad_out: Tensor, x: Tensor, row_range: Tensor = None) -> Tensor:
    """``grad_matrix[n] = grad_out[n] @ x[n].T`` (with ``row_range``: zero outside the diagonal blocks)."""
    dev = _lib.require_cuda(grad_out, x)
    n, d, c = x.shape
    gm = torch.empty(n, d, d, dtype=x.dtype, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().eqt_dense_rotation_grad_matrix(grad_out.data_ptr(), x.data_ptr(), gm.data_ptr(), n, d, c,
                                                             _lib.ptr(row_range), _lib.DTYPE_CODE[x.dtype],
                                                             _lib.stream_ptr(dev)),
                   "eqt_dense_rotation_grad_matrix")
    return gm


def rotation_supported(matrix: Tensor, x: Tensor) -> bool:
    if not (matrix.is_cuda and x.is_cuda and matrix.ndim == 3 and x.ndim == 3 and matrix.dtype == x.dtype
            and x.dtype in (torch.float32, torch.float64)):
        return False
    n, d, c = x.shape
    if matrix.shape != (n, d, d):
        return False
    es = x.element_size()
    d4, c4 = (d + 3) // 4 * 4, (c + 3) // 4 * 4
    return es * (d * d4 + d * c4) <= 200 * 1024 and es * (2 * c * d4 + d * d) <= 200 * 1024
