"""Real spherical harmonics on the GPU.  Same call as ``equitorch/ops/spherical_harmonics.py:69``
(``spherical_harmonics(input, l_max, dim=-1)``): component normalisation, m = -l..l,
``Y_1 = sqrt(3) (y, z, x)``, homogeneous polynomials for non-unit input.  Any ``l_max <= 64``
(the reference stops at 17).  Differentiable once (the gradient kernel is not itself
differentiable)."""
from __future__ import annotations

import ctypes as C
from typing import Dict, Tuple

import torch
from torch import Tensor

from .. import _lib, _profile
from ..sh_tables import sh_recurrence

_TABLES: Dict[Tuple[int, torch.device], Tuple[_lib.ShTable, tuple]] = {}


def device_table(l_max: int, device: torch.device) -> _lib.ShTable:
    """Upload (once per degree and device) the recurrence table; returns the C struct."""
    key = (l_max, device)
    if key not in _TABLES:
        t = sh_recurrence(l_max)
        keep = tuple(torch.from_numpy(a.copy()).to(device) for a in (t.ptr, t.m_out, t.m_in, t.axis, t.coef))
        _TABLES[key] = (_lib.ShTable(*(k.data_ptr() for k in keep), l_max, len(t.coef)), keep)
    return _TABLES[key][0]


def sh_forward(xyz: Tensor, l_max: int, normalize: bool, out_scale: float) -> Tensor:
    dev = _lib.require_cuda(xyz)
    if xyz.dtype not in (torch.float32, torch.float64):
        raise TypeError("spherical harmonics take float32 or float64 input")
    flat = xyz.reshape(-1, 3).contiguous()
    out = torch.empty(flat.shape[0], (l_max + 1) ** 2, dtype=xyz.dtype, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().eqt_sh_forward(_lib.DTYPE_CODE[xyz.dtype], flat.data_ptr(), out.data_ptr(), flat.shape[0],
                                             C.byref(device_table(l_max, dev)), int(normalize), float(out_scale),
                                             _lib.stream_ptr(dev)), "eqt_sh_forward")
    return out.view(*xyz.shape[:-1], (l_max + 1) ** 2)


def sh_backward(xyz: Tensor, grad_out: Tensor, l_max: int, normalize: bool, out_scale: float) -> Tensor:
    dev = _lib.require_cuda(xyz, grad_out)
    flat = xyz.reshape(-1, 3).contiguous()
    g = grad_out.to(xyz.dtype).reshape(-1, (l_max + 1) ** 2).contiguous()
    gx = torch.empty_like(flat)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().eqt_sh_backward(_lib.DTYPE_CODE[xyz.dtype], flat.data_ptr(), g.data_ptr(), gx.data_ptr(),
                                              flat.shape[0], C.byref(device_table(l_max, dev)), int(normalize),
                                              float(out_scale), _lib.stream_ptr(dev)), "eqt_sh_backward")
    return gx.view_as(xyz)


class _SphericalHarmonics(torch.autograd.Function):
    @staticmethod
    def forward(ctx, xyz, l_max, normalize, out_scale):
        ctx.save_for_backward(xyz)
        ctx.cfg = (l_max, normalize, out_scale)
        with _profile.timed("spherical_harmonics[fwd]"):
            return sh_forward(xyz, l_max, normalize, out_scale)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, grad_out):
        (xyz,) = ctx.saved_tensors
        with _profile.timed("spherical_harmonics[bwd]"):
            return sh_backward(xyz, grad_out, *ctx.cfg), None, None, None


def spherical_harmonics_fused(input: Tensor, l_max: int, normalize: bool = False, out_scale: float = 1.0) -> Tensor:
    """Normalisation, harmonics and the optional constant factor in one kernel (last axis = xyz)."""
    return _SphericalHarmonics.apply(input, l_max, normalize, out_scale)


def spherical_harmonics(input: Tensor, l_max: int, dim: int = -1) -> Tensor:
    if input.shape[dim] != 3:
        raise ValueError(f"dimension {dim} must have size 3, got {input.shape[dim]}")
    moved = input.movedim(dim, -1)
    return _SphericalHarmonics.apply(moved, l_max, False, 1.0).movedim(-1, dim)
