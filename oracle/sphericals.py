"""ORACLE (test infrastructure, never imported by the product path).

Real spherical harmonics and Wigner-D matrices restated independently of the
recurrences used by the CUDA kernels.

``spherical_harmonics`` reproduces ``equitorch/ops/spherical_harmonics.py:68-641``:
component normalisation (``sum_m Y_lm**2 = 2l+1`` on the unit sphere), components
ordered m = -l..l with the polar axis on **z** and ``Y_1 = sqrt(3) (y, z, x)``, and
for non-unit input the degree-l homogeneous polynomial (solid harmonic).  The
reference hard-codes polynomials generated with a CAS; here the same functions come
from the textbook construction

    Y_{l,+m} = N_lm * Q_l^m(z, r2) * Re (x + i y)^m * sqrt2
    Y_{l,-m} = N_lm * Q_l^m(z, r2) * Im (x + i y)^m * sqrt2
    Y_{l,0}  = N_l0 * Q_l^0(z, r2)

with ``Q_l^m`` the associated Legendre function stripped of ``sin^m`` and made
homogeneous with ``r2 = x^2+y^2+z^2`` (no Condon-Shortley phase) and
``N_lm = sqrt((2l+1) (l-m)!/(l+m)!)``.

``wigner_d`` restates ``D(a,b,c) = Dz(a) J Dz(b) J Dz(c)`` of
``equitorch/nn/functional/wigner_d.py:14-56`` with dense blocks.

Pinned against reference outputs in tests/golden.
"""
from __future__ import annotations

import math
from typing import List

import torch
from torch import Tensor


def spherical_harmonics(xyz: Tensor, l_max: int, dim: int = -1) -> Tensor:
    x, y, z = (xyz.narrow(dim, i, 1) for i in range(3))
    r2 = x * x + y * y + z * z
    # c[m] + i s[m] = (x + i y)^m
    c: List[Tensor] = [torch.ones_like(x)]
    s: List[Tensor] = [torch.zeros_like(x)]
    for m in range(1, l_max + 1):
        c_m = c[m - 1] * x - s[m - 1] * y
        s_m = s[m - 1] * x + c[m - 1] * y
        c.append(c_m)
        s.append(s_m)
    out = [[None] * (2 * l + 1) for l in range(l_max + 1)]

    def emit(l: int, m: int, q: Tensor) -> None:
        n = math.sqrt((2 * l + 1) * math.factorial(l - m) / math.factorial(l + m))
        if m == 0:
            out[l][l] = n * q
        else:
            out[l][l + m] = math.sqrt(2.0) * n * q * c[m]
            out[l][l - m] = math.sqrt(2.0) * n * q * s[m]

    for m in range(l_max + 1):
        below = torch.zeros_like(x)                                   # Q_{m-1}^m = 0
        here = torch.ones_like(x) * float(_double_factorial(2 * m - 1))  # Q_m^m = (2m-1)!!
        emit(m, m, here)
        for l in range(m + 1, l_max + 1):
            nxt = ((2 * l - 1) * z * here - (l + m - 1) * r2 * below) / (l - m)
            emit(l, m, nxt)
            below, here = here, nxt
    return torch.cat([t for row in out for t in row], dim=dim)


def _double_factorial(n: int) -> int:
    return 1 if n <= 0 else n * _double_factorial(n - 2)


def sincos(angle: Tensor, max_m: int) -> Tensor:
    """``[1, sin a, cos a, sin 2a, cos 2a, ...]`` (equitorch/nn/functional/angular.py:4-35)."""
    cols = [torch.ones_like(angle)]
    for m in range(1, max_m + 1):
        cols += [torch.sin(m * angle), torch.cos(m * angle)]
    return torch.stack(cols, dim=-1)


def _z_rotation_block(l: int, angle: Tensor) -> Tensor:
    """Dense (N, 2l+1, 2l+1) block of ``x'_m = cos(m a) x_m - sign(m) sin(|m| a) x_{-m}``
    (equitorch/utils/_structs.py:487-518)."""
    n = angle.shape[0]
    d = angle.new_zeros(n, 2 * l + 1, 2 * l + 1)
    d[:, l, l] = 1.0
    for m in range(1, l + 1):
        cm, sm = torch.cos(m * angle), torch.sin(m * angle)
        d[:, l + m, l + m] = cm
        d[:, l - m, l - m] = cm
        d[:, l + m, l - m] = -sm
        d[:, l - m, l + m] = sm
    return d


def wigner_d(ls: List[int], alpha: Tensor, beta: Tensor, gamma: Tensor, j_blocks) -> Tensor:
    """Block-diagonal ``Dz(alpha) J Dz(beta) J Dz(gamma)`` for the irreps with degrees ``ls``.

    ``j_blocks[l]`` is the (2l+1, 2l+1) J matrix as a tensor of the working dtype.
    """
    blocks = []
    for l in ls:
        J = j_blocks[l].to(alpha.dtype)
        blocks.append(_z_rotation_block(l, alpha) @ J @ _z_rotation_block(l, beta) @ J
                      @ _z_rotation_block(l, gamma))
    n = alpha.shape[0]
    dim = sum(2 * l + 1 for l in ls)
    out = alpha.new_zeros(n, dim, dim)
    o = 0
    for l, b in zip(ls, blocks):
        out[:, o:o + 2 * l + 1, o:o + 2 * l + 1] = b
        o += 2 * l + 1
    return out
