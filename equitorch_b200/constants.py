"""Real-basis Clebsch-Gordan coefficients and the J matrix, without a CAS.

The reference evaluates these symbolically (``equitorch/constants/__init__.py:12-105``:
``sympy.physics.wigner.clebsch_gordan`` + a complex->real change of basis, then
``float(...)``).  Here the same numbers come from

* the Racah closed form for the SU(2) coefficient, kept exact as
  ``sign * sqrt(Fraction)``;
* the same change of basis (columns = real index, an extra ``(-i)**l`` phase,
  reference :63-75) applied symbolically on ``(power of i, number of 1/sqrt2
  factors)`` pairs, so every real-basis entry is an integer combination of
  square roots of rationals;
* one final evaluation with 256-bit ``mpmath`` floats and a single rounding to
  float64.  Entries that vanish do so exactly (integer cancellation) or fall
  below 1e-60 and are flushed to 0.0, which keeps the reference's
  ``cg != 0.0`` sparsity test meaningful.

Index order of ``so3_clebsch_gordan(l, l1, l2)`` is ``[m_out, m1, m2]`` and each
``m_out`` slice has unit Frobenius norm.
"""
from __future__ import annotations

import functools
from fractions import Fraction
from math import factorial
from typing import Dict, List, Tuple

import mpmath
import numpy as np

_PREC_BITS = 256
_ZERO_BELOW = mpmath.mpf(10) ** -60


def _su2_cg_exact(j1: int, m1: int, j2: int, m2: int, j3: int, m3: int) -> Tuple[int, Fraction]:
    """<j1 m1 j2 m2 | j3 m3> for integer spins as (sign, value**2)."""
    if m3 != m1 + m2 or not abs(j1 - j2) <= j3 <= j1 + j2:
        return 0, Fraction(0)
    if abs(m1) > j1 or abs(m2) > j2 or abs(m3) > j3:
        return 0, Fraction(0)
    f = factorial
    pref = Fraction((2 * j3 + 1) * f(j3 + j1 - j2) * f(j3 - j1 + j2) * f(j1 + j2 - j3), f(j1 + j2 + j3 + 1))
    pref *= f(j3 + m3) * f(j3 - m3) * f(j1 - m1) * f(j1 + m1) * f(j2 - m2) * f(j2 + m2)
    lo = max(0, j2 - j3 - m1, j1 + m2 - j3)
    hi = min(j1 + j2 - j3, j1 - m1, j2 + m2)
    total = Fraction(0)
    for k in range(lo, hi + 1):
        den = (f(k) * f(j1 + j2 - j3 - k) * f(j1 - m1 - k) * f(j2 + m2 - k)
               * f(j3 - j2 + m1 + k) * f(j3 - j1 - m2 + k))
        total += Fraction(-1 if k % 2 else 1, den)
    if total == 0:
        return 0, Fraction(0)
    return (1 if total > 0 else -1), pref * total * total


def _real_to_complex_entries(l: int) -> Dict[int, List[Tuple[int, int, int]]]:
    """Non-zeros of the real->complex basis change, keyed by complex m.

    Value of an entry is ``i**power / sqrt(2)**halves``; each list item is
    ``(real_index, power, halves)``.  The global ``(-i)**l`` phase is folded in.
    """
    base = (3 * l) % 4  # (-i)**l == i**(3l)
    rows: Dict[int, List[Tuple[int, int, int]]] = {}
    for m in range(-l, l + 1):
        a = abs(m)
        if m == 0:
            rows[m] = [(l, base, 0)]
        elif m < 0:
            rows[m] = [(l + a, base, 1), (l - a, (base + 3) % 4, 1)]          # 1/√2 , -i/√2
        else:
            s = 2 if a % 2 else 0                                               # (-1)**m
            rows[m] = [(l + a, (base + s) % 4, 1), (l - a, (base + s + 1) % 4, 1)]  # ±1/√2 , ±i/√2
    return rows


@functools.lru_cache(maxsize=None)
def _so3_cg_mp(l: int, l1: int, l2: int):
    """Real-basis CG as a nested list of 256-bit mpmath numbers."""
    q_out, q1, q2 = _real_to_complex_entries(l), _real_to_complex_entries(l1), _real_to_complex_entries(l2)
    # accum[(a, b, c)][squared magnitude] = integer weight of the real part
    accum: Dict[Tuple[int, int, int], Dict[Fraction, int]] = {}
    for m1 in range(-l1, l1 + 1):
        for m2 in range(-l2, l2 + 1):
            m = m1 + m2
            if abs(m) > l:
                continue
            sgn, sq = _su2_cg_exact(l1, m1, l2, m2, l, m)
            if sgn == 0:
                continue
            for a, pa, ha in q_out[m]:
                for b, pb, hb in q1[m1]:
                    for c, pc, hc in q2[m2]:
                        power = (pb + pc - pa) % 4          # conj() on the output side
                        if power % 2:                        # purely imaginary: cancels in the sum
                            continue
                        term = sq / (2 ** (ha + hb + hc))
                        slot = accum.setdefault((a, b, c), {})
                        slot[term] = slot.get(term, 0) + sgn * (1 if power == 0 else -1)
    with mpmath.workprec(_PREC_BITS):
        out = [[[mpmath.mpf(0)] * (2 * l2 + 1) for _ in range(2 * l1 + 1)] for _ in range(2 * l + 1)]
        for (a, b, c), terms in accum.items():
            v = mpmath.mpf(0)
            for sq, w in terms.items():
                if w:
                    v += w * mpmath.sqrt(mpmath.mpf(sq.numerator) / sq.denominator)
            if abs(v) > _ZERO_BELOW:
                out[a][b][c] = v
    return out


@functools.lru_cache(maxsize=None)
def so3_clebsch_gordan(l: int, l1: int, l2: int) -> np.ndarray:
    """Real-basis CG tensor ``[m_out, m1, m2]`` as float64 (reference constants/__init__.py:40-61)."""
    mp = _so3_cg_mp(l, l1, l2)
    arr = np.array([[[float(v) for v in row] for row in mat] for mat in mp], dtype=np.float64)
    arr.setflags(write=False)
    return arr


@functools.lru_cache(maxsize=None)
def _j_matrix_mp(l: int):
    if l == 0:
        return [[mpmath.mpf(1)]]
    if l == 1:
        return [[mpmath.mpf(v) for v in row] for row in ((0, 1, 0), (1, 0, 0), (0, 0, -1))]
    cg = _so3_cg_mp(l, 1, l - 1)
    j1, jp = _j_matrix_mp(1), _j_matrix_mp(l - 1)
    n, npv = 2 * l + 1, 2 * l - 1
    with mpmath.workprec(_PREC_BITS):
        # t[k][I][J] = sum_{i,j} cg[k][i][j] * j1[i][I] * jp[j][J]
        t = [[[sum(cg[k][i][j] * j1[i][I] * jp[j][J] for i in range(3) for j in range(npv)
                   if cg[k][i][j] != 0 and j1[i][I] != 0)
               for J in range(npv)] for I in range(3)] for k in range(n)]
        return [[sum(t[k][I][J] * cg[K][I][J] for I in range(3) for J in range(npv) if cg[K][I][J] != 0)
                 for K in range(n)] for k in range(n)]


@functools.lru_cache(maxsize=None)
def j_matrix(l: int) -> np.ndarray:
    """Real-basis rotation block that swaps y/z and flips x, built by the CG
    recursion of the reference (constants/__init__.py:12-36).  Symmetric, J·J = 1."""
    arr = np.array([[float(v) for v in row] for row in _j_matrix_mp(l)], dtype=np.float64)
    arr.setflags(write=False)
    return arr
