"""Host-side builders of the sorted index tables (CG paths, CSR pointers).

These produce the same ``*Info`` tuples as ``equitorch/utils/_structs.py`` of the
reference (``tp_infos`` :318-333, ``sparse_product_info(s)`` :79-147,
``sparse_scale_info(s)`` :22-77, ``irreps_info`` :444-457, ``irreps_linear_infos``
:430-441, ``so2_linear_infos`` :784-786, ``wigner_d_info`` :638-654): integer
fields are bit-identical, ``scale`` agrees to the last float32 bit except where
the symbolic and the closed-form CG differ by one float64 ulp before rounding.

The reference sorts Python tuples and run-length-encodes Python lists; here the
tables are columns of NumPy arrays, ordered with a stable ``lexsort`` and
segmented with vectorised boundary detection.  The contract that matters to the
kernels is kept:

* rows are ordered by (output id, index1, index2, scale);
* ``seg_out`` has ``out_size + 1`` entries, empty outputs repeat the pointer;
* a field that would equal ``arange`` is replaced by ``None`` (identity gather /
  one entry per output), ``index_out`` and ``gather_index`` are always ``None``.

Two deliberate differences from the reference, both only visible when some
output row receives no table entry:

* the reference prepends zeros to its run pointer before re-indexing it when the
  smallest output id is not 0 (``_structs.py:105-108``), which yields all-empty
  segments; here the pointer is the correct CSR of the sorted rows;
* ``create_tp_info`` numbers the rows of the weight step by the *rank* of the
  output component among the components that occur (``_structs.py:228-231``), so a
  component without paths shifts every later one; here the component id itself is
  used.  For tables whose outputs are all populated both agree bit for bit.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .constants import j_matrix, so3_clebsch_gordan
from .irreps import Irreps, check_irreps, has_path, irrep_segments
from .structs import (IrrepsInfo, IrrepsLinearInfo, SparseProductInfo, SparseScaleInfo,
                      TensorProductInfo, WignerRotationInfo)

_I = np.int64


# --------------------------------------------------------------------------
# column helpers
# --------------------------------------------------------------------------
def _col(values, n: Optional[int] = None, dtype=_I) -> np.ndarray:
    if values is None:
        return np.arange(n, dtype=dtype)
    return np.asarray(values, dtype=dtype)


def _order(*cols: np.ndarray) -> np.ndarray:
    """Stable permutation sorting rows lexicographically by ``cols`` (first = major)."""
    if len(cols[0]) == 0:
        return np.zeros(0, dtype=_I)
    return np.lexsort(tuple(reversed(cols)))


def _runs(*cols: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    """Run-length segmentation of already ordered rows.

    Returns ``(run_id per row, start offsets of the runs plus the total length)``.
    """
    n = len(cols[0])
    if n == 0:
        return np.zeros(0, dtype=_I), np.zeros(1, dtype=_I)
    change = np.zeros(n, dtype=bool)
    change[0] = True
    for c in cols:
        change[1:] |= c[1:] != c[:-1]
    starts = np.flatnonzero(change)
    return np.cumsum(change) - 1, np.append(starts, n).astype(_I)


def _dense_rank(*cols: np.ndarray) -> Tuple[np.ndarray, List[np.ndarray]]:
    """Rank of every row among the sorted distinct rows, and those distinct rows."""
    perm = _order(*cols)
    sorted_cols = [c[perm] for c in cols]
    rid, ptr = _runs(*sorted_cols)
    rank = np.empty(len(perm), dtype=_I)
    rank[perm] = rid
    return rank, [c[ptr[:-1]] for c in sorted_cols]


def _csr(sorted_ids: np.ndarray, out_size: int) -> np.ndarray:
    """CSR pointer (``out_size + 1`` entries) of ascending output ids."""
    counts = np.bincount(sorted_ids, minlength=out_size)[:out_size] if len(sorted_ids) else np.zeros(out_size, _I)
    return np.concatenate([[0], np.cumsum(counts)]).astype(_I)


def _is_arange(a: np.ndarray, n: int) -> bool:
    return len(a) == n and bool(np.array_equal(a, np.arange(n, dtype=a.dtype)))


def _t(a: Optional[np.ndarray], floating: bool = False) -> Optional[torch.Tensor]:
    if a is None:
        return None
    if floating:
        return torch.tensor(np.asarray(a, dtype=np.float64).tolist(), dtype=torch.get_default_dtype())
    return torch.from_numpy(np.ascontiguousarray(a, dtype=_I))


def _first_len(*lists) -> int:
    for l in lists:
        if l is not None and len(l) > 0:
            return len(l)
    raise AssertionError("At least one of the indices should be not None")


# --------------------------------------------------------------------------
# generic sparse tables
# --------------------------------------------------------------------------
def sparse_scale_info(index=None, index_out=None, scale=None, out_size=None) -> SparseScaleInfo:
    """Table of ``z[index_out[t]] += scale[t] * x[index[t]]`` sorted by output row."""
    n = _first_len(index, index_out)
    src, dst = _col(index, n), _col(index_out, n)
    val = None if scale is None else np.asarray(scale, dtype=np.float64)
    perm = _order(dst, src) if val is None else _order(dst, src, val)
    src, dst = src[perm], dst[perm]
    val = None if val is None else val[perm]
    if out_size is None:
        out_size = len(np.unique(dst))
    ptr = _csr(dst, out_size)
    return SparseScaleInfo(
        scale=_t(val, floating=True),
        index=None if _is_arange(src, n) else _t(src),
        seg_out=None if _is_arange(ptr, out_size + 1) else _t(ptr),
        index_out=None,
        out_size=out_size)


def sparse_scale_infos(index=None, index_out=None, scale=None, out_size=None, in_size=None):
    """Forward table and its transpose (for the input gradient)."""
    return (sparse_scale_info(index, index_out, scale, out_size),
            sparse_scale_info(index_out, index, scale, in_size))


def sparse_product_info(index1=None, index2=None, index=None, scale=None, out_size=None) -> SparseProductInfo:
    """Table of ``z[index[t]] += scale[t] * x[index1[t]] (*) y[index2[t]]`` sorted by output row."""
    n = _first_len(index1, index2, index)
    a, b, o = _col(index1, n), _col(index2, n), _col(index, n)
    val = None if scale is None else np.asarray(scale, dtype=np.float64)
    perm = _order(o, a, b) if val is None else _order(o, a, b, val)
    a, b, o = a[perm], b[perm], o[perm]
    val = None if val is None else val[perm]
    if out_size is None:
        out_size = len(np.unique(o))
    ptr = _csr(o, out_size)
    return SparseProductInfo(
        scale=_t(val, floating=True),
        index1=None if _is_arange(a, n) else _t(a),
        index2=None if _is_arange(b, n) else _t(b),
        seg_out=None if _is_arange(ptr, out_size + 1) else _t(ptr),
        gather_index=None,
        index_out=None,
        out_size=out_size)


def sparse_product_infos(index1=None, index2=None, index=None, scale=None,
                         out_size=None, in1_size=None, in2_size=None):
    """Forward table plus the two role-rotated tables used by the input gradients:
    (x, y -> z), (y, z -> x), (z, x -> y)."""
    n = _first_len(index1, index2, index)
    index1 = list(range(n)) if index1 is None else index1
    index2 = list(range(n)) if index2 is None else index2
    index = list(range(n)) if index is None else index
    return (sparse_product_info(index1, index2, index, scale, out_size),
            sparse_product_info(index2, index, index1, scale, in1_size),
            sparse_product_info(index, index1, index2, scale, in2_size))


# --------------------------------------------------------------------------
# SO(3) tensor-product tables
# --------------------------------------------------------------------------
def generate_fully_connected_tp_paths(irreps_out: Irreps, irreps1: Irreps, irreps2: Irreps):
    """All allowed (k, i, j) = (out, in1, in2) irrep triples, k-major."""
    out, in1, in2 = list(irreps_out), list(irreps1), list(irreps2)
    return [(k, i, j) for k, ko in enumerate(out) for i, a in enumerate(in1)
            for j, b in enumerate(in2) if has_path(ko, a, b)]


def prepare_so3(irreps_out: Irreps, irreps1: Irreps, irreps2: Irreps, path=None,
                path_norm: bool = True, channel_norm: bool = False, channel_scale: float = 1.0):
    """Flat list of the non-zero, normalised CG entries of every path.

    Returns ``(cg, M, M1, M2, k, i, j, w_idx, num_paths)``.  ``path_norm`` divides by the
    square root of the number of *consecutive* paths sharing an output irrep
    (reference ``_structs.py:177-184``), ``channel_norm`` multiplies by ``channel_scale``.
    """
    if not path:
        path = generate_fully_connected_tp_paths(irreps_out, irreps1, irreps2)
    out, in1, in2 = list(irreps_out), list(irreps1), list(irreps2)
    off_out, off1, off2 = irrep_segments(irreps_out), irrep_segments(irreps1), irrep_segments(irreps2)

    fan: Dict[int, int] = {}
    prev = None
    for k, _, _ in path:
        fan[k] = fan[k] + 1 if k == prev else 1
        prev = k

    cols = [[] for _ in range(8)]
    for w, (k, i, j) in enumerate(path):
        cg = so3_clebsch_gordan(out[k].l, in1[i].l, in2[j].l)
        norm = (fan[k] ** (-0.5) if path_norm else 1.0) * (channel_scale if channel_norm else 1.0)
        vals = cg * norm
        mo, m1, m2 = np.nonzero(vals)          # C order == (m_out, m1, m2) nested loops
        cols[0].append(vals[mo, m1, m2])
        cols[1].append(mo + off_out[k])
        cols[2].append(m1 + off1[i])
        cols[3].append(m2 + off2[j])
        for c, v in zip(cols[4:], (k, i, j, w)):
            c.append(np.full(len(mo), v, dtype=_I))
    cat = [np.concatenate(c) if c else np.zeros(0) for c in cols]
    return (cat[0].tolist(), *(c.astype(_I).tolist() for c in cat[1:]), len(path))


def create_tp_info(cg_vals, M, M1, M2, k, i, j, w_idx, out_size, in1_size, in2_size) -> TensorProductInfo:
    """All tables of one role assignment (out, in1, in2) of a tensor product.

    Rows are ordered by (k, M, i, j, M1, M2, w, cg); a run of equal (k, M, i, j, w) is one
    row ``Mij`` of the intermediate that the CG contraction produces and the weight step
    consumes (reference ``_structs.py:219-291``).
    """
    cg = np.asarray(cg_vals, dtype=np.float64)
    M, M1, M2, k, i, j, w = (np.asarray(c, dtype=_I) for c in (M, M1, M2, k, i, j, w_idx))
    perm = _order(k, M, i, j, M1, M2, w, cg)
    cg, M, M1, M2, k, i, j, w = (c[perm] for c in (cg, M, M1, M2, k, i, j, w))

    # CG contraction: (x[M1], y[M2]) -> inter[Mij]
    mij, mij_ptr = _runs(k, M, i, j, w)
    head = mij_ptr[:-1]
    infos_inter = sparse_product_infos(M1.tolist(), M2.tolist(), mij.tolist(), cg.tolist(),
                                       in1_size=in1_size, in2_size=in2_size)
    # weight step: (inter[Mij], W[w]) -> out[M]
    infos_M = sparse_product_infos(index2=w[head].tolist(), index=M[head].tolist(), out_size=out_size)

    # "weights first" factorisation used for the gradient w.r.t. a channel-less operand:
    #   (x[M1], W[w]) -> u[kijM1] ; (u, y[M2]) -> v[kijM1M2] ; v -> out[M] scaled by cg
    q_id, (qk, qi, qj, qM1, qM2, qw) = _dense_rank(k, i, j, M1, M2, w)
    r_id, (rk, ri, rM1, rj, rw) = _dense_rank(qk, qi, qM1, qj, qw)
    infos_kM1j = sparse_product_infos(index1=rM1.tolist(), index2=rw.tolist(), in1_size=in1_size)
    infos_kM1M2 = sparse_product_infos(index1=r_id.tolist(), index2=qM2.tolist(), in2_size=in2_size)
    infos_M_kM1M2 = sparse_scale_infos(index=q_id.tolist(), index_out=M.tolist(), scale=cg.tolist(),
                                       out_size=out_size)
    return TensorProductInfo(*infos_inter, *infos_M, *infos_kM1j, *infos_kM1M2, *infos_M_kM1M2,
                             out_size=out_size)


def tp_infos(irreps_out: Irreps, irreps1: Irreps, irreps2: Irreps, path=None,
             path_norm: bool = True, channel_norm: bool = False, channel_scale: float = 1.0):
    """Forward tables and the two role rotations used by the backward passes.

    backward1 treats in1 as the output (roles out<-in1, in1<-in2, in2<-out), backward2
    treats in2 as the output; all three share the same scaled CG values.
    """
    cg, M, M1, M2, k, i, j, w, num_paths = prepare_so3(
        irreps_out, irreps1, irreps2, path, path_norm, channel_norm, channel_scale)
    d_out, d1, d2 = irreps_out.dim, irreps1.dim, irreps2.dim
    fwd = create_tp_info(cg, M, M1, M2, k, i, j, w, d_out, d1, d2)
    bwd1 = create_tp_info(cg, M1, M2, M, i, j, k, w, d1, d2, d_out)
    bwd2 = create_tp_info(cg, M2, M, M1, j, k, i, w, d2, d_out, d1)
    return fwd, bwd1, bwd2, num_paths


# --------------------------------------------------------------------------
# irrep-wise / irreps linear
# --------------------------------------------------------------------------
def irreps_info(irreps: Irreps) -> IrrepsInfo:
    irreps = check_irreps(irreps)
    dims = [ir.dim for ir in irreps]
    f = torch.get_default_dtype()
    return IrrepsInfo(
        torch.tensor([d ** (-0.5) for d in dims], dtype=f),
        torch.tensor([1 / d for d in dims], dtype=f),
        torch.tensor([n for n, d in enumerate(dims) for _ in range(d)], dtype=torch.long),
        torch.tensor(irrep_segments(irreps), dtype=torch.long),
        len(dims))


def generate_fully_connected_irreps_linear_paths(irreps_out: Irreps, irreps_in: Irreps):
    return [(a, b) for a, ir_o in enumerate(irreps_out) for b, ir_i in enumerate(irreps_in)
            if has_path(ir_o, ir_i)]


def prepare_irreps_linear(irreps_out, irreps_in, path, path_norm, channel_norm, channel_scale: float = 1.0):
    if not path:
        path = generate_fully_connected_irreps_linear_paths(irreps_out, irreps_in)
    out = list(irreps_out)
    off_out, off_in = irrep_segments(irreps_out), irrep_segments(irreps_in)
    fan: Dict[int, int] = {}
    prev = None
    for a, _ in path:
        fan[a] = fan[a] + 1 if a == prev else 1
        prev = a
    scales, Ms, M0s, i_s, i0_s, ws = [], [], [], [], [], []
    for w, (a, b) in enumerate(path):
        s = fan[a] ** (-0.5) if path_norm else 1
        if channel_norm:
            s *= channel_scale
        for m in range(out[a].dim):
            scales.append(s); Ms.append(off_out[a] + m); M0s.append(off_in[b] + m)
            i_s.append(a); i0_s.append(b); ws.append(w)
    return scales, Ms, M0s, i_s, i0_s, ws, len(path)


def create_irreps_linear_info(scales, M_s, M0_s, ii0_s, out_size) -> IrrepsLinearInfo:
    s = np.asarray(scales, dtype=np.float64)
    M, M0, w = (np.asarray(c, dtype=_I) for c in (M_s, M0_s, ii0_s))
    p = _order(M, M0, w, s)
    _, ptr = _runs(M[p])
    q = _order(w, M, M0, s)
    _, wptr = _runs(w[q], s[q])
    return IrrepsLinearInfo(
        _t(s[p], floating=True), _t(ptr), _t(w[p]), _t(M0[p]), _t(M[p]), _t(M[p][ptr[:-1]]),
        _t(wptr), _t(M[q]), _t(M0[q]), _t(s[q][wptr[:-1]], floating=True), out_size)


def irreps_linear_infos(irreps_out: Irreps, irreps_in: Irreps, path=None, path_norm: bool = True,
                        channel_norm: bool = False, channel_scale: float = 1.0):
    scales, M_s, M0_s, _, _, w, num_paths = prepare_irreps_linear(
        irreps_out, irreps_in, path, path_norm, channel_norm, channel_scale)
    return (create_irreps_linear_info(scales, M_s, M0_s, w, irreps_out.dim),
            create_irreps_linear_info(scales, M0_s, M_s, w, irreps_in.dim), num_paths)


def irreps_blocks_infos(irreps: Irreps):
    """Block-diagonal (per irrep) dense matrix application as a sparse product."""
    rows, cols = [], []
    base = 0
    for ir in check_irreps(irreps):
        for r in range(base, base + ir.dim):
            for c in range(base, base + ir.dim):
                rows.append(r); cols.append(c)
        base += ir.dim
    return sparse_product_infos(list(range(len(rows))), cols, rows)


# --------------------------------------------------------------------------
# Wigner rotation tables
# --------------------------------------------------------------------------
def _component_table(irreps) -> Tuple[List[Tuple[int, int, int]], Dict[Tuple[int, int, int], int]]:
    comps = [(n, ir.l, m) for n, ir in enumerate(irreps) for m in range(-ir.l, ir.l + 1)]
    return comps, {c: pos for pos, c in enumerate(comps)}


def prepare_z_rotation(irreps):
    """Entries of ``x'[M] = cos(m a) x[M] - sign(m) sin(|m| a) x[M(-m)]`` against the
    packed vector ``[1, sin a, cos a, sin 2a, cos 2a, ...]`` (reference ``_structs.py:460-520``)."""
    comps, where = _component_table(irreps)
    if irreps.dim != len(comps):
        raise RuntimeError("irreps.dim does not match the number of components")
    i1, i2, io, sc = [], [], [], []
    for M, (n, l, m) in enumerate(comps):
        if m == 0:
            io.append(M); sc.append(1.0); i1.append(M); i2.append(0)
            continue
        io += [M, M]
        sc += [1.0, -1.0 if m > 0 else 1.0]
        i1 += [M, where[(n, l, -m)]]
        i2 += [2 * abs(m), 2 * abs(m) - 1]
    max_l = max((l for _, l, _ in comps), default=0)
    return i1, i2, io, sc, 1 + 2 * max_l


def z_rotation_infos(irreps: Irreps):
    i1, i2, io, sc, cs_dim = prepare_z_rotation(irreps)
    return sparse_product_infos(index1=i1, index2=i2, index=io, scale=sc,
                                out_size=irreps.dim, in1_size=irreps.dim, in2_size=cs_dim)


def j_matrix_info(irreps: Irreps) -> SparseScaleInfo:
    """Block-diagonal J as a sparse row-scaled gather; entries below 1e-9 are dropped."""
    src, dst, val = [], [], []
    base = 0
    for ir in irreps:
        J = j_matrix(ir.l)
        r, c = np.nonzero(np.abs(J) > 1e-9)
        dst += (base + r).tolist(); src += (base + c).tolist(); val += J[r, c].tolist()
        base += ir.dim
    return sparse_scale_info(index=src, index_out=dst, scale=val, out_size=irreps.dim)


def wigner_d_info(irreps: Irreps) -> WignerRotationInfo:
    irreps = check_irreps(irreps)
    fwd, bwd_x, bwd_cs = z_rotation_infos(irreps)
    # reference quirk (_structs.py:645): iterating an Irrep yields (l, p), so `sign` holds two
    # entries per irrep; it is unused by every consumer and kept only for field parity.
    sign = [ir.p ** ir.l for ir in irreps for _ in ir]
    return WignerRotationInfo(j_matrix_info=j_matrix_info(irreps), rotate_z_info_fwd=fwd,
                              rotate_z_info_bwd_input=bwd_x, rotate_z_info_bwd_cs=bwd_cs,
                              sign=torch.tensor(sign), max_m=max(ir.l for ir in irreps))


# --------------------------------------------------------------------------
# SO(2) linear
# --------------------------------------------------------------------------
def prepare_so2_linear(irreps_out, irreps_in, path=None, path_norm=True, channel_norm=False, channel_scale=1.0):
    """Entries of the per-|m| 2x2 mixing ``[[w+, -w-], [w-, w+]]`` of an SO(2) linear layer.

    Weight ids are handed out per path and m in the order (m=0), (-1, +1), (-2, +2), ...
    The fan-in used by ``path_norm`` follows the reference's counting
    (``_structs.py:715-729``): for m > 0 the count under key (k, m) is re-derived from the
    never-written key (k, -m), so it stays 1 however many paths feed that output.
    """
    out, inn = list(irreps_out), list(irreps_in)
    if path is None:
        path = [(a, b) for a in range(len(out)) for b in range(len(inn))]
    _, pos_in = _component_table(inn)
    _, pos_out = _component_table(out)

    wid: Dict[Tuple[int, int, int], int] = {}
    fan: Dict[Tuple[int, int], int] = {}
    for a, b in path:
        for m in range(min(out[a].l, inn[b].l) + 1):
            if m == 0:
                wid[(a, b, 0)] = len(wid)
                fan[(a, 0)] = fan.get((a, 0), 0) + 1
            else:
                wid[(a, b, -m)] = len(wid)
                wid[(a, b, m)] = len(wid)
                fan[(a, m)] = fan.get((a, -m), 0) + 1

    i1, i2, io, sc = [], [], [], []
    for a, b in path:
        lo, li = out[a].l, inn[b].l
        for m in range(min(lo, li) + 1):
            if m == 0:
                sc.append(fan[(a, 0)] ** (-0.5) if path_norm else 1.0)
                io.append(pos_out[(a, lo, 0)]); i1.append(pos_in[(b, li, 0)]); i2.append(wid[(a, b, 0)])
                continue
            s = (fan[(a, m)] * 2) ** (-0.5) if path_norm else 2 ** (-0.5)
            for sign, mo, mi, mw in ((1, m, m, m), (1, -m, -m, m), (-1, m, -m, -m), (1, -m, m, -m)):
                sc.append(sign * s)
                io.append(pos_out[(a, lo, mo)]); i1.append(pos_in[(b, li, mi)]); i2.append(wid[(a, b, mw)])
    if channel_norm:
        sc = [s * channel_scale for s in sc]
    return i1, i2, io, sc, len(wid)


def so2_linear_info(irreps_out, irreps_in, path=None, path_norm=True, channel_norm=False, channel_scale=1.0):
    i1, i2, io, sc, nw = prepare_so2_linear(irreps_out, irreps_in, path, path_norm, channel_norm, channel_scale)
    return sparse_product_info(i1, i2, io, sc, irreps_out.dim), nw


def so2_linear_infos(irreps_out, irreps_in, path=None, path_norm=True, channel_norm=False, channel_scale=1.0):
    i1, i2, io, sc, nw = prepare_so2_linear(irreps_out, irreps_in, path, path_norm, channel_norm, channel_scale)
    return (*sparse_product_infos(i1, i2, io, sc, irreps_out.dim, irreps_in.dim, nw), nw)
