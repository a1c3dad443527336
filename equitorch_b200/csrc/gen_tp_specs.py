"""Generate ``generated/tp_specs.inc``: fully unrolled Clebsch-Gordan inner loops.

The fused tensor-product kernels keep the gathered feature rows, the per-edge CG
coefficients and the accumulators in registers.  Registers cannot be indexed at run time,
so for the index structures that matter (the registry below) the loop over the table
entries is emitted as straight-line code, one function per warp of the CTA: each warp
owns a contiguous range of intermediate rows (and hence of table entries), balanced by
entry count.  Only the *index structure* is baked in; the CG values stay run-time data
(``scale``), so path / channel normalisation do not need their own code.

A structure is identified by ``structure_key`` (a hash of T, R, D_feat, D_y and the three
index columns); ``equitorch_b200.fused`` computes the same key from a layer's tables and
falls back to the table-driven kernels when the key is not in the registry.

    python -m equitorch_b200.csrc.gen_tp_specs        # rewrites generated/tp_specs.inc
"""
from __future__ import annotations

import hashlib
import os
from typing import List, NamedTuple, Sequence

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "generated", "tp_specs.inc")
NUM_WARPS = 4

# (irreps_out, irreps_in1, irreps_in2) of layers whose inner loops are unrolled at build time.
# All role rotations (forward, gradient w.r.t. input1, gradient w.r.t. input2) are generated.
REGISTRY = [
    ("0e+1o", "0e+1o", "0e+1o"),
    ("0e+1o+2e", "0e+1o+2e", "0e+1o+2e"),
    ("0e+1o+2e+3o", "0e+1o+2e+3o", "0e+1o+2e+3o"),
]


class Structure(NamedTuple):
    """CG step of one role assignment: entry t adds ``scale[t] * feat[mf[t]] * y[my[t]]`` to row[t]."""
    mf: np.ndarray     # component of the channelled operand
    my: np.ndarray     # component of the channel-less operand
    row: np.ndarray    # intermediate row, ascending
    d_feat: int
    d_y: int
    num_rows: int


def structure_key(s: Structure) -> int:
    h = hashlib.sha256()
    h.update(np.asarray([len(s.mf), s.num_rows, s.d_feat, s.d_y], dtype=np.int64).tobytes())
    for col in (s.mf, s.my, s.row):
        h.update(np.ascontiguousarray(col, dtype=np.int64).tobytes())
    return int.from_bytes(h.digest()[:7], "little")


def structure_from_info(info, feat_is_input1: bool, d_feat: int, d_y: int) -> Structure:
    """``info`` is the ``info_Mij_fwd`` table of a TensorProductInfo (rows sorted by intermediate row)."""
    t = info.scale.numel()
    seg = info.seg_out.cpu().numpy() if info.seg_out is not None else np.arange(info.out_size + 1)
    row = np.repeat(np.arange(len(seg) - 1), np.diff(seg))
    i1 = info.index1.cpu().numpy() if info.index1 is not None else np.arange(t)
    i2 = info.index2.cpu().numpy() if info.index2 is not None else np.arange(t)
    mf, my = (i1, i2) if feat_is_input1 else (i2, i1)
    return Structure(mf.astype(np.int64), my.astype(np.int64), row.astype(np.int64), d_feat, d_y, info.out_size)


def partition(s: Structure, warps: int = NUM_WARPS):
    """Split the rows into ``warps`` contiguous groups with balanced entry counts."""
    t = len(s.row)
    starts = np.searchsorted(s.row, np.arange(s.num_rows + 1))      # first entry of each row
    wr = [0]
    for w in range(1, warps):
        target = t * w / warps
        r = int(np.argmin(np.abs(starts - target)))
        wr.append(max(r, wr[-1]))
    wr.append(s.num_rows)
    wt = [int(starts[r]) for r in wr]
    return wt, wr


def kernel_order(s: Structure, warps: int = NUM_WARPS) -> np.ndarray:
    """Order in which the unrolled code visits the table entries (a permutation of ``range(T)``).

    Inside a warp's range the entries are interleaved across rows (first entry of every row, then
    the second of every row, ...), so that consecutive FMAs hit different accumulators instead of
    forming one dependent chain per row.  The run-time arrays handed to the unrolled kernels
    (``scale``, ``m_y``) are stored in this order.
    """
    wt, _ = partition(s, warps)
    order = []
    for w in range(warps):
        ts = np.arange(wt[w], wt[w + 1])
        if len(ts) == 0:
            continue
        rows = s.row[ts]
        pos = ts - np.searchsorted(rows, rows, side="left") - wt[w]      # index of the entry within its row
        order.append(ts[np.lexsort((rows, pos))])
    return np.concatenate(order) if order else np.zeros(0, dtype=np.int64)


def _emit_segsum(s: Structure, order, wt, wr, w: int) -> List[str]:
    lines = []
    tb, te, rb = wt[w], wt[w + 1], wr[w]
    for q0 in range(tb, te, 4):
        lines.append(f"    c = cf[{(q0 - tb) // 4}];")
        for q in range(q0, min(q0 + 4, te)):
            comp, t = "xyzw"[q - q0], int(order[q])
            r, m = int(s.row[t]) - rb, int(s.mf[t])
            lines.append(f"    EQT_FMA_ROW(acc[{r}], c.{comp}, x[{m}]);")
    return lines


def _emit_inner(s: Structure, order, wt, wr, w: int) -> List[str]:
    lines = []
    tb, te, rb = wt[w], wt[w + 1], wr[w]
    for q0 in range(tb, te, 4):
        lines.append(f"    c = sc[{(q0 - tb) // 4}];")
        for q in range(q0, min(q0 + 4, te)):
            comp, t = "xyzw"[q - q0], int(order[q])
            r, m, k = int(s.row[t]) - rb, int(s.mf[t]), int(s.my[t])
            lines.append(f"    ay[{k}] = fmaf(c.{comp}, EQT_DOT_ROW(x[{m}], g[{r}]), ay[{k}]);")
    return lines


def emit_spec(idx: int, s: Structure, note: str) -> str:
    wt, wr = partition(s)
    order = kernel_order(s)
    maxr = max(wr[w + 1] - wr[w] for w in range(NUM_WARPS))
    maxt = max(wt[w + 1] - wt[w] for w in range(NUM_WARPS))
    out = [f"// {note}", f"struct Spec{idx} {{",
           f"  static constexpr uint64_t KEY = {structure_key(s)}ull;",
           f"  static constexpr int T = {len(s.row)}, R = {s.num_rows}, DF = {s.d_feat}, DY = {s.d_y};",
           f"  static constexpr int MAXR = {maxr}, MAXT = {((maxt + 3) // 4) * 4};",
           f"  static constexpr int WT[{NUM_WARPS + 1}] = {{{', '.join(map(str, wt))}}};",
           f"  static constexpr int WR[{NUM_WARPS + 1}] = {{{', '.join(map(str, wr))}}};"]
    for w in range(NUM_WARPS):
        out.append("  template <int CPL> __device__ __forceinline__ static void "
                   f"segsum_w{w}(float (&acc)[MAXR][CPL], const float (&x)[DF][CPL], const float4* cf) {{")
        out.append("    float4 c;")
        out += _emit_segsum(s, order, wt, wr, w)
        out.append("  }")
        out.append("  template <int CPL> __device__ __forceinline__ static void "
                   f"inner_w{w}(float (&ay)[DY], const float (&x)[DF][CPL], const float (&g)[MAXR][CPL], const float4* sc) {{")
        out.append("    float4 c;")
        out += _emit_inner(s, order, wt, wr, w)
        out.append("  }")
    out.append("};")
    return "\n".join(out)


def collect() -> List[tuple]:
    from ..irreps import Irreps
    from ..tables import tp_infos
    seen, specs = set(), []
    for o, a, b in REGISTRY:
        io, i1, i2 = Irreps(o), Irreps(a), Irreps(b)
        fwd, bwd1, bwd2, _ = tp_infos(io, i1, i2)
        # forward: feat = input1 (index1), y = input2.  gradient of input1: table of backward1, whose
        # input1 is the channel-less operand and input2 the incoming gradient (the channelled one).
        cands = [(structure_from_info(fwd.info_Mij_fwd, True, i1.dim, i2.dim), f"{a} (x) {b} -> {o}: forward"),
                 (structure_from_info(bwd1.info_Mij_fwd, False, io.dim, i2.dim), f"{a} (x) {b} -> {o}: grad of input1")]
        for s, note in cands:
            k = structure_key(s)
            if k not in seen:
                seen.add(k)
                specs.append((s, note))
    return specs


def generate(path: str = OUT) -> str:
    specs = collect()
    body = ["// AUTO-GENERATED by equitorch_b200/csrc/gen_tp_specs.py - do not edit.",
            "// Straight-line Clebsch-Gordan inner loops; see the generator for the layout.",
            "#pragma once", ""]
    for n, (s, note) in enumerate(specs):
        body.append(emit_spec(n, s, note))
        body.append("")
    body.append(f"#define EQT_NUM_SPECS {len(specs)}")
    body.append("#define EQT_FOR_EACH_SPEC(X) " + " ".join(f"X(Spec{n})" for n in range(len(specs))))
    text = "\n".join(body) + "\n"
    os.makedirs(os.path.dirname(path), exist_ok=True)
    if not os.path.exists(path) or open(path).read() != text:
        with open(path, "w") as fh:
            fh.write(text)
    return path


if __name__ == "__main__":
    print(generate())
