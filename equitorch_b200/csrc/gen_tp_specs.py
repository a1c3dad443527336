"""Generate ``generated/tp_specs.inc``: fully unrolled Clebsch-Gordan inner loops.

The fused tensor-product kernels keep the gathered feature row, the per-node outer-product
accumulators and the CG sums in registers.  Registers cannot be indexed at run time, so for
the index structures that matter (the registry below) the loops over the accumulator cells
and over the table entries are emitted as straight-line code, one set of functions per warp
role (see ``OuterPlan``).  Only the *index structure* is baked in; the CG values stay
run-time data (``scale``), so path / channel normalisation do not need their own code.

A structure is identified by ``structure_key`` (a hash of T, R, D_feat, D_y and the three
index columns); ``equitorch_b200.ops.fused_tp_op.TpTable`` computes the same key from a layer's tables and
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


NUM_ROLES = 4


class OuterPlan(NamedTuple):
    """Split of a structure for the outer-product kernels.

    The sum over the edges of a node commutes with the CG contraction:
    ``S[d, r] = sum_t scale[t] * Q_d[m_y[t], m_feat[t]]`` with ``Q_d = sum_e y_e (x) x_e``.  A *cell* is a
    pair (m_y, m_feat) that some entry uses.  Cells that share a row are tied together; the resulting
    groups (for irreps tables: the (l_y, l_feat) blocks) are dealt to ``NUM_ROLES`` warps so that every
    row is produced by exactly one warp from accumulators it holds itself.
    """
    cells: List[np.ndarray]      # per role: (n, 2) array of (m_y, m_feat), its accumulator order
    rows: List[np.ndarray]       # per role: rows it produces, ascending
    entries: List[np.ndarray]    # per role: entry ids sorted by row
    offsets: List[int]           # start of each role's block in the permuted scale array (multiples of 4)


def outer_plan(s: Structure, roles: int = NUM_ROLES) -> OuterPlan:
    cell_id = s.my * s.d_feat + s.mf
    parent = {int(c): int(c) for c in np.unique(cell_id)}

    def find(c):
        while parent[c] != c:
            parent[c] = parent[parent[c]]
            c = parent[c]
        return c

    starts = np.searchsorted(s.row, np.arange(s.num_rows + 1))
    for r in range(s.num_rows):
        cs = cell_id[starts[r]:starts[r + 1]]
        for c in cs[1:]:
            ra, rb = find(int(cs[0])), find(int(c))
            if ra != rb:
                parent[max(ra, rb)] = min(ra, rb)
    groups = {}
    for c in parent:
        groups.setdefault(find(c), []).append(c)
    # largest group first onto the lightest role (ties: lowest role) - deterministic
    order = sorted(groups.items(), key=lambda kv: (-len(kv[1]), kv[0]))
    load = [0] * roles
    owner = {}
    for root, members in order:
        w = min(range(roles), key=lambda i: (load[i], i))
        load[w] += len(members)
        for c in members:
            owner[c] = w
    cells, rows, entries, offsets = [], [], [], [0]
    for w in range(roles):
        cw = np.array(sorted(c for c in owner if owner[c] == w), dtype=np.int64)
        cells.append(np.stack([cw // s.d_feat, cw % s.d_feat], axis=1) if len(cw) else np.zeros((0, 2), np.int64))
        tw = np.array([t for t in range(len(s.row)) if owner[int(cell_id[t])] == w], dtype=np.int64)
        entries.append(tw)
        rw = set(int(r) for r in s.row[tw])
        if w == 0:                                     # rows without any entry are written (as zeros) by role 0
            rw |= set(range(s.num_rows)) - set(int(r) for r in s.row)
        rows.append(np.array(sorted(rw), dtype=np.int64))
        offsets.append(offsets[-1] + ((len(tw) + 3) // 4) * 4)
    return OuterPlan(cells, rows, entries, offsets)


def outer_order(s: Structure) -> np.ndarray:
    """Entry ids in the order the outer-product kernels read ``scale`` (-1 = padding to a multiple of 4)."""
    plan = outer_plan(s)
    out = np.full(plan.offsets[-1], -1, dtype=np.int64)
    for w, tw in enumerate(plan.entries):
        out[plan.offsets[w]:plan.offsets[w] + len(tw)] = tw
    return out


class TcPlan(NamedTuple):
    """Layout of a structure for the tensor-core segment-sum kernel (16 x 16 components, 64 channels).

    The per-node outer product Q[f, m_y] = sum_e x_e[f] y_e[m_y] (f = (m_feat, channel), 1024 features) is eight
    tcgen05 tiles of 128 features.  A thread of the contraction stage reads one TMEM lane of every tile, i.e. one
    channel of eight components m_feat; the components are dealt to the two lane halves so that every irrep of
    the channelled operand lies in one half, and with it every intermediate row: ``mlist[h][i]`` is the component
    held by tile ``i`` for the lanes of half ``h``."""
    mlist: List[List[int]]                 # [2][8]
    phases: List[List[dict]]               # per half: phases {tiles: [(i, cols kept)], rows: [(row, [(t, tile, m_y)])]}


def _groups(keys: np.ndarray, row: np.ndarray, size: int) -> List[List[int]]:
    """Components that share a row are one group (for irreps tables: the irreps)."""
    parent = list(range(size))

    def find(c):
        while parent[c] != c:
            parent[c] = parent[parent[c]]
            c = parent[c]
        return c
    for r in np.unique(row):
        ks = keys[row == r]
        for k in ks[1:]:
            a, b = find(int(ks[0])), find(int(k))
            if a != b:
                parent[max(a, b)] = min(a, b)
    out = {}
    for c in range(size):
        out.setdefault(find(c), []).append(c)
    return [sorted(v) for _, v in sorted(out.items())]


def tc_plan(s: Structure):
    if s.d_feat != 16 or s.d_y != 16:
        return None
    fgroups, ygroups = _groups(s.mf, s.row, s.d_feat), _groups(s.my, s.row, s.d_y)
    # split the groups of the channelled operand into two halves of exactly eight components
    import itertools
    halves = None
    for pick in range(1, len(fgroups)):
        for combo in itertools.combinations(range(len(fgroups)), pick):
            if sum(len(fgroups[g]) for g in combo) == 8:
                halves = (list(combo), [g for g in range(len(fgroups)) if g not in combo])
                break
        if halves:
            break
    if halves is None:
        return None
    group_of_f = {m: g for g, ms in enumerate(fgroups) for m in ms}
    group_of_y = {k: g for g, ks in enumerate(ygroups) for k in ks}
    mlist, phases = [], []
    for h in range(2):
        ms = [m for g in halves[h] for m in fgroups[g]]
        tile_of = {m: i for i, m in enumerate(ms)}
        mlist.append(ms)
        ph = []
        for g in halves[h]:
            for yg in range(len(ygroups)):
                rows = {}
                for t in range(len(s.row)):
                    if group_of_f[int(s.mf[t])] == g and group_of_y[int(s.my[t])] == yg:
                        rows.setdefault(int(s.row[t]), []).append((t, tile_of[int(s.mf[t])], int(s.my[t])))
                if rows:
                    ph.append(dict(tiles=[tile_of[m] for m in fgroups[g]], cols=list(ygroups[yg]), rows=sorted(rows.items())))
        phases.append(ph)
    return TcPlan(mlist, phases)


def _emit_tc(s: Structure, plan: TcPlan) -> List[str]:
    out = ["  // tensor-core segment sum: component of the channelled operand held by tile i for the lanes of half h",
           "  static constexpr bool HAS_TC = true;",
           "  __device__ __forceinline__ static int tc_mfeat(int h, int i) {",
           "    switch (i) {"]
    for i in range(8):
        out.append(f"      case {i}: return h ? {plan.mlist[1][i]} : {plan.mlist[0][i]};")
    out += ["      default: return 0;", "    }", "  }"]
    used = set(int(r) for r in s.row)
    for h in range(2):
        out.append("  // contraction of one node by a lane of half %d: tq = TMEM address of the lane's row of tile 0 (tiles 16 columns apart)," % h)
        out.append("  // sc = scales in shared memory (table order), o = the lane's channel of the node's first row (row stride C floats)")
        out.append(f"  template <int C> __device__ __forceinline__ static void tc_node_h{h}(uint32_t tq, const float* sc, float* o) {{")
        for pi, ph in enumerate(plan.phases[h]):
            cols = ph["cols"]
            # smallest power-of-two run of columns covering the phase's components; all tiles are requested before one wait
            lo, width = min(cols), 1
            while lo + width <= max(cols):
                width *= 2
            if lo + width > 16:
                lo = 16 - width
            out.append("    {")
            for i in ph["tiles"]:
                out.append(f"      uint32_t q{i}[{width}];")
                out.append(f"      tmem_ld_nowait<{width}>(tq + {16 * i + lo}, q{i});")
            out.append("      tmem_wait_ld();")
            for i in ph["tiles"]:
                out.append(f"      tmem_touch<{width}>(q{i});")
            for r, ents in ph["rows"]:
                terms = [(f"sc[{t}]", f"__uint_as_float(q{tile}[{k - lo}])") for t, tile, k in ents]
                expr = f"{terms[0][0]} * {terms[0][1]}"
                for a_, b_ in terms[1:]:
                    expr = f"fmaf({a_}, {b_}, {expr})"
                out.append(f"      o[{r} * C] = {expr};")
            out.append("    }")
        if h == 0:
            for r in range(s.num_rows):
                if r not in used:
                    out.append(f"    o[{r} * C] = 0.f;")
        out.append("  }")
    return out


def _emit_outer_role(s: Structure, plan: OuterPlan, w: int) -> List[str]:
    """Functions of warp role ``w``.  A lane holds CPL channels; ``xr`` points at its channels of the
    staged feature row (component stride C floats), loaded component by component just before use."""
    cells, tw = plan.cells[w], plan.entries[w]
    index = {(int(k), int(m)): i for i, (k, m) in enumerate(cells)}
    by_m = {}
    for i, (k, m) in enumerate(cells):
        by_m.setdefault(int(m), []).append((i, int(k)))
    out = []
    # per edge: q[cell] += x[m_feat] * y[m_y]
    out.append("  template <int CPL, int C> __device__ __forceinline__ static void "
               f"outer_r{w}(float (&q)[MAXCELL][CPL], const float* xr, const float (&y)[DY]) {{")
    out.append("    float x[CPL];")
    for m in sorted(by_m):
        out.append(f"    EQT_LDX(x, xr + {m} * C);")
        for i, k in by_m[m]:
            out.append(f"    EQT_FMA(q[{i}], x, y[{k}]);")
    out.append("  }")
    # per node: rows of this role from the accumulators
    out.append("  template <int CPL, int C> __device__ __forceinline__ static void "
               f"node_r{w}(const float (&q)[MAXCELL][CPL], const float4* sc, float* o) {{")
    out.append("    float4 c; float v[CPL];")
    pos = {int(t): i for i, t in enumerate(tw)}
    by_row = {}
    for t in tw:
        by_row.setdefault(int(s.row[t]), []).append(int(t))
    loaded = -1
    for r in plan.rows[w]:
        ts = by_row.get(int(r), [])
        if not ts:
            out.append(f"    EQT_ZERO(v); EQT_STX(o + {int(r)} * C, v);")
            continue
        for n, t in enumerate(ts):
            i = pos[t]
            if i // 4 != loaded:
                loaded = i // 4
                out.append(f"    c = sc[{loaded}];")
            term = f"c.{'xyzw'[i % 4]}"
            cell = index[(int(s.my[t]), int(s.mf[t]))]
            out.append(f"    EQT_MUL(v, q[{cell}], {term});" if n == 0 else f"    EQT_FMA(v, q[{cell}], {term});")
        out.append(f"    EQT_STX(o + {int(r)} * C, v);")
    out.append("  }")
    # adjoint, per node: h[cell] = sum_t scale[t] * g[row[t]]
    out.append("  template <int CPL, int C> __device__ __forceinline__ static void "
               f"hbuild_r{w}(float (&h)[MAXCELL][CPL], const float4* sc, const float* g) {{")
    out.append("    float4 c; float gr[CPL];")
    touched = set()
    loaded = -1
    for r in plan.rows[w]:
        ts = by_row.get(int(r), [])
        if not ts:
            continue
        out.append(f"    EQT_LDG(gr, g + {int(r)} * C);")
        for t in ts:
            i = pos[t]
            if i // 4 != loaded:
                loaded = i // 4
                out.append(f"    c = sc[{loaded}];")
            term = f"c.{'xyzw'[i % 4]}"
            cell = index[(int(s.my[t]), int(s.mf[t]))]
            if cell in touched:
                out.append(f"    EQT_FMA(h[{cell}], gr, {term});")
            else:
                touched.add(cell)
                out.append(f"    EQT_MUL(h[{cell}], gr, {term});")
    out.append("  }")
    # adjoint, per edge: ay[m_y] = sum over the role's cells of <x[m_feat], h[cell]> over the lane's channels
    kys = set(int(k) for k, _ in cells)
    out.append("  template <int CPL, int C> __device__ __forceinline__ static void "
               f"dot_r{w}(float (&ay)[DY], const float* xr, const float (&h)[MAXCELL][CPL]) {{")
    out.append("    float x[CPL];")
    first = set()
    for k in range(s.d_y):
        if k not in kys:
            out.append(f"    ay[{k}] = 0.f;")
    for m in sorted(by_m):
        out.append(f"    EQT_LDX(x, xr + {m} * C);")
        for i, k in by_m[m]:
            out.append(f"    EQT_DOT(ay[{k}], x, h[{i}]);" if k in first else f"    EQT_DOT0(ay[{k}], x, h[{i}]);")
            first.add(k)
    out.append("  }")
    return out


def emit_spec(idx: int, s: Structure, note: str) -> str:
    plan = outer_plan(s)
    maxcell = max(1, max(len(c) for c in plan.cells))
    out = [f"// {note}", f"struct Spec{idx} {{",
           f"  static constexpr uint64_t KEY = {structure_key(s)}ull;",
           f"  static constexpr int T = {len(s.row)}, R = {s.num_rows}, DF = {s.d_feat}, DY = {s.d_y};",
           f"  static constexpr int MAXCELL = {maxcell};",
           f"  static constexpr int NCELL[{NUM_ROLES}] = {{{', '.join(str(len(c)) for c in plan.cells)}}};",
           "  // start of each role's block in the permuted scale array, and its end",
           "  static constexpr int " + ", ".join(f"OT{w} = {o}" for w, o in enumerate(plan.offsets)) + ";"]
    for w in range(NUM_ROLES):
        out += _emit_outer_role(s, plan, w)
    tcp = tc_plan(s)
    if tcp is not None:
        out += _emit_tc(s, tcp)
    else:
        out.append("  static constexpr bool HAS_TC = false;")
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
