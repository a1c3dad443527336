"""Generate the golden fixtures in this directory by running the reference itself.

    python tests/golden/make_golden.py            # needs the reference checkout (see _reference_import)

Every fixture is a gzip-compressed ``torch.save`` dictionary of CPU tensors: seeded inputs, the
reference's outputs and, for differentiable layers, the reference's gradients for a
fixed random cotangent.  The tests load these files; they never need the reference.

Files written
-------------
tables.pt.gz  index tables (``tp_infos``, ``so2_linear_infos``, ``wigner_d_info``,
            ``irreps_info``, ``irreps_linear_infos``) flattened to ``{path: tensor|int|None}``
ops.pt.gz     the sparse ops on small ragged inputs, all flag combinations the library uses
layers.pt.gz  SO3Linear / TensorProduct / SO2Linear / IrrepWiseLinear / IrrepsLinear,
            SphericalHarmonics, WignerD, SparseWignerRotation: outputs and gradients (float64)
"""
from __future__ import annotations

import gzip
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from _reference_import import import_reference  # noqa: E402
from make_golden_shared import flatten  # noqa: E402

import_reference()
from equitorch.irreps import Irreps  # noqa: E402  (reference)
from equitorch.nn import (IrrepsLinear, IrrepWiseLinear, SO2Linear, SO3Linear, SparseWignerRotation,  # noqa: E402
                          SphericalHarmonics, TensorProduct, WignerD)
from equitorch.nn.functional.angular import sincos  # noqa: E402
from equitorch.ops import batched_sparse_dense_op as ref_ops  # noqa: E402
from equitorch.ops.indexed_scale_segment_op import indexed_scale_segment  # noqa: E402
from equitorch.ops.spherical_harmonics import spherical_harmonics  # noqa: E402
from equitorch.utils import _structs as ref_tables  # noqa: E402


def make_tables():
    fx = {}
    for tag, (o, a, b) in {
        "tp_l1": ("0e+1o", "0e+1o", "0e+1o"),
        "tp_l2": ("0e+1o+2e",) * 3,
        "tp_l3": ("0e+1o+2e+3o",) * 3,
        "tp_mul": ("4x0e+2x1o+2e", "0e+1o+2e", "4x0e+2x1o+2e"),
        "tp_so3": ("0+1+2", "0+1", "1+2"),
    }.items():
        for pn in (True, False):
            fx[f"{tag}/path_norm={pn}"] = dict(
                args=(o, a, b), kwargs=dict(path_norm=pn),
                out=flatten(ref_tables.tp_infos(Irreps(o), Irreps(a), Irreps(b), path_norm=pn)))
    fx["tp_l2/channel_norm"] = dict(
        args=("0e+1o+2e",) * 3, kwargs=dict(channel_norm=True, channel_scale=0.25),
        out=flatten(ref_tables.tp_infos(*(Irreps("0e+1o+2e"),) * 3, channel_norm=True, channel_scale=0.25)))
    for tag, (o, i) in {"so2_l2": ((0, 2), (0, 2)), "so2_l6": ((0, 6), (0, 6)), "so2_mixed": ("0e+1o+2e", "1o+2e+3o")}.items():
        fx[tag] = dict(args=(o, i), out=flatten(ref_tables.so2_linear_infos(Irreps(o), Irreps(i))))
    for tag, ir in {"wigner_l3": (0, 3), "wigner_l6": (0, 6), "wigner_mul": "2x0e+3x1o+2e"}.items():
        fx[tag] = dict(args=(ir,), out=flatten(ref_tables.wigner_d_info(Irreps(ir))))
        fx["irreps_info_" + tag] = dict(args=(ir,), out=flatten(ref_tables.irreps_info(Irreps(ir))))
    fx["irreps_linear"] = dict(args=("2x0e+1o+2e", "0e+2x1o+2e+2e"),
                               out=flatten(ref_tables.irreps_linear_infos(Irreps("2x0e+1o+2e"), Irreps("0e+2x1o+2e+2e"))))
    return fx


def make_ops():
    """Ragged sizes on purpose: N=5, C=3 / 2, empty segments, shared operands."""
    g = torch.Generator().manual_seed(1234)
    N, M1, M2, C, C2, T = 5, 6, 4, 3, 2, 11
    idx1 = torch.randint(0, M1, (T,), generator=g)
    idx2 = torch.randint(0, M2, (T,), generator=g)
    scale = torch.randn(T, generator=g, dtype=torch.float64)
    seg = torch.tensor([0, 2, 2, 5, 9, 11])           # 5 outputs, one empty
    gather = torch.randperm(T, generator=g)
    index_out = torch.tensor([4, 0, 6, 2, 3])         # scatter into 7 rows
    r = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)  # noqa: E731
    x, y = r(N, M1, C), r(N, M2, C)
    xs, ys = r(M1, C), r(M2, C)
    y2 = r(N, M2, C2)
    sca, scas = r(N, M2), r(M2)
    mat, mats = r(N, M2, C, C2), r(M2, C, C2)
    cases = []

    def add(op, a, b, **kw):
        fn = getattr(ref_ops, f"indexed_{op}_scale_gather")
        cases.append(dict(op=op, input1=a, input2=b, kwargs=kw, out=fn(a, b, **kw)))

    variants = [
        dict(scale=scale, index1=idx1, index2=idx2, seg=seg),
        dict(scale=scale, index1=idx1, index2=idx2, seg=seg, out_accumulated=True),
        dict(index1=idx1, index2=idx2),
        dict(scale=scale, index1=idx1, index2=idx2, seg=seg, gather_index=gather),
        dict(scale=scale, index1=idx1, index2=idx2, seg=seg, index_out=index_out, out_size=7),
    ]
    for kw in variants:
        add("mul", x, y, **kw)
        add("mul", xs, y, **kw)
        add("mul", x, ys, **kw)
        add("outer", x, y2, **kw)
        add("inner", x, y, **kw)
        add("inner", x, ys, **kw)
        add("vecmat", x, mat, **kw)
        add("vecmat", x, mats, **kw)
        add("vecmat", xs, mat, **kw)
        add("vecsca", x, sca, **kw)
        add("vecsca", xs, sca, **kw)
        add("vecsca", x, scas, **kw)
        add("scavec", sca, x, scale=kw.get("scale"),
            index1=idx2, index2=idx1, **{k: v for k, v in kw.items() if k not in ("scale", "index1", "index2")})
        add("mat_t_vec", mats, x, scale=kw.get("scale"), index1=idx2, index2=idx1,
            **{k: v for k, v in kw.items() if k not in ("scale", "index1", "index2")})
    # identity-indexed forms used by the weight step and the irrep-wise layers
    segM = torch.tensor([0, 1, 4, 6])
    add("mul", x, y[:, :1].expand(N, M1, C).contiguous(), seg=segM)
    add("vecmat", x, mats[torch.tensor([0, 1, 1, 2, 3, 3])], index2=None, seg=segM)
    add("outer", x, r(N, M1, C2), seg=segM, out_accumulated=True)
    ss = dict(op="scale_segment", input1=x, input2=None,
              kwargs=dict(scale=scale, index=idx1, seg=seg),
              out=indexed_scale_segment(x, scale, idx1, seg))
    cases.append(ss)
    return dict(cases=cases)


def _with_grads(fn, inputs, seed):
    """Run ``fn(*inputs)`` and back-propagate a seeded cotangent through it."""
    leaves = [t.clone().requires_grad_(True) for t in inputs]
    out = fn(*leaves)
    cot = torch.randn(out.shape, generator=torch.Generator().manual_seed(seed), dtype=out.dtype)
    grads = torch.autograd.grad(out, leaves, cot, allow_unused=True)
    return dict(inputs=[t.detach() for t in inputs], out=out.detach(), cotangent=cot,
                grads=[None if gr is None else gr.detach() for gr in grads])


def make_layers():
    torch.set_default_dtype(torch.float64)
    g = torch.Generator().manual_seed(2024)
    r = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)  # noqa: E731
    fx = {}
    N = 6
    # ---- SO3Linear
    for tag, (i1, i2, io, C) in {"l2": ("0e+1o+2e", "0e+1o+2e", "0e+1o+2e", 4),
                                 "l3": ("0e+1o+2e+3o", "0e+1o+2e+3o", "0e+1o+2e+3o", 3),
                                 "mul": ("4x0e+2x1o+2e", "0e+1o+2e", "4x0e+2x1o+2e", 2)}.items():
        d1, d2 = Irreps(i1).dim, Irreps(i2).dim
        for mode in ("uu", "uv"):
            for per_sample in (False, True):
                Cout = C if mode == "uu" else C + 1
                layer = SO3Linear(i1, i2, io, C, Cout, internal_weights=False, feature_mode=mode)
                wshape = (N, *layer.weight_shape) if per_sample else layer.weight_shape
                rec = _with_grads(lambda x, y, w: layer(x, y, w), [r(N, d1, C), r(N, d2), r(*wshape)], 7)
                rec["ctor"] = dict(irreps_in1=i1, irreps_in2=i2, irreps_out=io, channels_in=C,
                                   channels_out=Cout, feature_mode=mode)
                fx[f"so3linear/{tag}/{mode}/{'per_sample' if per_sample else 'shared'}"] = rec
    layer = SO3Linear("0e+1o+2e", "0e+1o+2e", "0e+1o+2e", 4, 5, internal_weights=False, feature_mode="uv",
                      channel_norm=True, path_norm=False)
    rec = _with_grads(lambda x, y, w: layer(x, y, w), [r(N, 9, 4), r(N, 9), r(*layer.weight_shape)], 8)
    rec["ctor"] = dict(irreps_in1="0e+1o+2e", irreps_in2="0e+1o+2e", irreps_out="0e+1o+2e", channels_in=4,
                       channels_out=5, feature_mode="uv", channel_norm=True, path_norm=False)
    fx["so3linear/l2/uv/channel_norm"] = rec
    # ---- TensorProduct
    for mode in ("uuu", "uvw"):
        for per_sample in (False, True):
            c1, c2, co = (3, 3, 3) if mode == "uuu" else (3, 2, 4)
            layer = TensorProduct("0e+1o+2e", "0e+1o", "0e+1o+2e", c1, c2, co, internal_weights=False, feature_mode=mode)
            wshape = (N, *layer.weight_shape) if per_sample else layer.weight_shape
            rec = _with_grads(lambda x, y, w: layer(x, y, w), [r(N, 9, c1), r(N, 4, c2), r(*wshape)], 9)
            rec["ctor"] = dict(irreps_in1="0e+1o+2e", irreps_in2="0e+1o", irreps_out="0e+1o+2e",
                               channels_in1=c1, channels_in2=c2, channels_out=co, feature_mode=mode)
            fx[f"tensorproduct/{mode}/{'per_sample' if per_sample else 'shared'}"] = rec
    # ---- SO2Linear
    for mode in ("uu", "uv"):
        layer = SO2Linear((0, 3), (0, 2), 3, 3 if mode == "uu" else 4, internal_weights=False, feature_mode=mode)
        rec = _with_grads(lambda x, w: layer(x, w), [r(N, 16, 3), r(*layer.weight_shape)], 10)
        rec["ctor"] = dict(irreps_in=(0, 3), irreps_out=(0, 2), channels_in=3,
                           channels_out=3 if mode == "uu" else 4, feature_mode=mode)
        fx[f"so2linear/{mode}"] = rec
    # ---- IrrepWiseLinear / IrrepsLinear
    layer = IrrepWiseLinear("2x0e+1o+2e", 3, 4, internal_weights=False)
    rec = _with_grads(lambda x, w: layer(x, w), [r(N, 10, 3), r(*layer.weight_shape)], 11)
    rec["ctor"] = dict(irreps="2x0e+1o+2e", channels_in=3, channels_out=4)
    fx["irrepwiselinear"] = rec
    layer = IrrepsLinear("0e+2x1o+2e", "2x0e+1o+2e", 3, 4, internal_weights=False)
    rec = _with_grads(lambda x, w: layer(x, w), [r(N, 12, 3), r(*layer.weight_shape)], 12)
    rec["ctor"] = dict(irreps_in="0e+2x1o+2e", irreps_out="2x0e+1o+2e", channels_in=3, channels_out=4)
    fx["irrepslinear"] = rec
    # ---- spherical harmonics (raw op on non-unit vectors, module on normalised ones)
    v = r(9, 3)
    fx["sh/op_l4"] = _with_grads(lambda t: spherical_harmonics(t, 4, -1), [v], 13)
    fx["sh/module_l3"] = _with_grads(lambda t: SphericalHarmonics(3)(t), [v], 14)
    fx["sh/module_l6_integral"] = _with_grads(lambda t: SphericalHarmonics(6, integral_normalize=True)(t), [v], 15)
    # ---- Wigner D
    a, b, c = (torch.rand(5, generator=g) * 6.0 - 3.0 for _ in range(3))
    wig = WignerD(Irreps((0, 3)))
    fx["wignerd/l3"] = _with_grads(lambda p, q, s: wig(p, q, s), [a, b, c], 16)
    wig2 = WignerD(Irreps("2x0e+1o+2e"))
    fx["wignerd/mul"] = _with_grads(lambda p, q, s: wig2(p, q, s), [a, b, c], 17)
    rot = SparseWignerRotation(Irreps((0, 2)))
    fx["sparse_wigner_rotation/l2"] = _with_grads(
        lambda x, p, q, s: rot(x, sincos(p, 2), sincos(q, 2), sincos(s, 2)), [r(5, 9, 3), a, b, c], 18)
    torch.set_default_dtype(torch.float32)
    return fx


if __name__ == "__main__":
    torch.manual_seed(0)
    for name, maker in (("tables", make_tables), ("ops", make_ops), ("layers", make_layers)):
        data = maker()
        path = os.path.join(HERE, f"{name}.pt.gz")
        with gzip.open(path, "wb", compresslevel=9) as fh:
            torch.save(data, fh)
        print(f"{name}: {os.path.getsize(path) / 1024:.1f} KiB")
