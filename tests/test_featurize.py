"""Edge featurisation: radial basis / cutoff modules and oracle against the fixture generated from the reference
(CPU); the cell-list radius graph and the fused per-edge features against the oracle (GPU)."""
import types

import pytest
import torch

from equitorch_b200 import nn as enn
from oracle import featurize as ofe
from tests.conftest import load_golden

GOLD = load_golden("radial")
DEV = "cuda:0"


def _module(name, kw):
    kind = name.split("/")[0]
    if kind == "bessel":
        return enn.BesselBasis(kw["r_max"], kw["num_basis"])
    if kind == "polynomial":
        return enn.PolynomialCutoff(kw["r_max"], kw["r_min"], kw["p"])
    if kind == "cosine":
        return enn.CosineCutoff(kw["r_max"], kw["r_min"])
    return enn.MollifierCutoff(kw["r_max"], kw["r_min"], kw["eps"])


@pytest.mark.parametrize("name", sorted(GOLD["cases"]))
def test_radial_modules_and_oracle_match_reference_fixture(name):
    case, x = GOLD["cases"][name], GOLD["x"].clone().requires_grad_(True)
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.float64)
    try:
        mod = _module(name, case["kwargs"])
    finally:
        torch.set_default_dtype(prev)
    out = mod(x)
    (gx,) = torch.autograd.grad(out.sum(), x)
    assert float((out - case["out"]).abs().max()) <= 1e-12 * max(1.0, float(case["out"].abs().max()))
    assert float((gx - case["gx"]).abs().max()) <= 1e-12 * max(1.0, float(case["gx"].abs().max()))
    kw, kind = case["kwargs"], name.split("/")[0]
    if kind == "bessel":
        w = torch.linspace(1.0, kw["num_basis"], kw["num_basis"], dtype=torch.float64) * torch.pi
        ref = ofe.bessel_basis(GOLD["x"], kw["r_max"], w)
    else:
        ref = ofe.cutoff(GOLD["x"], kind, kw["r_max"], kw.get("r_min", 0.0), kw.get("p", 6.0), kw.get("eps", 1e-7))
    assert float((ref - case["out"]).abs().max()) <= 1e-12 * max(1.0, float(case["out"].abs().max()))


def _points(n, graphs, box, seed):
    g = torch.Generator().manual_seed(seed)
    pos = torch.rand(n, 3, generator=g) * box
    batch = torch.sort(torch.randint(0, graphs, (n,), generator=g)).values if graphs > 1 else None
    return pos, batch


@pytest.mark.gpu
@pytest.mark.parametrize("n,graphs,box,r,cap,loop", [(960, 32, 6.0, 5.0, 64, False), (3000, 1, 12.0, 1.5, 32, False),
                                                      (500, 3, 4.0, 1.0, 8, True), (7, 1, 1.0, 0.3, 32, False)])
def test_radius_graph_matches_brute_force(n, graphs, box, r, cap, loop):
    """Index tables bit-exact: same edges in the same (target, source) order as the brute-force oracle, including
    the max_num_neighbors truncation and several graphs per batch."""
    from equitorch_b200.ops.featurize_op import radius_graph_features
    pos, batch = _points(n, graphs, box, n)
    src, dst = ofe.radius_graph(pos, r, batch, loop, cap)
    f = radius_graph_features(pos.to(DEV), r, None if batch is None else batch.to(DEV), loop, cap)
    assert torch.equal(f.src.cpu(), src) and torch.equal(f.dst.cpu(), dst)
    assert torch.equal(f.ptr.cpu()[1:], torch.cumsum(torch.bincount(dst, minlength=n), 0))
    assert torch.equal(f.vec.cpu(), pos[dst] - pos[src])


@pytest.mark.gpu
@pytest.mark.parametrize("l_max", [0, 1, 2, 3, 4])
def test_fused_edge_features_match_oracle(l_max):
    """Harmonics, Bessel basis and the three cutoffs written by the edge kernel against the float64 oracle on the
    same edges (molecular configuration: 32 graphs x 30 nodes, 6 A box, 5 A cutoff); error = max |a - b| / max |b|,
    bound 1e-5."""
    from equitorch_b200.transforms import EdgeFeaturizer
    pos, batch = _points(960, 32, 6.0, 3)
    src, dst = ofe.radius_graph(pos, 5.0, batch, False, 64)
    vec, length, sh = ofe.edge_features(pos.double(), src, dst, l_max, integral_normalize=l_max == 2)
    w = torch.linspace(1.0, 8, 8, dtype=torch.float64) * torch.pi
    for cut, kind in ((enn.PolynomialCutoff(5.0, 0.5, 6), "polynomial"), (enn.CosineCutoff(5.0), "cosine"),
                      (enn.MollifierCutoff(5.0), "mollifier")):
        data = types.SimpleNamespace(pos=pos.to(DEV), batch=batch.to(DEV))
        data = EdgeFeaturizer(5.0, l_max, enn.BesselBasis(5.0, 8).to(DEV), cut, max_num_neighbors=64,
                              integral_normalize=l_max == 2)(data)
        assert torch.equal(data.edge_index.cpu(), torch.stack([src, dst]))
        want = {"edge_sh": sh, "edge_norm": length, "edge_emb": ofe.bessel_basis(length, 5.0, w),
                "edge_cutoff": ofe.cutoff(length, kind, 5.0, cut.r_min, getattr(cut, "p", 6.0), getattr(cut, "eps", 1e-7))}
        for key, ref in want.items():
            got = getattr(data, key).double().cpu()
            assert got.shape == ref.shape, key
            assert float((got - ref).abs().max()) <= 1e-5 * max(1e-30, float(ref.abs().max())), (key, kind)


@pytest.mark.gpu
def test_transforms_chain_like_the_reference():
    """RadiusGraph -> AddVectorNorm -> AddSphericalHarmonics -> AddVectorLengthEmbedding with the reference's attribute
    names; differentiable with respect to the positions."""
    from equitorch_b200 import transforms as T
    pos, _ = _points(200, 1, 3.0, 5)
    data = types.SimpleNamespace(pos=pos.to(DEV).requires_grad_(True), batch=None)
    data = T.AddVectorLengthEmbedding(enn.BesselBasis(1.2, 8).to(DEV))(T.AddSphericalHarmonics(3)(T.AddVectorNorm()(T.RadiusGraph(1.2)(data))))
    src, dst = ofe.radius_graph(pos, 1.2)
    assert torch.equal(data.edge_index.cpu(), torch.stack([src, dst]))
    assert data.edge_sh.shape == (src.numel(), 16) and data.edge_emb.shape == (src.numel(), 8)
    (g,) = torch.autograd.grad(data.edge_emb.sum() + data.edge_sh.sum() + data.edge_norm.sum(), data.pos)
    po = pos.double().requires_grad_(True)
    vec, length, sh = ofe.edge_features(po, src, dst, 3)
    ref = ofe.bessel_basis(length, 1.2, torch.linspace(1.0, 8, 8, dtype=torch.float64) * torch.pi).sum() + sh.sum() + length.sum()
    (go,) = torch.autograd.grad(ref, po)
    assert float((g.double().cpu() - go).abs().max()) <= 1e-4 * float(go.abs().max())
