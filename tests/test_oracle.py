"""Pin the CPU oracle against outputs of the reference (tests/golden), float64, 1e-12."""
import pytest
import torch

from equitorch_b200 import constants, tables
from equitorch_b200.irreps import Irreps
from oracle import sparse_ops, sphericals, tensor_products as otp

TOL = dict(rtol=1e-12, atol=1e-12)


def _grads(fn, rec):
    leaves = [t.clone().requires_grad_(True) for t in rec["inputs"]]
    out = fn(*leaves)
    torch.testing.assert_close(out, rec["out"], **TOL)
    got = torch.autograd.grad(out, leaves, rec["cotangent"], allow_unused=True)
    for g, want in zip(got, rec["grads"]):
        if want is None:
            continue
        torch.testing.assert_close(g, want, **TOL)


def test_sparse_ops_match_reference(golden_ops):
    cases = golden_ops["cases"]
    assert len(cases) > 70
    for n, case in enumerate(cases):
        if case["op"] == "scale_segment":
            got = sparse_ops.indexed_scale_segment(case["input1"], **case["kwargs"])
        else:
            fn = getattr(sparse_ops, f"indexed_{case['op']}_scale_gather")
            got = fn(case["input1"], case["input2"], **case["kwargs"])
        torch.testing.assert_close(got, case["out"], **TOL, msg=lambda m: f"case {n} {case['op']}: {m}")


@pytest.mark.parametrize("form", ["dense", "sparse"])
def test_so3linear_matches_reference(golden_layers, form):
    torch.set_default_dtype(torch.float64)
    try:
        keys = [k for k in golden_layers if k.startswith("so3linear/")]
        assert len(keys) == 13
        for key in keys:
            rec = golden_layers[key]
            c = rec["ctor"]
            kw = dict(path_norm=c.get("path_norm", True), channel_norm=c.get("channel_norm", False),
                      channel_scale=c["channels_in"] ** -0.5)
            if form == "dense":
                fn = lambda x, y, w: otp.so3_linear_dense(x, y, w, c["irreps_in1"], c["irreps_in2"], c["irreps_out"],  # noqa: E731
                                                          feature_mode=c["feature_mode"], **kw)
            else:
                info = tables.tp_infos(Irreps(c["irreps_out"]), Irreps(c["irreps_in1"]), Irreps(c["irreps_in2"]), **kw)[0]
                fn = lambda x, y, w: otp.so3_linear_sparse(x, y, w, info, c["feature_mode"])  # noqa: E731
            _grads(fn, rec)
    finally:
        torch.set_default_dtype(torch.float32)


@pytest.mark.parametrize("form", ["dense", "sparse"])
def test_tensorproduct_matches_reference(golden_layers, form):
    torch.set_default_dtype(torch.float64)
    try:
        for key in [k for k in golden_layers if k.startswith("tensorproduct/")]:
            rec = golden_layers[key]
            c = rec["ctor"]
            if form == "dense":
                fn = lambda x, y, w: otp.tensor_product_dense(x, y, w, c["irreps_in1"], c["irreps_in2"], c["irreps_out"],  # noqa: E731
                                                              feature_mode=c["feature_mode"])
            else:
                info = tables.tp_infos(Irreps(c["irreps_out"]), Irreps(c["irreps_in1"]), Irreps(c["irreps_in2"]))[0]
                fn = lambda x, y, w: otp.tensor_product_sparse(x, y, w, info, c["feature_mode"])  # noqa: E731
            _grads(fn, rec)
    finally:
        torch.set_default_dtype(torch.float32)


def test_so2_and_irrepwise_match_reference(golden_layers):
    torch.set_default_dtype(torch.float64)
    try:
        for mode in ("uu", "uv"):
            rec = golden_layers[f"so2linear/{mode}"]
            c = rec["ctor"]
            info = tables.so2_linear_infos(Irreps(c["irreps_out"]), Irreps(c["irreps_in"]))[0]
            _grads(lambda x, w: otp.so2_linear_sparse(x, w, info, mode), rec)
        rec = golden_layers["irrepwiselinear"]
        ii = tables.irreps_info(Irreps(rec["ctor"]["irreps"]))
        _grads(lambda x, w: otp.irrep_wise_linear(x, w, ii.irrep_index), rec)
    finally:
        torch.set_default_dtype(torch.float32)


def test_spherical_harmonics_match_reference(golden_layers):
    _grads(lambda v: sphericals.spherical_harmonics(v, 4), golden_layers["sh/op_l4"])
    _grads(lambda v: sphericals.spherical_harmonics(torch.nn.functional.normalize(v, dim=-1), 3),
           golden_layers["sh/module_l3"])
    inv = 1.0 / (2.0 * torch.pi ** 0.5)
    _grads(lambda v: sphericals.spherical_harmonics(torch.nn.functional.normalize(v, dim=-1), 6) * inv,
           golden_layers["sh/module_l6_integral"])


def test_wigner_d_matches_reference(golden_layers):
    jb = {l: torch.from_numpy(constants.j_matrix(l).copy()) for l in range(4)}
    _grads(lambda a, b, c: sphericals.wigner_d([0, 1, 2, 3], a, b, c, jb), golden_layers["wignerd/l3"])
    _grads(lambda a, b, c: sphericals.wigner_d([0, 0, 1, 2], a, b, c, jb), golden_layers["wignerd/mul"])
    torch.set_default_dtype(torch.float64)
    try:
        info = tables.wigner_d_info(Irreps((0, 2)))
    finally:
        torch.set_default_dtype(torch.float32)
    sc = sphericals.sincos
    _grads(lambda x, a, b, c: otp.sparse_wigner_rotation(x, sc(a, 2), sc(b, 2), sc(c, 2), info),
           golden_layers["sparse_wigner_rotation/l2"])


def test_wigner_d_rotates_spherical_harmonics():
    """D(a,b,c) SH(v) = SH(R v) with R = Rz(a) Ry(b) Rz(c) (known-answer property)."""
    g = torch.Generator().manual_seed(5)
    a, b, c = (torch.rand(7, generator=g, dtype=torch.float64) * 6 - 3 for _ in range(3))
    v = torch.nn.functional.normalize(torch.randn(7, 3, generator=g, dtype=torch.float64), dim=-1)

    def rz(t):
        z, o = torch.zeros_like(t), torch.ones_like(t)
        return torch.stack([torch.cos(t), -torch.sin(t), z, torch.sin(t), torch.cos(t), z, z, z, o], -1).view(-1, 3, 3)

    def ry(t):
        z, o = torch.zeros_like(t), torch.ones_like(t)
        return torch.stack([torch.cos(t), z, torch.sin(t), z, o, z, -torch.sin(t), z, torch.cos(t)], -1).view(-1, 3, 3)

    rv = (rz(a) @ ry(b) @ rz(c) @ v.unsqueeze(-1)).squeeze(-1)
    jb = {l: torch.from_numpy(constants.j_matrix(l).copy()) for l in range(5)}
    d = sphericals.wigner_d([0, 1, 2, 3, 4], a, b, c, jb)
    lhs = (d @ sphericals.spherical_harmonics(v, 4).unsqueeze(-1)).squeeze(-1)
    torch.testing.assert_close(lhs, sphericals.spherical_harmonics(rv, 4), rtol=1e-11, atol=1e-11)


def test_message_passing_oracle_is_sum_of_edge_messages():
    g = torch.Generator().manual_seed(9)
    ir = "0e+1o+2e"
    nodes, edges, c = 7, 30, 3
    x = torch.randn(nodes, 9, c, generator=g, dtype=torch.float64)
    vec = torch.randn(edges, 3, generator=g, dtype=torch.float64)
    src = torch.randint(0, nodes, (edges,), generator=g)
    dst = torch.sort(torch.randint(0, nodes, (edges,), generator=g)).values
    w = torch.randn(11, c, c + 1, generator=g, dtype=torch.float64)
    out = otp.so3_linear_message_passing(x, vec, src, dst, w, ir, ir, ir, feature_mode="uv")
    y = sphericals.spherical_harmonics(torch.nn.functional.normalize(vec, dim=-1), 2)
    msg = otp.so3_linear_dense(x[src], y, w, ir, ir, ir, feature_mode="uv")
    want = torch.zeros_like(out)
    for e in range(edges):
        want[dst[e]] += msg[e]
    torch.testing.assert_close(out, want, rtol=1e-12, atol=1e-12)
