"""Parity of the module / functional layer on the GPU with the reference's outputs and gradients
(golden fixtures, float64 and float32) and with the CPU oracle at benchmark-like sizes."""
import pytest
import torch

from equitorch_b200 import nn as enn
from equitorch_b200.irreps import Irreps
from equitorch_b200.nn.functional import sincos
from equitorch_b200.ops.spherical_harmonics import spherical_harmonics
from oracle import tensor_products as otp

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = {torch.float64: 1e-10, torch.float32: 1e-5}


def _check(fn, rec, dtype, what):
    leaves = [t.to(DEV, dtype).requires_grad_(True) for t in rec["inputs"]]
    out = fn(*leaves)
    tol = TOL[dtype]

    def close(got, want, name):
        scale = float(want.abs().max().clamp_min(1e-30))
        err = float((got.detach().double().cpu() - want).abs().max()) / scale
        assert err < tol, f"{what}: {name} relative error {err:.2e} (tolerance {tol})"

    assert out.shape == rec["out"].shape, what
    close(out, rec["out"], "output")
    grads = torch.autograd.grad(out, leaves, rec["cotangent"].to(DEV, dtype), allow_unused=True)
    for n, (g, want) in enumerate(zip(grads, rec["grads"])):
        if want is not None:
            close(g, want, f"grad[{n}]")


def _module(cls, ctor, dtype, **extra):
    """Tables are built in the default dtype (as in the reference), so float64 runs build them in float64."""
    old = torch.get_default_dtype()
    torch.set_default_dtype(dtype)
    try:
        return cls(**ctor, internal_weights=False, **extra).to(DEV)
    finally:
        torch.set_default_dtype(old)


@pytest.mark.parametrize("dtype", [torch.float64, torch.float32])
def test_so3linear_fixtures(golden_layers, dtype):
    keys = [k for k in golden_layers if k.startswith("so3linear/")]
    assert len(keys) == 13
    for key in keys:
        rec = golden_layers[key]
        layer = _module(enn.SO3Linear, rec["ctor"], dtype)
        _check(lambda x, y, w: layer(x, y, w), rec, dtype, key)


@pytest.mark.parametrize("dtype", [torch.float64, torch.float32])
def test_tensorproduct_fixtures(golden_layers, dtype):
    for key in [k for k in golden_layers if k.startswith("tensorproduct/")]:
        rec = golden_layers[key]
        layer = _module(enn.TensorProduct, rec["ctor"], dtype)
        _check(lambda x, y, w: layer(x, y, w), rec, dtype, key)


@pytest.mark.parametrize("dtype", [torch.float64, torch.float32])
def test_so2_irrepwise_irrepslinear_fixtures(golden_layers, dtype):
    for mode in ("uu", "uv"):
        rec = golden_layers[f"so2linear/{mode}"]
        layer = _module(enn.SO2Linear, rec["ctor"], dtype)
        _check(lambda x, w: layer(x, w), rec, dtype, f"so2linear/{mode}")
    rec = golden_layers["irrepwiselinear"]
    layer = _module(enn.IrrepWiseLinear, rec["ctor"], dtype)
    _check(lambda x, w: layer(x, w), rec, dtype, "irrepwiselinear")
    rec = golden_layers["irrepslinear"]
    layer = _module(enn.IrrepsLinear, rec["ctor"], dtype)
    _check(lambda x, w: layer(x, w), rec, dtype, "irrepslinear")


@pytest.mark.parametrize("dtype", [torch.float64, torch.float32])
def test_spherical_harmonics_fixtures(golden_layers, dtype):
    _check(lambda v: spherical_harmonics(v, 4, -1), golden_layers["sh/op_l4"], dtype, "sh/op_l4")
    _check(lambda v: enn.SphericalHarmonics(3)(v), golden_layers["sh/module_l3"], dtype, "sh/module_l3")
    _check(lambda v: enn.SphericalHarmonics(6, integral_normalize=True)(v), golden_layers["sh/module_l6_integral"],
           dtype, "sh/module_l6_integral")


def test_spherical_harmonics_high_degree_and_other_axis():
    from oracle.sphericals import spherical_harmonics as osh
    v = torch.nn.functional.normalize(torch.randn(3, 1000, dtype=torch.float64), dim=0)
    got = spherical_harmonics(v.to(DEV), 17, 0)
    want = osh(v, 17, 0)
    assert got.shape == (18 * 18, 1000)
    torch.testing.assert_close(got.cpu(), want, rtol=1e-9, atol=1e-9)


@pytest.mark.parametrize("dtype", [torch.float64, torch.float32])
def test_wigner_fixtures(golden_layers, dtype):
    old = torch.get_default_dtype()
    torch.set_default_dtype(dtype)
    try:
        wig, wig2, rot = (enn.WignerD(Irreps((0, 3))).to(DEV), enn.WignerD(Irreps("2x0e+1o+2e")).to(DEV),
                          enn.SparseWignerRotation(Irreps((0, 2))).to(DEV))
    finally:
        torch.set_default_dtype(old)
    _check(lambda a, b, c: wig(a, b, c), golden_layers["wignerd/l3"], dtype, "wignerd/l3")
    _check(lambda a, b, c: wig2(a, b, c), golden_layers["wignerd/mul"], dtype, "wignerd/mul")
    _check(lambda x, a, b, c: rot(x, sincos(a, 2), sincos(b, 2), sincos(c, 2)),
           golden_layers["sparse_wigner_rotation/l2"], dtype, "sparse_wigner_rotation/l2")


@pytest.mark.parametrize("mode,per_sample", [("uu", False), ("uu", True), ("uv", False)])
def test_config1_like_against_oracle(mode, per_sample):
    """1024 samples, 0e+1o+2e, 16 channels, y = SH(lmax 2): forward + backward, float32, 1e-5."""
    g = torch.Generator().manual_seed(0)
    ir, N, C = "0e+1o+2e", 1024, 16
    x = torch.randn(N, 9, C, generator=g)
    v = torch.randn(N, 3, generator=g)
    shape = (11, C) if mode == "uu" else (11, C, C)
    w = torch.randn(*((N,) + shape if per_sample else shape), generator=g) / 4
    cot = torch.randn(N, 9, C, generator=g)
    # oracle in float64
    xo, vo, wo = (t.double().requires_grad_(True) for t in (x, v, w))
    from oracle.sphericals import spherical_harmonics as osh
    yo = osh(torch.nn.functional.normalize(vo, dim=-1), 2)
    out_o = otp.so3_linear_dense(xo, yo, wo, ir, ir, ir, feature_mode=mode)
    go = torch.autograd.grad(out_o, [xo, vo, wo], cot.double())
    # CUDA path in float32
    layer = enn.SO3Linear(ir, ir, ir, C, C, internal_weights=False, feature_mode=mode).to(DEV)
    xg, vg, wg = (t.to(DEV).requires_grad_(True) for t in (x, v, w))
    out_g = layer(xg, enn.SphericalHarmonics(2)(vg), wg)
    gg = torch.autograd.grad(out_g, [xg, vg, wg], cot.to(DEV))
    for name, a, b in [("out", out_g, out_o)] + [(f"grad{n}", a, b) for n, (a, b) in enumerate(zip(gg, go))]:
        err = float((a.detach().double().cpu() - b.detach()).abs().max() / b.detach().abs().max())
        assert err < 1e-5, f"{name}: relative error {err:.2e}"


def test_gradcheck_and_gradgradcheck_small():
    """Finite-difference check in float64 (tolerances of the reference's own test: 1e-5)."""
    torch.manual_seed(0)
    ir = "0e+1o"
    for cls, ctor, shapes in [
        (enn.SO3Linear, dict(irreps_in1=ir, irreps_in2=ir, irreps_out=ir, channels_in=2, channels_out=3, feature_mode="uv"),
         [(3, 4, 2), (3, 4)]),
        (enn.SO3Linear, dict(irreps_in1=ir, irreps_in2=ir, irreps_out=ir, channels_in=2, channels_out=2, feature_mode="uu"),
         [(3, 4, 2), (3, 4)]),
        (enn.TensorProduct, dict(irreps_in1=ir, irreps_in2=ir, irreps_out=ir, channels_in1=2, channels_in2=2,
                                 channels_out=2, feature_mode="uuu"), [(3, 4, 2), (3, 4, 2)]),
        (enn.TensorProduct, dict(irreps_in1=ir, irreps_in2=ir, irreps_out=ir, channels_in1=2, channels_in2=3,
                                 channels_out=2, feature_mode="uvw"), [(3, 4, 2), (3, 4, 3)]),
    ]:
        torch.set_default_dtype(torch.float64)
        try:
            layer = cls(**ctor, internal_weights=False).to(DEV)
        finally:
            torch.set_default_dtype(torch.float32)
        ins = [torch.randn(*s, dtype=torch.float64, device=DEV, requires_grad=True) for s in shapes]
        w = torch.randn(*layer.weight_shape, dtype=torch.float64, device=DEV, requires_grad=True)
        assert torch.autograd.gradcheck(lambda a, b, c: layer(a, b, c), (*ins, w), eps=1e-6, atol=1e-5, rtol=1e-5,
                                        nondet_tol=1e-9)
        assert torch.autograd.gradgradcheck(lambda a, b, c: layer(a, b, c), (*ins, w), eps=1e-6, atol=1e-5, rtol=1e-5,
                                            nondet_tol=1e-9)
