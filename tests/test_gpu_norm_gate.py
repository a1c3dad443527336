"""Gate, norm and RMS-normalisation layers on the GPU against the fixtures generated from the reference and
against the CPU oracle at a larger size."""
import types

import pytest
import torch

from equitorch_b200 import nn as enn
from equitorch_b200.irreps import Irreps
from equitorch_b200.nn import functional as F
from equitorch_b200.tables import irreps_info
from oracle import norm_gate as ong
from tests.conftest import load_golden
from tests.test_oracle_norm_gate import run_case

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
GOLD = load_golden("norm_gate")


def _impl(name, dtype):
    """The product functions behind the oracle's call signatures (dims -> this irreps' info on the GPU)."""
    ir = Irreps(name)
    prev = torch.get_default_dtype()
    torch.set_default_dtype(dtype)
    try:
        info = irreps_info(ir).to(DEV)
    finally:
        torch.set_default_dtype(prev)

    def gate(x, g, dims, activation, irrep_wise=True):
        mod = enn.Gate(ir, activation=activation, irrep_wise=irrep_wise).to(DEV)
        mod.irreps_info = info
        return mod(x, g)

    def batch_rms(x, run, dims, w, scaled, training, momentum, eps):
        run = run.clone()
        out = F.batch_rms_norm(x, run, info, w, scaled, training, momentum, eps)
        return out, run

    return types.SimpleNamespace(
        gate=gate,
        squared_norm=lambda x, d, s: F.squared_norm(x, info, s), norm=lambda x, d, s: F.norm(x, info, s),
        channel_mean_squared_norm=lambda x, d, s: F.channel_mean_squared_norm(x, info, s),
        batch_mean_squared_norm=lambda x, d, s: F.batch_mean_squared_norm(x, info, s),
        batch_rms_norm=batch_rms,
        layer_rms_norm=lambda x, d, w, s, eps: F.layer_rms_norm(x, info, w, s, eps))


@pytest.mark.parametrize("dtype,tol", [(torch.float64, 1e-11), (torch.float32, 1e-5)])
@pytest.mark.parametrize("key", sorted(GOLD["cases"]))
def test_matches_reference_fixture(key, dtype, tol):
    case = {k: (v.to(DEV, dtype) if torch.is_tensor(v) else v) for k, v in GOLD["cases"][key].items()}
    out, grads, extra = run_case(key, case, _impl(key.split("/")[0], dtype))
    want = [case["out"], case["gx"]] + ([case["gg"] if "gg" in case else case["gw"]] if len(grads) > 1 else [])
    got = [out.detach(), *grads]
    if "run1" in case:
        want.append(case["run1"])
        got.append(extra["run1"])
    for a, b in zip(got, want):
        assert a.shape == b.shape
        assert float((a - b).abs().max()) <= tol * max(1.0, float(b.abs().max()))


def test_layer_sizes_against_oracle():
    """cfg-sized features (l_max 3, 64 channels, 4096 nodes): modules against the oracle in float64 on CPU."""
    name, n, c = "0e+1o+2e+3o", 4096, 64
    ir = Irreps(name)
    dims = [i.dim for i in ir]
    g = torch.Generator().manual_seed(5)
    x = torch.randn(n, ir.dim, c, generator=g)
    gates = torch.randn(n, len(ir), c, generator=g)
    w = torch.rand(len(ir), c, generator=g) + 0.5
    cot = torch.randn(n, ir.dim, c, generator=g)

    def chain(xx, gg, ww, impl_gate, impl_bn, impl_ln):
        return impl_ln(impl_bn(impl_gate(xx, gg), ww), ww)

    xo, go, wo = (t.double().requires_grad_(True) for t in (x, gates, w))
    ref = chain(xo, go, wo, lambda a, b: ong.gate(a, b, dims, torch.sigmoid),
                lambda a, ww: ong.batch_rms_norm(a, torch.ones(len(ir), c, dtype=torch.float64), dims, ww, True, True, 0.1, 1e-5)[0],
                lambda a, ww: ong.layer_rms_norm(a, dims, ww, True, 1e-5))
    gref = torch.autograd.grad(ref, [xo, go, wo], cot.double())

    gate = enn.Gate(ir, activation=torch.nn.Sigmoid()).to(DEV)
    bn = enn.BatchRMSNorm(ir, c).to(DEV).train()
    ln = enn.LayerRMSNorm(ir, c).to(DEV)
    xg, gg, wg = (t.to(DEV).requires_grad_(True) for t in (x, gates, w))
    bn.weight, ln.weight = torch.nn.Parameter(wg.detach().clone()), torch.nn.Parameter(wg.detach().clone())
    out = ln(bn(gate(xg, gg)))
    grads = torch.autograd.grad(out, [xg, gg, bn.weight, ln.weight], cot.to(DEV))
    got = [out, grads[0], grads[1], grads[2] + grads[3]]
    for a, b in zip(got, [ref, *gref]):
        err = float((a.detach().double().cpu() - b.detach()).abs().max() / b.detach().abs().max())
        assert err < 1e-5


@pytest.mark.parametrize("key", sorted(k for k in GOLD["cases"] if "/layer_rms" in k))
def test_layer_rms_unfused_composition(key, monkeypatch):
    """The composition of per-irrep operators (used for higher-order derivatives) gives the same result."""
    from equitorch_b200.nn.functional import normalization
    monkeypatch.setattr(normalization, "FUSED_LAYER_RMS", False)
    case = {k: (v.to(DEV) if torch.is_tensor(v) else v) for k, v in GOLD["cases"][key].items()}
    out, grads, _ = run_case(key, case, _impl(key.split("/")[0], torch.float64))
    assert float((out.detach() - case["out"]).abs().max()) <= 1e-11
    assert float((grads[0] - case["gx"]).abs().max()) <= 1e-11 * max(1.0, float(case["gx"].abs().max()))


def test_bfloat16_layers_against_oracle():
    """bfloat16 features (the molecular configuration's dtype) run through the same layers: bfloat16 storage,
    float32 arithmetic.  Checked against the float64 oracle on the bfloat16-rounded inputs at the 2e-2 the
    tensor products use for bfloat16 (error = max |a - b| / max |b|)."""
    name, n, c = "4x0e+2x1o+2e", 512, 32
    ir = Irreps(name)
    dims = [i.dim for i in ir]
    g = torch.Generator().manual_seed(11)
    x = torch.randn(n, ir.dim, c, generator=g).bfloat16()
    gates = torch.randn(n, len(ir), c, generator=g).bfloat16()
    w = (torch.rand(len(ir), c, generator=g) + 0.5).bfloat16()
    cot = torch.randn(n, ir.dim, c, generator=g).bfloat16()

    xo, go, wo = (t.double().requires_grad_(True) for t in (x, gates, w))
    ref = ong.layer_rms_norm(ong.gate(xo, go, dims, torch.sigmoid), dims, wo, True, 1e-5)
    gref = torch.autograd.grad(ref, [xo, go, wo], cot.double())
    nref = ong.squared_norm(xo, dims, True)

    gate = enn.Gate(ir, activation=torch.nn.Sigmoid()).to(DEV)
    ln = enn.LayerRMSNorm(ir, c).to(DEV).to(torch.bfloat16)
    xg, gg = (t.to(DEV).requires_grad_(True) for t in (x, gates))
    ln.weight = torch.nn.Parameter(w.to(DEV))
    out = ln(gate(xg, gg))
    assert out.dtype == torch.bfloat16
    grads = torch.autograd.grad(out, [xg, gg, ln.weight], cot.to(DEV))
    info = irreps_info(ir).to(DEV)
    got_norm = F.squared_norm(xg.detach(), info, True)
    assert grads[0].dtype == torch.bfloat16
    for a, b in zip([out, *grads, got_norm], [ref, *gref, nref]):
        err = float((a.detach().double().cpu() - b.detach()).abs().max() / b.detach().abs().max())
        assert err < 2e-2, err
