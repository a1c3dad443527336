"""``TensorDot`` ('uu'): the oracle against the fixture generated from the reference (CPU), the CUDA module against
the fixture and against the oracle at a larger size (GPU)."""
import pytest
import torch

from equitorch_b200 import nn as enn
from oracle import tensor_products as otp
from tests.conftest import load_golden

GOLD = load_golden("tensor_dot")
DEV = "cuda:0"


@pytest.mark.parametrize("key", sorted(GOLD["cases"]))
def test_oracle_matches_reference_fixture(key):
    case = GOLD["cases"][key]
    a, b = (case[k].clone().requires_grad_(True) for k in ("a", "b"))
    out = otp.tensor_dot_uu(a, b, key.split("/")[0], case["scaled"])
    ga, gb = torch.autograd.grad(out, [a, b], case["cot"])
    for got, want in ((out, case["out"]), (ga, case["ga"]), (gb, case["gb"])):
        assert got.shape == want.shape
        assert float((got - want).abs().max()) <= 1e-12 * max(1.0, float(want.abs().max()))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,tol", [(torch.float64, 1e-11), (torch.float32, 1e-5)])
@pytest.mark.parametrize("key", sorted(GOLD["cases"]))
def test_module_matches_reference_fixture(key, dtype, tol):
    case = GOLD["cases"][key]
    prev = torch.get_default_dtype()
    torch.set_default_dtype(dtype)          # the 1 / sqrt(2l + 1) table is built in the default dtype, as in the reference
    try:
        mod = enn.TensorDot(key.split("/")[0], "uu", scaled=case["scaled"]).to(DEV)
    finally:
        torch.set_default_dtype(prev)
    a, b = (case[k].to(DEV, dtype).requires_grad_(True) for k in ("a", "b"))
    out = mod(a, b)
    ga, gb = torch.autograd.grad(out, [a, b], case["cot"].to(DEV, dtype))
    for got, want in ((out, case["out"]), (ga, case["ga"]), (gb, case["gb"])):
        want = want.to(DEV, dtype)
        assert got.shape == want.shape
        assert float((got - want).abs().max()) <= tol * max(1.0, float(want.abs().max()))


@pytest.mark.gpu
def test_module_against_oracle_at_layer_size():
    """4096 x 16 x 64 float32 against the float64 oracle, error = max |a - b| / max |b| <= 1e-5; a shared second
    operand takes the table-driven path."""
    name, n, c = "0e+1o+2e+3o", 4096, 64
    g = torch.Generator().manual_seed(9)
    a, b = torch.randn(n, 16, c, generator=g), torch.randn(n, 16, c, generator=g)
    cot = torch.randn(n, 4, c, generator=g)
    ao, bo = (t.double().requires_grad_(True) for t in (a, b))
    ref = otp.tensor_dot_uu(ao, bo, name, True)
    gref = torch.autograd.grad(ref, [ao, bo], cot.double())
    mod = enn.TensorDot(name, "uu", scaled=True).to(DEV)
    ag, bg = (t.to(DEV).requires_grad_(True) for t in (a, b))
    out = mod(ag, bg)
    grads = torch.autograd.grad(out, [ag, bg], cot.to(DEV))
    for got, want in zip([out, *grads], [ref, *gref]):
        err = float((got.detach().double().cpu() - want.detach()).abs().max() / want.detach().abs().max())
        assert err < 1e-5, err
    shared = mod(ag, bg[0].detach())
    want = otp.tensor_dot_uu(ao.detach(), bo[0].detach().expand(n, 16, c), name, True)
    assert float((shared.double().cpu() - want).abs().max() / want.abs().max()) < 1e-5
