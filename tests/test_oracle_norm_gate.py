"""The norm / gate oracle against fixtures generated from the reference itself (CPU, float64)."""
import pytest
import torch

from tests.conftest import load_golden
from equitorch_b200.irreps import Irreps
from oracle import norm_gate as ong

TOL = 1e-12
ACT = {"gate_irrepwise": torch.sigmoid, "gate_shared": None, "gate_global": torch.tanh, "gate_concat": torch.nn.functional.silu}


def _dims(name):
    return [ir.dim for ir in Irreps(name)]


def _close(a, b):
    assert a.shape == b.shape
    assert float((a - b).abs().max()) <= TOL * max(1.0, float(b.abs().max()))


def run_case(key, case, impl):
    """Evaluate one fixture case with ``impl`` (a namespace of functions with the oracle's signatures)."""
    name, kind = key.split("/")[0], key.split("/")[1]
    dims = _dims(name)
    scaled = key.endswith("scaled=True")
    x = case["x"].clone().requires_grad_(True)
    inputs, extra = [x], {}
    if kind.startswith("gate"):
        g = case["g"].clone().requires_grad_(True) if "g" in case else None
        out = impl.gate(x, g, dims, ACT[kind], irrep_wise=kind != "gate_global")
        if g is not None:
            inputs.append(g)
    elif kind == "squared_norm":
        out = impl.squared_norm(x, dims, scaled)
    elif kind in ("norm", "norm_zero_row"):
        out = impl.norm(x, dims, scaled if kind == "norm" else True)
    elif kind == "msn_channel":
        out = impl.channel_mean_squared_norm(x, dims, scaled)
    elif kind == "msn_batch":
        out = impl.batch_mean_squared_norm(x, dims, scaled)
    elif kind.startswith("batch_rms"):
        w = case["w"].clone().requires_grad_(True)
        out, run = impl.batch_rms_norm(x, case["run0"].clone(), dims, w, scaled, training=kind.endswith("train"),
                                       momentum=0.3, eps=1e-5)
        inputs.append(w)
        extra["run1"] = run
    elif kind == "layer_rms":
        w = case["w"].clone().requires_grad_(True)
        out = impl.layer_rms_norm(x, dims, w, scaled, eps=1e-5)
        inputs.append(w)
    elif kind == "layer_rms_noaffine":
        out = impl.layer_rms_norm(x, dims, None, True, eps=1e-5)
    else:
        raise AssertionError(key)
    grads = torch.autograd.grad(out, inputs, case["cot"].to(out.dtype).to(out.device))
    return out, grads, extra


GOLD = load_golden("norm_gate")


@pytest.mark.parametrize("key", sorted(GOLD["cases"]))
def test_oracle_matches_reference(key):
    case = GOLD["cases"][key]
    out, grads, extra = run_case(key, case, ong)
    _close(out.detach(), case["out"])
    _close(grads[0], case["gx"])
    if len(grads) > 1:
        _close(grads[1], case["gg"] if "gg" in case else case["gw"])
    if "run1" in case:
        _close(extra["run1"], case["run1"])
