"""Generate ``norm_gate.pt.gz``: outputs and gradients of the reference's gate, norm and RMS-normalisation
layers on seeded inputs (float64, CPU).

    python tests/golden/make_golden_norm_gate.py

Needs the reference checkout (``_reference_import.py``); the tests only read the fixture.
"""
from __future__ import annotations

import gzip
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from tests.golden._reference_import import import_reference  # noqa: E402

IRREPS = ["0e+1o+2e", "2x0e+1o+1e+3o", "1o"]
N, C = 5, 6


def _grads(out, inputs, gen):
    cot = torch.randn(out.shape, generator=gen, dtype=out.dtype)
    grads = torch.autograd.grad(out, inputs, cot, allow_unused=True)
    return cot, [None if g is None else g.detach() for g in grads]


def main():
    torch.set_default_dtype(torch.float64)
    eq = import_reference()
    from equitorch.irreps import Irreps
    from equitorch import nn as rnn
    cases = {}
    for name in IRREPS:
        ir = Irreps(name)
        gen = torch.Generator().manual_seed(len(name) * 7 + 1)
        x = torch.randn(N, ir.dim, C, generator=gen, requires_grad=True)
        k = len(ir)
        # --- gate: separate irrep-wise gates with an activation, shared gates, global gate, concatenated input
        g = torch.randn(N, k, C, generator=gen, requires_grad=True)
        out = rnn.Gate(ir, activation=torch.nn.Sigmoid())(x, g)
        cot, (gx, gg) = _grads(out, [x, g], gen)
        cases[f"{name}/gate_irrepwise"] = dict(x=x.detach(), g=g.detach(), out=out.detach(), cot=cot, gx=gx, gg=gg)
        gs = torch.randn(k, C, generator=gen, requires_grad=True)
        out = rnn.Gate(ir)(x, gs)
        cot, (gx, gg) = _grads(out, [x, gs], gen)
        cases[f"{name}/gate_shared"] = dict(x=x.detach(), g=gs.detach(), out=out.detach(), cot=cot, gx=gx, gg=gg)
        g1 = torch.randn(N, 1, C, generator=gen, requires_grad=True)
        out = rnn.Gate(ir, activation=torch.nn.Tanh(), irrep_wise=False)(x, g1)
        cot, (gx, gg) = _grads(out, [x, g1], gen)
        cases[f"{name}/gate_global"] = dict(x=x.detach(), g=g1.detach(), out=out.detach(), cot=cot, gx=gx, gg=gg)
        xc = torch.randn(N, ir.dim + k, C, generator=gen, requires_grad=True)
        out = rnn.Gate(ir, activation=torch.nn.SiLU())(xc)
        cot, (gx,) = _grads(out, [xc], gen)
        cases[f"{name}/gate_concat"] = dict(x=xc.detach(), out=out.detach(), cot=cot, gx=gx)
        # --- norms
        for scaled in (True, False):
            for label, mod in (("squared_norm", rnn.SquaredNorm(ir, scaled)), ("norm", rnn.Norm(ir, scaled)),
                               ("msn_channel", rnn.MeanSquaredNorm(ir, scaled, dim=-1)),
                               ("msn_batch", rnn.MeanSquaredNorm(ir, scaled, dim=0))):
                out = mod(x)
                cot, (gx,) = _grads(out, [x], gen)
                cases[f"{name}/{label}/scaled={scaled}"] = dict(x=x.detach(), out=out.detach(), cot=cot, gx=gx)
        # norm of a zero vector has zero gradient
        xz = x.detach().clone()
        xz[0] = 0.0
        xz.requires_grad_(True)
        out = rnn.Norm(ir, True)(xz)
        cot, (gx,) = _grads(out, [xz], gen)
        cases[f"{name}/norm_zero_row"] = dict(x=xz.detach(), out=out.detach(), cot=cot, gx=gx)
        # --- normalisation layers
        for scaled in (True, False):
            w = torch.rand(k, C, generator=gen) + 0.5
            bn = rnn.BatchRMSNorm(ir, C, eps=1e-5, momentum=0.3, affine=True, scaled=scaled)
            with torch.no_grad():
                bn.weight.copy_(w)
                bn.running_squared_norm.copy_(torch.rand(k, C, generator=gen) + 0.5)
            run0 = bn.running_squared_norm.clone()
            bn.train()
            out = bn(x)
            cot, (gx, gw) = _grads(out, [x, bn.weight], gen)
            cases[f"{name}/batch_rms_train/scaled={scaled}"] = dict(
                x=x.detach(), w=w, run0=run0, run1=bn.running_squared_norm.clone(), out=out.detach(), cot=cot, gx=gx, gw=gw)
            bn.eval()
            out = bn(x)
            cot, (gx, gw) = _grads(out, [x, bn.weight], gen)
            cases[f"{name}/batch_rms_eval/scaled={scaled}"] = dict(
                x=x.detach(), w=w, run0=bn.running_squared_norm.clone(), out=out.detach(), cot=cot, gx=gx, gw=gw)
            ln = rnn.LayerRMSNorm(ir, C, eps=1e-5, affine=True, scaled=scaled)
            with torch.no_grad():
                ln.weight.copy_(w)
            out = ln(x)
            cot, (gx, gw) = _grads(out, [x, ln.weight], gen)
            cases[f"{name}/layer_rms/scaled={scaled}"] = dict(x=x.detach(), w=w, out=out.detach(), cot=cot, gx=gx, gw=gw)
        ln = rnn.LayerRMSNorm(ir, C, affine=False)
        out = ln(x)
        cot, (gx,) = _grads(out, [x], gen)
        cases[f"{name}/layer_rms_noaffine"] = dict(x=x.detach(), out=out.detach(), cot=cot, gx=gx)
    path = os.path.join(HERE, "norm_gate.pt.gz")
    with gzip.open(path, "wb", compresslevel=9) as fh:
        torch.save({"n": N, "channels": C, "cases": cases}, fh)
    print(path, len(cases), "cases", os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
