"""Generate ``tensor_dot.pt.gz``: outputs and gradients of the reference's ``TensorDot`` ('uu', scaled and
unscaled; ``equitorch/nn/tensor_products.py:199-269``) on seeded inputs (float64, CPU).

    python tests/golden/make_golden_tensor_dot.py

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

IRREPS = ["0e+1o+2e", "2x0e+1o+1e+3o", "1o", "0e+1o+2e+3o"]
N, C = 7, 6


def main():
    torch.set_default_dtype(torch.float64)
    import_reference()
    from equitorch.irreps import Irreps
    from equitorch import nn as rnn
    cases = {}
    for name in IRREPS:
        ir = Irreps(name)
        gen = torch.Generator().manual_seed(len(name) * 13 + 5)
        for scaled in (True, False):
            a = torch.randn(N, ir.dim, C, generator=gen, requires_grad=True)
            b = torch.randn(N, ir.dim, C, generator=gen, requires_grad=True)
            out = rnn.TensorDot(ir, "uu", scaled=scaled)(a, b)
            cot = torch.randn(out.shape, generator=gen)
            ga, gb = torch.autograd.grad(out, [a, b], cot)
            cases[f"{name}/scaled={scaled}"] = dict(a=a.detach(), b=b.detach(), scaled=scaled, out=out.detach(), cot=cot,
                                                   ga=ga.detach(), gb=gb.detach())
    path = os.path.join(HERE, "tensor_dot.pt.gz")
    with gzip.open(path, "wb") as fh:
        torch.save({"cases": cases}, fh)
    print(path, len(cases), "cases")


if __name__ == "__main__":
    main()
