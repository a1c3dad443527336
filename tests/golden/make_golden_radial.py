"""Generate ``radial.pt.gz``: outputs of the reference's ``BesselBasis`` and cutoff modules (and the gradient of
their sum with respect to the distances) on seeded inputs (float64, CPU).

    python tests/golden/make_golden_radial.py

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


def main():
    torch.set_default_dtype(torch.float64)
    import_reference()
    from equitorch.nn.cutoffs import CosineCutoff, MollifierCutoff, PolynomialCutoff
    from equitorch.nn.radials import BesselBasis
    gen = torch.Generator().manual_seed(17)
    x = (torch.rand(64, generator=gen) * 6.0 + 0.05).requires_grad_(True)      # beyond r_max = 5 too
    cases = {}
    mods = {"bessel/8": (BesselBasis(5.0, 8), dict(r_max=5.0, num_basis=8)),
            "bessel/3": (BesselBasis(2.5, 3, trainable=False), dict(r_max=2.5, num_basis=3)),
            "polynomial/p6": (PolynomialCutoff(5.0), dict(r_max=5.0, r_min=0.0, p=6.0)),
            "polynomial/p3_rmin": (PolynomialCutoff(5.0, 1.0, 3), dict(r_max=5.0, r_min=1.0, p=3.0)),
            "cosine": (CosineCutoff(5.0, 0.5), dict(r_max=5.0, r_min=0.5)),
            "mollifier": (MollifierCutoff(5.0, 0.0, 1e-7), dict(r_max=5.0, r_min=0.0, eps=1e-7))}
    for name, (mod, kw) in mods.items():
        out = mod(x)
        (gx,) = torch.autograd.grad(out.sum(), x)
        cases[name] = dict(kwargs=kw, out=out.detach(), gx=gx.detach())
    path = os.path.join(HERE, "radial.pt.gz")
    with gzip.open(path, "wb") as fh:
        torch.save({"x": x.detach(), "cases": cases}, fh)
    print(path, len(cases), "cases")


if __name__ == "__main__":
    main()
