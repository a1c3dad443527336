"""Import the reference implementation from a read-only checkout.

Used by the fixture generators (``make_golden*.py``), by optional cross-checks that are
skipped when the checkout is absent, and by the CPU arm of ``bench.py``, which points
``EQUITORCH_REFERENCE_ROOT`` at the unmodified install of the reference under
``baseline/_ref`` to time the reference's own CPU code.  No test that runs on a GPU
machine needs the checkout.

The reference imports ``torch_geometric`` for two CPU reductions (``segment``,
``scatter``) and a few names it never calls on this path.  That package is not
installed, so small stand-ins written from the documented semantics are
registered under its name before the reference is imported:

* ``segment(src, ptr)``: CSR segment-sum along dimension ``ptr.dim() - 1``;
* ``scatter(src, index, dim, dim_size)``: index-add (sum) along ``dim``.
"""
from __future__ import annotations

import os
import sys
import types

import torch

# the checkout is looked for beside this repository unless EQUITORCH_REFERENCE_ROOT says otherwise
_REPO = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
REFERENCE_ROOT = os.environ.get("EQUITORCH_REFERENCE_ROOT", os.path.join(os.path.dirname(_REPO), "reference"))


def _segment(src: torch.Tensor, ptr: torch.Tensor, reduce: str = "sum") -> torch.Tensor:
    assert reduce == "sum"
    dim = ptr.dim() - 1
    p = ptr.reshape(-1)
    pieces = [src.narrow(dim, int(p[i]), int(p[i + 1] - p[i])).sum(dim=dim, keepdim=True)
              for i in range(p.numel() - 1)]
    if not pieces:
        shape = list(src.shape)
        shape[dim] = 0
        return src.new_zeros(shape)
    return torch.cat(pieces, dim=dim)


def _scatter(src: torch.Tensor, index: torch.Tensor, dim: int = 0, dim_size=None, reduce: str = "sum"):
    assert reduce == "sum"
    dim = dim % src.dim()
    size = int(index.max()) + 1 if dim_size is None else dim_size
    shape = list(src.shape)
    shape[dim] = size
    return src.new_zeros(shape).index_add_(dim, index, src)


def _install_stand_in() -> None:
    if "torch_geometric" in sys.modules:
        return
    root = types.ModuleType("torch_geometric")
    utils = types.ModuleType("torch_geometric.utils")
    utils.segment, utils.scatter = _segment, _scatter
    data = types.ModuleType("torch_geometric.data")
    data.Data = type("Data", (), {})
    pipes = types.ModuleType("torch_geometric.data.datapipes")
    pipes.functional_transform = lambda name: (lambda cls: cls)
    transforms = types.ModuleType("torch_geometric.transforms")
    transforms.BaseTransform = type("BaseTransform", (), {})
    nn = types.ModuleType("torch_geometric.nn")
    nn.radius_graph = None
    root.utils, root.data, root.transforms, root.nn = utils, data, transforms, nn
    data.datapipes = pipes
    for mod in (root, utils, data, pipes, transforms, nn):
        sys.modules[mod.__name__] = mod


def reference_available() -> bool:
    return os.path.isdir(os.path.join(REFERENCE_ROOT, "equitorch"))


def import_reference():
    """Return the reference's top-level package (``equitorch``)."""
    if not reference_available():
        raise RuntimeError(f"no reference checkout at {REFERENCE_ROOT}")
    _install_stand_in()
    if REFERENCE_ROOT not in sys.path:
        sys.path.insert(0, REFERENCE_ROOT)
    import equitorch  # noqa: WPS433  (the reference, not this repository's package)
    return equitorch
