"""The smaller benchmark configurations as self-contained steps (seeded synthetic inputs, forward + backward).

Each builder returns a :class:`Workload`: pinned host inputs, matching device tensors and a ``step`` that runs the
layer forward and backward on the device tensors and returns ``(loss, results)`` - the scalar ``<out, cotangent>``
and the gradients a training loop would read back.  ``bench.py`` times them; the tests run the same shapes
against the oracle.

* ``cfg1``  one weighted CG product with a channel-less second operand: 1024 samples, l_max 2, 16 channels, 'uu'
            weights shared by the batch, spherical harmonics of 1024 random vectors (the CPU-runnable case).
* ``cfg3``  molecular-style message passing: 32 graphs x 30 nodes in a 6 A box, radius graph at 5 A, 8 Bessel
            functions -> 2-layer MLP -> per-edge 'uu' weights, node irreps 128x0e+64x1o+32x2e (4x0e+2x1o+2e with 32
            channels), l_max 2 harmonics, bfloat16 operands with float32 sums.
* ``cfg4``  Wigner-rotated SO(2) linear layer: 100k edges, 32 channels for l = 0..6, Haar rotations, D x -> per-m
            channel mixing 32 -> 32 -> D^T, float32.
"""
from __future__ import annotations

import math
from typing import Callable, List, NamedTuple, Sequence

import torch
from torch import Tensor


class Workload(NamedTuple):
    label: str
    unit: str                         # what `units` counts ("samples", "edges")
    units: int
    dtype: str
    algorithmic_bytes_per_unit: float  # minimal traffic of one forward + backward pass per unit
    host_inputs: List[Tensor]         # pinned; copied into dev_inputs at the start of an end-to-end step
    dev_inputs: List[Tensor]
    step: Callable[[], tuple]         # -> (loss (1,), [tensors a trainer reads back])
    note: str


def _pin(t: Tensor) -> Tensor:
    return t.contiguous().pin_memory() if torch.cuda.is_available() else t.contiguous()


def molecular_graph(graphs: int = 32, nodes_per_graph: int = 30, box: float = 6.0, cutoff: float = 5.0, seed: int = 0):
    """Batched radius graphs: (src, dst ascending, edge_vec = pos[dst] - pos[src], num_nodes)."""
    g = torch.Generator().manual_seed(seed)
    pos = torch.rand(graphs, nodes_per_graph, 3, generator=g) * box
    diff = pos[:, :, None, :] - pos[:, None, :, :]                  # [graph, dst, src]
    mask = (diff.norm(dim=-1) < cutoff) & ~torch.eye(nodes_per_graph, dtype=torch.bool)
    gi, dst, src = mask.nonzero(as_tuple=True)
    off = gi * nodes_per_graph
    order = torch.argsort(off + dst, stable=True)
    return (off + src)[order], (off + dst)[order], diff[gi, dst, src][order], graphs * nodes_per_graph


def bessel(r: Tensor, cutoff: float = 5.0, n: int = 8) -> Tensor:
    k = torch.arange(1, n + 1, dtype=r.dtype, device=r.device) * math.pi / cutoff
    return math.sqrt(2.0 / cutoff) * torch.sin(k * r[:, None]) / r[:, None]


def euler_from_quaternion(q: Tensor):
    """ZYZ angles (a, b, c) with R(q) = Rz(a) Ry(b) Rz(c)."""
    w, x, y, z = q.unbind(-1)
    r22 = 1 - 2 * (x * x + y * y)
    b = torch.acos(r22.clamp(-1, 1))
    a = torch.atan2(2 * (y * z - x * w), 2 * (x * z + y * w))
    c = torch.atan2(2 * (y * z + x * w), -2 * (x * z - y * w))
    return a, b, c


def cfg1(dev) -> Workload:
    from .. import nn as enn
    n, c, ir = 1024, 16, "0e+1o+2e"
    g = torch.Generator().manual_seed(0)
    x, v = torch.randn(n, 9, c, generator=g), torch.randn(n, 3, generator=g)
    w = torch.randn(11, c, generator=g) / 4
    cot = torch.randn(n, 9, c, generator=g).to(dev)
    layer = enn.SO3Linear(ir, ir, ir, c, c, internal_weights=False, feature_mode="uu").to(dev)
    sh = enn.SphericalHarmonics(2)
    xd, vd = x.to(dev).requires_grad_(True), v.to(dev).requires_grad_(True)
    wd = w.to(dev).requires_grad_(True)

    def step():
        out = layer(xd, sh(vd), wd)
        gx, gv, gw = torch.autograd.grad(out, [xd, vd, wd], cot)
        return torch.dot(out.reshape(-1), cot.reshape(-1)).reshape(1), [gw, gx, gv]

    return Workload("cfg1: SO3Linear 'uu', 1024 samples, l_max 2, 16 channels, shared weights, harmonics of random vectors",
                    "samples", n, "f32", 2916.0, [_pin(x), _pin(v)], [xd, vd], step,
                    "2916 B/sample: x, v, out forward; g, x, v, gx, gv backward")


def cfg3(dev) -> Workload:
    from .. import nn as enn
    from ..ops.graph_ops import segment_sum
    src, dst, vec, nodes = molecular_graph()
    edges = src.numel()
    ir, ir_y, c = "4x0e+2x1o+2e", "0e+1o+2e", 32
    g = torch.Generator().manual_seed(1)
    x = torch.randn(nodes, 15, c, generator=g).bfloat16()
    w1 = (torch.randn(8, 64, generator=g) / 8 ** 0.5).to(dev).requires_grad_(True)
    w2 = (torch.randn(64, 54 * c, generator=g) / 8).to(dev).requires_grad_(True)
    cot = torch.randn(nodes, 15, c, generator=g).to(dev)
    layer = enn.SO3Linear(ir, ir_y, ir, c, c, internal_weights=False, feature_mode="uu").to(dev)
    sh = enn.SphericalHarmonics(2)
    srcd, dstd = src.to(dev), dst.to(dev)
    ptr = torch.zeros(nodes + 1, dtype=torch.long, device=dev)
    ptr[1:] = torch.cumsum(torch.bincount(dstd, minlength=nodes), 0)
    xd, vd = x.to(dev).requires_grad_(True), vec.to(dev)

    def step():
        wts = (torch.nn.functional.silu(bessel(vd.norm(dim=-1)) @ w1) @ w2).bfloat16().view(edges, 54, c)
        msg = layer(xd[srcd], sh(vd).bfloat16(), wts)
        out = segment_sum(msg.float(), ptr)
        gx, g1, g2 = torch.autograd.grad(out, [xd, w1, w2], cot)
        return torch.dot(out.reshape(-1), cot.reshape(-1)).reshape(1), [g1, g2, gx]

    return Workload(f"cfg3: 32 graphs x 30 nodes, radius 5 A ({edges} edges), Bessel(8) -> MLP(64) -> per-edge 'uu' weights, "
                    "irreps 4x0e+2x1o+2e x 32 channels, l_max 2, bfloat16 operands / float32 sums",
                    "edges", edges, "bf16", 12300.0, [_pin(x), _pin(vec)], [xd, vd], step,
                    "12.3 KB/edge: x row 960 B + per-edge weights 3456 B + vector forward; g row, x, weights read and "
                    "weight gradient 3456 B written backward")


def cfg4(dev, edges: int = 100_000) -> Workload:
    from .. import nn as enn
    from ..irreps import Irreps
    c, ir = 32, Irreps((0, 6))
    g = torch.Generator().manual_seed(3)
    x = torch.randn(edges, 49, c, generator=g)
    q = torch.nn.functional.normalize(torch.randn(edges, 4, generator=g), dim=-1)
    ang = torch.stack(euler_from_quaternion(q.double()), dim=-1).float()            # (E, 3)
    layer = enn.SO2Linear(ir, ir, c, c, internal_weights=False, feature_mode="uv").to(dev)
    w = (torch.randn(*layer.weight_shape, generator=g) / c ** 0.5).to(dev).requires_grad_(True)
    cot = torch.randn(edges, 49, c, generator=g).to(dev)
    wig, dense = enn.WignerD(ir).to(dev), enn.DenseWignerRotation(ir)
    xd, ad = x.to(dev).requires_grad_(True), ang.to(dev).requires_grad_(True)

    def step():
        d = wig(ad[:, 0], ad[:, 1], ad[:, 2])
        out = dense(layer(dense(xd, d), w), d.transpose(-1, -2))
        gx, ga, gw = torch.autograd.grad(out, [xd, ad, w], cot)
        return torch.dot(out.reshape(-1), cot.reshape(-1)).reshape(1), [gw, gx, ga]

    return Workload(f"cfg4: {edges} edges, 32 channels for l = 0..6 (49 components), Haar rotations as ZYZ angles, "
                    "D x -> SO2Linear 'uv' 32 -> 32 -> D^T", "edges", edges, "f32", 31400.0,
                    [_pin(x), _pin(ang)], [xd, ad], step,
                    "31.4 KB/edge fused: x 6272 + angles 12 + out 6272 forward; g, x, gx 6272 each + 12 backward")


def featurize(dev, nodes: int = 100_000, box: float = 27.56, cutoff: float = 1.0) -> Workload:
    """Edge featurisation of the scaling graph's point cloud: 100k points uniform in a cube of side 27.56, cutoff 1.0
    (about 2M directed edges): radius graph + edge vectors + harmonics l_max 3 + 8 Bessel functions + polynomial
    cutoff in two kernel passes (no gradient)."""
    from .. import nn as enn
    from ..transforms import EdgeFeaturizer
    g = torch.Generator().manual_seed(0)
    pos = torch.rand(nodes, 3, generator=g) * box
    feat = EdgeFeaturizer(cutoff, 3, enn.BesselBasis(cutoff, 8).to(dev), enn.PolynomialCutoff(cutoff), max_num_neighbors=64)
    pd = pos.to(dev)
    edges = int(feat.features(pd).src.numel())

    def step():
        f = feat.features(pd)
        return f.cutoff.sum().reshape(1), [f.ptr[-1:].float()]

    return Workload(f"featurize: {nodes} points uniform in a cube of side {box}, cutoff {cutoff} ({edges} directed edges), harmonics "
                    "l_max 3, 8 Bessel functions, polynomial cutoff", "edges", edges, "f32", 132.0, [_pin(pos)], [pd], step,
                    "132 B written per edge: source and target 16, vector 12, length 4, harmonics 64, Bessel 32, cutoff 4")


BUILDERS = {"cfg1": cfg1, "cfg3": cfg3, "cfg4": cfg4, "featurize": featurize}
