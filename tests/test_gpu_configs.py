"""Parity at the shapes of the remaining benchmark configurations (3: molecular-style layer with
per-edge weights in bfloat16; 4: Wigner-rotated SO(2) linear path, l = 0..6), against the CPU oracle."""
import math

import pytest
import torch

from equitorch_b200 import constants
from equitorch_b200 import nn as enn
from equitorch_b200.irreps import Irreps
from equitorch_b200.ops.graph_ops import gather_rows, segment_sum
from equitorch_b200.tables import so2_linear_infos
from oracle import sphericals as osph
from oracle import tensor_products as otp

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _molecular_graph(graphs=32, nodes_per_graph=30, box=6.0, cutoff=5.0, seed=0):
    g = torch.Generator().manual_seed(seed)
    pos = torch.rand(graphs, nodes_per_graph, 3, generator=g) * box
    diff = pos[:, :, None, :] - pos[:, None, :, :]                  # [graph, dst, src]
    dist = diff.norm(dim=-1)
    mask = (dist < cutoff) & ~torch.eye(nodes_per_graph, dtype=torch.bool)
    gi, dst, src = mask.nonzero(as_tuple=True)
    off = gi * nodes_per_graph
    vec = diff[gi, dst, src]
    order = torch.argsort(off + dst, stable=True)
    return (off + src)[order], (off + dst)[order], vec[order], graphs * nodes_per_graph


def _bessel(r, cutoff=5.0, n=8):
    k = torch.arange(1, n + 1, dtype=r.dtype, device=r.device) * math.pi / cutoff
    return math.sqrt(2.0 / cutoff) * torch.sin(k * r[:, None]) / r[:, None]


def test_config3_molecular_layer_bf16_inputs():
    """32 graphs x 30 nodes, radius graph, Bessel -> MLP -> per-edge uu weights, node irreps
    128x0e+64x1o+32x2e (= 4x0e+2x1o+2e with 32 channels), SH l_max 2, bfloat16 inputs, float32 sums."""
    src, dst, vec, nodes = _molecular_graph()
    edges = src.numel()
    assert 15000 < edges < 26000
    ir, ir_y, c = "4x0e+2x1o+2e", "0e+1o+2e", 32
    g = torch.Generator().manual_seed(1)
    x = torch.randn(nodes, 15, c, generator=g)
    w1, w2 = torch.randn(8, 64, generator=g) / 8 ** 0.5, torch.randn(64, 54 * c, generator=g) / 8
    cot = torch.randn(nodes, 15, c, generator=g)

    def weights_of(v):
        return torch.nn.functional.silu(_bessel(v.norm(dim=-1)) @ w1.to(v)) @ w2.to(v)

    # oracle: float64 on the bfloat16-rounded inputs
    xb = x.bfloat16()
    xo = xb.double().requires_grad_(True)
    wo = weights_of(vec.double()).bfloat16().double().view(edges, 54, c).requires_grad_(True)
    yo = osph.spherical_harmonics(torch.nn.functional.normalize(vec.double(), dim=-1), 2).bfloat16().double()
    msg = otp.so3_linear_dense(xo[src], yo, wo, ir, ir_y, ir, feature_mode="uu")
    out_o = torch.zeros(nodes, 15, c, dtype=torch.float64).index_add(0, dst, msg)
    gx_o, gw_o = torch.autograd.grad(out_o, [xo, wo], cot.double())

    layer = enn.SO3Linear(ir, ir_y, ir, c, c, internal_weights=False, feature_mode="uu").to(DEV)
    srcg, dstg = src.to(DEV), dst.to(DEV)
    ptr = torch.zeros(nodes + 1, dtype=torch.long, device=DEV)
    ptr[1:] = torch.cumsum(torch.bincount(dstg, minlength=nodes), 0)
    xg = xb.to(DEV).requires_grad_(True)
    wg = weights_of(vec.to(DEV)).bfloat16().view(edges, 54, c).requires_grad_(True)
    yg = enn.SphericalHarmonics(2)(vec.to(DEV)).bfloat16()
    msg_g = layer(xg[srcg], yg, wg)
    assert msg_g.dtype == torch.bfloat16
    out_g = segment_sum(msg_g.float(), ptr)
    gx_g, gw_g = torch.autograd.grad(out_g, [xg, wg], cot.to(DEV))
    for name, a, b in (("out", out_g, out_o), ("grad_x", gx_g, gx_o), ("grad_w", gw_g, gw_o)):
        err = float((a.detach().double().cpu() - b.detach()).abs().max() / b.detach().abs().max())
        assert err < 2e-2, f"{name}: relative error {err:.2e}"


def _rel(a, b):
    """max |a - b| / max |b| (the error norm of every bound in this file)."""
    return float((a.detach().double().cpu() - b.detach().double().cpu()).abs().max() / b.detach().double().abs().max())


def _config4_inputs(e, c=32, seed=3):
    from equitorch_b200.utils.workloads import euler_from_quaternion
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(e, 49, c, generator=g)
    q = torch.nn.functional.normalize(torch.randn(e, 4, generator=g), dim=-1)
    a, b, cc = euler_from_quaternion(q.double())
    cot = torch.randn(e, 49, c, generator=g)
    return g, x, (a, b, cc), cot


def test_config4_wigner_d_generation():
    """D(alpha, beta, gamma) for l = 0..6 at 20k Haar rotations and the angle gradients of <D, cotangent>, float32
    kernel against the float64 oracle product Z J Z J Z, bound 1e-5; D is orthogonal (size-independent property)."""
    e, ir = 20_000, Irreps((0, 6))
    g, _, (a, b, c), _ = _config4_inputs(e)
    cot = torch.randn(e, 49, 49, generator=g)
    jb = {l: torch.from_numpy(constants.j_matrix(l).copy()) for l in range(7)}
    ao, bo, co = (t.clone().requires_grad_(True) for t in (a, b, c))
    d_o = osph.wigner_d(list(range(7)), ao, bo, co, jb)
    go = torch.autograd.grad(d_o, [ao, bo, co], cot.double())
    wig = enn.WignerD(ir).to(DEV)
    ag, bg, cg = (t.float().to(DEV).requires_grad_(True) for t in (a, b, c))
    d_g = wig(ag, bg, cg)
    gg = torch.autograd.grad(d_g, [ag, bg, cg], cot.to(DEV))
    assert _rel(d_g, d_o) < 1e-5
    scale = max(float(t.abs().max()) for t in go)
    for u, v in zip(gg, go):
        assert float((u.double().cpu() - v).abs().max()) / scale < 1e-5
    eye = torch.eye(49, device=DEV).expand(e, 49, 49)
    assert float((d_g.detach() @ d_g.detach().transpose(-1, -2) - eye).abs().max()) < 1e-5
    # the sparse z-rotation route (packed sin/cos inputs, higher derivatives) gives the same matrices
    from equitorch_b200.nn.functional import wigner_d as fw
    fw.FORCE_SPARSE = True
    try:
        d_s = wig(ag[:512], bg[:512], cg[:512])
    finally:
        fw.FORCE_SPARSE = False
    assert _rel(d_s, d_g[:512]) < 1e-5


@pytest.mark.parametrize("block_diagonal", [False, True])
def test_config4_dense_rotation(block_diagonal):
    """D x, D^T x and their gradients with respect to x and D at 20k samples (49 x 49 matrices, 32 channels), own
    kernels against float64 matmul, bound 1e-5.  Dense matrices with ``block_diagonal=False``; matrices that are block
    diagonal over l = 0..6 with the default, where only the blocks are read and the matrix gradient is the float64
    gradient restricted to the blocks."""
    e, c = 20_000, 32
    g, x, _, cot = _config4_inputs(e, c)
    d = torch.randn(e, 49, 49, generator=g) / 7
    mask = torch.zeros(49, 49)
    for l in range(7):
        mask[l * l:(l + 1) ** 2, l * l:(l + 1) ** 2] = 1
    if block_diagonal:
        d = d * mask
    rot = enn.DenseWignerRotation(Irreps((0, 6)), block_diagonal=block_diagonal)
    for transposed in (False, True):
        xo, do = x.double().requires_grad_(True), d.double().requires_grad_(True)
        ref = (do.transpose(-1, -2) if transposed else do) @ xo
        gro = list(torch.autograd.grad(ref, [xo, do], cot.double()))
        if block_diagonal:
            gro[1] = gro[1] * mask.double()
        xg, dg = x.to(DEV).requires_grad_(True), d.to(DEV).requires_grad_(True)
        out = rot(xg, dg.transpose(-1, -2) if transposed else dg)
        grg = torch.autograd.grad(out, [xg, dg], cot.to(DEV))
        for u, v in [(out, ref), *zip(grg, gro)]:
            assert _rel(u, v) < 1e-5
        if block_diagonal:
            assert bool((grg[1].cpu() * (1 - mask) == 0).all())


def test_config4_so2_linear():
    """SO2Linear 'uv' 32 -> 32 for l = 0..6 on 20k samples against the sparse restatement in float64, bound 1e-5."""
    e, c, ir = 20_000, 32, Irreps((0, 6))
    g, x, _, cot = _config4_inputs(e, c)
    layer = enn.SO2Linear(ir, ir, c, c, internal_weights=False, feature_mode="uv")
    w = torch.randn(*layer.weight_shape, generator=g) / c ** 0.5
    torch.set_default_dtype(torch.float64)
    try:
        info64 = so2_linear_infos(ir, ir)[0]
    finally:
        torch.set_default_dtype(torch.float32)
    xo, wo = x.double().requires_grad_(True), w.double().requires_grad_(True)
    ref = otp.so2_linear_sparse(xo, wo, info64, "uv")
    gro = torch.autograd.grad(ref, [xo, wo], cot.double())
    layer = layer.to(DEV)
    xg, wg = x.to(DEV).requires_grad_(True), w.to(DEV).requires_grad_(True)
    out = layer(xg, wg)
    grg = torch.autograd.grad(out, [xg, wg], cot.to(DEV))
    for u, v in [(out, ref), *zip(grg, gro)]:
        assert _rel(u, v) < 1e-5


def test_config4_wigner_rotated_so2_linear():
    """The whole chain at 20k edges: x (E, 49, 32), Haar quaternions -> ZYZ angles -> D = WignerD(l = 0..6); D x ->
    SO2Linear uv 32 -> 32 -> D^T; forward and backward in float32 against the float64 oracle.  Each stage meets 1e-5
    on its own (tests above); the chain of three float32 stages (two 49-term rotations around a 413-term mixing) is
    held to 2e-5."""
    e, c, ir = 20_000, 32, Irreps((0, 6))
    g, x, (a, b, cc), cot = _config4_inputs(e, c)
    layer = enn.SO2Linear(ir, ir, c, c, internal_weights=False, feature_mode="uv")
    w = torch.randn(*layer.weight_shape, generator=g) / c ** 0.5

    jb = {l: torch.from_numpy(constants.j_matrix(l).copy()) for l in range(7)}
    torch.set_default_dtype(torch.float64)
    try:
        info64 = so2_linear_infos(ir, ir)[0]
    finally:
        torch.set_default_dtype(torch.float32)
    xo, wo = x.double().requires_grad_(True), w.double().requires_grad_(True)
    ao, bo, co = (t.clone().requires_grad_(True) for t in (a, b, cc))
    d_o = osph.wigner_d(list(range(7)), ao, bo, co, jb)
    out_o = d_o.transpose(-1, -2) @ otp.so2_linear_sparse(d_o @ xo, wo, info64, "uv")
    grads_o = torch.autograd.grad(out_o, [xo, wo, ao, bo, co], cot.double())

    layer = layer.to(DEV)
    wig, rot = enn.WignerD(ir).to(DEV), enn.DenseWignerRotation(ir)
    xg, wg = x.to(DEV).requires_grad_(True), w.to(DEV).requires_grad_(True)
    ag, bg, cg = (t.float().to(DEV).requires_grad_(True) for t in (a, b, cc))
    d_g = wig(ag, bg, cg)
    out_g = rot(layer(rot(xg, d_g), wg), d_g.transpose(-1, -2))
    grads_g = torch.autograd.grad(out_g, [xg, wg, ag, bg, cg], cot.to(DEV))
    for name, u, v in [("out", out_g, out_o), ("grad_x", grads_g[0], grads_o[0]), ("grad_w", grads_g[1], grads_o[1])]:
        assert _rel(u, v) < 2e-5, f"{name}: relative error {_rel(u, v):.2e}"
    # the layer commutes with the outermost z-rotation, so d/d(alpha) vanishes identically: compare the three
    # angle gradients on their common scale
    ang_g = torch.stack([t.double().cpu() for t in grads_g[2:]])
    ang_o = torch.stack([t.detach() for t in grads_o[2:]])
    err = float((ang_g - ang_o).abs().max() / ang_o.abs().max())
    assert err < 1e-4, f"angle gradients: relative error {err:.2e}"
