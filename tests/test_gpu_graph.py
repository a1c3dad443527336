"""Fused graph layer (gather -> CG -> segment sum -> channel mix) against the CPU oracle."""
import pytest
import torch

from equitorch_b200 import nn as enn
from equitorch_b200.graph import EdgeGraph
from equitorch_b200.ops.fused_tp_op import check_status
from oracle import tensor_products as otp
from oracle.sphericals import spherical_harmonics as osh

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _case(seed, nodes, edges, sort_dst=True, isolated=0):
    g = torch.Generator().manual_seed(seed)
    src = torch.randint(0, nodes, (edges,), generator=g)
    dst = torch.randint(0, max(1, nodes - isolated), (edges,), generator=g)
    if sort_dst:
        dst = torch.sort(dst).values
    vec = torch.randn(edges, 3, generator=g)
    return g, src, dst, vec


@pytest.mark.parametrize("irreps,lmax,c,mode", [
    ("0e+1o+2e+3o", 3, 64, "uv"), ("0e+1o+2e+3o", 3, 64, "uu"), ("0e+1o+2e+3o", 3, 32, "uv"),
    ("0e+1o+2e", 2, 64, "uv"), ("0e+1o", 1, 32, "uu"),
    ("0e+1o+2e+3o", 3, 16, "uv"),          # channel count without unrolled kernel -> table-driven path
    ("0e+1e+1o+2e", 2, 64, "uv"),          # structure not in the registry -> table-driven path
])
@pytest.mark.parametrize("sort_dst", [True, False])
def test_fused_graph_layer_matches_oracle(irreps, lmax, c, mode, sort_dst):
    nodes, edges = 97, 1531
    g, src, dst, vec = _case(hash((irreps, c, mode)) % 1000, nodes, edges, sort_dst, isolated=5)
    ir_y = {1: "0e+1o", 2: "0e+1o+2e", 3: "0e+1o+2e+3o"}[lmax]
    dim = sum(2 * int(t[0]) + 1 for t in irreps.split("+"))
    x = torch.randn(nodes, dim, c, generator=g)
    layer = enn.SO3LinearGraph(irreps, ir_y, irreps, c, c, internal_weights=False, feature_mode=mode).to(DEV)
    w = torch.randn(*layer.weight_shape, generator=g) / (c ** 0.5 if mode == "uv" else 1.0)
    cot = torch.randn(nodes, dim, c, generator=g)

    xo, vo, wo = (t.double().requires_grad_(True) for t in (x, vec, w))
    ref = otp.so3_linear_message_passing(xo, vo, src, dst, wo, irreps, ir_y, irreps, feature_mode=mode)
    gref = torch.autograd.grad(ref, [xo, vo, wo], cot.double())

    graph = EdgeGraph(src.to(DEV), dst.to(DEV), nodes)
    xg, vg, wg = (t.to(DEV).requires_grad_(True) for t in (x, vec, w))
    out = layer(xg, enn.SphericalHarmonics(lmax)(vg), graph, wg)
    grads = torch.autograd.grad(out, [xg, vg, wg], cot.to(DEV))
    check_status()
    assert out.shape == ref.shape
    for name, a, b in [("out", out, ref)] + [(f"grad{n}", a, b) for n, (a, b) in enumerate(zip(grads, gref))]:
        err = float((a.detach().double().cpu() - b.detach()).abs().max() / b.detach().abs().max())
        assert err < 1e-5, f"{name}: relative error {err:.2e}"
    assert torch.count_nonzero(out[nodes - 5:]) == 0     # nodes without incoming edges


def test_fused_graph_layer_equals_per_edge_layer_plus_scatter():
    """Same numbers as the drop-in per-edge SO3Linear followed by an index_add over destinations."""
    nodes, edges, c, ir = 50, 700, 64, "0e+1o+2e+3o"
    g, src, dst, vec = _case(11, nodes, edges)
    x = torch.randn(nodes, 16, c, generator=g).to(DEV)
    fused = enn.SO3LinearGraph(ir, ir, ir, c, c, feature_mode="uv").to(DEV)
    plain = enn.SO3Linear(ir, ir, ir, c, c, feature_mode="uv").to(DEV)
    plain.load_state_dict(fused.state_dict())
    y = enn.SphericalHarmonics(3)(vec.to(DEV))
    out = fused(x, y, EdgeGraph(src.to(DEV), dst.to(DEV), nodes))
    msg = plain(x[src.to(DEV)], y)
    want = torch.zeros_like(out).index_add_(0, dst.to(DEV), msg)
    check_status()
    err = float((out - want).abs().max() / want.abs().max())
    assert err < 1e-5, f"relative error {err:.2e}"


def test_forward_sharded_on_one_rank_equals_forward():
    """`forward_sharded` with a one-rank plan (no halo rows, no process group): same output and the same three
    gradients as `forward`, although its backward pass runs the passes in another order (local-row gradient first)."""
    from equitorch_b200.dist import plan_shards
    nodes, edges, c, ir = 60, 900, 64, "0e+1o+2e+3o"
    g, src, dst, vec = _case(12, nodes, edges)
    order = torch.argsort(dst, stable=True)
    src, dst, vec = src[order], dst[order], vec[order]
    plan = plan_shards(src, dst, nodes, 1)[0]
    assert plan.num_local == nodes and plan.send_index.numel() == 0
    layer = enn.SO3LinearGraph(ir, ir, ir, c, c, feature_mode="uv").to(DEV)
    graph = EdgeGraph(plan.src_local.to(DEV), plan.dst_local.to(DEV), plan.num_local, plan.num_owned)
    cot = torch.randn(nodes, 16, c, generator=g).to(DEV)
    results = []
    for sharded in (False, True):
        x = torch.randn(nodes, 16, c, generator=torch.Generator().manual_seed(5)).to(DEV).requires_grad_(True)
        v = vec.to(DEV).requires_grad_(True)
        y = enn.SphericalHarmonics(3)(v)
        out = layer.forward_sharded(x, y, graph, plan) if sharded else layer(x, y, graph)
        results.append((out, *torch.autograd.grad(out, [x, v, layer.weight], cot)))
    check_status()
    for a, b in zip(*results):
        torch.testing.assert_close(a, b, rtol=0, atol=0)


def test_fused_graph_layer_no_edges_and_rectangular():
    ir, c = "0e+1o+2e", 64
    layer = enn.SO3LinearGraph(ir, ir, ir, c, c, feature_mode="uv").to(DEV)
    x = torch.randn(7, 9, c, device=DEV)
    empty = torch.zeros(0, dtype=torch.long, device=DEV)
    out = layer(x, torch.zeros(0, 9, device=DEV), EdgeGraph(empty, empty, 7))
    assert out.shape == (7, 9, c) and torch.count_nonzero(out) == 0
    # more source rows (owned + halo) than destination rows
    g = torch.Generator().manual_seed(2)
    src = torch.randint(0, 7, (40,), generator=g).to(DEV)
    dst = torch.sort(torch.randint(0, 3, (40,), generator=g)).values.to(DEV)
    y = torch.randn(40, 9, device=DEV)
    out = layer(x, y, EdgeGraph(src, dst, 7, 3))
    assert out.shape == (3, 9, c)
    plain = enn.SO3Linear(ir, ir, ir, c, c, feature_mode="uv").to(DEV)
    plain.load_state_dict(layer.state_dict())
    want = torch.zeros(3, 9, c, device=DEV).index_add_(0, dst, plain(x[src], y))
    check_status()
    assert float((out - want).abs().max() / want.abs().max()) < 1e-5


def test_large_graph_properties():
    """Benchmark-sized graph (200k edges, 10k nodes, l_max 3, C 64): linearity in the node features and
    agreement of the two edge orders - properties that need no oracle run at this size."""
    nodes, edges, c, ir = 10_000, 200_000, 64, "0e+1o+2e+3o"
    g, src, dst, vec = _case(5, nodes, edges)
    layer = enn.SO3LinearGraph(ir, ir, ir, c, c, feature_mode="uv").to(DEV)
    y = enn.SphericalHarmonics(3)(vec.to(DEV))
    graph = EdgeGraph(src.to(DEV), dst.to(DEV), nodes)
    x1 = torch.randn(nodes, 16, c, generator=g).to(DEV)
    x2 = torch.randn(nodes, 16, c, generator=g).to(DEV)
    o1, o2, o12 = layer(x1, y, graph), layer(x2, y, graph), layer(x1 + 2 * x2, y, graph)
    torch.testing.assert_close(o12, o1 + 2 * o2, rtol=1e-4, atol=1e-4)
    perm = torch.randperm(edges, generator=g).to(DEV)
    shuffled = EdgeGraph(src.to(DEV)[perm], dst.to(DEV)[perm], nodes)
    o1s = layer(x1, y[perm], shuffled)
    check_status()
    torch.testing.assert_close(o1s, o1, rtol=1e-4, atol=1e-4)


def test_profiling_size_graph_prefix_against_oracle():
    """The quarter-size benchmark graph (25k nodes, ~500k edges, l_max 3, C 64, uv) through the fused layer, output
    and all three gradients against the float64 oracle on the first ~32k destination-contiguous edges - the slice
    the CPU baseline of the benchmark times.  The cotangent is zero outside the prefix nodes, so every gradient
    depends on the prefix edges only.  Error = max |a - b| / max |b|, bound 1e-5."""
    from equitorch_b200.utils.synthetic import node_features, radius_graph
    ir, c = "0e+1o+2e+3o", 64
    graph, _ = radius_graph(25_000, 500_000, seed=0)
    nodes, edges = graph.num_nodes, graph.src.numel()
    n_pre = 32768
    last = int(graph.dst[n_pre - 1])
    n_pre = int(torch.searchsorted(graph.dst, torch.tensor(last), right=True))
    g = torch.Generator().manual_seed(4)
    x = node_features(nodes, 16, c, seed=1)
    w = (torch.rand(23, c, c, generator=g) * 2 - 1) * (3.0 / c) ** 0.5
    cot = torch.randn(nodes, 16, c, generator=g)
    cot[last + 1:] = 0

    layer = enn.SO3LinearGraph(ir, ir, ir, c, c, internal_weights=False, feature_mode="uv").to(DEV)
    eg = EdgeGraph(graph.src.to(DEV), graph.dst.to(DEV), nodes)
    xg, vg, wg = (t.to(DEV).requires_grad_(True) for t in (x, graph.edge_vec, w))
    out = layer(xg, enn.SphericalHarmonics(3)(vg), eg, wg)
    gx, gv, gw = torch.autograd.grad(out, [xg, vg, wg], cot.to(DEV))
    check_status()

    xo, wo = x.double().requires_grad_(True), w.double().requires_grad_(True)
    vo = graph.edge_vec[:n_pre].double().requires_grad_(True)
    ref = otp.so3_linear_message_passing(xo, vo, graph.src[:n_pre], graph.dst[:n_pre], wo, ir, ir, ir, feature_mode="uv",
                                         num_out_nodes=last + 1)
    rx, rv, rw = torch.autograd.grad(ref, [xo, vo, wo], cot[: last + 1].double())
    assert torch.count_nonzero(gv[n_pre:]) == 0          # edges into nodes with a zero cotangent
    pairs = [("out", out[: last + 1], ref), ("grad_x", gx, rx), ("grad_vec", gv[:n_pre], rv), ("grad_w", gw, rw)]
    for name, a, b in pairs:
        err = float((a.detach().double().cpu() - b.detach()).abs().max() / b.detach().abs().max())
        assert err < 1e-5, f"{name}: relative error {err:.2e}"
