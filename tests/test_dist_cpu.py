"""Sharding by destination range and the halo exchange, on CPU with the gloo backend (world size 2 and 3).

Each rank runs the CPU oracle on its shard (owned rows + halo rows fetched from the other rank); the
concatenated outputs and the summed gradients must equal the single-process result."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from equitorch_b200.dist import halo_exchange, partition_nodes_by_edges, plan_shards, replicated, sharded_layer
from equitorch_b200.utils.synthetic import radius_graph, random_graph
from oracle import tensor_products as otp

IR = "0e+1o+2e"


def _inputs():
    g, _ = radius_graph(num_nodes=300, target_edges=3000, seed=3, tolerance=0.2)
    gen = torch.Generator().manual_seed(0)
    x = torch.randn(g.num_nodes, 9, 4, generator=gen, dtype=torch.float64)
    w = torch.randn(11, 4, 5, generator=gen, dtype=torch.float64)
    cot = torch.randn(g.num_nodes, 9, 5, generator=gen, dtype=torch.float64)
    return g, x, w, cot


def _single():
    g, x, w, cot = _inputs()
    x, w = x.requires_grad_(True), w.requires_grad_(True)
    v = g.edge_vec.double().requires_grad_(True)
    out = otp.so3_linear_message_passing(x, v, g.src, g.dst, w, IR, IR, IR, feature_mode="uv")
    gx, gv, gw = torch.autograd.grad(out, [x, v, w], cot)
    return out.detach(), gx, gv, gw


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g, x, w, cot = _inputs()
        plan = plan_shards(g.src, g.dst, g.num_nodes, world)[rank]
        owned = x[plan.node_lo:plan.node_hi].clone().requires_grad_(True)
        wr = w.clone().requires_grad_(True)
        v = g.edge_vec[plan.edge_lo:plan.edge_hi].double().requires_grad_(True)
        local = halo_exchange(owned, plan)
        assert local.shape[0] == plan.num_local
        torch.testing.assert_close(local[plan.num_owned:], x[plan.halo_global])
        out = otp.so3_linear_message_passing(local, v, plan.src_local, plan.dst_local, replicated(wr), IR, IR, IR,
                                             feature_mode="uv", num_out_nodes=plan.num_owned)
        gx, gv, gw = torch.autograd.grad(out, [owned, v, wr], cot[plan.node_lo:plan.node_hi])
        ret[rank] = (plan.node_lo, plan.node_hi, plan.edge_lo, plan.edge_hi, out.detach(), gx, gv, gw)
    finally:
        dist.destroy_process_group()


class _OracleOps:
    """The layer as separate passes, computed by the CPU oracle (stands in for the CUDA passes of FusedGraphOps)."""

    def __init__(self, plan):
        self.plan = plan

    def forward(self, local_x, y, weight):
        with torch.enable_grad():
            leaves = [t.detach().clone().requires_grad_(True) for t in (local_x, y, weight)]
            out = otp.so3_linear_message_passing(leaves[0], leaves[1], self.plan.src_local, self.plan.dst_local, leaves[2],
                                                 IR, IR, IR, feature_mode="uv", num_out_nodes=self.plan.num_owned)
        return out.detach(), (leaves, out)

    def _grad(self, state, grad, which):
        leaves, out = state
        return torch.autograd.grad(out, leaves[which], grad, retain_graph=True)[0]

    def grad_x(self, state, grad):
        return self._grad(state, grad, 0)

    def grad_y(self, state, grad):
        return self._grad(state, grad, 1)

    def grad_weight(self, state, grad):
        return self._grad(state, grad, 2)


def _worker_fused(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g, x, w, cot = _inputs()
        plan = plan_shards(g.src, g.dst, g.num_nodes, world)[rank]
        local = torch.full((plan.num_local, *x.shape[1:]), float("nan"), dtype=x.dtype)     # halo rows start as garbage
        local[:plan.num_owned] = x[plan.node_lo:plan.node_hi]
        local.requires_grad_(True)
        wr = w.clone().requires_grad_(True)
        v = g.edge_vec[plan.edge_lo:plan.edge_hi].double().requires_grad_(True)
        out = sharded_layer(local, v, wr, _OracleOps(plan), plan)
        torch.testing.assert_close(local.detach()[plan.num_owned:], x[plan.halo_global])
        gx, gv, gw = torch.autograd.grad(out, [local, v, wr], cot[plan.node_lo:plan.node_hi])
        assert bool((gx[plan.num_owned:] == 0).all())
        ret[rank] = (plan.node_lo, plan.node_hi, plan.edge_lo, plan.edge_hi, out.detach(), gx[:plan.num_owned], gv, gw)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_layer_in_place_exchange_equals_single_process(world):
    """`sharded_layer`: halo rows received into the preallocated buffer, halo gradients returned and the weight
    gradient all-reduced asynchronously inside one backward pass."""
    ref_out, ref_gx, ref_gv, ref_gw = _single()
    ret = mp.Manager().dict()
    mp.spawn(_worker_fused, args=(world, _free_port(), ret), nprocs=world, join=True)
    assert sorted(ret.keys()) == list(range(world))
    for rank in range(world):
        lo, hi, e0, e1, out, gx, gv, gw = ret[rank]
        torch.testing.assert_close(out, ref_out[lo:hi], rtol=1e-12, atol=1e-12)
        torch.testing.assert_close(gx, ref_gx[lo:hi], rtol=1e-12, atol=1e-12)
        torch.testing.assert_close(gv, ref_gv[e0:e1], rtol=1e-12, atol=1e-12)
        torch.testing.assert_close(gw, ref_gw, rtol=1e-12, atol=1e-12)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_layer_equals_single_process(world):
    ref_out, ref_gx, ref_gv, ref_gw = _single()
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    assert sorted(ret.keys()) == list(range(world))
    for rank in range(world):
        lo, hi, e0, e1, out, gx, gv, gw = ret[rank]
        torch.testing.assert_close(out, ref_out[lo:hi], rtol=1e-12, atol=1e-12)
        torch.testing.assert_close(gx, ref_gx[lo:hi], rtol=1e-12, atol=1e-12)
        torch.testing.assert_close(gv, ref_gv[e0:e1], rtol=1e-12, atol=1e-12)
        torch.testing.assert_close(gw, ref_gw, rtol=1e-12, atol=1e-12)   # all-reduced: identical on every rank


def test_partition_balances_edges_and_covers_everything():
    g = random_graph(1000, 20000, seed=1)
    for world in (1, 2, 4, 8):
        b = partition_nodes_by_edges(g.dst, g.num_nodes, world)
        assert b[0] == 0 and b[-1] == g.num_nodes and all(x <= y for x, y in zip(b, b[1:]))
        plans = plan_shards(g.src, g.dst, g.num_nodes, world)
        sizes = [p.edge_hi - p.edge_lo for p in plans]
        assert sum(sizes) == 20000 and max(sizes) - min(sizes) <= 0.05 * 20000 / world + 40
        for p in plans:
            assert p.recv_counts[p.rank] == 0 and p.send_counts[p.rank] == 0
            assert int(p.dst_local.max()) < p.num_owned and int(p.src_local.max()) < p.num_local
            assert sum(p.recv_counts) == p.halo_global.numel()
        for r in range(world):   # what r sends to q is what q expects from r
            assert [plans[r].send_counts[q] for q in range(world)] == [plans[q].recv_counts[r] for q in range(world)]


def test_morton_order_keeps_halo_small():
    g, _ = radius_graph(num_nodes=20000, target_edges=400000, seed=0)
    plans = plan_shards(g.src, g.dst, g.num_nodes, 8)
    worst = max(p.halo_global.numel() / p.num_owned for p in plans)
    assert worst < 1.0, f"halo is {worst:.2f}x the owned rows"
