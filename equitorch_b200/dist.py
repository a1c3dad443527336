"""Sharding a graph layer over the GPUs of one box (one process per GPU, ``torch.distributed``).

Edges are partitioned by destination-node range: rank ``r`` owns a contiguous range of nodes
(chosen so that every rank gets the same number of edges), all edges pointing into that range,
and the output rows of those nodes - so the sum over incoming edges never crosses ranks.  What
does cross ranks is the *input* of edges whose source lives elsewhere ("halo" nodes):

* forward: every rank receives the feature rows of its halo nodes from their owners (one
  variable-size all-to-all; NCCL over NVLink on GPUs, gloo on CPU) into a buffer appended to its
  owned rows; edge sources are renumbered into that local buffer, so kernels only read local memory;
* backward: gradients of halo rows are sent back to their owners and added there; gradients of
  weights shared by all ranks are all-reduced.

Two forms.  ``halo_exchange`` + ``replicated`` are differentiable building blocks around any per-rank layer.
``sharded_layer`` runs the exchange and a layer given as separate passes (``forward``, ``grad_x``, ``grad_weight``,
``grad_y``) as one operation on a preallocated ``[owned | halo]`` buffer: halo rows are received in place (no
concatenation), the backward computes the gradient of the local rows first, sends the halo part back and all-reduces
the weight gradient asynchronously while the remaining gradients are computed, and adds the returned rows with one
``index_add_``.

The reference has no multi-GPU mode; this module is the sharding the benchmark's scaling
configuration asks for.  All planning happens once on the host from the global edge list.
"""
from __future__ import annotations

from typing import List, NamedTuple, Optional

import torch
import torch.distributed as dist
from torch import Tensor


def partition_nodes_by_edges(dst_sorted: Tensor, num_nodes: int, world_size: int) -> List[int]:
    """Node boundaries ``b[0]=0 <= ... <= b[world]=num_nodes`` balancing the edges per range."""
    counts = torch.bincount(dst_sorted, minlength=num_nodes)
    cum = torch.cumsum(counts, 0)
    total = int(cum[-1]) if num_nodes else 0
    bounds = [0]
    for r in range(1, world_size):
        target = total * r // world_size
        b = int(torch.searchsorted(cum, torch.tensor(target), right=False)) + 1 if total else 0
        bounds.append(min(max(b, bounds[-1]), num_nodes))
    bounds.append(num_nodes)
    return bounds


class ShardPlan(NamedTuple):
    """Everything rank ``rank`` needs, with node ids local to the rank."""
    rank: int
    world_size: int
    node_lo: int                 # first owned global node id
    node_hi: int                 # one past the last owned global node id
    edge_lo: int                 # slice of the global (destination sorted) edge list owned by the rank
    edge_hi: int
    src_local: Tensor            # (E_r,) source ids into [owned rows | halo rows]
    dst_local: Tensor            # (E_r,) destination ids into the owned rows, ascending
    halo_global: Tensor          # (H_r,) global ids of the halo rows, grouped by owner, ascending within owner
    recv_counts: List[int]       # halo rows received from each rank
    send_index: Tensor           # local owned-row ids this rank sends, grouped by destination rank
    send_counts: List[int]

    @property
    def num_owned(self) -> int:
        return self.node_hi - self.node_lo

    @property
    def num_local(self) -> int:
        return self.num_owned + self.halo_global.numel()


def plan_shards(src: Tensor, dst_sorted: Tensor, num_nodes: int, world_size: int) -> List[ShardPlan]:
    """Plans for all ranks (cheap; every rank can call this on the same global edge list)."""
    bounds = partition_nodes_by_edges(dst_sorted, num_nodes, world_size)
    bt = torch.tensor(bounds)
    edge_bounds = torch.searchsorted(dst_sorted, bt).tolist()
    halos, halo_owner_counts = [], []
    for r in range(world_size):
        lo, hi = bounds[r], bounds[r + 1]
        s = src[edge_bounds[r]:edge_bounds[r + 1]]
        remote = torch.unique(s[(s < lo) | (s >= hi)])           # ascending => grouped by owner
        owner = torch.bucketize(remote, bt[1:-1], right=True) if world_size > 1 else torch.zeros_like(remote)
        halos.append(remote)
        halo_owner_counts.append(torch.bincount(owner, minlength=world_size).tolist())
    plans = []
    for r in range(world_size):
        lo, hi = bounds[r], bounds[r + 1]
        e0, e1 = edge_bounds[r], edge_bounds[r + 1]
        s, d = src[e0:e1], dst_sorted[e0:e1]
        remote = halos[r]
        owned = (s >= lo) & (s < hi)
        src_local = torch.where(owned, s - lo, (hi - lo) + torch.searchsorted(remote, s).clamp_max(max(remote.numel() - 1, 0)))
        send_lists, send_counts = [], []
        for q in range(world_size):
            hq = halos[q]
            mine = hq[(hq >= lo) & (hq < hi)] - lo
            send_lists.append(mine)
            send_counts.append(int(mine.numel()))
        plans.append(ShardPlan(r, world_size, lo, hi, e0, e1, src_local, d - lo, remote, halo_owner_counts[r],
                               torch.cat(send_lists) if send_lists else torch.zeros(0, dtype=torch.long), send_counts))
    return plans


def _all_to_all(send: Tensor, send_counts: List[int], recv_counts: List[int], group=None) -> Tensor:
    recv = send.new_empty((sum(recv_counts), *send.shape[1:]))
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_to_all_single(recv, send.contiguous(), recv_counts, send_counts, group=group)
    else:
        recv.copy_(send[: recv.shape[0]])
    return recv


class _HaloExchange(torch.autograd.Function):
    """owned rows (num_owned, ...) -> local rows [owned | halo]; the backward returns halo gradients to
    their owners and adds them to the owned rows' gradients."""

    @staticmethod
    def forward(ctx, owned: Tensor, plan: ShardPlan, send_index: Tensor, group):
        ctx.plan, ctx.group = plan, group
        ctx.save_for_backward(send_index)
        halo = _all_to_all(owned.index_select(0, send_index), plan.send_counts, plan.recv_counts, group)
        return torch.cat([owned, halo], dim=0)

    @staticmethod
    def backward(ctx, grad_local: Tensor):
        plan = ctx.plan
        (send_index,) = ctx.saved_tensors
        grad_owned = grad_local[: plan.num_owned].clone()
        back = _all_to_all(grad_local[plan.num_owned:].contiguous(), plan.recv_counts, plan.send_counts, ctx.group)
        grad_owned.index_add_(0, send_index, back)
        return grad_owned, None, None, None


def halo_exchange(owned: Tensor, plan: ShardPlan, send_index: Optional[Tensor] = None, group=None) -> Tensor:
    """Differentiable: append the halo rows fetched from their owners to this rank's owned rows."""
    if send_index is None:
        send_index = plan.send_index.to(owned.device)
    return _HaloExchange.apply(owned, plan, send_index, group)


class _AllReduceGrad(torch.autograd.Function):
    """Identity in the forward pass; sums the gradient over all ranks in the backward pass (for
    parameters replicated on every rank)."""

    @staticmethod
    def forward(ctx, w: Tensor, group):
        ctx.group = group
        return w.view_as(w)

    @staticmethod
    def backward(ctx, grad: Tensor):
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(ctx.group) > 1:
            grad = grad.contiguous()
            dist.all_reduce(grad, group=ctx.group)
        return grad, None


def replicated(weight: Tensor, group=None) -> Tensor:
    return _AllReduceGrad.apply(weight, group)


def _distributed(group=None) -> bool:
    return dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1


class _ShardedLayer(torch.autograd.Function):
    """``local_x`` is the rank's ``(num_local, ...)`` buffer whose first ``num_owned`` rows are the owned rows; the
    halo rows behind them are overwritten by the forward pass.  The returned gradient has the buffer's shape: owned
    rows carry the full gradient (own edges + what other ranks returned), halo rows are zero."""

    @staticmethod
    def forward(ctx, local_x: Tensor, y: Tensor, weight: Tensor, ops, plan: ShardPlan, send_index: Tensor, group):
        n_owned = plan.num_owned
        if local_x.shape[0] != plan.num_local:
            raise ValueError(f"local buffer has {local_x.shape[0]} rows, the plan needs {plan.num_local}")
        buf = local_x.detach()
        if _distributed(group):
            dist.all_to_all_single(buf[n_owned:], buf[:n_owned].index_select(0, send_index), plan.recv_counts,
                                   plan.send_counts, group=group)
        elif buf.shape[0] > n_owned:
            raise RuntimeError("the plan has halo rows, but no process group with more than one rank is initialised")
        out, state = ops.forward(buf, y, weight)
        ctx.ops, ctx.plan, ctx.group, ctx.state = ops, plan, group, state
        ctx.save_for_backward(send_index)
        return out

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, grad: Tensor):
        ops, plan, group, state = ctx.ops, ctx.plan, ctx.group, ctx.state
        (send_index,) = ctx.saved_tensors
        n_owned = plan.num_owned
        grad = grad.contiguous()
        multi = _distributed(group)
        gx = gy = gw = back = work_x = work_w = None
        if ctx.needs_input_grad[0]:
            gx = ops.grad_x(state, grad)                       # (num_local, ...): own edges' contribution to every local row
            if multi:
                back = gx.new_empty((send_index.shape[0], *gx.shape[1:]))
                work_x = dist.all_to_all_single(back, gx[n_owned:], plan.send_counts, plan.recv_counts, group=group,
                                                async_op=True)
        if ctx.needs_input_grad[2]:
            gw = ops.grad_weight(state, grad).contiguous()
            if multi:
                work_w = dist.all_reduce(gw, group=group, async_op=True)
        if ctx.needs_input_grad[1]:
            gy = ops.grad_y(state, grad)
        if gx is not None:
            if work_x is not None:
                work_x.wait()
                gx[:n_owned].index_add_(0, send_index, back)
            gx[n_owned:].zero_()
        if work_w is not None:
            work_w.wait()
        return gx, gy, gw, None, None, None, None


def sharded_layer(local_x: Tensor, y: Tensor, weight: Tensor, ops, plan: ShardPlan, send_index: Optional[Tensor] = None,
                  group=None) -> Tensor:
    """Halo exchange + layer + gradient exchange as one differentiable operation.

    ``ops`` supplies the layer as four passes over the local rows: ``forward(local_x, y, weight) -> (out, state)``,
    ``grad_x(state, grad) -> (num_local, ...)``, ``grad_weight(state, grad)`` and ``grad_y(state, grad)``
    (``equitorch_b200.nn.functional.graph_tp.FusedGraphOps`` on a GPU).  ``local_x`` is modified in place (its halo
    rows); the weight gradient comes back summed over ranks."""
    if send_index is None:
        send_index = plan.send_index.to(local_x.device)
    return _ShardedLayer.apply(local_x, y, weight, ops, plan, send_index, group)
