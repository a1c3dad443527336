"""``SO3Linear`` evaluated on the edges of a graph and summed into destination nodes, fused.

    out[d] = sum_{e: dst(e) = d}  SO3Linear(node_x[src(e)], y[e]; W)

The reference offers the per-edge layer only; users gather ``node_x[edge_index[0]]`` before it and
scatter-add after it (``equitorch/nn/linears.py:145-187`` surrounded by the
``edge_index`` convention of ``equitorch/transforms/__init__.py:99-101``).  Here the three steps
are one operation, and because the weights are shared by all edges the sum over edges is moved
*in front of* the channel mixing: the CG contraction is accumulated per destination node
(``S[d, r, :]``, one row per (output component, path)) and the ``C_in x C_out`` matrices are
applied once per node instead of once per edge - the result is the same sum, evaluated in a
different order.  The same holds for every gradient:

    grad_W        = sum_d  S[d]^T g[d]                       (node level)
    G[d]          = g[d] W^T                                 (node level, gradient w.r.t. S)
    grad_y[e]     = <CG, node_x[src(e)], G[dst(e)]>          (edge pass, grouped by destination)
    grad_node_x[s]= (sum_{e: src(e)=s} CG' (g[dst(e)], y[e])) W^T   (edge pass grouped by source, then node level)

No per-edge tensor with a channel axis is ever written to memory.
"""
from __future__ import annotations

import os
from typing import Optional

import torch
from torch import Tensor
from torch.autograd import Function

from ... import _profile
from ...graph import EdgeGraph
from ...ops import batched_sparse_dense_op as _ops
from ...ops.fused_tp_op import TpTable, cg_inner, cg_segment_sum, check_status
from ...ops.mix_tc_op import (MixPlan, mix_tc, mix_tc_transposed, wgrad_tc, supported as _tc_supported,
                              supported_transposed as _tc_supported_t, supported_wgrad as _tc_supported_w)
from ...structs import TensorProductInfo


# The fused kernels bound every wait on an asynchronous copy; a wait that runs out raises a per-device status
# word and the kernel returns with partial output.  `fused_tp_op.check_status()` turns the word into an
# exception (it synchronises, so it is not called on the hot path); EQT_CHECK_STATUS=1 makes every forward and
# backward of the fused layer call it.
_CHECK_EVERY_CALL = os.environ.get("EQT_CHECK_STATUS", "0") not in ("", "0")


class GraphTPPlan:
    """Device tables of one layer for the fused graph kernels (built once per layer and device)."""

    def __init__(self, tp_info_forward: TensorProductInfo, tp_info_backward1: TensorProductInfo,
                 d_in1: int, d_in2: int, d_out: int, device, out_dims=None, in1_dims=None):
        f, b1 = tp_info_forward, tp_info_backward1
        self.fwd_table = TpTable(f.info_Mij_fwd, True, d_in1, d_in2, device)
        # backward-1 tables: input1 is the channel-less operand, input2 the incoming gradient
        self.bwd1_table = TpTable(b1.info_Mij_fwd, False, d_out, d_in2, device)
        self.mix_fwd, self.mix_bwd1, self.mix_bwd2 = (t.to(device) for t in (f.info_M_fwd, f.info_M_bwd1, f.info_M_bwd2))
        self.mix_src = b1.info_M_fwd.to(device)
        self.d_in1, self.d_in2, self.d_out = d_in1, d_in2, d_out
        self.device = torch.device(device)
        # block structure of the two weight steps for the tensor-core GEMM (None: CUDA-core kernel)
        self.tc_fwd = MixPlan(f.info_M_fwd, out_dims, device) if out_dims is not None else None
        self.tc_src = MixPlan(b1.info_M_fwd, in1_dims, device) if in1_dims is not None else None


def _mix(s: Tensor, w: Tensor, info, mode: str, tc: "MixPlan | None" = None) -> Tensor:
    if (mode == "uv" and tc is not None and tc.regular and s.dtype == torch.float32
            and _tc_supported(w.shape[-2], w.shape[-1])):
        return mix_tc(s, w, tc)
    op = _ops.indexed_vecmat_scale_gather if mode == "uv" else _ops.indexed_mul_scale_gather
    return op(s, w, info.scale, info.index1, info.index2, info.seg_out, out_size=info.out_size)


class FusedGraphOps:
    """The passes of the fused layer as separate calls, so that a caller can order them (the sharded layer sends halo
    gradients back while the other gradients are computed).  ``state`` is what ``forward`` returns second."""

    def __init__(self, graph: EdgeGraph, plan: GraphTPPlan, mode: str):
        self.graph, self.plan, self.mode = graph, plan, mode

    def forward(self, node_x: Tensor, y: Tensor, weight: Tensor):
        graph, plan = self.graph, self.plan
        with _profile.timed("cg_segment_sum[fwd]"):
            s = cg_segment_sum(plan.fwd_table, node_x, y, graph.src_by_dst, graph.dst_order, graph.dst_ptr,
                               graph.num_dst)
        with _profile.timed("channel_mix[fwd]"):
            out = _mix(s, weight, plan.mix_fwd, self.mode, plan.tc_fwd)
        return out, (node_x, y, weight, s if weight.requires_grad else None)

    def _wt(self, weight: Tensor) -> Tensor:
        return weight.transpose(-1, -2).contiguous() if self.mode == "uv" else weight

    def grad_weight(self, state, grad: Tensor) -> Tensor:
        _, _, weight, s = state
        plan, mode, b2 = self.plan, self.mode, self.plan.mix_bwd2
        with _profile.timed("weight_grad"):
            tcw = plan.tc_fwd
            if (mode == "uv" and tcw is not None and tcw.regular and grad.dtype == torch.float32
                    and _tc_supported_w(weight.shape[-2], weight.shape[-1])):
                return wgrad_tc(s, grad, tcw, weight.shape[0])
            if mode == "uv":   # (P, Cout, Cin) summed over nodes, then transposed to the weight's layout
                gw = _ops.indexed_outer_scale_gather(grad, s, b2.scale, b2.index1, b2.index2, b2.seg_out,
                                                     out_accumulated=True, out_size=b2.out_size)
                return gw.transpose(-1, -2).contiguous()
            return _ops.indexed_mul_scale_gather(grad, s, b2.scale, b2.index1, b2.index2, b2.seg_out,
                                                 out_accumulated=True, out_size=b2.out_size)

    def grad_y(self, state, grad: Tensor) -> Tensor:
        node_x, y, weight, _ = state
        graph, plan, mode, b1 = self.graph, self.plan, self.mode, self.plan.mix_bwd1
        # gradient w.r.t. the node-level intermediate: G[d, r] = g[d, M(r)] W[w(r)]^T
        with _profile.timed("channel_mix[grad_inter]"):
            tc = plan.tc_fwd
            if (mode == "uv" and tc is not None and tc.regular
                    and _tc_supported_t(weight.shape[-2], weight.shape[-1])):
                g_inter = mix_tc_transposed(grad, weight, tc)
            elif mode == "uv":
                g_inter = _ops.indexed_vecmat_scale_gather(grad, self._wt(weight), b1.scale, b1.index2, b1.index1,
                                                           b1.seg_out, out_size=b1.out_size)
            else:
                g_inter = _ops.indexed_mul_scale_gather(weight, grad, b1.scale, b1.index1, b1.index2, b1.seg_out,
                                                        out_size=b1.out_size)
        with _profile.timed("cg_inner[grad_y]"):
            return cg_inner(plan.fwd_table, node_x, g_inter, graph.src_by_dst, graph.dst_ptr, graph.dst_sorted,
                            graph.dst_order, y.shape[0])

    def grad_x(self, state, grad: Tensor) -> Tensor:
        _, y, weight, _ = state
        graph, plan = self.graph, self.plan
        with _profile.timed("cg_segment_sum[grad_x]"):
            sx = cg_segment_sum(plan.bwd1_table, grad, y, graph.dst_by_src, graph.src_order, graph.src_ptr,
                                graph.num_src)
        with _profile.timed("channel_mix[grad_x]"):
            return _mix(sx, self._wt(weight), plan.mix_src, self.mode, plan.tc_src)


class SO3LinearGraphFunction(Function):
    @staticmethod
    def forward(ctx, node_x: Tensor, y: Tensor, weight: Tensor, graph: EdgeGraph, plan: GraphTPPlan, mode: str):
        ctx.ops = FusedGraphOps(graph, plan, mode)
        out, state = ctx.ops.forward(node_x, y, weight)
        ctx.save_for_backward(*state)
        if _CHECK_EVERY_CALL:
            check_status(node_x.device)
        return out

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, grad: Tensor):
        state, ops = ctx.saved_tensors, ctx.ops
        grad = grad.contiguous()
        gw = ops.grad_weight(state, grad) if ctx.needs_input_grad[2] else None
        gy = ops.grad_y(state, grad) if ctx.needs_input_grad[1] else None
        gx = ops.grad_x(state, grad) if ctx.needs_input_grad[0] else None
        if _CHECK_EVERY_CALL:
            check_status(grad.device)
        return gx, gy, gw, None, None, None


def so3_linear_graph(node_x: Tensor, y: Tensor, weight: Tensor, graph: EdgeGraph, plan: GraphTPPlan,
                     feature_mode: str = "uv") -> Tensor:
    """Fused gather -> ``SO3Linear`` -> sum over incoming edges.  ``node_x`` (num_src, D1, Cin) float32,
    ``y`` (E, D2) in the caller's edge order, shared ``weight``; returns (num_dst, Dout, Cout)."""
    if weight.ndim != (3 if feature_mode == "uv" else 2):
        raise ValueError("the fused graph layer needs weights shared by all edges")
    return SO3LinearGraphFunction.apply(node_x, y, weight, graph, plan, feature_mode)
