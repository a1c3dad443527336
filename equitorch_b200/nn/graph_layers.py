"""Graph form of ``SO3Linear``: gather by edge source, tensor product with the edge's spherical
harmonics, sum into the destination node - one fused operation (see ``functional.graph_tp``)."""
from __future__ import annotations

from typing import Dict, Optional

import torch
from torch import Tensor

from ..graph import EdgeGraph
from .functional.graph_tp import FusedGraphOps, GraphTPPlan, so3_linear_graph
from .linears import SO3Linear


class SO3LinearGraph(SO3Linear):
    """``out[d] = sum_{e -> d} SO3Linear(node_x[src(e)], y[e])`` with weights shared by all edges.

    Same constructor, parameters and state dict as :class:`SO3Linear`; ``forward`` takes node
    features ``(num_nodes, irreps_in1.dim, channels_in)``, per-edge harmonics ``(E, irreps_in2.dim)``
    in the caller's edge order and an :class:`~equitorch_b200.graph.EdgeGraph`.
    """

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self._plans: Dict[torch.device, GraphTPPlan] = {}

    def plan(self, device) -> GraphTPPlan:
        device = torch.device(device)
        if device not in self._plans:
            self._plans[device] = GraphTPPlan(self.tp_info_forward, self.tp_info_backward1,
                                              self.irreps_in1_dim, self.irreps_in2_dim, self.irreps_out_dim, device,
                                              out_dims=[ir.dim for ir in self.irreps_out],
                                              in1_dims=[ir.dim for ir in self.irreps_in1])
        return self._plans[device]

    def _apply(self, fn, *args, **kwargs):
        module = super()._apply(fn, *args, **kwargs)
        module._plans = {}
        return module

    def forward(self, node_x: Tensor, edge_sh: Tensor, graph: EdgeGraph, weight: Optional[Tensor] = None) -> Tensor:
        assert node_x.shape[-2] == self.irreps_in1_dim and edge_sh.shape[-1] == self.irreps_in2_dim
        assert node_x.shape[0] == graph.num_src and edge_sh.shape[0] == graph.num_edges
        weight = self._resolve_weight(weight)
        return so3_linear_graph(node_x, edge_sh, weight, graph, self.plan(node_x.device), self.feature_mode)

    def forward_sharded(self, local_x: Tensor, edge_sh: Tensor, graph: EdgeGraph, shard, send_index: Optional[Tensor] = None,
                        weight: Optional[Tensor] = None, group=None) -> Tensor:
        """One rank's part of the layer on a graph sharded by destination range (``equitorch_b200.dist``):
        ``local_x`` is the rank's ``[owned | halo]`` buffer (halo rows are filled in place from their owners),
        ``graph`` its local edges; returns the owned output rows.  Gradients: owned rows of ``local_x`` (including
        what other ranks' edges contribute), ``edge_sh``, and the weight gradient summed over ranks."""
        from ..dist import sharded_layer
        weight = self._resolve_weight(weight)
        if weight.ndim != (3 if self.feature_mode == "uv" else 2):
            raise ValueError("the fused graph layer needs weights shared by all edges")
        ops = FusedGraphOps(graph, self.plan(local_x.device), self.feature_mode)
        return sharded_layer(local_x, edge_sh, weight, ops, shard, send_index, group)
