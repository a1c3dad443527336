"""The fused layer's step (forward + backward) replayed as a CUDA graph gives the eager results, also after
the inputs have been overwritten in place."""
import pytest
import torch

from equitorch_b200 import nn as enn
from equitorch_b200.graph import EdgeGraph
from equitorch_b200.ops.fused_tp_op import check_status
from equitorch_b200.utils.cuda_graph import GraphedStep

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_graphed_step_matches_eager():
    irreps, lmax, c, nodes, edges = "0e+1o+2e+3o", 3, 64, 300, 5000
    g = torch.Generator().manual_seed(11)
    src = torch.randint(0, nodes, (edges,), generator=g)
    dst = torch.sort(torch.randint(0, nodes, (edges,), generator=g)).values
    graph = EdgeGraph(src.to(DEV), dst.to(DEV), nodes)
    layer = enn.SO3LinearGraph(irreps, irreps, irreps, c, c, internal_weights=False, feature_mode="uv").to(DEV)
    sh = enn.SphericalHarmonics(lmax)
    x = torch.randn(nodes, 16, c, generator=g).to(DEV).requires_grad_(True)
    vec = torch.randn(edges, 3, generator=g).to(DEV).requires_grad_(True)
    w = (torch.randn(*layer.weight_shape, generator=g) / c ** 0.5).to(DEV).requires_grad_(True)
    cot = torch.randn(nodes, 16, c, generator=g).to(DEV)

    def step():
        out = layer(x, sh(vec), graph, w)
        return (out,) + torch.autograd.grad(out, [x, vec, w], cot)

    graphed = GraphedStep(step, DEV)
    for trial in range(2):
        if trial == 1:                      # new inputs in the same buffers
            with torch.no_grad():
                x.copy_(torch.randn(nodes, 16, c, generator=g))
                vec.copy_(torch.randn(edges, 3, generator=g))
        want = [t.clone() for t in step()]
        got = graphed.replay()
        torch.cuda.synchronize()
        check_status()
        for a, b in zip(got, want):
            assert torch.equal(a, b)        # same kernels on the same data: bit-identical
