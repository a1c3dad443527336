"""Tensor-core (tcgen05, 3xTF32) weight step against the CUDA-core kernel and a float64 einsum."""
import pytest
import torch

from equitorch_b200.irreps import Irreps
from equitorch_b200.ops import batched_sparse_dense_op as gops
from equitorch_b200.ops.fused_tp_op import check_status
from equitorch_b200.ops.mix_tc_op import MixPlan, mix_tc, mix_tc_transposed, wgrad_tc
from equitorch_b200.tables import tp_infos

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("irreps,n,cin,cout", [
    ("0e+1o+2e+3o", 1000, 64, 64), ("0e+1o+2e+3o", 37, 64, 64), ("0e+1o+2e", 513, 32, 48),
    ("0e+1o+2e+3o", 20011, 64, 64), ("2x0e+1o", 300, 64, 128),
])
def test_mix_tc_matches_float64(irreps, n, cin, cout):
    ir = Irreps(irreps)
    fwd, _, _, paths = tp_infos(ir, ir, Irreps("0e+1o+2e+3o"))
    info = fwd.info_M_fwd.to(DEV)
    plan = MixPlan(info, [i.dim for i in ir], DEV)
    assert plan.regular
    g = torch.Generator().manual_seed(n)
    s = torch.randn(n, plan.rows, cin, generator=g).to(DEV)
    w = (torch.randn(paths, cin, cout, generator=g) / cin ** 0.5).to(DEV)
    got = mix_tc(s, w, plan)
    check_status()
    simt = gops.indexed_vecmat_scale_gather(s, w, None, None, info.index2, info.seg_out, out_size=info.out_size)
    sel = w.double()[info.index2]                                    # (rows, cin, cout)
    per_row = torch.einsum("nri,rio->nro", s.double(), sel)
    seg = info.seg_out.cpu() if info.seg_out is not None else torch.arange(info.out_size + 1)
    want = torch.stack([per_row[:, seg[m]:seg[m + 1]].sum(1) for m in range(info.out_size)], 1)
    scale = float(want.abs().max())
    err_tc = float((got.double() - want).abs().max()) / scale
    err_simt = float((simt.double() - want).abs().max()) / scale
    # the float32 accumulation inside the tensor core is not round-to-nearest: a few 1e-6 of the largest
    # element is what the hardware gives; the parity bar for float32 results is 1e-5
    assert err_tc < 8e-6, f"tensor-core path: relative error {err_tc:.2e} (CUDA-core path {err_simt:.2e})"


@pytest.mark.parametrize("irreps,n,cin,cout", [("0e+1o+2e+3o", 1000, 64, 64), ("0e+1o+2e", 77, 48, 32),
                                               ("0e+1o+2e+3o", 20011, 64, 64)])
def test_mix_tc_transposed_is_the_adjoint(irreps, n, cin, cout):
    ir = Irreps(irreps)
    fwd, _, _, paths = tp_infos(ir, ir, Irreps("0e+1o+2e+3o"))
    info = fwd.info_M_fwd.to(DEV)
    plan = MixPlan(info, [i.dim for i in ir], DEV)
    gen = torch.Generator().manual_seed(n + 1)
    g = torch.randn(n, plan.comps, cout, generator=gen).to(DEV)
    w = (torch.randn(paths, cin, cout, generator=gen) / cout ** 0.5).to(DEV)
    got = mix_tc_transposed(g, w, plan)
    check_status()
    seg = info.seg_out.cpu() if info.seg_out is not None else torch.arange(info.out_size + 1)
    comp_of_row = torch.repeat_interleave(torch.arange(info.out_size), seg[1:] - seg[:-1]).to(DEV)
    want = torch.einsum("nro,rio->nri", g.double()[:, comp_of_row], w.double()[info.index2])
    err = float((got.double() - want).abs().max() / want.abs().max())
    assert got.shape == want.shape and err < 8e-6, f"relative error {err:.2e}"


@pytest.mark.parametrize("irreps,n,cin,cout", [("0e+1o+2e+3o", 1000, 64, 64), ("0e+1o+2e", 77, 32, 32),
                                               ("0e+1o+2e+3o", 20011, 64, 64), ("0e+1o+2e+3o", 5, 64, 64)])
def test_wgrad_tc_matches_float64_and_is_reproducible(irreps, n, cin, cout):
    ir = Irreps(irreps)
    fwd, _, _, paths = tp_infos(ir, ir, Irreps("0e+1o+2e+3o"))
    info = fwd.info_M_fwd.to(DEV)
    plan = MixPlan(info, [i.dim for i in ir], DEV)
    gen = torch.Generator().manual_seed(n + 2)
    s = torch.randn(n, plan.rows, cin, generator=gen).to(DEV)
    g = torch.randn(n, plan.comps, cout, generator=gen).to(DEV)
    got = wgrad_tc(s, g, plan, paths)
    again = wgrad_tc(s, g, plan, paths)
    check_status()
    assert torch.equal(got, again)
    seg = info.seg_out.cpu() if info.seg_out is not None else torch.arange(info.out_size + 1)
    comp_of_row = torch.repeat_interleave(torch.arange(info.out_size), seg[1:] - seg[:-1]).to(DEV)
    per_row = torch.einsum("nri,nro->rio", s.double(), g.double()[:, comp_of_row])
    want = torch.zeros(paths, cin, cout, dtype=torch.float64, device=DEV).index_add_(0, info.index2, per_row)
    err = float((got.double() - want).abs().max() / want.abs().max())
    assert err < 8e-6, f"relative error {err:.2e}"
