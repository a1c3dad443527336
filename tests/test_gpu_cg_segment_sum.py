"""Gather + CG + segment-sum step (``eqt_tp_cg_segment_sum``) against a float64 restatement of its sum."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from equitorch_b200.irreps import Irreps
from equitorch_b200.tables import tp_infos
from equitorch_b200.ops.fused_tp_op import TpTable, cg_segment_sum, check_status


def _irreps(lmax):
    return Irreps("+".join(f"{l}{'e' if l % 2 == 0 else 'o'}" for l in range(lmax + 1)))


def _reference(table, feat, y, fidx, yidx, ptr, num_out):
    """float64: out[d, row[t]] += scale[t] * y[yidx[e], m_y[t]] * feat[fidx[e], m_feat[t]] over e in node d."""
    f = feat.double()[fidx]                                     # (E, DF, C)
    yy = y.double()[yidx] if yidx is not None else y.double()   # (E, DY)
    rp = table.row_ptr.cpu().numpy()
    row = torch.from_numpy(np.repeat(np.arange(table.num_rows), np.diff(rp))).to(feat.device)
    term = table.scale.double()[None, :, None] * yy[:, table.m_y][:, :, None] * f[:, table.m_feat]
    inter = torch.zeros(f.shape[0], table.num_rows, f.shape[2], dtype=torch.float64, device=feat.device)
    inter.index_add_(1, row, term)
    node = torch.repeat_interleave(torch.arange(num_out, device=feat.device), ptr[1:] - ptr[:-1])
    out = torch.zeros(num_out, table.num_rows, f.shape[2], dtype=torch.float64, device=feat.device)
    out.index_add_(0, node, inter)
    return out


@pytest.mark.parametrize("lmax,c,role", [(3, 64, "fwd"), (3, 64, "bwd1"), (2, 32, "fwd"), (1, 128, "fwd"), (3, 96, "fwd")])
def test_cg_segment_sum(lmax, c, role):
    dev = torch.device("cuda:0")
    ir = _irreps(lmax)
    fwd, bwd1, _, _ = tp_infos(ir, ir, ir)
    table = (TpTable(fwd.info_Mij_fwd, True, ir.dim, ir.dim, dev) if role == "fwd"
             else TpTable(bwd1.info_Mij_fwd, False, ir.dim, ir.dim, dev))
    g = torch.Generator().manual_seed(1234 + lmax + c)
    n_nodes, n_feat = 700, 650
    deg = torch.randint(0, 9, (n_nodes,), generator=g)          # empty, odd and even segments
    deg[5] = 37
    deg[n_nodes - 1] = 0
    ptr = torch.zeros(n_nodes + 1, dtype=torch.int64)
    ptr[1:] = torch.cumsum(deg, 0)
    e = int(ptr[-1])
    fidx = torch.randint(0, n_feat, (e,), generator=g).to(dev)
    yidx = torch.randperm(e, generator=g).to(dev)
    feat = torch.randn(n_feat, ir.dim, c, generator=g).to(dev)
    y = torch.randn(e, ir.dim, generator=g).to(dev)
    ptr = ptr.to(dev)
    want = _reference(table, feat, y, fidx, yidx, ptr, n_nodes)
    got = cg_segment_sum(table, feat, y, fidx, yidx, ptr, n_nodes)
    check_status(dev)
    scale = want.abs().max().item()
    # float32 tolerance of the path: 1e-5 of the largest entry
    assert (got.double() - want).abs().max().item() <= 1e-5 * scale
    assert torch.all(got[deg.to(dev) == 0] == 0)


def test_cg_segment_sum_identity_indices():
    """No gather indices: edge e reads feature row e and harmonics row e."""
    dev = torch.device("cuda:0")
    ir = _irreps(3)
    fwd, _, _, _ = tp_infos(ir, ir, ir)
    table = TpTable(fwd.info_Mij_fwd, True, ir.dim, ir.dim, dev)
    g = torch.Generator().manual_seed(7)
    n_nodes = 300
    ptr = torch.arange(0, 3 * n_nodes + 1, 3, dtype=torch.int64, device=dev)
    e = 3 * n_nodes
    feat = torch.randn(e, ir.dim, 64, generator=g).to(dev)
    y = torch.randn(e, ir.dim, generator=g).to(dev)
    want = _reference(table, feat, y, torch.arange(e, device=dev), None, ptr, n_nodes)
    got = cg_segment_sum(table, feat, y, None, None, ptr, n_nodes)
    check_status(dev)
    assert (got.double() - want).abs().max().item() <= 1e-5 * want.abs().max().item()
