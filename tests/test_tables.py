"""Index tables against the reference's own output (tests/golden/tables.pt.gz).

Integer fields and segment pointers must be bit-identical, ``None``-ness of every field
must agree (kernels branch on it), float scales must agree to one float32 ulp.
"""
import numpy as np
import pytest
import torch

from equitorch_b200 import constants, tables
from equitorch_b200.irreps import Irreps
from tests.golden.make_golden_shared import flatten

BUILDERS = {
    "tp": lambda a, kw: tables.tp_infos(*(Irreps(s) for s in a), **kw),
    "so2": lambda a, kw: tables.so2_linear_infos(*(Irreps(s) for s in a), **kw),
    "wigner": lambda a, kw: tables.wigner_d_info(Irreps(a[0])),
    "irreps_info": lambda a, kw: tables.irreps_info(Irreps(a[0])),
    "irreps_linear": lambda a, kw: tables.irreps_linear_infos(*(Irreps(s) for s in a), **kw),
}


def _builder(tag):
    for prefix in ("irreps_info", "irreps_linear", "tp", "so2", "wigner"):
        if tag.startswith(prefix):
            return BUILDERS[prefix]
    raise KeyError(tag)


def _check(ours, ref, where):
    assert ours.keys() == ref.keys(), where
    for key, want in ref.items():
        got = ours[key]
        if want is None or isinstance(want, int):
            assert got == want, f"{where}:{key}: {got} != {want}"
            continue
        assert isinstance(got, torch.Tensor), f"{where}:{key} should be a tensor"
        assert got.dtype == want.dtype and got.shape == want.shape, f"{where}:{key}"
        if want.is_floating_point():
            ulp = torch.finfo(want.dtype).eps * want.abs().clamp_min(1e-30)
            assert bool(((got - want).abs() <= ulp).all()), f"{where}:{key}"
        else:
            assert torch.equal(got, want), f"{where}:{key}"


def test_tables_match_reference(golden_tables):
    assert len(golden_tables) >= 20
    for tag, rec in golden_tables.items():
        ours = flatten(_builder(tag)(rec["args"], rec.get("kwargs", {})))
        _check(ours, rec["out"], tag)


def test_appendix_mini_example():
    """Hand-checkable case: 0e+1o (x) 0e+1o -> 0e+1o, path_norm."""
    fwd, bwd1, bwd2, n = tables.tp_infos(*(Irreps("0e+1o"),) * 3)
    assert n == 4
    assert fwd.info_Mij_fwd.index1.tolist() == [0, 1, 2, 3, 0, 1, 0, 2, 0, 3]
    assert fwd.info_Mij_fwd.index2.tolist() == [0, 1, 2, 3, 1, 0, 2, 0, 3, 0]
    assert fwd.info_Mij_fwd.seg_out.tolist() == [0, 1, 4, 5, 6, 7, 8, 9, 10]
    assert fwd.info_M_fwd.index1 is None and fwd.info_M_fwd.scale is None
    assert fwd.info_M_fwd.index2.tolist() == [0, 1, 2, 3, 2, 3, 2, 3]
    assert fwd.info_M_fwd.seg_out.tolist() == [0, 2, 4, 6, 8]
    assert fwd.info_M_bwd1.seg_out is None and fwd.info_M_bwd1.out_size == 8
    assert fwd.info_M_bwd2.seg_out.tolist() == [0, 1, 2, 5, 8]
    s = fwd.info_Mij_fwd.scale
    assert s.dtype == torch.float32
    np.testing.assert_allclose(s[:4].numpy(), [2 ** -0.5] + [6 ** -0.5] * 3, rtol=1e-7)


def test_config_sizes():
    """Sizes quoted for the benchmark configurations (lmax 2 and lmax 3, all paths)."""
    f2 = tables.tp_infos(*(Irreps("0e+1o+2e"),) * 3)
    f3 = tables.tp_infos(*(Irreps("0e+1o+2e+3o"),) * 3)
    assert f2[3] == 11 and f2[0].info_Mij_fwd.scale.numel() == 83 and f2[0].info_Mij_fwd.out_size == 35
    assert f3[3] == 23 and f3[0].info_Mij_fwd.scale.numel() == 353 and f3[0].info_Mij_fwd.out_size == 99
    assert f3[0].info_kM1M2_fwd.out_size == 311


def test_empty_output_rows_keep_csr_shape():
    """An output irrep without any path still gets (repeated) pointers."""
    info = tables.sparse_product_info(index1=[0, 1], index2=[1, 0], index=[1, 3], scale=[1.0, 2.0], out_size=5)
    assert info.seg_out.tolist() == [0, 0, 1, 1, 2, 2]
    fwd, *_ = tables.tp_infos(Irreps("1o+0e"), Irreps("0e"), Irreps("0e"))
    assert fwd.info_M_fwd.out_size == 4
    assert fwd.info_M_fwd.seg_out.tolist() == [0, 0, 0, 0, 1]


@pytest.mark.parametrize("l,l1,l2", [(0, 0, 0), (1, 1, 0), (1, 1, 1), (2, 1, 1), (3, 2, 1), (4, 2, 2), (6, 3, 3), (5, 6, 2)])
def test_cg_orthonormal_rows(l, l1, l2):
    cg = constants.so3_clebsch_gordan(l, l1, l2)
    gram = np.einsum("mab,nab->mn", cg, cg)
    np.testing.assert_allclose(gram, np.eye(2 * l + 1), atol=1e-14)


def test_cg_full_decomposition_is_orthogonal():
    """Stacking all l in |l1-l2|..l1+l2 gives an orthogonal (2l1+1)(2l2+1) matrix."""
    l1, l2 = 2, 3
    rows = [constants.so3_clebsch_gordan(l, l1, l2).reshape(2 * l + 1, -1) for l in range(abs(l1 - l2), l1 + l2 + 1)]
    q = np.concatenate(rows)
    np.testing.assert_allclose(q @ q.T, np.eye(q.shape[0]), atol=1e-14)


@pytest.mark.parametrize("l", range(0, 7))
def test_j_matrix_symmetric_involution(l):
    j = constants.j_matrix(l)
    np.testing.assert_allclose(j, j.T, atol=1e-14)
    np.testing.assert_allclose(j @ j, np.eye(2 * l + 1), atol=1e-13)


def test_info_movement_keeps_int64():
    fwd, *_ = tables.tp_infos(*(Irreps("0e+1o"),) * 3)
    moved = fwd.to(torch.float64)
    assert moved.info_Mij_fwd.scale.dtype == torch.float64
    assert moved.info_Mij_fwd.index1.dtype == torch.int64
    assert moved.info_M_fwd.scale is None and moved.out_size == fwd.out_size
