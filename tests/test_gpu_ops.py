"""Parity of the CUDA operator layer with the reference (golden fixtures) and the CPU oracle."""
import pytest
import torch

from equitorch_b200.ops import batched_sparse_dense_op as gops
from equitorch_b200.ops.graph_ops import gather_rows, segment_sum
from equitorch_b200.ops.indexed_scale_segment_op import indexed_scale_segment
from oracle import sparse_ops as oops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
# relative tolerances per storage type; float64/float32 follow the 1e-5 parity bar (float64 far tighter)
TOL = {torch.float64: dict(rtol=1e-11, atol=1e-11), torch.float32: dict(rtol=1e-5, atol=1e-5),
       torch.bfloat16: dict(rtol=2e-2, atol=2e-2)}


def _cuda(v, dtype=None):
    if isinstance(v, torch.Tensor):
        v = v.to(DEV)
        return v.to(dtype) if (dtype is not None and v.is_floating_point()) else v
    return v


def _run(case, dtype):
    kw = {k: _cuda(v, dtype) for k, v in case["kwargs"].items()}
    if case["op"] == "scale_segment":
        return indexed_scale_segment(_cuda(case["input1"], dtype), **kw)
    fn = getattr(gops, f"indexed_{case['op']}_scale_gather")
    return fn(_cuda(case["input1"], dtype), _cuda(case["input2"], dtype), **kw)


@pytest.mark.parametrize("dtype", [torch.float64, torch.float32, torch.bfloat16])
def test_ops_match_reference_fixtures(golden_ops, dtype):
    for n, case in enumerate(golden_ops["cases"]):
        got = _run(case, dtype)
        assert got.dtype == dtype and got.shape == case["out"].shape, f"case {n} {case['op']}"
        want = case["out"]
        if dtype == torch.bfloat16:   # compare with the reference evaluated on the rounded inputs
            rounded = dict(case, input1=case["input1"].to(dtype).double(),
                           input2=None if case["input2"] is None else case["input2"].to(dtype).double())
            if case["op"] == "scale_segment":
                want = oops.indexed_scale_segment(rounded["input1"], **case["kwargs"])
            else:
                want = getattr(oops, f"indexed_{case['op']}_scale_gather")(rounded["input1"], rounded["input2"], **case["kwargs"])
        scale = max(1.0, float(want.abs().max()))
        tol = TOL[dtype]
        torch.testing.assert_close(got.double().cpu(), want, rtol=tol["rtol"], atol=tol["atol"] * scale,
                                   msg=lambda m: f"case {n} {case['op']} {sorted(case['kwargs'])}: {m}")


@pytest.mark.parametrize("op", ["mul", "outer", "inner", "vecmat", "vecsca"])
@pytest.mark.parametrize("shared", [(False, False), (True, False), (False, True)])
@pytest.mark.parametrize("accumulated", [False, True])
def test_ops_ragged_sizes_vs_oracle(op, shared, accumulated):
    """Odd sizes of the reference's own sweep (N=135, C=97, C1=35, C2=21), float32."""
    g = torch.Generator().manual_seed(hash((op, shared, accumulated)) % 2**31)
    N, M1, M2, T, O = 135, 9, 16, 83, 35
    C, C2 = (35, 21) if op in ("outer", "vecmat") else (97, 0)
    i1 = torch.randint(0, M1, (T,), generator=g)
    i2 = torch.randint(0, M2, (T,), generator=g)
    scale = torch.randn(T, generator=g)
    cuts = torch.sort(torch.randint(0, T + 1, (O - 1,), generator=g)).values
    seg = torch.cat([torch.tensor([0]), cuts, torch.tensor([T])])
    r = lambda *s: torch.randn(*s, generator=g)  # noqa: E731
    x = r(M1, C) if shared[0] else r(N, M1, C)
    tail = {"mul": (C,), "inner": (C,), "outer": (C2,), "vecsca": (), "vecmat": (C, C2)}[op]
    y = r(M2, *tail) if shared[1] else r(N, M2, *tail)
    kw = dict(scale=scale, index1=i1, index2=i2, seg=seg, out_accumulated=accumulated)
    want = getattr(oops, f"indexed_{op}_scale_gather")(x.double(), y.double(), **{**kw, "scale": scale.double()})
    got = getattr(gops, f"indexed_{op}_scale_gather")(x.to(DEV), y.to(DEV), **{k: _cuda(v) for k, v in kw.items()})
    assert got.shape == want.shape
    err = (got.double().cpu() - want).abs().max() / want.abs().max().clamp_min(1e-30)
    assert err < 1e-5, f"relative error {err:.2e}"


def test_empty_batch_and_empty_segments():
    x = torch.zeros(0, 4, 8, device=DEV)
    y = torch.zeros(0, 4, 8, device=DEV)
    assert gops.indexed_mul_scale_gather(x, y).shape == (0, 4, 8)
    x = torch.randn(3, 4, 8, device=DEV)
    seg = torch.tensor([0, 0, 4, 4], device=DEV)
    out = gops.indexed_mul_scale_gather(x, x, seg=seg)
    assert out.shape == (3, 3, 8)
    assert torch.count_nonzero(out[:, 0]) == 0 and torch.count_nonzero(out[:, 2]) == 0
    torch.testing.assert_close(out[:, 1], (x * x).sum(1))


def test_non_atomic_paths_are_bitwise_deterministic():
    g = torch.Generator().manual_seed(3)
    x = torch.randn(257, 16, 64, generator=g).to(DEV)
    y = torch.randn(257, 16, generator=g).to(DEV)
    i1 = torch.randint(0, 16, (353,), generator=g).to(DEV)
    i2 = torch.randint(0, 16, (353,), generator=g).to(DEV)
    seg = torch.arange(0, 354, 3).clamp_max(353).to(DEV)
    a = gops.indexed_vecsca_scale_gather(x, y, index1=i1, index2=i2, seg=seg)
    b = gops.indexed_vecsca_scale_gather(x, y, index1=i1, index2=i2, seg=seg)
    assert torch.equal(a, b)


def test_gather_and_segment_sum():
    g = torch.Generator().manual_seed(4)
    nodes, edges = 50, 400
    x = torch.randn(nodes, 9, 8, generator=g)
    src = torch.randint(0, nodes, (edges,), generator=g)
    dst = torch.sort(torch.randint(0, nodes, (edges,), generator=g)).values
    ptr = torch.zeros(nodes + 1, dtype=torch.long)
    ptr[1:] = torch.cumsum(torch.bincount(dst, minlength=nodes), 0)
    xe = gather_rows(x.to(DEV), src.to(DEV))
    assert torch.equal(xe.cpu(), x[src])
    got = segment_sum(xe, ptr.to(DEV))
    want = torch.zeros(nodes, 9, 8, dtype=torch.float64).index_add_(0, dst, x[src].double())
    torch.testing.assert_close(got.double().cpu(), want, rtol=1e-5, atol=1e-5)
    perm = torch.randperm(edges, generator=g)
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(edges)
    got2 = segment_sum(xe[perm], ptr.to(DEV), inv.to(DEV))
    torch.testing.assert_close(got2, got, rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("use_perm", [False, True])
def test_segment_sum_gradient(use_perm):
    """Gradient of the segment sum against index_add on float64, with rows before ptr[0] and after ptr[-1] that
    belong to no segment (their gradient is zero)."""
    g = torch.Generator().manual_seed(5)
    nodes, edges, lead, trail = 37, 300, 5, 7
    dst = torch.sort(torch.randint(0, nodes, (edges,), generator=g)).values
    ptr = torch.zeros(nodes + 1, dtype=torch.long)
    ptr[1:] = torch.cumsum(torch.bincount(dst, minlength=nodes), 0)
    ptr += lead
    rows = lead + edges + trail
    x = torch.randn(rows, 4, 8, generator=g)
    cot = torch.randn(nodes, 4, 8, generator=g)
    perm = torch.randperm(rows, generator=g) if use_perm else None
    xd = x.to(DEV).requires_grad_(True)
    out = segment_sum(xd, ptr.to(DEV), None if perm is None else perm.to(DEV))
    (gx,) = torch.autograd.grad(out, xd, cot.to(DEV))
    xr = x.double().requires_grad_(True)
    src_rows = xr if perm is None else xr[perm]
    want = torch.zeros(nodes, 4, 8, dtype=torch.float64).index_add_(0, dst, src_rows[lead:lead + edges])
    torch.testing.assert_close(out.double().cpu(), want.detach(), rtol=1e-5, atol=1e-5)
    (gr,) = torch.autograd.grad(want, xr, cot.double())
    torch.testing.assert_close(gx.double().cpu(), gr, rtol=1e-6, atol=1e-6)
