"""The tensor-core paths behind ``indexed_vecmat_scale_gather`` (shared matrix operand) and accumulated
``indexed_outer_scale_gather``: against the float64 oracle and against the table-driven CUDA-core kernels, on random
tables with empty segments, missing index arrays and ragged batch sizes; and the layers that reach them through
the reference's own entry points (IrrepWiseLinear, IrrepsLinear, SO2Linear, per-edge SO3Linear 'uv').
Error norm: max |a - b| / max |b|, bound 1e-5 (float32, 3xTF32 products with float32 accumulation)."""
import pytest
import torch

from equitorch_b200 import nn as enn
from equitorch_b200.ops import batched_sparse_dense_op as gops
from equitorch_b200.ops import indexed_tc_op as tc
from equitorch_b200.ops.fused_tp_op import check_status
from oracle import sparse_ops as oops
from oracle import tensor_products as otp

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _rel(a, b):
    return float((a.detach().double().cpu() - b.detach().double().cpu()).abs().max() / max(1e-30, float(b.detach().abs().max())))


def _table(g, entries, rows1, rows2, num_out, with_index1=True, with_index2=True, with_scale=True):
    # sorted output rows with some empty segments
    owner = torch.sort(torch.randint(0, num_out, (entries,), generator=g)).values
    owner = owner[owner != num_out // 2] if num_out > 2 else owner          # one row without entries
    entries = owner.numel()
    seg = torch.zeros(num_out + 1, dtype=torch.long)
    seg[1:] = torch.cumsum(torch.bincount(owner, minlength=num_out), 0)
    i1 = torch.randint(0, rows1, (entries,), generator=g) if with_index1 else None
    i2 = torch.randint(0, rows2, (entries,), generator=g) if with_index2 else None
    sc = torch.randn(entries, generator=g) if with_scale else None
    return sc, i1, i2, seg, entries


@pytest.mark.parametrize("n,cin,cout", [(1000, 32, 32), (777, 64, 48), (4096, 32, 64), (513, 96, 128)])
@pytest.mark.parametrize("variant", ["full", "no_index2", "no_scale"])
def test_vecmat_shared_weights(n, cin, cout, variant):
    g = torch.Generator().manual_seed(n + cin + cout)
    rows1, rows2, num_out = 13, 9, 11
    sc, i1, i2, seg, entries = _table(g, 40, rows1, rows2, num_out, with_index2=variant != "no_index2",
                                      with_scale=variant != "no_scale")
    if i2 is None:
        rows2 = entries
    x = torch.randn(n, rows1, cin, generator=g)
    w = torch.randn(rows2, cin, cout, generator=g) / cin ** 0.5
    want = oops.indexed_vecmat_scale_gather(x.double(), w.double(), sc if sc is None else sc.double(), i1, i2, seg)
    dev = lambda t: None if t is None else t.to(DEV)
    assert tc.vecmat_supported(x.to(DEV), w.to(DEV), None, None, False, num_out, num_out)
    got = gops.indexed_vecmat_scale_gather(x.to(DEV), w.to(DEV), dev(sc), dev(i1), dev(i2), dev(seg))
    check_status()
    assert got.shape == want.shape and _rel(got, want) < 1e-5
    assert torch.count_nonzero(got[:, num_out // 2]) == 0                       # the row without entries
    # operands swapped: the matrix-transposed-vector alias reaches the same kernel
    got2 = gops.indexed_mat_t_vec_scale_gather(w.to(DEV), x.to(DEV), dev(sc), dev(i2), dev(i1), dev(seg))
    assert torch.equal(got, got2)


@pytest.mark.parametrize("n,c1,c2", [(1000, 32, 32), (999, 64, 32), (5000, 32, 64), (640, 64, 128)])
@pytest.mark.parametrize("variant", ["full", "no_scale"])
def test_outer_accumulated(n, c1, c2, variant):
    g = torch.Generator().manual_seed(n + c1 + c2)
    rows1, rows2, num_w = 7, 5, 9
    sc, i1, i2, seg, entries = _table(g, 30, rows1, rows2, num_w, with_scale=variant != "no_scale")
    a, b = torch.randn(n, rows1, c1, generator=g), torch.randn(n, rows2, c2, generator=g)
    want = oops.indexed_outer_scale_gather(a.double(), b.double(), sc if sc is None else sc.double(), i1, i2, seg,
                                           out_accumulated=True)
    dev = lambda t: None if t is None else t.to(DEV)
    assert tc.outer_supported(a.to(DEV), b.to(DEV), None, None, True, num_w, num_w)
    got = gops.indexed_outer_scale_gather(a.to(DEV), b.to(DEV), dev(sc), dev(i1), dev(i2), dev(seg), out_accumulated=True)
    again = gops.indexed_outer_scale_gather(a.to(DEV), b.to(DEV), dev(sc), dev(i1), dev(i2), dev(seg), out_accumulated=True)
    check_status()
    assert got.shape == want.shape and _rel(got, want) < 1e-5
    assert torch.equal(got, again)                                              # fixed summation order
    assert torch.count_nonzero(got[num_w // 2]) == 0


def test_layers_reach_tensor_cores_and_match_table_driven_kernels(monkeypatch):
    """IrrepWiseLinear, IrrepsLinear, SO2Linear and the per-edge SO3Linear 'uv' at 4096 samples: output and all
    gradients through the tensor-core paths against the same layers on the table-driven kernels (1e-5) and the
    number of tensor-core launches."""
    from equitorch_b200 import _lib
    g = torch.Generator().manual_seed(1)
    n, c = 4096, 32
    cases = [
        ("irrepwise", enn.IrrepWiseLinear("0e+1o+2e", c, c, internal_weights=False), 9),
        ("irreps", enn.IrrepsLinear("0e+1o+2e", "0e+1o+1o+2e", c, c, internal_weights=False), 9),
        ("so2", enn.SO2Linear("0e+1o+2e+3o", "0e+1o+2e+3o", c, c, internal_weights=False, feature_mode="uv"), 16),
    ]
    for name, layer, dim in cases:
        layer = layer.to(DEV)
        x = torch.randn(n, dim, c, generator=g).to(DEV).requires_grad_(True)
        w = (torch.randn(*layer.weight_shape, generator=g) / c ** 0.5).to(DEV).requires_grad_(True)
        out = layer(x, w)
        cot = torch.randn(out.shape, generator=g).to(DEV)
        grads = torch.autograd.grad(out, [x, w], cot)
        check_status()
        monkeypatch.setattr(tc, "MIN_BATCH", 1 << 60)                          # table-driven kernels
        ref = layer(x, w)
        ref_grads = torch.autograd.grad(ref, [x, w], cot)
        monkeypatch.setattr(tc, "MIN_BATCH", 512)
        for u, v in [(out, ref), *zip(grads, ref_grads)]:
            assert _rel(u, v) < 1e-5, name


def test_tensor_product_uvw_sliced_over_samples(monkeypatch):
    """TensorProduct 'uvw' (both operands channelled, 32 x 32 -> 32 channels, l_max 2) with the intermediate limit
    lowered so that the batch is processed in slices: output and all three gradients against the float64 oracle
    (dense path form) and against the unsliced chain; bound 1e-5."""
    from equitorch_b200.nn.functional import tensor_products as ftp
    ir, n, c = "0e+1o+2e", 1536, 32
    g = torch.Generator().manual_seed(2)
    layer = enn.TensorProduct(ir, ir, ir, c, c, c, internal_weights=False, feature_mode="uvw").to(DEV)
    x1, x2 = torch.randn(n, 9, c, generator=g), torch.randn(n, 9, c, generator=g)
    w = torch.randn(*layer.weight_shape, generator=g) / c
    cot = torch.randn(n, 9, c, generator=g)
    a, b, ww = (t.to(DEV).requires_grad_(True) for t in (x1, x2, w))
    whole = layer(a, b, ww)
    gwhole = torch.autograd.grad(whole, [a, b, ww], cot.to(DEV))
    monkeypatch.setattr(ftp, "UVW_INTERMEDIATE_LIMIT", 512 * 35 * c * c * 4)       # slices of 512 samples
    sliced = layer(a, b, ww)
    gsliced = torch.autograd.grad(sliced, [a, b, ww], cot.to(DEV))
    check_status()
    for u, v in [(sliced, whole), *zip(gsliced, gwhole)]:
        assert _rel(u, v) < 1e-5
    m = 256                                                                      # oracle on the first samples
    ao, bo, wo = x1[:m].double().requires_grad_(True), x2[:m].double().requires_grad_(True), w.double().requires_grad_(True)
    ref = otp.tensor_product_dense(ao, bo, wo, ir, ir, ir, feature_mode="uvw")
    assert _rel(sliced[:m], ref) < 1e-5
    cot0 = cot.clone()
    cot0[m:] = 0
    gx1, gx2, gw = torch.autograd.grad(layer(a, b, ww), [a, b, ww], cot0.to(DEV))
    ro = torch.autograd.grad(ref, [ao, bo, wo], cot[:m].double())
    for u, v in zip((gx1[:m], gx2[:m], gw), ro):
        assert _rel(u, v) < 1e-5
