"""The allocation-free weight-gradient entry point (``eqt_wgrad_tc_static``) against the regular one.

Some callers of the C ABI cannot give the library a scratch buffer: a plain C host without an
allocator at hand, or a plug-in inside a framework that owns all device memory and forbids later
``cudaMalloc``.  For them the library carries its scratch as a static device array.  This test calls
both entry points through ctypes on the same inputs, twice in a row (the second call reuses the
array the first one left dirty), and expects bit-identical results: the arithmetic is the same and
the reduction order is fixed.  It is collected last on purpose.
"""
import ctypes as C

import pytest
import torch

from equitorch_b200 import _lib
from equitorch_b200.irreps import Irreps
from equitorch_b200.ops.mix_tc_op import MixPlan
from equitorch_b200.tables import tp_infos

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _call_both(n, cin, cout, seed):
    ir = Irreps("0e+1o+2e+3o")
    fwd, _, _, paths = tp_infos(ir, ir, ir)
    plan = MixPlan(fwd.info_M_fwd.to(DEV), [i.dim for i in ir], DEV)
    gen = torch.Generator().manual_seed(seed)
    s = torch.randn(n, plan.rows, cin, generator=gen).to(DEV)
    g = torch.randn(n, plan.comps, cout, generator=gen).to(DEV)
    blocks = plan.structs(cin, cout)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    lib = _lib.lib()
    stream = torch.cuda.current_stream().cuda_stream
    # regular entry point: the caller brings the scratch
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    scratch = torch.empty(128 * cout * sms, dtype=torch.float32, device=DEV)
    want = torch.full((paths, cin, cout), float("nan"), device=DEV)
    rc = lib.eqt_wgrad_tc(s.data_ptr(), g.data_ptr(), want.data_ptr(), scratch.data_ptr(), scratch.numel(), n,
                          plan.rows, plan.comps, cin, cout, blocks, len(blocks), status.data_ptr(), stream)
    assert rc == 0, lib.eqt_last_error()
    # allocation-free entry point: inputs and output only
    got = torch.full((paths, cin, cout), float("nan"), device=DEV)
    rc = lib.eqt_wgrad_tc_static(s.data_ptr(), g.data_ptr(), got.data_ptr(), n, plan.rows, plan.comps, cin, cout,
                                 blocks, len(blocks), status.data_ptr(), stream)
    assert rc == 0, lib.eqt_last_error()
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    return got, want, s, g, plan, paths


def test_static_scratch_entry_point_matches_regular_one_twice():
    for seed, n in ((1, 3000), (2, 777)):          # two calls in a row, different sizes
        got, want, s, g, plan, paths = _call_both(n, 64, 64, seed)
        assert not torch.isnan(got).any()
        assert torch.equal(got, want)
    # and against float64 arithmetic, at the tolerance of the other tensor-core tests
    info = plan
    ref = torch.zeros(paths, 64, 64, dtype=torch.float64, device=DEV)
    for in0, out0, dim, npaths, first in plan.blocks_host:
        a = s.double()[:, in0:in0 + dim * npaths].reshape(-1, dim, npaths, 64)
        b = g.double()[:, out0:out0 + dim]
        ref[plan.path_gather[first:first + npaths]] += torch.einsum("nmpi,nmo->pio", a, b)
    err = float((got.double() - ref).abs().max() / ref.abs().max())
    assert err < 8e-6, f"relative error {err:.2e}"


def test_static_scratch_entry_point_rejects_oversize_requests():
    lib = _lib.lib()
    assert lib.eqt_wgrad_tc_static_capacity() == 148 * 128 * 64
    ir = Irreps("0e+1o")
    fwd, _, _, paths = tp_infos(ir, ir, ir)
    plan = MixPlan(fwd.info_M_fwd.to(DEV), [i.dim for i in ir], DEV)
    s = torch.zeros(4, plan.rows, 32, device=DEV)
    g = torch.zeros(4, plan.comps, 128, device=DEV)
    out = torch.zeros(paths, 32, 128, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    blocks = plan.structs(32, 128)
    rc = lib.eqt_wgrad_tc_static(s.data_ptr(), g.data_ptr(), out.data_ptr(), 4, plan.rows, plan.comps, 32, 128,
                                 blocks, len(blocks), status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 2 and b"limit of 64" in lib.eqt_last_error()
