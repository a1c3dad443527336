"""The C-ABI library loads on a machine without a GPU and exports every function the header declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    names = []
    for fn in sorted(os.listdir(os.path.join(ROOT, "include"))):
        if not fn.endswith(".h"):
            continue
        text = open(os.path.join(ROOT, "include", fn)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names += re.findall(r"\b(eqt_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


def test_header_declares_entry_points():
    names = declared_functions()
    for must in ("eqt_sparse_product", "eqt_sh_forward", "eqt_sh_backward", "eqt_segment_sum", "eqt_gather_rows"):
        assert must in names


def test_library_exports_every_declared_symbol():
    from equitorch_b200 import _lib
    from equitorch_b200.csrc.build import build
    build()
    handle = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared_functions():
        assert hasattr(handle, name), f"{name} is declared in include/ but not exported"
    assert set(_lib.SIGNATURES) == set(declared_functions())
    assert _lib.lib().eqt_version() >= 100


def test_bad_arguments_are_reported_not_crashed():
    from equitorch_b200 import _lib
    rc = _lib.lib().eqt_sparse_product(None, None)
    assert rc == 1 and b"NULL" in _lib.lib().eqt_last_error()
    args = _lib.ProductArgs(op=99, dtype=0, n=-1)
    assert _lib.lib().eqt_sparse_product(ctypes.byref(args), None) == 1


def test_cpu_tensors_are_rejected_loudly():
    import torch
    from equitorch_b200.ops.batched_sparse_dense_op import indexed_mul_scale_gather
    with pytest.raises(_import_error()):
        indexed_mul_scale_gather(torch.zeros(2, 3, 4), torch.zeros(2, 3, 4))


def _import_error():
    from equitorch_b200._lib import EqtError
    return EqtError
