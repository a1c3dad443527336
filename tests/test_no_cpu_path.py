"""The product path has no CPU fallback: CPU tensors are refused with a clear error (no GPU needed)."""
import pytest
import torch

from equitorch_b200 import _lib
from equitorch_b200 import nn as enn
from equitorch_b200.ops import irrep_ops


def test_irrep_ops_refuse_cpu_tensors():
    x = torch.randn(3, 4, 8)
    with pytest.raises(_lib.EqtError):
        irrep_ops.irrep_scale(x, torch.randn(2, 8), torch.tensor([0, 1, 1, 1]), irrep_ops.SHARED)
    with pytest.raises(_lib.EqtError):
        irrep_ops.irrep_dot(x, x, torch.tensor([0, 1, 4]))


def test_layers_refuse_cpu_tensors():
    with pytest.raises(_lib.EqtError):
        enn.Gate("0e+1o")(torch.randn(3, 4, 8), torch.randn(3, 2, 8))
    with pytest.raises(_lib.EqtError):
        enn.LayerRMSNorm("0e+1o", 8)(torch.randn(3, 4, 8))
    with pytest.raises(_lib.EqtError):
        enn.BatchRMSNorm("0e+1o", 8)(torch.randn(3, 4, 8))


def test_shape_checks_come_before_the_device_check():
    with pytest.raises(ValueError):
        enn.LayerRMSNorm("0e+1o", 8)(torch.randn(3, 5, 8))
    with pytest.raises(ValueError):
        enn.Norm("0e+1o")(torch.randn(3, 5, 8))
