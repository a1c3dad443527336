"""Module API of the tensor-product path (same class names as ``equitorch.nn``)."""
from . import functional  # noqa: F401
from .angular import SinCos
from .graph_layers import SO3LinearGraph
from .linears import IrrepsLinear, IrrepWiseLinear, SO2Linear, SO3Linear
from .sphericals import SphericalHarmonics
from .tensor_products import TensorDot, TensorProduct
from .wigner_d import DenseWignerRotation, SparseWignerRotation, WignerD

__all__ = ["SinCos", "IrrepsLinear", "IrrepWiseLinear", "SO2Linear", "SO3Linear", "SO3LinearGraph", "SphericalHarmonics",
           "TensorDot", "TensorProduct", "DenseWignerRotation", "SparseWignerRotation", "WignerD", "functional"]
