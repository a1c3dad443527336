"""Module API of the tensor-product path (same class names as ``equitorch.nn``)."""
from . import functional  # noqa: F401
from .activations import Gate
from .cutoffs import CosineCutoff, MollifierCutoff, PolynomialCutoff
from .radials import BesselBasis
from .angular import SinCos
from .graph_layers import SO3LinearGraph
from .linears import IrrepsLinear, IrrepWiseLinear, SO2Linear, SO3Linear
from .norm import MeanSquaredNorm, Norm, SquaredNorm
from .normalization import BatchRMSNorm, LayerRMSNorm
from .sphericals import SphericalHarmonics
from .tensor_products import TensorDot, TensorProduct
from .wigner_d import DenseWignerRotation, SparseWignerRotation, WignerD

__all__ = ["Gate", "MeanSquaredNorm", "Norm", "SquaredNorm", "BatchRMSNorm", "LayerRMSNorm", "SinCos", "IrrepsLinear", "IrrepWiseLinear", "SO2Linear", "SO3Linear", "SO3LinearGraph", "SphericalHarmonics",
           "TensorDot", "TensorProduct", "DenseWignerRotation", "SparseWignerRotation", "WignerD", "functional"]
