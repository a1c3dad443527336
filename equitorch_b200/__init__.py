"""B200-native implementation of Equitorch's sparse Clebsch-Gordan tensor-product path."""
from .irreps import Irrep, Irreps, check_irreps, has_path  # noqa: F401

__version__ = "0.1.0"
