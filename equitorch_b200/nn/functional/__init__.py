"""Functional API (same names as ``equitorch.nn.functional`` for the tensor-product path)."""
from .activations import gating
from .angular import sincos
from .linears import (irrep_wise_linear, irreps_linear, so2_linear_uu, so2_linear_uv, so3_linear_uu, so3_linear_uv,
                      tensor_product_1uu, tensor_product_1vu, tensor_product_u1u, tensor_product_u1v,
                      tensor_product_uu1, tensor_product_vu1)
from .norm import batch_mean_squared_norm, channel_mean_squared_norm, norm, squared_norm
from .normalization import batch_rms_norm, layer_rms_norm
from .sparse_product import (sparse_inner, sparse_mat_t_vec, sparse_mul, sparse_outer, sparse_scavec, sparse_vecmat,
                             sparse_vecsca)
from .sparse_scale import sparse_scale
from .sphericals import spherical_harmonics
from .tensor_products import tensor_dot_uu, tensor_dot_uv, tensor_product_uuu, tensor_product_uvw
from .wigner_d import dense_wigner_rotation, sparse_wigner_rotation, wigner_d_matrix

__all__ = [n for n in dir() if not n.startswith("_")]
