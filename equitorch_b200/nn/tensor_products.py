"""``TensorProduct`` and ``TensorDot`` modules (``equitorch/nn/tensor_products.py:19-269``)."""
from __future__ import annotations

from typing import Optional

from torch import Tensor, nn

from ..irreps import check_irreps
from ..tables import irreps_info, tp_infos
from ._base import _WeightedTableModule
from .functional.tensor_products import tensor_dot_uu, tensor_dot_uv, tensor_product_uuu, tensor_product_uvw
from .init import initialize_tensor_product


class TensorProduct(_WeightedTableModule):
    """Weighted Clebsch-Gordan tensor product of two channelled feature tensors.

    ``'uvw'``: ``(N, D1, C1) x (N, D2, C2)`` with weight ``(num_paths, C1, C2, Cout)`` -> ``(N, Dout, Cout)``.
    ``'uuu'``: equal channel counts, weight ``(num_paths, C)``, channels are not mixed.
    """
    _table_attrs = ("tp_info_forward", "tp_info_backward1", "tp_info_backward2")

    def __init__(self, irreps_in1, irreps_in2, irreps_out, channels_in1=None, channels_in2=None,
                 channels_out=None, internal_weights=True, feature_mode="uuu", path_norm=True,
                 channel_norm=False, path=None):
        super().__init__()
        self.irreps_in1, self.irreps_in2, self.irreps_out = (check_irreps(irreps_in1), check_irreps(irreps_in2),
                                                             check_irreps(irreps_out))
        self.irreps_in1_dim, self.irreps_in2_dim, self.irreps_out_dim = (
            self.irreps_in1.dim, self.irreps_in2.dim, self.irreps_out.dim)
        assert not internal_weights or None not in (channels_in1, channels_in2, channels_out)
        if feature_mode not in ("uvw", "uuu"):
            raise ValueError(f'Feature_mode should be in ["uvw", "uuu"], got {feature_mode}.')
        self.channels_in1, self.channels_in2, self.channels_out = channels_in1, channels_in2, channels_out
        self.feature_mode, self.path_norm = feature_mode, path_norm
        self.channel_norm = channel_norm and feature_mode == "uvw"
        fan_in = channels_in1 * channels_in2 if feature_mode == "uvw" else 1
        (self.tp_info_forward, self.tp_info_backward1, self.tp_info_backward2, self.num_paths) = tp_infos(
            self.irreps_out, self.irreps_in1, self.irreps_in2, path=path, path_norm=path_norm,
            channel_norm=self.channel_norm, channel_scale=fan_in ** (-0.5))
        shape = ((self.num_paths, channels_in1, channels_in2, channels_out) if feature_mode == "uvw"
                 else (self.num_paths, channels_out))
        self._setup_weight(shape, internal_weights,
                           lambda w: initialize_tensor_product(w, feature_mode, channel_normed=self.channel_norm))

    def forward(self, input1: Tensor, input2: Tensor, weight: Optional[Tensor] = None) -> Tensor:
        assert input1.shape[-2] == self.irreps_in1_dim, \
            f"Input1 spherical dim mismatch: expected {self.irreps_in1_dim}, got {input1.shape[-2]}"
        assert input2.shape[-2] == self.irreps_in2_dim, \
            f"Input2 spherical dim mismatch: expected {self.irreps_in2_dim}, got {input2.shape[-2]}"
        if self.feature_mode == "uvw":
            assert self.channels_in1 is None or input1.shape[-1] == self.channels_in1, "Input1 channel dim mismatch"
            assert self.channels_in2 is None or input2.shape[-1] == self.channels_in2, "Input2 channel dim mismatch"
        else:
            assert input1.shape[-1] == input2.shape[-1], "Input channel dims must match in 'uuu' mode"
        weight = self._resolve_weight(weight)
        fn = tensor_product_uuu if self.feature_mode == "uuu" else tensor_product_uvw
        return fn(input1, input2, weight, self.tp_info_forward, self.tp_info_backward1, self.tp_info_backward2)

    def __repr__(self):
        ch = (f"channels={self.channels_in1}" if self.feature_mode == "uuu" else
              f"channels_in1={self.channels_in1}, channels_in2={self.channels_in2}, channels_out={self.channels_out}")
        return (f"{type(self).__name__}(irreps_in1={self.irreps_in1.short_repr()}, "
                f"irreps_in2={self.irreps_in2.short_repr()}, irreps_out={self.irreps_out.short_repr()}, {ch}, "
                f"feature_mode={self.feature_mode}, path_norm={self.path_norm}, channel_norm={self.channel_norm}, "
                f"internal_weights={self.internal_weights}, num_paths={self.num_paths})")


class TensorDot(nn.Module):
    """Irrep-wise dot product ``(N, D, C) x (N, D, C) -> (N, len(irreps), C)`` (``'uu'``)."""

    def __init__(self, irreps, feature_mode, scaled=False):
        super().__init__()
        self.irreps = check_irreps(irreps)
        self.irreps_dim = self.irreps.dim
        self.irreps_info = irreps_info(self.irreps)
        assert feature_mode in ["uv", "uu"]
        self.feature_mode, self.scaled = feature_mode, scaled

    def forward(self, input1: Tensor, input2: Tensor) -> Tensor:
        assert input1.shape[-2] == self.irreps_dim and input2.shape[-2] == self.irreps_dim, "spherical dim mismatch"
        if self.feature_mode == "uu":
            assert input1.shape[-1] == input2.shape[-1], "Input channel dims must match in 'uu' mode"
            return tensor_dot_uu(input1, input2, self.irreps_info, self.scaled)
        return tensor_dot_uv(input1, input2, self.irreps_info, self.scaled)

    def _apply(self, fn, *args, **kwargs):
        module = super()._apply(fn, *args, **kwargs)
        module.irreps_info = self.irreps_info._apply(fn)
        return module

    def __repr__(self):
        return f"{type(self).__name__}(irreps={self.irreps.short_repr()}, feature_mode={self.feature_mode}, scaled={self.scaled})"
