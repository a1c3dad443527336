"""Equivariant linear layers: ``SO3Linear``, ``IrrepWiseLinear``, ``IrrepsLinear``, ``SO2Linear``.

Constructor arguments, attribute names, weight shapes and forward signatures are those of
``equitorch/nn/linears.py`` (SO3Linear :26-212, IrrepWiseLinear :215-301, IrrepsLinear :303-411,
SO2Linear :413-571), so state dicts and call sites carry over.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from ..irreps import check_irreps
from ..tables import irreps_info, irreps_linear_infos, so2_linear_infos, tp_infos
from ._base import _WeightedTableModule
from .functional.linears import irrep_wise_linear, irreps_linear, so3_linear_uu, so3_linear_uv
from .functional.sparse_product import sparse_mul, sparse_vecmat
from .init import initialize_linear, initialize_so3_so2_linear


class SO3Linear(_WeightedTableModule):
    r"""Tensor product of channelled features with a channel-less second operand
    (typically spherical harmonics of an edge direction).

    ``feature_mode='uv'``: input1 ``(N, irreps_in1.dim, channels_in)``, input2 ``(N, irreps_in2.dim)``,
    weight ``(num_paths, channels_in, channels_out)`` -> ``(N, irreps_out.dim, channels_out)``.
    ``feature_mode='uu'``: weight ``(num_paths, channels)``, channels are not mixed.
    A weight with a leading batch dimension is applied per sample.  ``path_norm`` divides each
    path by the square root of the number of paths into its output irrep; ``channel_norm``
    (``'uv'`` only) divides by ``sqrt(channels_in)``.
    """
    _table_attrs = ("tp_info_forward", "tp_info_backward1", "tp_info_backward2")

    def __init__(self, irreps_in1, irreps_in2, irreps_out, channels_in=None, channels_out=None,
                 internal_weights=True, feature_mode="uu", path_norm=True, channel_norm=False, path=None):
        super().__init__()
        self.irreps_in1 = check_irreps(irreps_in1)
        self.irreps_in2 = check_irreps(irreps_in2)
        self.irreps_out = check_irreps(irreps_out)
        self.irreps_in1_dim, self.irreps_in2_dim, self.irreps_out_dim = (
            self.irreps_in1.dim, self.irreps_in2.dim, self.irreps_out.dim)
        assert not internal_weights or (channels_in is not None and channels_out is not None)
        if feature_mode not in ("uv", "uu"):
            raise ValueError(f'Feature_mode should be in ["uv", "uu"], got {feature_mode}.')
        self.channels_in, self.channels_out = channels_in, channels_out
        self.feature_mode = feature_mode
        self.path_norm = path_norm
        self.channel_norm = channel_norm and feature_mode == "uv"
        fan_in = channels_in if feature_mode == "uv" else 1
        (self.tp_info_forward, self.tp_info_backward1, self.tp_info_backward2, self.num_paths) = tp_infos(
            self.irreps_out, self.irreps_in1, self.irreps_in2, path=path, path_norm=path_norm,
            channel_norm=self.channel_norm, channel_scale=fan_in ** (-0.5) if fan_in else 1.0)
        shape = (self.num_paths, channels_in, channels_out) if feature_mode == "uv" else (self.num_paths, channels_out)
        self._setup_weight(shape, internal_weights,
                           lambda w: initialize_so3_so2_linear(w, feature_mode, channel_normed=self.channel_norm))

    def forward(self, input1: Tensor, input2: Tensor, weight: Optional[Tensor] = None) -> Tensor:
        assert input1.shape[-2] == self.irreps_in1_dim, \
            f"Input1 spherical dim mismatch: expected {self.irreps_in1_dim}, got {input1.shape[-2]}"
        assert input2.shape[-1] == self.irreps_in2_dim, \
            f"Input2 spherical dim mismatch: expected {self.irreps_in2_dim}, got {input2.shape[-1]}"
        assert input2.ndim == input1.ndim - 1, \
            f"Input2 should have one less dimension than Input1. Got input1 ndim={input1.ndim}, input2 ndim={input2.ndim}"
        assert self.channels_in is None or input1.shape[-1] == self.channels_in, \
            f"Input1 channel dim mismatch: expected {self.channels_in}, got {input1.shape[-1]}"
        weight = self._resolve_weight(weight)
        fn = so3_linear_uu if self.feature_mode == "uu" else so3_linear_uv
        return fn(input1, input2, weight, self.tp_info_forward, self.tp_info_backward1, self.tp_info_backward2)

    def __repr__(self):
        ch = (f"channels={self.channels_in}" if self.feature_mode == "uu"
              else f"channels_in={self.channels_in}, channels_out={self.channels_out}")
        return (f"{type(self).__name__}(irreps_in1={self.irreps_in1.short_repr()}, "
                f"irreps_in2={self.irreps_in2.short_repr()}, irreps_out={self.irreps_out.short_repr()}, {ch}, "
                f"feature_mode={self.feature_mode}, path_norm={self.path_norm}, channel_norm={self.channel_norm}, "
                f"internal_weights={self.internal_weights}, num_paths={self.num_paths})")


class IrrepWiseLinear(_WeightedTableModule):
    """One ``channels_in x channels_out`` matrix per irrep of ``irreps`` applied to all its
    components: ``(N, irreps.dim, channels_in) -> (N, irreps.dim, channels_out)``."""
    _table_attrs = ("irreps_info",)

    def __init__(self, irreps, channels_in, channels_out, internal_weights=True, channel_norm: bool = False):
        super().__init__()
        self.irreps = check_irreps(irreps)
        self.irreps_dim = self.irreps.dim
        self.channels_in, self.channels_out = channels_in, channels_out
        self.irreps_info = irreps_info(self.irreps)
        self.channel_norm = channel_norm
        self.num_paths = len(self.irreps)
        self._setup_weight((self.num_paths, channels_in, channels_out), internal_weights,
                           lambda w: initialize_linear(w, channel_normed=channel_norm))

    def forward(self, input: Tensor, weight: Optional[Tensor] = None) -> Tensor:
        assert input.shape[-2] == self.irreps_dim, \
            f"Input spherical dim mismatch: expected {self.irreps_dim}, got {input.shape[-2]}"
        assert input.shape[-1] == self.channels_in, \
            f"Input channel dim mismatch: expected {self.channels_in}, got {input.shape[-1]}"
        out = irrep_wise_linear(input, self._resolve_weight(weight), self.irreps_info)
        return out / (self.channels_in ** 0.5) if self.channel_norm else out

    def __repr__(self):
        return (f"{type(self).__name__}(irreps={self.irreps.short_repr()}, channels_in={self.channels_in}, "
                f"channels_out={self.channels_out}, channel_norm={self.channel_norm}, "
                f"internal_weights={self.internal_weights})")


class IrrepsLinear(_WeightedTableModule):
    """Channel mixing between every (input irrep, output irrep) pair of equal degree and parity:
    ``(N, irreps_in.dim, channels_in) -> (N, irreps_out.dim, channels_out)``.

    As in the reference constructor (``equitorch/nn/linears.py:369-370``) the fifth positional
    argument handed to the table builder under ``channel_norm`` is ``channels_in`` itself.
    """
    _table_attrs = ("forward_info", "backward_info")

    def __init__(self, irreps_in, irreps_out, channels_in, channels_out, internal_weights=True,
                 path_norm=True, channel_norm=False, path=None):
        super().__init__()
        self.irreps_in, self.irreps_out = check_irreps(irreps_in), check_irreps(irreps_out)
        self.irreps_in_dim, self.irreps_out_dim = self.irreps_in.dim, self.irreps_out.dim
        self.channels_in, self.channels_out = channels_in, channels_out
        self.channel_norm, self.path_norm = channel_norm, path_norm
        self.forward_info, self.backward_info, self.num_paths = irreps_linear_infos(
            self.irreps_out, self.irreps_in, path, path_norm, channel_norm, channels_in)
        self._setup_weight((self.num_paths, channels_in, channels_out), internal_weights,
                           lambda w: initialize_linear(w, channel_normed=channel_norm))

    def forward(self, input: Tensor, weight: Optional[Tensor] = None) -> Tensor:
        assert input.shape[-2] == self.irreps_in_dim, \
            f"Input spherical dim mismatch: expected {self.irreps_in_dim}, got {input.shape[-2]}"
        assert input.shape[-1] == self.channels_in, \
            f"Input channel dim mismatch: expected {self.channels_in}, got {input.shape[-1]}"
        return irreps_linear(input, self._resolve_weight(weight), self.forward_info, self.backward_info)

    def __repr__(self):
        return (f"{type(self).__name__}(irreps_in={self.irreps_in.short_repr()}, "
                f"irreps_out={self.irreps_out.short_repr()}, channels_in={self.channels_in}, "
                f"channels_out={self.channels_out}, path_norm={self.path_norm}, channel_norm={self.channel_norm}, "
                f"internal_weights={self.internal_weights}, num_paths={self.num_paths})")


class SO2Linear(_WeightedTableModule):
    """SO(2)-equivariant linear map on features expressed in an edge-aligned frame: components of
    equal ``|m|`` mix through 2x2 rotation-like blocks.  ``'uv'``: weight ``(num_weights, Cin, Cout)``;
    ``'uu'``: weight ``(num_weights, C)``."""
    _table_attrs = ("info_forward", "info_backward1", "info_backward2")

    def __init__(self, irreps_in, irreps_out, channels_in=None, channels_out=None, internal_weights=True,
                 feature_mode="uu", path_norm=True, channel_norm=False, path=None):
        super().__init__()
        self.irreps_in, self.irreps_out = check_irreps(irreps_in), check_irreps(irreps_out)
        assert not internal_weights or (channels_in is not None and channels_out is not None)
        if feature_mode not in ("uv", "uu"):
            raise ValueError(f'Feature_mode should be in ["uv", "uu"], got {feature_mode}.')
        self.channels_in, self.channels_out = channels_in, channels_out
        self.feature_mode, self.path_norm = feature_mode, path_norm
        self.channel_norm = channel_norm and feature_mode == "uv"
        scale = channels_in ** (-0.5) if self.channel_norm else 1.0
        (self.info_forward, self.info_backward1, self.info_backward2, self.num_weights) = so2_linear_infos(
            self.irreps_out, self.irreps_in, path=path, path_norm=path_norm,
            channel_norm=self.channel_norm, channel_scale=scale)
        shape = (self.num_weights, channels_in, channels_out) if feature_mode == "uv" else (self.num_weights, channels_out)
        self._setup_weight(shape, internal_weights,
                           lambda w: initialize_so3_so2_linear(w, feature_mode, channel_normed=self.channel_norm))

    def forward(self, input: Tensor, weight: Optional[Tensor] = None) -> Tensor:
        assert input.shape[-2] == self.irreps_in.dim, \
            f"Input spherical dim mismatch: expected {self.irreps_in.dim}, got {input.shape[-2]}"
        assert self.channels_in is None or input.shape[-1] == self.channels_in, \
            f"Input channel dim mismatch: expected {self.channels_in}, got {input.shape[-1]}"
        fn = sparse_mul if self.feature_mode == "uu" else sparse_vecmat
        return fn(input, self._resolve_weight(weight), self.info_forward, self.info_backward1, self.info_backward2)

    def __repr__(self):
        ch = (f"channels={self.channels_in}" if self.feature_mode == "uu"
              else f"channels_in={self.channels_in}, channels_out={self.channels_out}")
        return (f"{type(self).__name__}(irreps_in={self.irreps_in.short_repr()}, "
                f"irreps_out={self.irreps_out.short_repr()}, {ch}, feature_mode={self.feature_mode}, "
                f"path_norm={self.path_norm}, channel_norm={self.channel_norm}, "
                f"internal_weights={self.internal_weights}, num_weights={self.num_weights})")
