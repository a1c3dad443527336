"""Common plumbing of the weighted equivariant layers: optional internal weight, reshaping of
externally supplied (possibly per-sample) weights, and moving the index tables together with the
module (they are plain attributes, not buffers, exactly as in the reference:
``equitorch/nn/tensor_products.py:173-178``)."""
from __future__ import annotations

import math
from typing import Optional, Sequence

import torch
from torch import Tensor, nn
from torch.nn import Parameter


class _WeightedTableModule(nn.Module):
    _table_attrs: Sequence[str] = ()

    def _setup_weight(self, weight_shape, internal_weights: bool, initializer) -> None:
        self.weight_shape = tuple(weight_shape)
        self.weight_numel = math.prod(self.weight_shape)
        self.internal_weights = internal_weights
        if internal_weights:
            self.weight = Parameter(torch.empty(*self.weight_shape))
            initializer(self.weight)
        else:
            self.weight = None

    def _resolve_weight(self, weight: Optional[Tensor]) -> Tensor:
        if self.internal_weights:
            assert weight is None, "Do not pass the weight when self.internal_weights is True."
            return self.weight
        assert weight is not None, "Please pass the weight when self.internal_weights is False."
        if weight.numel() > self.weight_numel:
            return weight.view(-1, *self.weight_shape)
        return weight.view(*self.weight_shape)

    def _apply(self, fn, *args, **kwargs):
        module = super()._apply(fn, *args, **kwargs)
        for name in self._table_attrs:
            setattr(module, name, getattr(self, name)._apply(fn))
        return module
