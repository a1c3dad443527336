"""Shared scaffolding of the two-step tensor-product Functions.

Every tensor-product flavour of the reference is "CG contraction of the two inputs into an
intermediate with one row per (output component, path)" followed by "weight step from the
intermediate to the output" (``equitorch/nn/functional/tensor_products.py:9-172``,
``linears.py:16-492``).  The Functions return the intermediate as a second output so that its
gradient can flow when somebody differentiates a backward pass; when nobody does, autograd
hands ``None`` for it (``set_materialize_grads(False)``) and the corresponding terms are
skipped instead of being computed on zeros.
"""
from __future__ import annotations

import torch
from torch import Tensor


def save_for_tp_backward(ctx, input1: Tensor, input2: Tensor, weight: Tensor, inter: Tensor, infos) -> None:
    g1, g2, gw = input1.requires_grad, input2.requires_grad, weight.requires_grad
    ctx.weight_ndim = weight.ndim
    ctx.inter_shape = inter.shape if inter is not None else None
    ctx.save_for_backward(input1 if g2 else None, input2 if g1 else None,
                          weight if (g1 or g2) else None, inter if gw else None)
    ctx.tp_info = infos
    ctx.set_materialize_grads(False)


def add(a, b):
    if a is None:
        return b
    if b is None:
        return a
    return a + b


def expand_like_inter(ctx, grad_inter):
    if grad_inter is None:
        return None
    return torch.broadcast_to(grad_inter, ctx.inter_shape)
