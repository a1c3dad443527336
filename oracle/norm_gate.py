"""ORACLE (test infrastructure, never imported by the product path).

CPU restatement of the reference's gate, norm and RMS-normalisation functions in plain PyTorch (dense
per-irrep slices, autograd for the gradients).  Follows

* ``gating``                      equitorch/nn/functional/activations.py:9-36 and the module logic of
  ``Gate.forward``                equitorch/nn/activations.py:95-155
* ``squared_norm`` / ``norm`` / ``channel_mean_squared_norm`` / ``batch_mean_squared_norm``
                                  equitorch/nn/functional/norm.py:14-276
* ``batch_rms_norm`` / ``layer_rms_norm``   equitorch/nn/functional/normalization.py:8-160

``dims`` is the list of irrep dimensions ``[2l + 1, ...]`` (multiplicity-expanded); features are
``(N, sum(dims), C)``.  Pinned against outputs of the reference itself
(tests/golden/norm_gate.pt.gz, made by tests/golden/make_golden_norm_gate.py).
"""
from __future__ import annotations

from typing import Callable, List, Optional

import torch
from torch import Tensor


def _blocks(dims: List[int]):
    start = 0
    for d in dims:
        yield start, start + d
        start += d


def gate(x: Tensor, g: Optional[Tensor], dims: List[int], activation: Optional[Callable] = None,
         irrep_wise: bool = True) -> Tensor:
    """``Gate.forward``: separate gates (N|shared, K, C) / (N, 1, C), or gates concatenated after the features."""
    d, k = sum(dims), len(dims)
    if g is None:
        x, g = x[..., :d, :], x[..., d:d + k, :]
    if not irrep_wise:
        g = g.reshape(-1, 1, x.shape[-1])
        return x * (activation(g) if activation else g)
    g = g.reshape(-1, k, x.shape[-1]) if g.numel() > k * x.shape[-1] else g.reshape(k, x.shape[-1])
    if activation:
        g = activation(g)
    return torch.cat([x[..., a:b, :] * g[..., n:n + 1, :] for n, (a, b) in enumerate(_blocks(dims))], dim=-2)


def squared_norm(x: Tensor, dims: List[int], scaled: bool = True) -> Tensor:
    out = torch.stack([x[..., a:b, :].pow(2).sum(-2) for a, b in _blocks(dims)], dim=-2)
    if scaled:
        out = out / torch.tensor(dims, dtype=x.dtype).unsqueeze(-1)
    return out


def norm(x: Tensor, dims: List[int], scaled: bool = True) -> Tensor:
    """sqrt of the unscaled squared norm, times ``dim^-1/2`` if scaled; zero gradient at a zero block."""
    sq = squared_norm(x, dims, scaled=False)
    safe = torch.where(sq > 0, sq, torch.ones_like(sq))
    out = torch.where(sq > 0, safe.sqrt(), torch.zeros_like(sq))
    if scaled:
        out = out * torch.tensor(dims, dtype=x.dtype).rsqrt().unsqueeze(-1)
    return out


def channel_mean_squared_norm(x: Tensor, dims: List[int], scaled: bool = True) -> Tensor:
    return squared_norm(x, dims, scaled).mean(-1)


def batch_mean_squared_norm(x: Tensor, dims: List[int], scaled: bool = True) -> Tensor:
    return squared_norm(x, dims, scaled).mean(0)


def _scale_blocks(x: Tensor, s: Tensor, dims: List[int]) -> Tensor:
    """x[..., block k, :] * s[..., k, :] (s broadcast over the block's components)."""
    return torch.cat([x[..., a:b, :] * s[..., n:n + 1, :] for n, (a, b) in enumerate(_blocks(dims))], dim=-2)


def batch_rms_norm(x: Tensor, running: Tensor, dims: List[int], weight: Optional[Tensor] = None, scaled: bool = True,
                   training: bool = False, momentum: float = 0.1, eps: float = 1e-5):
    """Returns (output, new running statistic)."""
    if training:
        stat = squared_norm(x, dims, scaled).mean(0)
        running = torch.lerp(running, stat.detach(), momentum)
    else:
        stat = running
    s = torch.rsqrt(stat + eps)
    if weight is not None:
        s = weight * s
    return _scale_blocks(x, s, dims), running


def layer_rms_norm(x: Tensor, dims: List[int], weight: Optional[Tensor] = None, scaled: bool = True,
                   eps: float = 1e-5) -> Tensor:
    r = torch.rsqrt(channel_mean_squared_norm(x, dims, scaled) + eps).unsqueeze(-1)     # (N, K, 1)
    out = _scale_blocks(x, r, dims)
    if weight is not None:
        out = _scale_blocks(out, weight, dims)
    return out
