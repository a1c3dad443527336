"""Per-irrep streaming operators (operator layer over ``eqt_irrep_scale`` / ``eqt_irrep_dot``)."""
from __future__ import annotations

import torch
from torch import Tensor

from .. import _lib

#: layout of the scale operand of :func:`irrep_scale`
PER_SAMPLE_CHANNEL, SHARED, PER_SAMPLE = 0, 1, 2


def _check(x: Tensor) -> None:
    if x.ndim != 3:
        raise ValueError(f"features must be (N, components, channels), got {tuple(x.shape)}")
    if x.dtype not in (torch.float32, torch.float64, torch.bfloat16):
        raise TypeError(f"float32, float64 or bfloat16 features expected, got {x.dtype}")


def irrep_scale(x: Tensor, s: Tensor, irrep_index: Tensor, mode: int) -> Tensor:
    """``out[n, i, c] = x[n, i, c] * s(n, irrep_index[i], c)`` with ``s`` of shape (N, K, C) (mode 0), (K, C)
    (mode 1) or (N, K) (mode 2)."""
    _check(x)
    dev = _lib.require_cuda(x, s, irrep_index)
    x, s = x.contiguous(), s.to(x.dtype).contiguous()
    n, d, c = x.shape
    k = s.shape[-2] if mode != PER_SAMPLE else s.shape[-1]
    want = {PER_SAMPLE_CHANNEL: (n, k, c), SHARED: (k, c), PER_SAMPLE: (n, k)}[mode]
    if tuple(s.shape) != want:
        raise ValueError(f"scale operand of mode {mode} must be {want}, got {tuple(s.shape)}")
    out = torch.empty_like(x)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().eqt_irrep_scale(x.data_ptr(), s.data_ptr(), out.data_ptr(), irrep_index.data_ptr(), n, d, k, c,
                                              mode, _lib.DTYPE_CODE[x.dtype], _lib.stream_ptr(dev)), "eqt_irrep_scale")
    return out


def irrep_dot(a: Tensor, b: Tensor, irrep_seg: Tensor) -> Tensor:
    """``out[n, k, c] = sum_{i in irrep k} a[n, i, c] * b[n, i, c]`` -> (N, num_irreps, C)."""
    _check(a)
    dev = _lib.require_cuda(a, b, irrep_seg)
    if a.shape != b.shape or a.dtype != b.dtype:
        raise ValueError("operands of irrep_dot must have the same shape and dtype")
    same = a is b
    a = a.contiguous()
    b = a if same else b.contiguous()
    n, d, c = a.shape
    k = irrep_seg.numel() - 1
    out = torch.empty(n, k, c, dtype=a.dtype, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().eqt_irrep_dot(a.data_ptr(), b.data_ptr(), out.data_ptr(), irrep_seg.data_ptr(), n, d, k, c,
                                            _lib.DTYPE_CODE[a.dtype], _lib.stream_ptr(dev)), "eqt_irrep_dot")
    return out


def layer_rms_supported(x: Tensor, num_irreps: int) -> bool:
    """Whether the fused LayerRMSNorm kernels take this input."""
    if not (x.is_cuda and x.ndim == 3 and x.dtype in (torch.float32, torch.float64)):
        return False
    v = 4 if x.dtype == torch.float32 else 2
    c = x.shape[-1]
    return num_irreps <= 16 and x.shape[1] <= 1024 and c % v == 0 and 32 % (c // v) == 0


def layer_rms_forward(x: Tensor, weight, irrep_seg: Tensor, scaled: bool, eps: float):
    """Returns (out, rsigma (N, K)); ``weight`` (K, C) or None."""
    dev = _lib.require_cuda(x, weight, irrep_seg)
    x = x.contiguous()
    w = None if weight is None else weight.to(x.dtype).contiguous()
    n, d, c = x.shape
    k = irrep_seg.numel() - 1
    out = torch.empty_like(x)
    rsigma = torch.empty(n, k, dtype=x.dtype, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().eqt_layer_rms_forward(x.data_ptr(), _lib.ptr(w), out.data_ptr(), rsigma.data_ptr(),
                                                    irrep_seg.data_ptr(), n, d, k, c, int(scaled), float(eps),
                                                    _lib.DTYPE_CODE[x.dtype], _lib.stream_ptr(dev)), "eqt_layer_rms_forward")
    return out, rsigma


def layer_rms_backward(x: Tensor, grad_out: Tensor, weight, rsigma: Tensor, irrep_seg: Tensor, scaled: bool,
                       need_weight_grad: bool):
    """Returns (grad_x, grad_weight or None)."""
    dev = _lib.require_cuda(x, grad_out, weight, rsigma, irrep_seg)
    x, grad_out = x.contiguous(), grad_out.to(x.dtype).contiguous()
    w = None if weight is None else weight.to(x.dtype).contiguous()
    n, d, c = x.shape
    k = irrep_seg.numel() - 1
    gx = torch.empty_like(x)
    partial = None
    if need_weight_grad:
        partial = torch.empty(_lib.lib().eqt_layer_rms_num_partials(n), k, c, dtype=x.dtype, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().eqt_layer_rms_backward(x.data_ptr(), grad_out.data_ptr(), _lib.ptr(w), rsigma.data_ptr(),
                                                     gx.data_ptr(), _lib.ptr(partial), irrep_seg.data_ptr(), n, d, k, c,
                                                     int(scaled), _lib.DTYPE_CODE[x.dtype], _lib.stream_ptr(dev)),
                   "eqt_layer_rms_backward")
    return gx, (None if partial is None else partial.sum(dim=0))
