"""Uniform weight initialisers (``equitorch/nn/init.py:3-119``): bound ``sqrt(3 / fan_in) * gain``,
or ``sqrt(3) * gain`` when the layer already divides by ``sqrt(fan_in)`` (channel norm) or mixes
no channels."""
import torch


def _uniform(weight, fan_in, gain, channel_normed):
    bound = (3.0 ** 0.5) * gain if (channel_normed or fan_in is None) else (3.0 / fan_in) ** 0.5 * gain
    torch.nn.init.uniform_(weight, -bound, bound)


def initialize_tensor_product(weight, feature_mode, gain=1, channel_normed=False):
    if feature_mode == "uvw":
        _uniform(weight, weight.shape[-2] * weight.shape[-3], gain, channel_normed)
    elif feature_mode == "uuu":
        _uniform(weight, None, gain, channel_normed)
    else:
        raise ValueError(f"Unknown feature_mode '{feature_mode}' for initialize_tensor_product")


def initialize_so3_so2_linear(weight, feature_mode, gain=1, channel_normed=False):
    if feature_mode == "uv":
        _uniform(weight, weight.shape[-2], gain, channel_normed)
    elif feature_mode == "uu":
        _uniform(weight, None, gain, channel_normed)
    else:
        raise ValueError(f"Unknown feature_mode '{feature_mode}' for initialize_so3_so2_linear")


def initialize_linear(weight, gain=1, channel_normed=False):
    _uniform(weight, weight.shape[-2], gain, channel_normed)
