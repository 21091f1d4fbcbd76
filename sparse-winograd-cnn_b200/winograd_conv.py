"""Layer wrapper WinogradConv, signature as in the reference
(ResNet-18-var/winograd_conv.py:15-28): a (16, in_channel, out_channel) Winograd-domain weight,
optionally multiplied by a pruning mask, applied to a transformed input."""
import math as _math

import torch

from winograd2x2_conv.winograd2x2_conv import winograd2x2_conv

__all__ = ["WinogradConv", "WinogradConvLayer", "default_W_init"]


def default_W_init(shape, generator=None, device=None):
    """tf.contrib.layers.variance_scaling_initializer(factor=2*9/32), the reference default
    (winograd_conv.py:18-19): truncated normal, mode FAN_IN.  TensorFlow takes fan_in of a
    3-D shape (16, Cin, Cout) as 16*Cin and widens the stddev by 1/0.8796 to undo the
    truncation at two sigma."""
    fan_in = shape[0] * shape[1]
    std = _math.sqrt(1.3 * (2.0 * 9.0 / 32.0) / fan_in)
    w = torch.empty(shape, dtype=torch.float32, device=device)
    torch.nn.init.trunc_normal_(w, mean=0.0, std=std, a=-2 * std, b=2 * std, generator=generator)
    return w


class WinogradConvLayer(torch.nn.Module):
    """Owns the variable `W` that the reference creates with tf.get_variable('W', [16, Cin, Cout])."""

    def __init__(self, in_channel, out_channel, mask=None, W_init=None, device=None):
        super().__init__()
        shape = (16, in_channel, out_channel)
        w = W_init(shape) if W_init is not None else default_W_init(shape, device=device)
        self.W = torch.nn.Parameter(torch.as_tensor(w, dtype=torch.float32, device=device).contiguous())
        if mask is not None:
            self.register_buffer("mask", torch.as_tensor(mask, dtype=torch.float32, device=device).contiguous())
        else:
            self.mask = None

    def forward(self, x, out_hw=None, data_format="NHWC", math="fp32"):
        W = self.W if self.mask is None else self.W * self.mask
        return winograd2x2_conv(x, W, out_hw=out_hw, data_format=data_format, math=math)


_layers = {}


def WinogradConv(x, in_channel, out_channel, mask=None, W_init=None, name=None, **kw):
    """Functional form with the reference's argument order.  tensorpack's @layer_register puts
    the variable in a scope named by the layer; here `name` keys a process-wide table of
    WinogradConvLayer modules (a fresh anonymous layer when name is None)."""
    layer = _layers.get(name) if name is not None else None
    if layer is None:
        layer = WinogradConvLayer(in_channel, out_channel, mask=mask, W_init=W_init, device=x.device)
        if name is not None:
            _layers[name] = layer
    return layer(x, **kw)
