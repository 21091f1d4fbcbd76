"""Layer wrapper WinogradImTrans, signature as in the reference
(ResNet-18-var/winograd_imtrans.py:15-17): the input transform followed by a nonlinearity."""
import torch

from winograd2x2_imTrans.winograd2x2_imTrans import winograd2x2_imTrans, winograd2x2_imTrans_relu

__all__ = ["WinogradImTrans"]

_RELUS = (torch.relu, torch.nn.functional.relu)


def _identity(x):
    return x


def WinogradImTrans(x, nl=_identity, data_format="NHWC"):
    """nl(winograd2x2_imTrans(x)).  When nl is torch's ReLU the two steps run as one kernel
    (forward and backward); any other callable is applied to the transform's output."""
    if nl in _RELUS or isinstance(nl, torch.nn.ReLU):
        return winograd2x2_imTrans_relu(x, data_format=data_format)
    return nl(winograd2x2_imTrans(x, data_format=data_format))
