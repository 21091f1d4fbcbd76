"""Drop-in for the reference module of the same path (winograd2x2_cublas/winograd2x2_imTrans/
winograd2x2_imTrans.py:13-33): same function names and tensor shapes, on torch CUDA tensors.

    winograd2x2_imTrans(I)        I (B,H,W,C) -> (16,B,nH,nW,C); differentiable
    winograd2x2_imTrans_grad(g)   the gradient op on its own: (16,B,nH,nW,C) -> (B,2nH,2nW,C)

The reference registers the gradient with TensorFlow (`@ops.RegisterGradient`, :29-33); here the
same pairing is a torch.autograd.Function.  `data_format="NCHW"` is an extension; the default is
the reference's NHWC.
"""
import torch

from wg2x2 import ops as _ops


class _ImTrans(torch.autograd.Function):
    @staticmethod
    def forward(ctx, I, relu, data_format):
        I = I.contiguous()
        V = _ops.imtrans_fwd(I, relu=relu, layout=data_format)
        if data_format == "NHWC":
            ctx.hw = (I.shape[1], I.shape[2])
        else:
            ctx.hw = (I.shape[2], I.shape[3])
        ctx.data_format = data_format
        ctx.relu = relu
        if relu:
            ctx.save_for_backward(V)
        return V

    @staticmethod
    def backward(ctx, grad):
        V = ctx.saved_tensors[0] if ctx.relu else None
        H, W = ctx.hw
        return _ops.imtrans_bwd(grad.contiguous(), H, W, V_relu=V, layout=ctx.data_format), None, None


def winograd2x2_imTrans(I, data_format="NHWC"):
    return _ImTrans.apply(I, False, data_format)


def winograd2x2_imTrans_relu(I, data_format="NHWC"):
    """Transform followed by the Winograd-domain ReLU in one kernel (what the layer wrapper
    computes with nl=relu); the backward pass applies the ReLU mask inside the gather."""
    return _ImTrans.apply(I, True, data_format)


def winograd2x2_imTrans_grad(grad, data_format="NHWC"):
    # like the reference op, the image size is taken as 2nH x 2nW
    # (winograd2x2_imTrans_grad_op.cc:45-46)
    _, _, nH, nW, _ = grad.shape
    return _ops.imtrans_bwd(grad.contiguous(), 2 * nH, 2 * nW, layout=data_format)
