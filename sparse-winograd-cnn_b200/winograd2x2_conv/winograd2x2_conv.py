"""Drop-in for the reference module of the same path (winograd2x2_cublas/winograd2x2_conv/
winograd2x2_conv.py:13-36): same function names and tensor shapes, on torch CUDA tensors.

    winograd2x2_conv(I, W)              I (16,B,nH,nW,C), W (16,C,K) -> (B,2nH,2nW,K); differentiable
    winograd2x2_conv_grad(i1, i2, grad) -> (grad wrt I, grad wrt W)

`math` selects the FP32 FFMA kernels ("fp32") or the tcgen05 TF32 kernels ("tf32");
`out_hw` crops the output to odd image sizes; `data_format="NCHW"` is an extension.
"""
import torch

from wg2x2 import ops as _ops


class _Conv(torch.autograd.Function):
    @staticmethod
    def forward(ctx, I, W, out_hw, data_format, math):
        I = I.contiguous()
        W = W.contiguous()
        oh, ow = out_hw if out_hw is not None else (None, None)
        Y = _ops.conv_fwd(I, W, oh, ow, layout=data_format, math=math)
        ctx.save_for_backward(I, W)
        ctx.data_format = data_format
        ctx.math = math
        return Y

    @staticmethod
    def backward(ctx, grad):
        I, W = ctx.saved_tensors
        dV, dW = _ops.conv_bwd(I, W, grad.contiguous(), layout=ctx.data_format, math=ctx.math,
                               need_dV=ctx.needs_input_grad[0], need_dW=ctx.needs_input_grad[1])
        return dV, dW, None, None, None


def winograd2x2_conv(I, W, out_hw=None, data_format="NHWC", math="fp32"):
    return _Conv.apply(I, W, out_hw, data_format, math)


def winograd2x2_conv_grad(i1, i2, grad, data_format="NHWC", math="fp32"):
    return _ops.conv_bwd(i1.contiguous(), i2.contiguous(), grad.contiguous(), layout=data_format, math=math)
