"""Torch-facing calls into the C ABI: device memory and streams come from PyTorch, the
arithmetic is entirely in libwinograd2x2_b200.so."""
import torch

from . import _lib
from ._lib import MATH_FP32, MATH_TF32, NCHW, NHWC, lib

_LAYOUTS = {"NHWC": NHWC, "NCHW": NCHW, NHWC: NHWC, NCHW: NCHW}
_MATHS = {"fp32": MATH_FP32, "tf32": MATH_TF32, MATH_FP32: MATH_FP32, MATH_TF32: MATH_TF32}


def _chk(t, name):
    if not (isinstance(t, torch.Tensor) and t.is_cuda and t.dtype == torch.float32 and t.is_contiguous()):
        raise TypeError("%s must be a contiguous float32 CUDA tensor" % name)
    return t


def _chk_shape(t, shape, name):
    """Optional tensor `t` must be a contiguous float32 CUDA tensor of exactly `shape`."""
    if t is None:
        return None
    _chk(t, name)
    if tuple(t.shape) != tuple(shape):
        raise ValueError("%s has shape %s, expected %s" % (name, tuple(t.shape), tuple(shape)))
    return t


def _chk_prepared(prepared, C, K):
    """`prepared` comes from prepare_weights for exactly this (C, K): the kernels build their TMA maps over it
    from C and K alone, so a buffer made for other sizes would be read past its end."""
    if not (isinstance(prepared, torch.Tensor) and prepared.is_cuda and prepared.dtype == torch.uint8):
        raise TypeError("prepared must be the buffer returned by prepare_weights")
    ck = getattr(prepared, "_wg_ck", None)
    if ck is not None and ck != (C, K):
        raise ValueError("prepared weights are for (C, K) = %s, the call has %s" % (ck, (C, K)))
    if prepared.numel() < lib.wg2x2_prepared_weights_bytes(C, K):
        raise ValueError("prepared weight buffer too small for C=%d K=%d" % (C, K))
    return prepared


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _ptr(t):
    return None if t is None else t.data_ptr()


def _img_dims(x, layout):
    if layout == NHWC:
        B, H, W, C = x.shape
    else:
        B, C, H, W = x.shape
    return B, H, W, C


def _img_shape(B, H, W, C, layout):
    return (B, H, W, C) if layout == NHWC else (B, C, H, W)


def _workspace(nbytes, device):
    return torch.empty(max(int(nbytes), 1), dtype=torch.uint8, device=device) if nbytes else None


def imtrans_fwd(x, relu=False, layout="NHWC", out=None, in_scale=None, in_shift=None):
    """x (B,H,W,C) or (B,C,H,W) -> V (16,B,nH,nW,C); in_scale/in_shift (C,) apply x*scale+shift to the pixels first."""
    layout = _LAYOUTS[layout]
    _chk(x, "x")
    B, H, W, C = _img_dims(x, layout)
    V = out if out is not None else torch.empty((16, B, (H + 1) // 2, (W + 1) // 2, C), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        if in_scale is not None:
            _chk(in_scale, "in_scale"); _chk(in_shift, "in_shift")
            _lib.check(lib.wg2x2_imtrans_fwd_affine(_ptr(x), _ptr(in_scale), _ptr(in_shift), _ptr(V), B, H, W, C, layout,
                                                    int(bool(relu)), _stream()), "wg2x2_imtrans_fwd_affine")
        else:
            _lib.check(lib.wg2x2_imtrans_fwd(_ptr(x), _ptr(V), B, H, W, C, layout, int(bool(relu)), _stream()), "wg2x2_imtrans_fwd")
    return V


def imtrans_bwd(dV, H, W, V_relu=None, layout="NHWC"):
    """dV (16,B,nH,nW,C) -> dX; V_relu, if given, applies the ReLU mask V>0 first."""
    layout = _LAYOUTS[layout]
    _chk(dV, "dV")
    _, B, nH, nW, C = dV.shape
    if (H + 1) // 2 != nH or (W + 1) // 2 != nW:
        raise ValueError("H, W do not match the tile grid of dV")
    if V_relu is not None:
        _chk(V_relu, "V_relu")
    dX = torch.empty(_img_shape(B, H, W, C, layout), dtype=torch.float32, device=dV.device)
    with torch.cuda.device(dV.device):
        _lib.check(lib.wg2x2_imtrans_bwd(_ptr(dV), _ptr(V_relu), _ptr(dX), B, H, W, C, layout, _stream()), "wg2x2_imtrans_bwd")
    return dX


def conv_fwd(V, Wt, out_h=None, out_w=None, layout="NHWC", math="fp32", out=None, workspace=None):
    """V (16,B,nH,nW,C), Wt (16,C,K) -> Y (B,out_h,out_w,K) / (B,K,out_h,out_w)."""
    layout, math = _LAYOUTS[layout], _MATHS[math]
    _chk(V, "V"); _chk(Wt, "Wt")
    _, B, nH, nW, C = V.shape
    K = Wt.shape[2]
    if tuple(Wt.shape) != (16, C, K):
        raise ValueError("Wt must be (16, C, K)")
    out_h = 2 * nH if out_h is None else out_h
    out_w = 2 * nW if out_w is None else out_w
    Y = out if out is not None else torch.empty(_img_shape(B, out_h, out_w, K, layout), dtype=torch.float32, device=V.device)
    nbytes = lib.wg2x2_conv_fwd_workspace_bytes(B, nH, nW, C, K, math)
    ws = workspace if workspace is not None else _workspace(nbytes, V.device)
    with torch.cuda.device(V.device):
        _lib.check(lib.wg2x2_conv_fwd(_ptr(V), _ptr(Wt), _ptr(Y), B, nH, nW, C, K, out_h, out_w, layout, math,
                                      _ptr(ws), ws.numel() if ws is not None else 0, _stream()), "wg2x2_conv_fwd")
    return Y


def prepare_weights(Wt):
    """Wt (16,C,K) -> opaque device buffer for conv_fwd_prepared (TF32 tensor-core path)."""
    _chk(Wt, "Wt")
    _, C, K = Wt.shape
    n = lib.wg2x2_prepared_weights_bytes(C, K)
    buf = torch.empty(n, dtype=torch.uint8, device=Wt.device)
    with torch.cuda.device(Wt.device):
        _lib.check(lib.wg2x2_weights_prepare(_ptr(Wt), C, K, _ptr(buf), n, _stream()), "wg2x2_weights_prepare")
    buf._wg_ck = (C, K)
    return buf


def conv_fwd_prepared(V, prepared, K, out_h=None, out_w=None, layout="NHWC", out=None, out_scale=None, out_shift=None,
                      residual=None, workspace=None, wide=True):
    """As conv_fwd(math="tf32") with weights already prepared by prepare_weights; optionally
    Y = acc*out_scale[k] + out_shift[k] + residual in the kernel's epilogue."""
    layout = _LAYOUTS[layout]
    _chk(V, "V")
    _, B, nH, nW, C = V.shape
    _chk_prepared(prepared, C, K)
    out_h = 2 * nH if out_h is None else out_h
    out_w = 2 * nW if out_w is None else out_w
    yshape = _img_shape(B, out_h, out_w, K, layout)
    Y = _chk_shape(out, yshape, "out") if out is not None else torch.empty(yshape, dtype=torch.float32, device=V.device)
    _chk_shape(out_scale, (K,), "out_scale"); _chk_shape(out_shift, (K,), "out_shift"); _chk_shape(residual, yshape, "residual")
    nws = lib.wg2x2_conv_fwd_prepared_workspace_bytes(B, nH, nW, C, K) if wide else 0
    if nws:   # many channels: products as wide GEMMs into scratch memory, then the output transform
        ws = workspace if workspace is not None and workspace.numel() >= nws else torch.empty(nws, dtype=torch.uint8, device=V.device)
        with torch.cuda.device(V.device):
            _lib.check(lib.wg2x2_conv_fwd_prepared_ws(_ptr(V), _ptr(prepared), _ptr(Y), B, nH, nW, C, K, out_h, out_w, layout,
                                                      _ptr(out_scale), _ptr(out_shift), _ptr(residual), _ptr(ws), ws.numel(),
                                                      _stream()), "wg2x2_conv_fwd_prepared_ws")
        return Y
    with torch.cuda.device(V.device):
        if out_scale is None and residual is None:
            _lib.check(lib.wg2x2_conv_fwd_prepared(_ptr(V), _ptr(prepared), _ptr(Y), B, nH, nW, C, K, out_h, out_w, layout,
                                                   _stream()), "wg2x2_conv_fwd_prepared")
        else:
            _lib.check(lib.wg2x2_conv_fwd_prepared_fused(_ptr(V), _ptr(prepared), _ptr(Y), B, nH, nW, C, K, out_h, out_w, layout,
                                                         _ptr(out_scale), _ptr(out_shift), _ptr(residual), _stream()),
                       "wg2x2_conv_fwd_prepared_fused")
    return Y


def conv_bwd(V, Wt, dY, mask=None, layout="NHWC", relu=False, math="fp32", need_dV=True, need_dW=True):
    """Gradients (dV, dW) of conv_fwd for dY (B,H,W,K) / (B,K,H,W)."""
    layout, math = _LAYOUTS[layout], _MATHS[math]
    _chk(V, "V"); _chk(Wt, "Wt"); _chk(dY, "dY")
    _, B, nH, nW, C = V.shape
    K = Wt.shape[2]
    Bd, H, W, Kd = _img_dims(dY, layout)
    if (Bd, Kd) != (B, K) or (H + 1) // 2 != nH or (W + 1) // 2 != nW:
        raise ValueError("dY does not match V / Wt")
    if mask is not None:
        _chk(mask, "mask")
    dV = torch.empty_like(V) if need_dV else None
    dW = torch.empty_like(Wt) if need_dW else None
    nbytes = lib.wg2x2_conv_bwd_workspace_bytes(B, H, W, C, K, math, int(need_dW))
    ws = _workspace(nbytes, V.device)
    with torch.cuda.device(V.device):
        _lib.check(lib.wg2x2_conv_bwd(_ptr(V), _ptr(Wt), _ptr(dY), _ptr(mask), _ptr(dV), _ptr(dW), B, H, W, C, K, layout,
                                      int(bool(relu)), math, _ptr(ws), ws.numel() if ws is not None else 0, _stream()),
                   "wg2x2_conv_bwd")
    return dV, dW


def layer_fwd(x, Wt, relu=True, layout="NHWC", math="fp32", keep_V=False, out=None, workspace=None):
    """Whole Winograd-ReLU layer X -> Y (and V when keep_V)."""
    layout, math = _LAYOUTS[layout], _MATHS[math]
    _chk(x, "x"); _chk(Wt, "Wt")
    B, H, W, C = _img_dims(x, layout)
    K = Wt.shape[2]
    if tuple(Wt.shape) != (16, C, K):
        raise ValueError("Wt must be (16, C, K)")
    Y = out if out is not None else torch.empty(_img_shape(B, H, W, K, layout), dtype=torch.float32, device=x.device)
    V = torch.empty((16, B, (H + 1) // 2, (W + 1) // 2, C), dtype=torch.float32, device=x.device) if keep_V else None
    nbytes = lib.wg2x2_layer_fwd_workspace_bytes(B, H, W, C, K, math, int(keep_V))
    ws = workspace if workspace is not None else _workspace(nbytes, x.device)
    with torch.cuda.device(x.device):
        _lib.check(lib.wg2x2_layer_fwd(_ptr(x), _ptr(Wt), _ptr(Y), _ptr(V), B, H, W, C, K, layout, int(bool(relu)), math,
                                       _ptr(ws), ws.numel() if ws is not None else 0, _stream()), "wg2x2_layer_fwd")
    return (Y, V) if keep_V else Y


def fused_supported(B, H, W, C, K, layout="NCHW"):
    return bool(lib.wg2x2_layer_fwd_fused_supported(B, H, W, C, K, _LAYOUTS[layout]))


def layer_fwd_prepared(x, prepared, K, relu=True, layout="NHWC", out=None, V_scratch=None, out_scale=None, out_shift=None,
                       residual=None, workspace=None):
    """Whole layer with prepared weights: one fused kernel where supported (V never stored), else transform +
    product through V_scratch (allocated here when not given); layers with C, K >= 256 take the wide product path
    through `workspace` (allocated here when not given; layer_fwd_prepared_workspace_bytes)."""
    layout = _LAYOUTS[layout]
    _chk(x, "x")
    B, H, W, C = _img_dims(x, layout)
    _chk_prepared(prepared, C, K)
    yshape = _img_shape(B, H, W, K, layout)
    Y = _chk_shape(out, yshape, "out") if out is not None else torch.empty(yshape, dtype=torch.float32, device=x.device)
    _chk_shape(out_scale, (K,), "out_scale"); _chk_shape(out_shift, (K,), "out_shift"); _chk_shape(residual, yshape, "residual")
    if V_scratch is not None:
        _chk_shape(V_scratch, (16, B, (H + 1) // 2, (W + 1) // 2, C), "V_scratch")
    nws = lib.wg2x2_layer_fwd_prepared_workspace_bytes(B, H, W, C, K)
    if V_scratch is None and (nws or not lib.wg2x2_layer_fwd_fused_supported(B, H, W, C, K, layout)):
        V_scratch = torch.empty((16, B, (H + 1) // 2, (W + 1) // 2, C), dtype=torch.float32, device=x.device)
    if nws and (workspace is None or workspace.numel() < nws):
        workspace = torch.empty(nws, dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(lib.wg2x2_layer_fwd_prepared_ws(_ptr(x), _ptr(prepared), _ptr(Y), _ptr(V_scratch), B, H, W, C, K, layout,
                                                   int(bool(relu)), _ptr(out_scale), _ptr(out_shift), _ptr(residual),
                                                   _ptr(workspace) if nws else None, nws, _stream()),
                   "wg2x2_layer_fwd_prepared_ws")
    return Y


def layer_fwd_prepared_workspace_bytes(B, H, W, C, K):
    return int(lib.wg2x2_layer_fwd_prepared_workspace_bytes(B, H, W, C, K))


def layer_fwd_fused(x, prepared, K, relu=True, out=None, out_scale=None, out_shift=None, residual=None,
                    in_scale=None, in_shift=None):
    """The one-kernel layer forward (NCHW); raises Wg2x2Error(UNSUPPORTED) for other shapes.  in_scale/in_shift:
    per-input-channel affine map applied to the image in front of the transform (the padding stays zero)."""
    _chk(x, "x")
    B, C, H, W = x.shape
    _chk_prepared(prepared, C, K)
    Y = _chk_shape(out, (B, K, H, W), "out") if out is not None else torch.empty((B, K, H, W), dtype=torch.float32, device=x.device)
    _chk_shape(out_scale, (K,), "out_scale"); _chk_shape(out_shift, (K,), "out_shift"); _chk_shape(residual, (B, K, H, W), "residual")
    _chk_shape(in_scale, (C,), "in_scale"); _chk_shape(in_shift, (C,), "in_shift")
    with torch.cuda.device(x.device):
        if in_scale is None and in_shift is None:
            _lib.check(lib.wg2x2_layer_fwd_fused(_ptr(x), _ptr(prepared), _ptr(Y), B, H, W, C, K, int(bool(relu)), _ptr(out_scale),
                                                 _ptr(out_shift), _ptr(residual), _stream()), "wg2x2_layer_fwd_fused")
        else:
            _lib.check(lib.wg2x2_layer_fwd_fused_affine(_ptr(x), _ptr(prepared), _ptr(Y), B, H, W, C, K, int(bool(relu)),
                                                        _ptr(in_scale), _ptr(in_shift), _ptr(out_scale), _ptr(out_shift),
                                                        _ptr(residual), _stream()), "wg2x2_layer_fwd_fused_affine")
    return Y


def maxpool3x3s2_same(x, with_relu=False, relu_scale=None, relu_shift=None):
    """3x3 / stride 2 max-pooling with TensorFlow's SAME padding of a (B,C,H,W) tensor into NCHW outputs; with_relu=True
    returns (pooled, relu(relu_scale[c] * pooled + relu_shift[c])) from the same pass (scale 1, shift 0 when not given).
    x may be contiguous (NCHW) or channels-last (e.g. the output of a channels-last convolution)."""
    B, C, H, W = x.shape
    entry, name = lib.wg2x2_maxpool3x3s2_same, "wg2x2_maxpool3x3s2_same"
    if not x.is_contiguous() and x.is_contiguous(memory_format=torch.channels_last) and x.is_cuda and x.dtype == torch.float32:
        entry, name = lib.wg2x2_maxpool3x3s2_same_nhwc_in, "wg2x2_maxpool3x3s2_same_nhwc_in"
    else:
        _chk(x, "x")
    _chk_shape(relu_scale, (C,), "relu_scale"); _chk_shape(relu_shift, (C,), "relu_shift")
    y = torch.empty((B, C, (H + 1) // 2, (W + 1) // 2), dtype=torch.float32, device=x.device)
    yr = torch.empty_like(y) if with_relu else None
    with torch.cuda.device(x.device):
        _lib.check(entry(_ptr(x), _ptr(y), _ptr(yr), _ptr(relu_scale), _ptr(relu_shift), B, C, H, W, _stream()), name)
    return (y, yr) if with_relu else y


def stem_supported(H, W):
    """Image sizes the fused 7x7/2 convolution + pool kernel takes: multiples of 4, at most 224 wide."""
    return H >= 4 and W >= 4 and H % 4 == 0 and W % 4 == 0 and W <= 224


def stem_prepare(w):
    """(64,3,7,7) stem weights -> the arrangement stem7x7s2_pool reads (TF32-rounded, in fragment order)."""
    _chk(w, "w")
    if tuple(w.shape) != (64, 3, 7, 7):
        raise ValueError("stem weights must have shape (64,3,7,7), got %s" % (tuple(w.shape),))
    wp = torch.empty(lib.wg2x2_stem_prepared_floats(), dtype=torch.float32, device=w.device)
    with torch.cuda.device(w.device):
        _lib.check(lib.wg2x2_stem_prepare(_ptr(w), _ptr(wp), _stream()), "wg2x2_stem_prepare")
    return wp


def stem7x7s2_pool(x, prepared, with_relu=False, relu_scale=None, relu_shift=None):
    """pool1(conv1(x)) of the ResNet-18-var graph in one kernel: x (B,3,H,W) -> (B,64,H/4,W/4); with_relu=True also
    returns relu(relu_scale[c] * pooled + relu_shift[c]).  `prepared` comes from stem_prepare."""
    _chk(x, "x")
    B, C, H, W = x.shape
    if C != 3:
        raise ValueError("stem input must have 3 channels, got %d" % C)
    if not stem_supported(H, W):
        raise ValueError("stem kernel needs H and W multiples of 4 and W <= 224, got %dx%d" % (H, W))
    _chk_shape(prepared, (lib.wg2x2_stem_prepared_floats(),), "prepared")
    _chk_shape(relu_scale, (64,), "relu_scale"); _chk_shape(relu_shift, (64,), "relu_shift")
    y = torch.empty((B, 64, H // 4, W // 4), dtype=torch.float32, device=x.device)
    yr = torch.empty_like(y) if with_relu else None
    with torch.cuda.device(x.device):
        _lib.check(lib.wg2x2_stem7x7s2_pool(_ptr(x), _ptr(prepared), _ptr(y), _ptr(yr), _ptr(relu_scale), _ptr(relu_shift),
                                            B, H, W, _stream()), "wg2x2_stem7x7s2_pool")
    return (y, yr) if with_relu else y


def last_device_status():
    """(status, where) of the bounded device-side waits since the last reading; synchronises the current stream.
    The tensor-core calls above do not read it themselves (that would cost a synchronisation per call): after a
    time-out their outputs are incomplete, so a caller that must know polls here after its last launch."""
    import ctypes
    where = ctypes.c_uint(0)
    st = lib.wg2x2_last_device_status(_stream(), ctypes.byref(where))
    return st, where.value
