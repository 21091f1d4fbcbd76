"""ctypes doorway to the CPU oracle (oracle/wg_oracle.c) plus an independent numpy twin.

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the benchmark's
CPU-baseline / reference arm.  The product package never imports this module.

All arrays use the reference's layouts: X (B,H,W,C); V (16,B,nH,nW,C); W (16,C,K);
Y (B,H,W,K).  `dtype` picks the float32 or float64 build of the C code.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def build(force=False):
    """Compile oracle/libwg_oracle.so (make -C oracle oracle)."""
    so = os.path.join(_HERE, "libwg_oracle.so")
    src = os.path.join(_HERE, "wg_oracle.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "oracle"], stdout=subprocess.DEVNULL)
        for o in ("wg_oracle_f32.o", "wg_oracle_f64.o"):
            p = os.path.join(_HERE, o)
            if os.path.exists(p):
                os.remove(p)
    return so


def lib():
    global _LIB
    if _LIB is None:
        so = os.path.join(_HERE, "libwg_oracle.so")
        if not os.path.exists(so):
            build()
        _LIB = ctypes.CDLL(so)
    return _LIB


def set_threads(n=None):
    """Use n OpenMP threads (default: every core this process may run on); returns the count in effect."""
    n = len(os.sched_getaffinity(0)) if n is None else int(n)
    lib().wgo_set_threads(n)
    return int(lib().wgo_get_max_threads())


def _suf(dtype):
    dtype = np.dtype(dtype)
    if dtype == np.float32:
        return "_f32", ctypes.c_float
    if dtype == np.float64:
        return "_f64", ctypes.c_double
    raise TypeError(dtype)


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p) if a is not None else None


def _c(a, dtype):
    return None if a is None else np.ascontiguousarray(a, dtype=dtype)


def imtrans_fwd(X, relu=False, dtype=np.float64):
    """V = [relu](B^T d B); see wgo_imtrans_fwd in wg_oracle.c."""
    suf, _ = _suf(dtype)
    X = _c(X, dtype)
    B, H, W, C = X.shape
    nH, nW = (H + 1) // 2, (W + 1) // 2
    V = np.empty((16, B, nH, nW, C), dtype=dtype)
    getattr(lib(), "wgo_imtrans_fwd" + suf)(_p(X), _p(V), B, H, W, C, int(bool(relu)))
    return V


def conv_fwd(V, Wt, out_h=None, out_w=None, dtype=np.float64):
    """Y = A^T (V_t . W_t) A, cropped to (out_h, out_w); see wgo_conv_fwd."""
    suf, _ = _suf(dtype)
    V, Wt = _c(V, dtype), _c(Wt, dtype)
    _, B, nH, nW, C = V.shape
    K = Wt.shape[2]
    assert Wt.shape == (16, C, K)
    out_h = 2 * nH if out_h is None else out_h
    out_w = 2 * nW if out_w is None else out_w
    Y = np.empty((B, out_h, out_w, K), dtype=dtype)
    scratch = np.empty(16 * B * nH * nW * K, dtype=dtype)
    getattr(lib(), "wgo_conv_fwd" + suf)(_p(V), _p(Wt), _p(Y), _p(scratch), B, nH, nW, C, K, out_h, out_w)
    return Y


def conv_bwd(V, Wt, dY, mask=None, dtype=np.float64):
    """(dV, dW) of conv_fwd; dY is (B,H,W,K) with H in {2nH-1, 2nH}; see wgo_conv_bwd."""
    suf, _ = _suf(dtype)
    V, Wt, dY, mask = _c(V, dtype), _c(Wt, dtype), _c(dY, dtype), _c(mask, dtype)
    _, B, nH, nW, C = V.shape
    K = Wt.shape[2]
    Bd, H, W, Kd = dY.shape
    assert (Bd, Kd) == (B, K) and (H + 1) // 2 == nH and (W + 1) // 2 == nW
    dV = np.empty_like(V)
    dW = np.empty_like(Wt)
    scratch = np.empty(16 * B * nH * nW * K, dtype=dtype)
    getattr(lib(), "wgo_conv_bwd" + suf)(_p(V), _p(Wt), _p(dY), _p(mask), _p(dV), _p(dW), _p(scratch),
                                        B, H, W, C, K)
    return dV, dW


def imtrans_bwd(dV, H, W, Vmask=None, dtype=np.float64):
    """dX of imtrans_fwd (with the ReLU mask V>0 when Vmask is given); see wgo_imtrans_bwd."""
    suf, _ = _suf(dtype)
    dV, Vmask = _c(dV, dtype), _c(Vmask, dtype)
    _, B, nH, nW, C = dV.shape
    assert (H + 1) // 2 == nH and (W + 1) // 2 == nW
    dX = np.empty((B, H, W, C), dtype=dtype)
    getattr(lib(), "wgo_imtrans_bwd" + suf)(_p(dV), _p(Vmask), _p(dX), B, H, W, C)
    return dX


def layer_fwd(X, Wt, relu=True, dtype=np.float32, bufs=None):
    """Whole layer X -> Y (transform, ReLU, 16 GEMMs, output transform); see wgo_layer_fwd.

    `bufs` may carry preallocated (Y, Vbuf, scratch) so that a timing loop allocates nothing."""
    suf, _ = _suf(dtype)
    X, Wt = _c(X, dtype), _c(Wt, dtype)
    B, H, W, C = X.shape
    K = Wt.shape[2]
    P = B * ((H + 1) // 2) * ((W + 1) // 2)
    if bufs is None:
        bufs = (np.empty((B, H, W, K), dtype=dtype), np.empty(16 * P * C, dtype=dtype),
                np.empty(16 * P * K, dtype=dtype))
    Y, Vbuf, scratch = bufs
    getattr(lib(), "wgo_layer_fwd" + suf)(_p(X), _p(Wt), _p(Y), _p(Vbuf), _p(scratch), B, H, W, C, K,
                                         int(bool(relu)))
    return Y


# ---------------------------------------------------------------------------------------
# numpy twin: the same math from the transform matrices with einsum, written independently
# of the C loops so that each checks the other.
# ---------------------------------------------------------------------------------------
BT = np.array([[1, 0, -1, 0], [0, 1, 1, 0], [0, -1, 1, 0], [0, 1, 0, -1]], dtype=np.float64)
AT = np.array([[1, 1, 1, 0], [0, 1, -1, -1]], dtype=np.float64)
# G of F(2x2,3x3), as expanded term by term in kernel_transform_num
# (winograd2x2_cublas/winograd2x2_imTrans/winograd2x2_imTrans_test.py:8-25).
G = np.array([[1, 0, 0], [0.5, 0.5, 0.5], [0.5, -0.5, 0.5], [0, 0, 1]], dtype=np.float64)


def kernel_transform(g_hwck):
    """Spatial 3x3 kernel (3,3,C,K) -> Winograd-domain weights (16,C,K) = G g G^T."""
    w = np.einsum("iy,yxck,jx->ijck", G, np.asarray(g_hwck, np.float64), G)
    return w.reshape(16, *w.shape[2:])


def np_patches(X):
    B, H, W, C = X.shape
    nH, nW = (H + 1) // 2, (W + 1) // 2
    Xp = np.zeros((B, 2 * nH + 2, 2 * nW + 2, C), dtype=np.float64)
    Xp[:, 1:H + 1, 1:W + 1] = X
    d = np.empty((B, nH, nW, 4, 4, C), dtype=np.float64)
    for y in range(4):
        for x in range(4):
            d[:, :, :, y, x] = Xp[:, y:y + 2 * nH:2, x:x + 2 * nW:2]
    return d


def np_imtrans_fwd(X, relu=False):
    d = np_patches(np.asarray(X, np.float64))
    V = np.einsum("iy,bhwyxc,jx->ijbhwc", BT, d, BT)
    V = V.reshape(16, *V.shape[2:])
    return np.maximum(V, 0) if relu else V


def np_conv_fwd(V, Wt, out_h=None, out_w=None):
    V = np.asarray(V, np.float64)
    _, B, nH, nW, C = V.shape
    M = np.einsum("tbhwc,tck->tbhwk", V, np.asarray(Wt, np.float64)).reshape(4, 4, B, nH, nW, -1)
    Y = np.einsum("ai,ijbhwk,ej->bhawek", AT, M, AT).reshape(B, 2 * nH, 2 * nW, -1)
    return Y[:, :out_h, :out_w]


def rel_l1(a, b):
    """The reference tests' error metric, sum|a-b| / (sum|a| + sum|b|)
    (winograd2x2_cublas/winograd2x2_imTrans/winograd2x2_imTrans_test.py:192)."""
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return float(np.abs(a - b).sum() / (np.abs(a).sum() + np.abs(b).sum() + 1e-300))


def max_rel(a, b):
    """max|a-b| / max|b| : the tolerance metric used by the parity tests."""
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return float(np.abs(a - b).max() / (np.abs(b).max() + 1e-300))
