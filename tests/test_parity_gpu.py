"""GPU parity: every op of the C ABI against the float64 CPU oracle on the same seeded inputs.

Tolerance (FP32 FFMA path): max|a-b| / max|b| <= 1e-5; the reference tests' relative-L1 metric
is checked alongside (<= 1e-6).
"""
import ctypes
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL_FP32 = 1e-5
TOL_L1 = 1e-6

# (B, H, W, C, K): the reference's test shapes, odd sizes, ragged channel counts, tile-edge cases
SHAPES = [
    (3, 6, 6, 32, 32), (3, 6, 6, 32, 64), (3, 6, 6, 5, 7),
    (2, 7, 7, 16, 24), (1, 1, 1, 4, 4), (1, 2, 3, 3, 5), (2, 5, 8, 4, 6),
    (1, 14, 14, 64, 64), (2, 9, 13, 33, 17), (1, 66, 70, 8, 12), (5, 8, 8, 128, 96),
]


@pytest.fixture(scope="module")
def wg():
    import wg2x2
    return wg2x2


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda()


def _to_layout(a_nhwc, layout):
    return a_nhwc if layout == "NHWC" else np.ascontiguousarray(np.transpose(a_nhwc, (0, 3, 1, 2)))


def _from_layout(t, layout):
    a = t.cpu().numpy()
    return a if layout == "NHWC" else np.transpose(a, (0, 2, 3, 1))


def _check(got, want, tol=TOL_FP32, tol_l1=TOL_L1, what=""):
    from oracle.wg_oracle import max_rel, rel_l1
    assert got.shape == want.shape, what
    assert np.isfinite(got).all(), what
    e, l1 = max_rel(got, want), rel_l1(got, want)
    assert e <= tol and l1 <= tol_l1, "%s: max_rel %.3g rel_l1 %.3g" % (what, e, l1)


def _inputs(shape, seed=0):
    B, H, W, C, K = shape
    rng = np.random.default_rng(seed + 1000 * sum(shape))
    X = rng.standard_normal((B, H, W, C)).astype(np.float32)
    Wt = (0.05 * rng.standard_normal((16, C, K))).astype(np.float32)
    dY = rng.standard_normal((B, H, W, K)).astype(np.float32)
    mask = (rng.random((16, C, K)) < 0.3).astype(np.float32)
    return X, Wt, dY, mask


@pytest.mark.parametrize("layout", ["NHWC", "NCHW"])
@pytest.mark.parametrize("relu", [False, True])
@pytest.mark.parametrize("shape", SHAPES)
def test_imtrans_fwd(wg, oracle, shape, relu, layout):
    X, _, _, _ = _inputs(shape)
    V = wg.imtrans_fwd(_dev(_to_layout(X, layout)), relu=relu, layout=layout).cpu().numpy()
    _check(V, oracle.imtrans_fwd(X, relu=relu), what="imtrans_fwd")
    if relu:
        # the ReLU pattern itself must agree wherever the float64 value is clearly non-zero
        ref = oracle.imtrans_fwd(X, relu=False)
        clear = np.abs(ref) > 1e-4
        assert ((V > 0) == (ref > 0))[clear].all()


@pytest.mark.parametrize("layout", ["NHWC", "NCHW"])
@pytest.mark.parametrize("shape", SHAPES)
def test_conv_fwd_fp32(wg, oracle, shape, layout):
    B, H, W, C, K = shape
    X, Wt, _, _ = _inputs(shape)
    V = oracle.imtrans_fwd(X, relu=True, dtype=np.float32)
    for oh, ow in {(H, W), (2 * ((H + 1) // 2), 2 * ((W + 1) // 2))}:
        Y = wg.conv_fwd(_dev(V), _dev(Wt), oh, ow, layout=layout, math="fp32")
        _check(_from_layout(Y, layout), oracle.conv_fwd(V, Wt, oh, ow), what="conv_fwd %dx%d" % (oh, ow))


@pytest.mark.parametrize("layout", ["NHWC", "NCHW"])
@pytest.mark.parametrize("shape", SHAPES)
def test_layer_fwd_fp32(wg, oracle, shape, layout):
    B, H, W, C, K = shape
    X, Wt, _, _ = _inputs(shape)
    Y, V = wg.layer_fwd(_dev(_to_layout(X, layout)), _dev(Wt), relu=True, layout=layout, math="fp32", keep_V=True)
    Vo = oracle.imtrans_fwd(X, relu=True)
    _check(V.cpu().numpy(), Vo, what="layer V")
    _check(_from_layout(Y, layout), oracle.conv_fwd(Vo, Wt, H, W), what="layer Y")
    Y2 = wg.layer_fwd(_dev(_to_layout(X, layout)), _dev(Wt), relu=True, layout=layout, math="fp32")
    assert torch.equal(Y, Y2)


@pytest.mark.parametrize("layout", ["NHWC", "NCHW"])
@pytest.mark.parametrize("use_mask", [False, True])
@pytest.mark.parametrize("shape", SHAPES)
def test_conv_bwd_fp32(wg, oracle, shape, use_mask, layout):
    B, H, W, C, K = shape
    X, Wt, dY, mask = _inputs(shape)
    if use_mask:
        Wt = Wt * mask
    V = oracle.imtrans_fwd(X, relu=True, dtype=np.float32)
    dVo, dWo = oracle.conv_bwd(V, Wt, dY, mask=mask if use_mask else None)
    dV, dW = wg.conv_bwd(_dev(V), _dev(Wt), _dev(_to_layout(dY, layout)), mask=_dev(mask) if use_mask else None,
                         layout=layout)
    _check(dV.cpu().numpy(), dVo, what="dV")
    _check(dW.cpu().numpy(), dWo, what="dW")
    # relu folded into the op: dV is zero wherever V is
    dVr, _ = wg.conv_bwd(_dev(V), _dev(Wt), _dev(_to_layout(dY, layout)), layout=layout, relu=True, need_dW=False)
    _check(dVr.cpu().numpy(), dVo * (V > 0), what="dV relu")


@pytest.mark.parametrize("layout", ["NHWC", "NCHW"])
def test_conv_bwd_fp32_conv5_width(wg, oracle, layout):
    """The FP32 gradient kernels at the width of the conv5_x backward workload (C = K = 512, 7 x 7, a batch slice of 8):
    dW runs split over the tiles with the deterministic reduction pass, dV with eight channel blocks."""
    shape = (8, 7, 7, 512, 512)
    B, H, W, C, K = shape
    X, Wt, dY, mask = _inputs(shape)
    Wt = Wt * mask
    V = oracle.imtrans_fwd(X, relu=True, dtype=np.float32)
    dVo, dWo = oracle.conv_bwd(V, Wt, dY, mask=mask)
    assert wg._lib.lib.wg2x2_conv_bwd_workspace_bytes(B, H, W, C, K, 0, 1) > 0      # split-P scratch is in use
    dV, dW = wg.conv_bwd(_dev(V), _dev(Wt), _dev(_to_layout(dY, layout)), mask=_dev(mask), layout=layout, relu=True)
    _check(dV.cpu().numpy(), dVo * (V > 0), what="dV")
    _check(dW.cpu().numpy(), dWo, what="dW")
    dX = wg.imtrans_bwd(dV, H, W, layout=layout)
    _check(_from_layout(dX, layout), oracle.imtrans_bwd(dVo * (V > 0), H, W), what="dX")


@pytest.mark.parametrize("layout", ["NHWC", "NCHW"])
@pytest.mark.parametrize("use_mask", [False, True])
@pytest.mark.parametrize("shape", SHAPES)
def test_imtrans_bwd(wg, oracle, shape, use_mask, layout):
    B, H, W, C, K = shape
    X, _, _, _ = _inputs(shape)
    rng = np.random.default_rng(7)
    nH, nW = (H + 1) // 2, (W + 1) // 2
    dV = rng.standard_normal((16, B, nH, nW, C)).astype(np.float32)
    V = oracle.imtrans_fwd(X, relu=True, dtype=np.float32) if use_mask else None
    dX = wg.imtrans_bwd(_dev(dV), H, W, V_relu=_dev(V) if use_mask else None, layout=layout)
    _check(_from_layout(dX, layout), oracle.imtrans_bwd(dV, H, W, Vmask=V), what="imtrans_bwd")


# The NCHW transform kernels with four channels per lane are chosen only where their grid fills the GPU (at least
# four CTAs per SM), so these shapes are sized to select them: 128 channels per CTA in bands, 128 per CTA with the
# whole image as one band, 64 per CTA (image too wide for 128), 64 per CTA with a ragged last block.
_VEC_BWD = [(40, 13, 14, 640), (150, 7, 7, 512), (16, 27, 56, 192), (150, 13, 14, 100)]
_VEC_FWD = [(150, 7, 7, 512), (160, 5, 8, 388), (30, 13, 14, 640), (150, 13, 14, 100)]   # the first two take the 128-channel kernel


@pytest.mark.parametrize("use_mask", [False, True])
@pytest.mark.parametrize("shape", _VEC_BWD + [(3, 7, 7, 132), (2, 9, 11, 68), (1, 12, 100, 64), (2, 6, 6, 130), (150, 7, 7, 255)])
def test_imtrans_bwd_nchw_channel_vector_paths(wg, oracle, shape, use_mask):
    """The NCHW gather's 16-byte-load variants (and small shapes that fall back from them), odd sizes included; the first
    shapes with small images take the whole-image kernels (two channels per lane; one per lane for the odd channel count)."""
    B, H, W, C = shape
    rng = np.random.default_rng(23)
    nH, nW = (H + 1) // 2, (W + 1) // 2
    dV = rng.standard_normal((16, B, nH, nW, C), dtype=np.float32)
    V = rng.standard_normal((16, B, nH, nW, C), dtype=np.float32) if use_mask else None
    dX = wg.imtrans_bwd(_dev(dV), H, W, V_relu=_dev(V) if use_mask else None, layout="NCHW")
    _check(_from_layout(dX, "NCHW"), oracle.imtrans_bwd(dV, H, W, Vmask=V, dtype=np.float32), what="imtrans_bwd NCHW %s" % (shape,))


@pytest.mark.parametrize("affine", [False, True])
@pytest.mark.parametrize("shape", _VEC_FWD + [(3, 7, 7, 132), (2, 9, 11, 68), (2, 6, 6, 130)])
def test_imtrans_fwd_nchw_channel_vector_paths(wg, oracle, shape, affine):
    """The NCHW input transform's 16-byte-store variants, with and without the folded per-channel affine map and ReLU."""
    B, H, W, C = shape
    rng = np.random.default_rng(29)
    X = rng.standard_normal((B, H, W, C), dtype=np.float32)
    kw, Xo = {}, X
    if affine:
        s_in, b_in = (1 + 0.2 * rng.standard_normal(C)).astype(np.float32), (0.3 * rng.standard_normal(C)).astype(np.float32)
        kw = dict(in_scale=_dev(s_in), in_shift=_dev(b_in))
        Xo = X.astype(np.float64) * s_in + b_in
    for relu in (True, False):
        V = wg.imtrans_fwd(_dev(_to_layout(X, "NCHW")), relu=relu, layout="NCHW", **kw).cpu().numpy()
        _check(V, oracle.imtrans_fwd(Xo, relu=relu), what="imtrans_fwd NCHW %s relu=%s" % (shape, relu))


def test_exhaustive_small_sizes(wg, oracle):
    """All H, W in 1..9 for a few channel counts, forward and backward, NHWC."""
    rng = np.random.default_rng(11)
    for C, K in [(1, 1), (3, 5), (32, 8)]:
        Wt = (0.1 * rng.standard_normal((16, C, K))).astype(np.float32)
        for H in range(1, 10):
            for W in range(1, 10):
                X = rng.standard_normal((2, H, W, C)).astype(np.float32)
                dY = rng.standard_normal((2, H, W, K)).astype(np.float32)
                Y, V = wg.layer_fwd(_dev(X), _dev(Wt), relu=True, keep_V=True)
                Vo = oracle.imtrans_fwd(X, relu=True)
                _check(Y.cpu().numpy(), oracle.conv_fwd(Vo, Wt, H, W), what="Y %dx%d" % (H, W))
                dV, dW = wg.conv_bwd(V, _dev(Wt), _dev(dY), relu=True)
                dVo, dWo = oracle.conv_bwd(Vo, Wt, dY)
                _check(dW.cpu().numpy(), dWo, what="dW %dx%d" % (H, W))
                dX = wg.imtrans_bwd(dV, H, W)
                _check(dX.cpu().numpy(), oracle.imtrans_bwd(dVo, H, W, Vmask=Vo), what="dX %dx%d" % (H, W))


def test_layer_equals_direct_convolution(wg, oracle):
    """The reference tests' level-1 identity on the GPU path: with G g G^T weights and no ReLU the
    layer is a 3x3 SAME convolution (winograd2x2_imTrans_test.py:179-192)."""
    rng = np.random.default_rng(3)
    for (B, H, W, C, K) in [(3, 6, 6, 32, 32), (2, 7, 9, 8, 16)]:
        X = rng.standard_normal((B, H, W, C)).astype(np.float32)
        g = rng.standard_normal((3, 3, C, K))
        Wt = oracle.kernel_transform(g).astype(np.float32)
        Y = wg.layer_fwd(_dev(X), _dev(Wt), relu=False).cpu().numpy()
        ref = torch.nn.functional.conv2d(torch.from_numpy(X).double().permute(0, 3, 1, 2),
                                         torch.from_numpy(g).permute(3, 2, 0, 1), padding=1).permute(0, 2, 3, 1).numpy()
        _check(Y, ref, what="conv2d identity")


def test_autograd_wrappers(wg, oracle):
    """The reference-named modules and layer wrappers, forward and backward through torch.autograd."""
    from winograd_conv import WinogradConvLayer
    from winograd_imtrans import WinogradImTrans
    from winograd2x2_conv.winograd2x2_conv import winograd2x2_conv, winograd2x2_conv_grad
    from winograd2x2_imTrans.winograd2x2_imTrans import winograd2x2_imTrans, winograd2x2_imTrans_grad
    B, H, W, C, K = 2, 6, 8, 16, 24
    X, Wt, dY, mask = _inputs((B, H, W, C, K))
    x = _dev(X).requires_grad_(True)
    layer = WinogradConvLayer(C, K, mask=mask, W_init=lambda shape: torch.from_numpy(Wt)).cuda()
    y = layer(WinogradImTrans(x, torch.relu))
    assert tuple(y.shape) == (B, H, W, K)
    y.backward(_dev(dY))
    Vo = oracle.imtrans_fwd(X, relu=True)
    Wm = Wt * mask
    _check(y.detach().cpu().numpy(), oracle.conv_fwd(Vo, Wm, H, W), what="wrapper Y")
    dVo, dWo = oracle.conv_bwd(Vo, Wm, dY, mask=mask)
    _check(layer.W.grad.cpu().numpy(), dWo, what="wrapper dW")
    _check(x.grad.cpu().numpy(), oracle.imtrans_bwd(dVo, H, W, Vmask=Vo), what="wrapper dX")
    # the bare ops, with the reference's shapes
    V = winograd2x2_imTrans(_dev(X))
    assert tuple(V.shape) == (16, B, H // 2, W // 2, C)
    assert tuple(winograd2x2_conv(V, _dev(Wt)).shape) == (B, H, W, K)
    g1, g2 = winograd2x2_conv_grad(V, _dev(Wt), _dev(dY))
    assert g1.shape == V.shape and tuple(g2.shape) == (16, C, K)
    assert tuple(winograd2x2_imTrans_grad(g1).shape) == (B, H, W, C)


def test_reference_named_launchers(wg, oracle):
    """The four C++ launcher symbols with the reference's names and argument lists."""
    from wg2x2._lib import lib
    B, H, W, C, K = 3, 6, 6, 32, 64
    X, Wt, dY, _ = _inputs((B, H, W, C, K))
    nH, nW = H // 2, W // 2
    x, wt, dy = _dev(X), _dev(Wt), _dev(dY)
    V = torch.empty((16, B, nH, nW, C), device="cuda")
    P = ctypes.c_void_p
    lib._Z33Winograd2x2ImTransComputeLauncherPKfPfiiiiii(P(x.data_ptr()), P(V.data_ptr()), C, B, H, W, 1, 1)
    Y = torch.empty((B, H, W, K), device="cuda")
    tmp = torch.zeros(16 * B * nH * nW * K, device="cuda")
    ptrs = torch.zeros(80, dtype=torch.int64, device="cuda")
    lib._Z30Winograd2x2ConvComputeLauncherPKfS0_PfS1_PKxiiiiiii(P(V.data_ptr()), P(wt.data_ptr()), P(Y.data_ptr()),
                                                              P(tmp.data_ptr()), P(ptrs.data_ptr()), C, B, nH, nW, K, 1, 1)
    dV = torch.empty_like(V)
    dW = torch.empty_like(wt)
    lib._Z34Winograd2x2ConvGradComputeLauncherPKfS0_S0_PfS1_S1_Pxiiiiiii(
        P(V.data_ptr()), P(wt.data_ptr()), P(dy.data_ptr()), P(dV.data_ptr()), P(dW.data_ptr()), P(tmp.data_ptr()),
        P(ptrs.data_ptr()), C, B, H, W, K, 1, 1)
    dV_before = dV.clone()
    dX = torch.empty_like(x)
    lib._Z37Winograd2x2ImTransGradComputeLauncherPKfPfiiiiii(P(dV.data_ptr()), P(dX.data_ptr()), C, B, H, W, 1, 1)
    torch.cuda.synchronize()
    Vo = oracle.imtrans_fwd(X)
    _check(V.cpu().numpy(), Vo, what="launcher V")
    _check(Y.cpu().numpy(), oracle.conv_fwd(Vo, Wt), what="launcher Y")
    dVo, dWo = oracle.conv_bwd(Vo, Wt, dY)
    _check(dV.cpu().numpy(), dVo, what="launcher dV")
    _check(dW.cpu().numpy(), dWo, what="launcher dW")
    _check(dX.cpu().numpy(), oracle.imtrans_bwd(dVo, H, W), what="launcher dX")
    assert torch.equal(dV, dV_before), "the gradient launcher must not write its input"


def test_against_upstream_cuda_kernels(wg, oracle):
    """Oracle pin: the reference's own kernels, compiled unmodified (oracle/_ref), on this GPU."""
    so = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "libwg_ref_cuda.so")
    if not os.path.exists(so):
        pytest.skip("oracle/_ref not built (make -C oracle ref)")
    ref = ctypes.CDLL(so)
    P = ctypes.c_void_p
    for shape in [(3, 6, 6, 32, 32), (2, 8, 12, 16, 24), (4, 56, 56, 64, 64)]:
        B, H, W, C, K = shape
        X, Wt, dY, _ = _inputs(shape)
        nH, nW = H // 2, W // 2
        x, wt, dy = _dev(X), _dev(Wt), _dev(dY)
        V = torch.empty((16, B, nH, nW, C), device="cuda")
        ref.wgref_imtrans(P(x.data_ptr()), P(V.data_ptr()), C, B, H, W)
        Y = torch.empty((B, H, W, K), device="cuda")
        tmp = torch.empty(16 * B * nH * nW * K, device="cuda")
        ptrs = torch.empty(80, dtype=torch.int64, device="cuda")
        ref.wgref_conv(P(V.data_ptr()), P(wt.data_ptr()), P(Y.data_ptr()), P(tmp.data_ptr()), P(ptrs.data_ptr()), C, B, nH, nW, K)
        dV = torch.empty_like(V)
        dW = torch.empty_like(wt)
        ref.wgref_conv_grad(P(V.data_ptr()), P(wt.data_ptr()), P(dy.data_ptr()), P(dV.data_ptr()), P(dW.data_ptr()),
                            P(tmp.data_ptr()), P(ptrs.data_ptr()), C, B, H, W, K)
        dVc = dV.clone()
        dX = torch.empty_like(x)
        ref.wgref_imtrans_grad(P(dVc.data_ptr()), P(dX.data_ptr()), C, B, H, W)
        torch.cuda.synchronize()
        Vo = oracle.imtrans_fwd(X)
        _check(V.cpu().numpy(), Vo, what="upstream V vs oracle")
        _check(Y.cpu().numpy(), oracle.conv_fwd(Vo, Wt), what="upstream Y vs oracle")
        dVo, dWo = oracle.conv_bwd(Vo, Wt, dY)
        _check(dV.cpu().numpy(), dVo, what="upstream dV vs oracle")
        _check(dW.cpu().numpy(), dWo, what="upstream dW vs oracle")
        _check(dX.cpu().numpy(), oracle.imtrans_bwd(dVo, H, W), what="upstream dX vs oracle")
        # and this library against the upstream kernels directly
        _check(wg.imtrans_fwd(x).cpu().numpy(), V.cpu().numpy(), what="V vs upstream")
        _check(wg.conv_fwd(V, wt).cpu().numpy(), Y.cpu().numpy(), what="Y vs upstream")


def test_determinism_and_canaries(wg):
    """Two runs give identical bits (no atomics), and nothing is written outside the outputs."""
    from wg2x2._lib import NHWC, lib
    B, H, W, C, K = 3, 7, 9, 20, 28
    X, Wt, dY, mask = _inputs((B, H, W, C, K))
    nH, nW = (H + 1) // 2, (W + 1) // 2
    pad = 1024
    x, wt, dy = _dev(X), _dev(Wt), _dev(dY)

    def padded(n):
        buf = torch.full((n + 2 * pad,), 1234.5, device="cuda")
        return buf, buf[pad:pad + n]

    st = torch.cuda.current_stream().cuda_stream
    results = []
    for _ in range(2):
        Vb, V = padded(16 * B * nH * nW * C)
        Yb, Y = padded(B * H * W * K)
        dVb, dV = padded(V.numel())
        dWb, dW = padded(wt.numel())
        dXb, dX = padded(x.numel())
        nws = lib.wg2x2_conv_bwd_workspace_bytes(B, H, W, C, K, 0, 1)
        wsb, ws = padded((nws + 3) // 4 + 1)
        P = ctypes.c_void_p
        assert lib.wg2x2_imtrans_fwd(P(x.data_ptr()), P(V.data_ptr()), B, H, W, C, NHWC, 1, P(st)) == 0
        assert lib.wg2x2_conv_fwd(P(V.data_ptr()), P(wt.data_ptr()), P(Y.data_ptr()), B, nH, nW, C, K, H, W, NHWC, 0, None, 0, P(st)) == 0
        assert lib.wg2x2_conv_bwd(P(V.data_ptr()), P(wt.data_ptr()), P(dy.data_ptr()), None, P(dV.data_ptr()), P(dW.data_ptr()),
                                  B, H, W, C, K, NHWC, 1, 0, P(ws.data_ptr()), nws, P(st)) == 0
        assert lib.wg2x2_imtrans_bwd(P(dV.data_ptr()), None, P(dX.data_ptr()), B, H, W, C, NHWC, P(st)) == 0
        torch.cuda.synchronize()
        for buf in (Vb, Yb, dVb, dWb, dXb, wsb):
            assert (buf[:pad] == 1234.5).all() and (buf[-pad:] == 1234.5).all(), "write outside the buffer"
        results.append([t.clone() for t in (V, Y, dV, dW, dX)])
    for a, b in zip(*results):
        assert torch.equal(a, b)


@pytest.mark.parametrize("layout", ["NHWC", "NCHW"])
def test_host_pipeline_equals_resident_call(wg, oracle, layout):
    """The chunked host-buffer pipeline gives the bits of the one-shot device call, on repeated use."""
    B, H, W, C, K = 10, 14, 14, 32, 64
    X, Wt, _, _ = _inputs((B, H, W, C, K))
    xl = _to_layout(X, layout)
    want = wg.layer_fwd(_dev(xl), _dev(Wt), relu=True, layout=layout, math="tf32")
    pipe = wg.HostLayerPipeline(B, H, W, C, K, layout=layout, math="tf32", chunks=4)
    xh = torch.from_numpy(np.ascontiguousarray(xl)).pin_memory()
    yh = torch.empty(tuple(want.shape)).pin_memory()
    wt = _dev(Wt)
    for _ in range(3):
        yh.zero_()
        pipe(xh, wt, yh)
        torch.cuda.current_stream().synchronize()
        assert torch.equal(yh, want.cpu())
    _check(_from_layout(yh, layout), oracle.conv_fwd(oracle.imtrans_fwd(X, relu=True), Wt, H, W), tol=5e-3, tol_l1=5e-3,
           what="pipeline vs oracle")
    # back-to-back submissions with different inputs and two output buffers: every result must be its own batch's
    xs = [xh, (xh * 0.5 + 1.0).pin_memory(), (xh * -1.0).pin_memory()]
    ys = [torch.empty_like(yh).pin_memory() for _ in xs]
    evs = [pipe.submit(xi, wt, yi) for xi, yi in zip(xs, ys)]
    for e in evs:
        e.synchronize()
    for xi, yi in zip(xs, ys):
        assert torch.equal(yi, wg.layer_fwd(xi.cuda(), wt, relu=True, layout=layout, math="tf32").cpu())
