"""GPU parity of the tcgen05 TF32 path against the float64 oracle.  Tolerance 5e-3 on
max|a-b| / max|b| (TF32 keeps 10 mantissa bits per operand; accumulation is fp32 in TMEM)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL_TF32 = 5e-3

SHAPES = [  # B, H, W, C, K
    (2, 14, 14, 64, 64),      # one partial m-tile
    (4, 56, 56, 64, 64),      # the small 56x56 layer
    (3, 6, 6, 32, 32), (3, 6, 6, 32, 64),
    (2, 7, 7, 64, 128),       # odd size, two channel blocks
    (1, 28, 28, 128, 96),     # K not a multiple of 64
    (2, 9, 13, 36, 20),       # C not a multiple of 32, K < 64
    (3, 14, 14, 256, 256),    # conv4_x shape
    (1, 30, 34, 8, 8),
]


@pytest.fixture(scope="module")
def wg():
    import wg2x2
    return wg2x2


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda()


def _inputs(shape, density=1.0):
    B, H, W, C, K = shape
    rng = np.random.default_rng(sum(shape))
    X = rng.standard_normal((B, H, W, C)).astype(np.float32)
    Wt = (0.05 * rng.standard_normal((16, C, K))).astype(np.float32)
    if density < 1.0:
        Wt *= (rng.random((16, C, K)) < density)
    return X, Wt.astype(np.float32)


def _status_ok(wg):
    st, where = wg.last_device_status()
    assert st == 0, "device-side wait gave up at 0x%x" % where


@pytest.mark.parametrize("layout", ["NHWC", "NCHW"])
@pytest.mark.parametrize("shape", SHAPES)
def test_conv_fwd_tf32(wg, oracle, shape, layout):
    B, H, W, C, K = shape
    X, Wt = _inputs(shape)
    V = oracle.imtrans_fwd(X, relu=True, dtype=np.float32)
    Y = wg.conv_fwd(_dev(V), _dev(Wt), H, W, layout=layout, math="tf32")
    _status_ok(wg)
    got = Y.cpu().numpy()
    if layout == "NCHW":
        got = np.transpose(got, (0, 2, 3, 1))
    want = oracle.conv_fwd(V, Wt, H, W)
    assert np.isfinite(got).all()
    err = oracle.max_rel(got, want)
    assert err <= TOL_TF32, "max_rel %.3g" % err
    assert oracle.rel_l1(got, want) <= TOL_TF32


def test_tf32_matches_fp32_path_closely(wg, oracle):
    """Same inputs through both math modes: they differ only by TF32 rounding."""
    shape = (4, 56, 56, 64, 64)
    X, Wt = _inputs(shape)
    x, wt = _dev(X), _dev(Wt)
    y32 = wg.layer_fwd(x, wt, relu=True, math="fp32")
    ytf = wg.layer_fwd(x, wt, relu=True, math="tf32")
    _status_ok(wg)
    assert oracle.max_rel(ytf.cpu().numpy(), y32.cpu().numpy()) <= TOL_TF32
    assert not torch.equal(y32, ytf)   # the tensor-core path really ran


def test_pruned_weights_and_block_skipping(wg, oracle):
    """Unstructured mask (density 0.3, the conv4_x benchmark shape) and a block-structured mask whose
    all-zero 64x32 blocks are skipped by the kernel: both must equal the dense arithmetic."""
    shape = (2, 14, 14, 256, 256)
    B, H, W, C, K = shape
    X, Wt = _inputs(shape, density=0.3)
    V = oracle.imtrans_fwd(X, relu=True, dtype=np.float32)
    Y = wg.conv_fwd(_dev(V), _dev(Wt), H, W, math="tf32").cpu().numpy()
    assert oracle.max_rel(Y, oracle.conv_fwd(V, Wt, H, W)) <= TOL_TF32
    rng = np.random.default_rng(9)
    blocks = rng.random((16, C // 32, K // 64)) < 0.4
    blocks[:, 0, :] |= rng.random((16, K // 64)) < 0.5    # some first chunks empty as well
    Wb = Wt * np.repeat(np.repeat(blocks, 32, axis=1), 64, axis=2)
    prepared = wg.prepare_weights(_dev(Wb))
    Yb = wg.conv_fwd_prepared(_dev(V), prepared, K, H, W, wide=False).cpu().numpy()   # the row-walk kernel, which skips blocks
    _status_ok(wg)
    assert oracle.max_rel(Yb, oracle.conv_fwd(V, Wb, H, W)) <= TOL_TF32
    # the wide path (products as GEMMs with 256 output channels per unit) consults the same map
    Yw = wg.conv_fwd_prepared(_dev(V), prepared, K, H, W, wide=True).cpu().numpy()
    _status_ok(wg)
    assert oracle.max_rel(Yw, oracle.conv_fwd(V, Wb, H, W)) <= TOL_TF32
    # all-zero weights: the output must be exactly zero, not stale accumulator contents
    Yz = wg.conv_fwd(_dev(V), _dev(np.zeros_like(Wt)), H, W, math="tf32")
    assert float(Yz.abs().max()) == 0.0
    Yz = wg.conv_fwd_prepared(_dev(V), wg.prepare_weights(_dev(np.zeros_like(Wt))), K, H, W, wide=False)
    assert float(Yz.abs().max()) == 0.0


@pytest.mark.parametrize("shape", [(2, 14, 14, 256, 256), (3, 8, 8, 320, 192), (2, 7, 7, 128, 64)])
def test_block_skipping_in_the_gradient_products(wg, oracle, shape):
    """dV on the tensor cores skips contraction chunks whose weight blocks are all zero (the map is rebuilt from the
    weights on every call): block-structured, unstructured and all-zero weights must equal the dense arithmetic."""
    B, H, W, C, K = shape
    X, Wt = _inputs(shape, density=0.5)
    rng = np.random.default_rng(5 + sum(shape))
    dY = rng.standard_normal((B, H, W, K)).astype(np.float32)
    V = oracle.imtrans_fwd(X, relu=True, dtype=np.float32)
    blocks = rng.random((16, (C + 31) // 32, (K + 63) // 64)) < 0.4
    blocks[:, :, 0] |= rng.random((16, (C + 31) // 32)) < 0.5
    Wb = Wt * np.repeat(np.repeat(blocks, 32, axis=1), 64, axis=2)[:, :C, :K]
    for Wc in (Wb, Wt, np.zeros_like(Wt)):
        dV, _ = wg.conv_bwd(_dev(V), _dev(Wc), _dev(dY), math="tf32", need_dW=False)
        _status_ok(wg)
        want = oracle.conv_bwd(V, Wc, dY)[0]
        if not Wc.any():
            assert float(dV.abs().max()) == 0.0
        else:
            assert oracle.max_rel(dV.cpu().numpy(), want) <= TOL_TF32


@pytest.mark.parametrize("shape", [(2, 16, 16, 128, 128), (1, 28, 28, 256, 64), (3, 8, 12, 96, 192)])
def test_block_skipping_in_the_one_kernel_layer(wg, oracle, shape):
    """The one-kernel layer's MMA issuers leave out the weight tiles the zero-block map marks empty."""
    B, H, W, C, K = shape
    X, Wt = _inputs(shape, density=0.5)
    rng = np.random.default_rng(7 + sum(shape))
    blocks = rng.random((16, (C + 31) // 32, (K + 63) // 64)) < 0.4
    blocks[:, 0, :] |= rng.random((16, (K + 63) // 64)) < 0.5
    Wb = Wt * np.repeat(np.repeat(blocks, 32, axis=1), 64, axis=2)[:, :C, :K]
    Xc = _dev(np.ascontiguousarray(np.transpose(X, (0, 3, 1, 2))))
    V = oracle.imtrans_fwd(X, relu=True)
    for Wc in (Wb, np.zeros_like(Wt)):
        Y = wg.layer_fwd_fused(Xc, wg.prepare_weights(_dev(Wc)), K, relu=True)
        _status_ok(wg)
        if not Wc.any():
            assert float(Y.abs().max()) == 0.0
        else:
            assert oracle.max_rel(np.transpose(Y.cpu().numpy(), (0, 2, 3, 1)), oracle.conv_fwd(V, Wc, H, W)) <= TOL_TF32


def test_prepared_weights_reused(wg, oracle):
    shape = (2, 28, 28, 128, 128)
    B, H, W, C, K = shape
    X, Wt = _inputs(shape)
    prepared = wg.prepare_weights(_dev(Wt))
    V = wg.imtrans_fwd(_dev(X), relu=True)
    Y1 = wg.conv_fwd_prepared(V, prepared, K, H, W)
    Y2 = wg.conv_fwd_prepared(V, prepared, K, H, W)
    assert torch.equal(Y1, Y2)
    want = oracle.conv_fwd(oracle.imtrans_fwd(X, relu=True), Wt, H, W)
    assert oracle.max_rel(Y1.cpu().numpy(), want) <= TOL_TF32


def test_unsupported_shape_reports(wg):
    """C % 4 != 0 cannot be described to TMA: the TF32 mode says so instead of falling back."""
    V = torch.zeros((16, 1, 2, 2, 6), device="cuda")
    Wt = torch.zeros((16, 6, 8), device="cuda")
    with pytest.raises(wg.Wg2x2Error) as e:
        wg.conv_fwd(V, Wt, math="tf32")
    assert e.value.status == -5


BWD_SHAPES = [  # B, H, W, C, K
    (2, 14, 14, 64, 64), (3, 6, 6, 32, 64), (2, 7, 7, 64, 128), (1, 28, 28, 128, 96), (2, 9, 13, 36, 20),
    (3, 14, 14, 256, 256), (4, 56, 56, 64, 64), (16, 7, 7, 512, 512), (2, 8, 8, 320, 288),
]


@pytest.mark.parametrize("layout", ["NHWC", "NCHW"])
@pytest.mark.parametrize("shape", BWD_SHAPES)
def test_conv_bwd_tf32(wg, oracle, shape, layout):
    """dV (with the ReLU mask) and masked dW from the tensor-core gradient kernels."""
    B, H, W, C, K = shape
    X, Wt = _inputs(shape)
    rng = np.random.default_rng(1 + sum(shape))
    dY = rng.standard_normal((B, H, W, K)).astype(np.float32)
    mask = (rng.random((16, C, K)) < 0.3).astype(np.float32)
    Wm = Wt * mask
    V = oracle.imtrans_fwd(X, relu=True, dtype=np.float32)
    dVo, dWo = oracle.conv_bwd(V, Wm, dY, mask=mask)
    dyl = dY if layout == "NHWC" else np.ascontiguousarray(np.transpose(dY, (0, 3, 1, 2)))
    dV, dW = wg.conv_bwd(_dev(V), _dev(Wm), _dev(dyl), mask=_dev(mask), layout=layout, relu=True, math="tf32")
    _status_ok(wg)
    dV, dW = dV.cpu().numpy(), dW.cpu().numpy()
    assert np.isfinite(dV).all() and np.isfinite(dW).all()
    e_dv = oracle.max_rel(dV, dVo * (V > 0))
    e_dw = oracle.max_rel(dW, dWo)
    assert e_dv <= TOL_TF32 and e_dw <= TOL_TF32, "dV %.3g dW %.3g" % (e_dv, e_dw)
    assert (dV[V <= 0] == 0).all() and (dW[mask == 0] == 0).all()
    # dV alone, without the mask, and dW alone
    dV2, none = wg.conv_bwd(_dev(V), _dev(Wm), _dev(dyl), layout=layout, math="tf32", need_dW=False)
    assert none is None and oracle.max_rel(dV2.cpu().numpy(), dVo) <= TOL_TF32
    none, dW2 = wg.conv_bwd(_dev(V), _dev(Wm), _dev(dyl), layout=layout, math="tf32", need_dV=False)
    assert none is None and oracle.max_rel(dW2.cpu().numpy(), oracle.conv_bwd(V, Wm, dY)[1]) <= TOL_TF32
    _status_ok(wg)


@pytest.mark.parametrize("layout", ["NHWC", "NCHW"])
@pytest.mark.parametrize("shape", [(2, 14, 14, 64, 64), (2, 7, 7, 64, 128), (2, 9, 13, 36, 20), (1, 28, 28, 128, 96)])
def test_fused_affine_and_residual(wg, oracle, shape, layout):
    """Input affine folded into the transform, output affine + residual folded into the product's epilogue."""
    B, H, W, C, K = shape
    X, Wt = _inputs(shape)
    rng = np.random.default_rng(5)
    s_in, b_in = (1 + 0.2 * rng.standard_normal(C)).astype(np.float32), (0.3 * rng.standard_normal(C)).astype(np.float32)
    s_out, b_out = (1 + 0.2 * rng.standard_normal(K)).astype(np.float32), (0.3 * rng.standard_normal(K)).astype(np.float32)
    R = rng.standard_normal((B, H, W, K)).astype(np.float32)
    to_l = (lambda a: a) if layout == "NHWC" else (lambda a: np.ascontiguousarray(np.transpose(a, (0, 3, 1, 2))))
    V = wg.imtrans_fwd(_dev(to_l(X)), relu=True, layout=layout, in_scale=_dev(s_in), in_shift=_dev(b_in))
    Vo = oracle.imtrans_fwd(X.astype(np.float64) * s_in + b_in, relu=True)
    assert oracle.max_rel(V.cpu().numpy(), Vo) <= 1e-5
    prepared = wg.prepare_weights(_dev(Wt))
    want = oracle.conv_fwd(Vo, Wt, H, W) * s_out + b_out + R
    for kw in (dict(out_scale=_dev(s_out), out_shift=_dev(b_out), residual=_dev(to_l(R))),):
        Y = wg.conv_fwd_prepared(V, prepared, K, H, W, layout=layout, **kw).cpu().numpy()
        got = Y if layout == "NHWC" else np.transpose(Y, (0, 2, 3, 1))
        assert oracle.max_rel(got, want) <= TOL_TF32
    Y2 = wg.conv_fwd_prepared(V, prepared, K, H, W, layout=layout, residual=_dev(to_l(R))).cpu().numpy()
    got2 = Y2 if layout == "NHWC" else np.transpose(Y2, (0, 2, 3, 1))
    assert oracle.max_rel(got2, oracle.conv_fwd(Vo, Wt, H, W) + R) <= TOL_TF32
    _status_ok(wg)


FUSED_SHAPES = [  # B, H, W, C, K  (NCHW, W % 4 == 0, C % 16 == 0)
    (2, 56, 56, 64, 64), (3, 28, 28, 128, 128), (5, 8, 8, 32, 64), (2, 12, 16, 16, 24), (9, 4, 4, 64, 96),
    (1, 56, 72, 32, 32), (2, 7, 8, 48, 64), (1, 6, 136, 16, 32), (2, 1, 4, 16, 16), (3, 2, 8, 32, 64), (1, 33, 60, 64, 72),
]


@pytest.mark.parametrize("shape", FUSED_SHAPES)
def test_fused_layer_forward(wg, oracle, shape):
    """One-kernel layer forward (V never stored) against the float64 oracle, with and without the epilogue extras."""
    B, H, W, C, K = shape
    assert wg.fused_supported(B, H, W, C, K, "NCHW")
    X, Wt = _inputs(shape)
    xl = np.ascontiguousarray(np.transpose(X, (0, 3, 1, 2)))
    prepared = wg.prepare_weights(_dev(Wt))
    want = oracle.conv_fwd(oracle.imtrans_fwd(X, relu=True), Wt, H, W)
    Y = wg.layer_fwd_fused(_dev(xl), prepared, K, relu=True)
    _status_ok(wg)
    got = np.transpose(Y.cpu().numpy(), (0, 2, 3, 1))
    Yauto = wg.layer_fwd_prepared(_dev(xl), prepared, K, relu=True, layout="NCHW")   # picks a path by shape
    assert oracle.max_rel(np.transpose(Yauto.cpu().numpy(), (0, 2, 3, 1)), want) <= TOL_TF32
    assert np.isfinite(got).all()
    err = oracle.max_rel(got, want)
    assert err <= TOL_TF32, "max_rel %.3g" % err
    # no ReLU, plus affine output and residual
    rng = np.random.default_rng(3)
    s_out, b_out = (1 + 0.2 * rng.standard_normal(K)).astype(np.float32), (0.3 * rng.standard_normal(K)).astype(np.float32)
    R = rng.standard_normal((B, H, W, K)).astype(np.float32)
    Y2 = wg.layer_fwd_fused(_dev(xl), prepared, K, relu=False, out_scale=_dev(s_out), out_shift=_dev(b_out),
                            residual=_dev(np.ascontiguousarray(np.transpose(R, (0, 3, 1, 2)))))
    want2 = oracle.conv_fwd(oracle.imtrans_fwd(X, relu=False), Wt, H, W) * s_out + b_out + R
    assert oracle.max_rel(np.transpose(Y2.cpu().numpy(), (0, 2, 3, 1)), want2) <= TOL_TF32
    _status_ok(wg)


@pytest.mark.parametrize("shape", FUSED_SHAPES + [(3, 9, 12, 32, 64), (2, 56, 56, 64, 128)])
def test_fused_layer_forward_input_affine(wg, oracle, shape):
    """BatchNorm-like map in front of the transform, inside the one kernel: the padding must stay zero, so the
    oracle is fed s * x + t and pads that itself."""
    B, H, W, C, K = shape
    X, Wt = _inputs(shape)
    rng = np.random.default_rng(5)
    s_in, t_in = (1 + 0.3 * rng.standard_normal(C)).astype(np.float32), (0.5 * rng.standard_normal(C)).astype(np.float32)
    s_out, b_out = (1 + 0.2 * rng.standard_normal(K)).astype(np.float32), (0.3 * rng.standard_normal(K)).astype(np.float32)
    R = rng.standard_normal((B, H, W, K)).astype(np.float32)
    xl = np.ascontiguousarray(np.transpose(X, (0, 3, 1, 2)))
    prepared = wg.prepare_weights(_dev(Wt))
    Xa = X.astype(np.float64) * s_in + t_in
    for relu in (True, False):
        want = oracle.conv_fwd(oracle.imtrans_fwd(Xa, relu=relu), Wt, H, W)
        Y = wg.layer_fwd_fused(_dev(xl), prepared, K, relu=relu, in_scale=_dev(s_in), in_shift=_dev(t_in))
        assert oracle.max_rel(np.transpose(Y.cpu().numpy(), (0, 2, 3, 1)), want) <= TOL_TF32
    Y2 = wg.layer_fwd_fused(_dev(xl), prepared, K, relu=True, in_scale=_dev(s_in), in_shift=_dev(t_in), out_scale=_dev(s_out),
                            out_shift=_dev(b_out), residual=_dev(np.ascontiguousarray(np.transpose(R, (0, 3, 1, 2)))))
    want2 = oracle.conv_fwd(oracle.imtrans_fwd(Xa, relu=True), Wt, H, W) * s_out + b_out + R
    assert oracle.max_rel(np.transpose(Y2.cpu().numpy(), (0, 2, 3, 1)), want2) <= TOL_TF32
    _status_ok(wg)


@pytest.mark.parametrize("seed", range(16))
def test_fused_random_shapes(wg, oracle, seed):
    """Random geometry (segments, row blocks, images per unit, ragged ends, channel counts) against the oracle,
    plain and with every optional map at once."""
    rng = np.random.default_rng(1000 + seed)
    B, H = int(rng.integers(1, 7)), int(rng.integers(1, 40))
    W = 4 * int(rng.integers(1, 40))
    C, K = 16 * int(rng.integers(1, 7)), int(rng.integers(1, 150))
    shape = (B, H, W, C, K)
    assert wg.fused_supported(B, H, W, C, K, "NCHW"), shape
    X, Wt = _inputs(shape)
    xl = np.ascontiguousarray(np.transpose(X, (0, 3, 1, 2)))
    prepared = wg.prepare_weights(_dev(Wt))
    Y = wg.layer_fwd_fused(_dev(xl), prepared, K, relu=True)
    want = oracle.conv_fwd(oracle.imtrans_fwd(X, relu=True), Wt, H, W)
    err = oracle.max_rel(np.transpose(Y.cpu().numpy(), (0, 2, 3, 1)), want)
    assert err <= TOL_TF32, (shape, err)
    s_in, t_in = (1 + 0.3 * rng.standard_normal(C)).astype(np.float32), (0.5 * rng.standard_normal(C)).astype(np.float32)
    s_out, b_out = (1 + 0.2 * rng.standard_normal(K)).astype(np.float32), (0.3 * rng.standard_normal(K)).astype(np.float32)
    R = rng.standard_normal((B, H, W, K)).astype(np.float32)
    y = _dev(np.ascontiguousarray(np.transpose(R, (0, 3, 1, 2))))          # the shortcut, added to in place
    Y2 = wg.layer_fwd_fused(_dev(xl), prepared, K, relu=True, out=y, in_scale=_dev(s_in), in_shift=_dev(t_in),
                            out_scale=_dev(s_out), out_shift=_dev(b_out), residual=y)
    want2 = oracle.conv_fwd(oracle.imtrans_fwd(X.astype(np.float64) * s_in + t_in, relu=True), Wt, H, W) * s_out + b_out + R
    err2 = oracle.max_rel(np.transpose(Y2.cpu().numpy(), (0, 2, 3, 1)), want2)
    assert err2 <= TOL_TF32, (shape, err2)
    _status_ok(wg)


@pytest.mark.parametrize("shape,launches", [((256, 56, 56, 64, 64), 1500), ((40, 28, 28, 128, 128), 1500)])
def test_fused_many_units_per_cta_repeated(wg, oracle, shape, launches):
    """Many units per CTA, many launches: every launch on the same input must give the same bits, the device
    status must stay clean, and a sample of the result must match the oracle.  (The rings inside the kernel wrap
    around many times per launch here; a lost or mis-attributed barrier phase shows up as a changed result, a
    time-out status or a failed launch.)"""
    import torch
    B, H, W, C, K = shape
    gen = torch.Generator(device="cuda").manual_seed(11)
    Xs = [torch.randn((B, C, H, W), generator=gen, device="cuda") for _ in range(3)]
    Wt = 0.05 * torch.randn((16, C, K), generator=gen, device="cuda")
    prepared = wg.prepare_weights(Wt)
    Y = torch.empty((B, K, H, W), device="cuda")
    first = [None] * 3
    for it in range(launches):
        wg.layer_fwd_fused(Xs[it % 3], prepared, K, relu=True, out=Y)
        if it < 3 or it % 250 < 3 or it >= launches - 3:
            if first[it % 3] is None:
                first[it % 3] = Y.clone()
            else:
                assert torch.equal(Y, first[it % 3]), "launch %d differs from the first launch on the same input" % it
    _status_ok(wg)
    # two images of the first input against the float64 oracle
    xs = np.ascontiguousarray(np.transpose(Xs[0][:2].cpu().numpy(), (0, 2, 3, 1)))
    want = oracle.conv_fwd(oracle.imtrans_fwd(xs, relu=True), Wt.cpu().numpy(), H, W)
    got = np.transpose(first[0][:2].cpu().numpy(), (0, 2, 3, 1))
    assert oracle.max_rel(got, want) <= TOL_TF32


@pytest.mark.parametrize("layout", ["NCHW", "NHWC"])
def test_two_kernel_path_at_full_conv2_batch(wg, oracle, layout):
    """Input transform + product kernel at the full batch of the conv2_x workload (64 x 64 x 56 x 56, K = 64), where
    the product kernel shrinks its units so that they divide evenly over the SMs: sampled images against the
    float64 oracle, every image against the one-kernel path."""
    B, H, W, C, K = 64, 56, 56, 64, 64
    gen = torch.Generator(device="cuda").manual_seed(17)
    X = torch.randn((B, C, H, W), generator=gen, device="cuda")
    Wt = 0.05 * torch.randn((16, C, K), generator=gen, device="cuda")
    prepared = wg.prepare_weights(Wt)
    xin = X if layout == "NCHW" else X.permute(0, 2, 3, 1).contiguous()
    V = wg.imtrans_fwd(xin, relu=True, layout=layout)
    Y = wg.conv_fwd_prepared(V, prepared, K, H, W, layout=layout)
    _status_ok(wg)
    Yn = Y if layout == "NHWC" else Y.permute(0, 2, 3, 1)
    for b in (0, 17, 38, 63):        # first, last and two images whose tiles straddle unit boundaries
        xs = np.ascontiguousarray(X[b:b + 1].permute(0, 2, 3, 1).cpu().numpy())
        want = oracle.conv_fwd(oracle.imtrans_fwd(xs, relu=True), Wt.cpu().numpy(), H, W)
        assert oracle.max_rel(Yn[b:b + 1].cpu().numpy(), want) <= TOL_TF32, b
    Yf = wg.layer_fwd_fused(X, prepared, K, relu=True)
    assert oracle.max_rel(Yn.permute(0, 3, 1, 2).cpu().numpy(), Yf.cpu().numpy()) <= 2e-3
    _status_ok(wg)


def test_layer_fwd_prepared_falls_back_to_two_kernels(wg, oracle):
    shape = (2, 7, 7, 36, 20)        # odd width: not a fused shape
    B, H, W, C, K = shape
    assert not wg.fused_supported(B, H, W, C, K, "NCHW")
    X, Wt = _inputs(shape)
    prepared = wg.prepare_weights(_dev(Wt))
    Y = wg.layer_fwd_prepared(_dev(X), prepared, K, relu=True, layout="NHWC")
    assert oracle.max_rel(Y.cpu().numpy(), oracle.conv_fwd(oracle.imtrans_fwd(X, relu=True), Wt, H, W)) <= TOL_TF32


@pytest.mark.parametrize("layout", ["NHWC", "NCHW"])
def test_layer_fwd_prepared_takes_the_wide_path(wg, oracle, layout):
    """The whole-layer call with prepared weights: for C, K >= 256 it asks for product scratch and gives the result of the
    wide path (bit for bit what input transform + conv_fwd_prepared give)."""
    shape = (4, 14, 14, 256, 256)
    B, H, W, C, K = shape
    X, Wt = _inputs(shape)
    assert wg.layer_fwd_prepared_workspace_bytes(B, H, W, C, K) == 16 * B * 7 * 7 * K * 4
    assert wg.layer_fwd_prepared_workspace_bytes(B, 56, 56, 64, 64) == 0
    x = _dev(X if layout == "NHWC" else np.ascontiguousarray(np.transpose(X, (0, 3, 1, 2))))
    prepared = wg.prepare_weights(_dev(Wt))
    Y = wg.layer_fwd_prepared(x, prepared, K, relu=True, layout=layout)
    _status_ok(wg)
    V = wg.imtrans_fwd(x, relu=True, layout=layout)
    assert torch.equal(Y, wg.conv_fwd_prepared(V, prepared, K, H, W, layout=layout, wide=True))
    got = Y.cpu().numpy() if layout == "NHWC" else np.transpose(Y.cpu().numpy(), (0, 2, 3, 1))
    assert oracle.max_rel(got, oracle.conv_fwd(oracle.imtrans_fwd(X, relu=True), Wt, H, W)) <= TOL_TF32


@pytest.mark.parametrize("layout", ["NHWC", "NCHW"])
@pytest.mark.parametrize("shape", [(3, 14, 14, 256, 256), (16, 7, 7, 512, 512), (2, 9, 13, 260, 264), (1, 28, 28, 256, 320)])
def test_wide_forward_path(wg, oracle, shape, layout):
    """Layers with many channels: products as wide GEMMs into scratch memory + output transform pass, against the
    oracle and against the single-kernel path; with the epilogue extras too."""
    B, H, W, C, K = shape
    X, Wt = _inputs(shape)
    V = oracle.imtrans_fwd(X, relu=True, dtype=np.float32)
    want = oracle.conv_fwd(V, Wt, H, W)
    prepared = wg.prepare_weights(_dev(Wt))
    fix = (lambda a: a) if layout == "NHWC" else (lambda a: np.transpose(a, (0, 2, 3, 1)))
    to_l = (lambda a: a) if layout == "NHWC" else (lambda a: np.ascontiguousarray(np.transpose(a, (0, 3, 1, 2))))
    assert wg._lib.lib.wg2x2_conv_fwd_prepared_workspace_bytes(B, (H + 1) // 2, (W + 1) // 2, C, K) > 0
    Yw = wg.conv_fwd_prepared(_dev(V), prepared, K, H, W, layout=layout).cpu().numpy()
    Yn = wg.conv_fwd_prepared(_dev(V), prepared, K, H, W, layout=layout, wide=False).cpu().numpy()
    assert oracle.max_rel(fix(Yw), want) <= TOL_TF32 and oracle.max_rel(fix(Yn), want) <= TOL_TF32
    assert oracle.max_rel(Yw, Yn) <= 1e-5          # same TF32 products, fp32 sums in a different order
    rng = np.random.default_rng(8)
    s_out, b_out = (1 + 0.2 * rng.standard_normal(K)).astype(np.float32), (0.3 * rng.standard_normal(K)).astype(np.float32)
    R = rng.standard_normal((B, H, W, K)).astype(np.float32)
    Ye = wg.conv_fwd_prepared(_dev(V), prepared, K, H, W, layout=layout, out_scale=_dev(s_out), out_shift=_dev(b_out),
                              residual=_dev(to_l(R))).cpu().numpy()
    assert oracle.max_rel(fix(Ye), want * s_out + b_out + R) <= TOL_TF32
    Yc = wg.conv_fwd(_dev(V), _dev(Wt), H, W, layout=layout, math="tf32").cpu().numpy()      # raw-weight entry point
    assert oracle.max_rel(fix(Yc), want) <= TOL_TF32
    _status_ok(wg)


_PAIR_CHILD = r"""
import sys, numpy as np, torch
sys.path.insert(0, sys.argv[1])
import wg2x2
g = torch.Generator().manual_seed(7)
B, C, K, H, W = 70, 512, 512, 7, 7          # P = 1120 tiles: nine row blocks, the last pair half empty; contraction 1120 / 512
X = torch.randn((B, C, H, W), generator=g).cuda()
Wt = (0.05 * torch.randn((16, C, K), generator=g)).cuda()
dY = torch.randn((B, K, H, W), generator=g).cuda()
V = wg2x2.imtrans_fwd(X, relu=True, layout="NCHW")
dV, dW = wg2x2.conv_bwd(V, Wt, dY, layout="NCHW", relu=False, math="tf32")
Y = wg2x2.conv_fwd_prepared(V, wg2x2.prepare_weights(Wt), K, H, W, layout="NCHW")
st, where = wg2x2.last_device_status()
assert st == 0, hex(where)
np.savez(sys.argv[2], dV=dV.cpu().numpy(), dW=dW.cpu().numpy(), Y=Y.cpu().numpy())
"""


def test_pair_of_sms_kernel_equals_the_one_cta_kernel(tmp_path):
    """The GEMM on pairs of SMs (tcgen05 cta_group::2: dW, and products over 512 channels) against the one-CTA kernel
    (WG2X2_GEMM_PAIR=0) on the same inputs, each in its own process: every output element is the same sum in the same
    order, so the results are equal bit for bit.  Nine row blocks: the last pair works with one CTA's rows out of range."""
    import os
    import subprocess
    import sys
    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "sparse-winograd-cnn_b200")
    outs = []
    for flag in ("1", "0"):
        path = str(tmp_path / ("pair%s.npz" % flag))
        env = dict(os.environ, WG2X2_GEMM_PAIR=flag)
        r = subprocess.run([sys.executable, "-c", _PAIR_CHILD, root, path], env=env, capture_output=True, text=True, timeout=300)
        assert r.returncode == 0, r.stderr[-2000:]
        outs.append(np.load(path))
    for key in ("dV", "dW", "Y"):
        assert np.array_equal(outs[0][key], outs[1][key]), key
    assert np.isfinite(outs[0]["dW"]).all() and float(np.abs(outs[0]["dW"]).max()) > 0


def test_pair_of_sms_kernel_repeated_launches(wg):
    """300 back-to-back gradient and wide-forward products on the pair kernel (dW contracts over 1120 tiles, the
    products over 512 channels): the cross-CTA barriers keep their phases from launch to launch, every result
    equals the first bit for bit and no bounded wait gives up."""
    g = torch.Generator().manual_seed(5)
    B, C, K, H, W = 70, 512, 512, 7, 7
    X = torch.randn((B, C, H, W), generator=g).cuda()
    Wt = (0.05 * torch.randn((16, C, K), generator=g)).cuda()
    dY = torch.randn((B, K, H, W), generator=g).cuda()
    V = wg.imtrans_fwd(X, relu=True, layout="NCHW")
    prep = wg.prepare_weights(Wt)
    dV0, dW0 = wg.conv_bwd(V, Wt, dY, layout="NCHW", relu=False, math="tf32")
    Y0 = wg.conv_fwd_prepared(V, prep, K, H, W, layout="NCHW")
    for i in range(300):
        dV, dW = wg.conv_bwd(V, Wt, dY, layout="NCHW", relu=False, math="tf32")
        Y = wg.conv_fwd_prepared(V, prep, K, H, W, layout="NCHW")
        if i % 60 == 59:
            _status_ok(wg)
            assert torch.equal(dV, dV0) and torch.equal(dW, dW0) and torch.equal(Y, Y0), i
