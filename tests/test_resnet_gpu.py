"""ResNet-18-var forward graph: the Winograd layers on this library's kernels against the same graph with
the layers computed from the transform matrices in float64 (torch einsum)."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("layout", ["NHWC", "NCHW"])
@pytest.mark.parametrize("math,tol,fused", [("fp32", 2e-4, False), ("tf32", 2e-2, False), ("tf32", 2e-2, True)])
@pytest.mark.parametrize("stage5_pool", [True, False])
def test_forward_matches_einsum_graph(math, tol, fused, stage5_pool, layout):
    from resnet18_var import ResNet18Var
    torch.manual_seed(0)
    model = ResNet18Var(stage5_pool=stage5_pool, seed=3, math=math, fused=fused, layout=layout).cuda().eval()
    x = torch.randn((2, 3, 96, 96), device="cuda")       # 24x24 at stage 2 ... 3x3 (odd) at stage 5
    with torch.no_grad():
        got = model(x)
        want = model(x, reference=True)
    assert got.shape == (2, 1000) and torch.isfinite(got).all()
    err = float((got - want).abs().max() / want.abs().max())
    assert err <= tol, err   # 16 layers deep: per-layer 1e-5 / 5e-3 compounds


def test_winograd_flops_count():
    from resnet18_var import ResNet18Var
    m = ResNet18Var(stage5_pool=True)
    assert abs(m.winograd_flops(1) / 1e6 - 1600.2) < 1.0      # MFLOP per image, stage 5 at 7x7
    assert abs(ResNet18Var(stage5_pool=False).winograd_flops(1) / 1e6 - 2569.0) < 1.5   # at 14x14, as the reference runs it


def test_load_weights_and_masks_by_reference_names():
    import numpy as np
    import wg_weights as ww
    from resnet18_var import ResNet18Var
    model = ResNet18Var(seed=1).cuda().eval()
    layers = model.winograd_layers()
    assert tuple(sorted(layers)) == tuple(sorted(ww.RESNET18_LAYER_NAMES))
    rng = np.random.default_rng(0)
    weights = {n: rng.standard_normal(tuple(l.W.shape)).astype(np.float32) for n, l in layers.items()}
    pruned, masks = ww.prune_layers(weights, 0.3)
    model.load_winograd_weights(weights, masks)
    for n, l in layers.items():
        assert np.array_equal(l.W.cpu().numpy(), pruned[n]) and abs(float(l.mask.mean()) - 0.3) < 1e-3
    x = torch.randn((1, 3, 64, 64), device="cuda")
    with torch.no_grad():
        assert torch.isfinite(model(x)).all()


def test_same_pool_matches_tensorflow_padding():
    """3x3/2 SAME max-pool: explicit -inf padding as TensorFlow places it vs the copy-free form used by the model."""
    import torch.nn.functional as F
    from resnet18_var import _same_pool
    for H, W in [(112, 112), (7, 7), (14, 9), (5, 8)]:
        x = torch.randn(2, 3, H, W)
        ph = max((-(-H // 2) - 1) * 2 + 3 - H, 0)
        pw = max((-(-W // 2) - 1) * 2 + 3 - W, 0)
        ref = F.max_pool2d(F.pad(x, (pw // 2, pw - pw // 2, ph // 2, ph - ph // 2), value=float("-inf")), 3, 2)
        assert torch.equal(_same_pool(x), ref)


@pytest.mark.parametrize("shape", [(3, 8, 112, 112), (2, 64, 32, 40), (1, 96, 9, 11), (2, 5, 56, 56), (2, 4, 28, 28), (1, 3, 9, 12), (2, 2, 13, 20), (2, 3, 14, 14), (2, 3, 7, 7), (1, 2, 14, 9),
                                   (1, 2, 5, 8), (2, 3, 9, 16), (1, 1, 1, 1), (1, 2, 2, 3)])
def test_pool_kernel_matches_torch(shape):
    """wg2x2_maxpool3x3s2_same (the vector path for widths that are multiples of 8, the general path elsewhere, odd
    sizes included) against the torch form of the same pooling: the maxima bit for bit, the extra ReLU output too, the
    affine ReLU output to rounding."""
    import wg2x2
    from resnet18_var import _same_pool
    g = torch.Generator(device="cuda").manual_seed(sum(shape))
    x = torch.randn(shape, device="cuda", generator=g)
    want = _same_pool(x)
    got = wg2x2.maxpool3x3s2_same(x)
    assert torch.equal(got, want)
    got2, relu = wg2x2.maxpool3x3s2_same(x, with_relu=True)
    assert torch.equal(got2, want) and torch.equal(relu, torch.relu(want))
    sc = 1 + 0.2 * torch.randn(shape[1], device="cuda", generator=g)
    sh = 0.3 * torch.randn(shape[1], device="cuda", generator=g)
    got3, bnrelu = wg2x2.maxpool3x3s2_same(x, with_relu=True, relu_scale=sc, relu_shift=sh)
    ref = torch.relu(want * sc.view(1, -1, 1, 1) + sh.view(1, -1, 1, 1))
    assert torch.equal(got3, want) and float((bnrelu - ref).abs().max()) <= 1e-6 * max(1.0, float(ref.abs().max()))
    # the same from a channels-last input (the layout a channels-last stem convolution leaves): NCHW outputs
    xcl = x.contiguous(memory_format=torch.channels_last)
    got4, bnrelu4 = wg2x2.maxpool3x3s2_same(xcl, with_relu=True, relu_scale=sc, relu_shift=sh)
    assert got4.is_contiguous() and torch.equal(got4, want)
    assert float((bnrelu4 - ref).abs().max()) <= 1e-6 * max(1.0, float(ref.abs().max()))
    assert torch.equal(wg2x2.maxpool3x3s2_same(xcl), want)


def _tf32(x):
    """Round to TF32, nearest with ties away from zero (cvt.rna.tf32.f32)."""
    return ((x.contiguous().view(torch.int32) + 0x1000) & ~0x1FFF).view(torch.float32)


@pytest.mark.parametrize("shape", [(2, 224, 224), (3, 64, 48), (1, 32, 224), (5, 100, 36), (1, 4, 4), (2, 8, 12), (37, 56, 56)])
def test_stem_kernel_matches_dense_conv_and_pool(shape):
    """wg2x2_stem7x7s2_pool (7x7/2 SAME convolution of a 3-channel image into 64 channels + 3x3/2 SAME max-pool in one
    tensor-core kernel) against float64 convolution of the TF32-rounded operands followed by the torch pooling: only
    the FP32 accumulation order differs, so 2e-5 of the largest value; the BNReLU output to the same bound."""
    import wg2x2
    from resnet18_var import _same_pool
    B, H, W = shape
    g = torch.Generator(device="cuda").manual_seed(B + H + W)
    x = torch.randn((B, 3, H, W), device="cuda", generator=g)
    w = torch.randn((64, 3, 7, 7), device="cuda", generator=g) * 0.1
    sc = 1 + 0.2 * torch.randn(64, device="cuda", generator=g)
    sh = 0.3 * torch.randn(64, device="cuda", generator=g)
    assert wg2x2.stem_supported(H, W)
    prep = wg2x2.stem_prepare(w)
    conv = F.conv2d(F.pad(_tf32(x).double(), (2, 3, 2, 3)), _tf32(w).double(), stride=2)
    want = _same_pool(conv.float())
    got, bnrelu = wg2x2.stem7x7s2_pool(x, prep, with_relu=True, relu_scale=sc, relu_shift=sh)
    tol = 2e-5 * float(want.abs().max())
    assert got.shape == want.shape and float((got - want).abs().max()) <= tol
    ref = torch.relu(want * sc.view(1, -1, 1, 1) + sh.view(1, -1, 1, 1))
    assert float((bnrelu - ref).abs().max()) <= 2 * tol
    assert torch.equal(wg2x2.stem7x7s2_pool(x, prep), got)
    # against the plain FP32 convolution: TF32 operand rounding, 2e-3 of the largest value
    keep = torch.backends.cudnn.allow_tf32
    torch.backends.cudnn.allow_tf32 = False
    try:
        plain = _same_pool(F.conv2d(F.pad(x, (2, 3, 2, 3)), w, stride=2))
    finally:
        torch.backends.cudnn.allow_tf32 = keep
    assert float((got - plain).abs().max()) <= 2e-3 * float(plain.abs().max())


def test_stem_kernel_rejects_other_sizes():
    import wg2x2
    assert not wg2x2.stem_supported(226, 224) and not wg2x2.stem_supported(224, 228) and not wg2x2.stem_supported(224, 256)
    x = torch.zeros((1, 3, 30, 32), device="cuda")
    with pytest.raises(ValueError):
        wg2x2.stem7x7s2_pool(x, wg2x2.stem_prepare(torch.zeros((64, 3, 7, 7), device="cuda")))
