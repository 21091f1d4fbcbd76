"""CPU checks that pin the oracle (oracle/wg_oracle.c) before anything is compared with it."""
import glob
import os

import numpy as np
import pytest
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
# the reference test scripts' own shapes (B=3, 6x6, (C,K) = (32,32), (32,64), (5,7)), then odd / ragged ones
REF_SHAPES = [(3, 6, 6, 32, 32), (3, 6, 6, 32, 64), (3, 6, 6, 5, 7)]
MORE_SHAPES = [(2, 7, 7, 5, 7), (1, 1, 1, 3, 2), (2, 5, 8, 4, 6), (1, 9, 4, 6, 3)]


def _conv2d(X, g):
    return torch.nn.functional.conv2d(torch.from_numpy(X).permute(0, 3, 1, 2), torch.from_numpy(g).permute(3, 2, 0, 1),
                                      padding=1).permute(0, 2, 3, 1).numpy()


@pytest.mark.parametrize("shape", REF_SHAPES + MORE_SHAPES)
def test_identity_with_direct_convolution(oracle, shape):
    """Level 1 of the reference tests: Winograd layer with G g G^T weights == 3x3 SAME conv
    (winograd2x2_imTrans_test.py:179-192); their metric is the relative L1 error."""
    B, H, W, C, K = shape
    rng = np.random.default_rng(sum(shape))
    X = rng.standard_normal((B, H, W, C))
    g = rng.standard_normal((3, 3, C, K))
    Wt = oracle.kernel_transform(g)
    Y = oracle.conv_fwd(oracle.imtrans_fwd(X), Wt, H, W)
    ref = _conv2d(X, g)
    assert oracle.rel_l1(Y, ref) < 1e-14 and oracle.max_rel(Y, ref) < 1e-13
    Y32 = oracle.layer_fwd(X.astype(np.float32), Wt.astype(np.float32), relu=False, dtype=np.float32)
    assert oracle.max_rel(Y32, ref) < 2e-6


@pytest.mark.parametrize("shape", REF_SHAPES + MORE_SHAPES)
def test_c_oracle_equals_numpy_twin(oracle, shape):
    B, H, W, C, K = shape
    rng = np.random.default_rng(1 + sum(shape))
    X = rng.standard_normal((B, H, W, C))
    Wt = rng.standard_normal((16, C, K))
    for relu in (False, True):
        V = oracle.imtrans_fwd(X, relu=relu)
        assert np.allclose(V, oracle.np_imtrans_fwd(X, relu=relu), rtol=0, atol=1e-13)
    assert np.allclose(oracle.conv_fwd(V, Wt, H, W), oracle.np_conv_fwd(V, Wt, H, W), rtol=0, atol=1e-11)
    assert V.shape == (16, B, (H + 1) // 2, (W + 1) // 2, C)


def _torch_layer(X, Wt, oracle, relu=True):
    """The reference tests' pure-TF graph (image_transform + winograd_conv,
    winograd2x2_imTrans_test.py:27-156) restated with torch so that autograd gives the gradients."""
    B, H, W, C = X.shape
    nH, nW = (H + 1) // 2, (W + 1) // 2
    BT, AT = torch.tensor(oracle.BT), torch.tensor(oracle.AT)
    Xp = torch.nn.functional.pad(X, (0, 0, 1, 2 * nW + 1 - W, 1, 2 * nH + 1 - H))
    d = torch.stack([torch.stack([Xp[:, y:y + 2 * nH:2, x:x + 2 * nW:2] for x in range(4)], 3) for y in range(4)], 3)
    V = torch.einsum("iy,bhwyxc,jx->ijbhwc", BT, d, BT).reshape(16, B, nH, nW, C)
    Vr = torch.relu(V) if relu else V
    Vr.retain_grad()
    M = torch.einsum("tbhwc,tck->tbhwk", Vr, Wt).reshape(4, 4, B, nH, nW, -1)
    Y = torch.einsum("ai,ijbhwk,ej->bhawek", AT, M, AT).reshape(B, 2 * nH, 2 * nW, -1)[:, :H, :W]
    return Vr, Y


@pytest.mark.parametrize("shape", REF_SHAPES + MORE_SHAPES)
def test_gradients_equal_autodiff(oracle, shape):
    """Level 2 for the gradient ops (winograd2x2_conv_grad_test.py:205-227,
    winograd2x2_imTrans_grad_test.py:194-216): compare with autodiff of the restated graph."""
    B, H, W, C, K = shape
    rng = np.random.default_rng(2 + sum(shape))
    X = torch.tensor(rng.standard_normal((B, H, W, C)), requires_grad=True)
    mask = (rng.random((16, C, K)) < 0.5).astype(np.float64)
    Wraw = torch.tensor(rng.standard_normal((16, C, K)), requires_grad=True)
    dY = rng.standard_normal((B, H, W, K))
    Vr, Y = _torch_layer(X, Wraw * torch.tensor(mask), oracle)
    (Y * torch.tensor(dY)).sum().backward()
    Vo = oracle.imtrans_fwd(X.detach().numpy(), relu=True)
    Wm = Wraw.detach().numpy() * mask
    assert oracle.rel_l1(oracle.conv_fwd(Vo, Wm, H, W), Y.detach().numpy()) < 1e-14
    dV, dW = oracle.conv_bwd(Vo, Wm, dY, mask=mask)
    dX = oracle.imtrans_bwd(dV, H, W, Vmask=Vo)
    assert oracle.rel_l1(dV, Vr.grad.numpy()) < 1e-14
    assert oracle.rel_l1(dW, Wraw.grad.numpy()) < 1e-14
    assert oracle.rel_l1(dX, X.grad.numpy()) < 1e-14


def test_adjoint_identities(oracle):
    """<imtrans(x), g> == <x, imtrans_bwd(g)> and the same for the product op, odd sizes included."""
    rng = np.random.default_rng(5)
    for (B, H, W, C, K) in [(2, 7, 7, 3, 4), (1, 6, 9, 4, 2)]:
        nH, nW = (H + 1) // 2, (W + 1) // 2
        x = rng.standard_normal((B, H, W, C))
        g = rng.standard_normal((16, B, nH, nW, C))
        assert abs((oracle.imtrans_fwd(x) * g).sum() - (x * oracle.imtrans_bwd(g, H, W)).sum()) < 1e-10
        V = rng.standard_normal((16, B, nH, nW, C))
        Wt = rng.standard_normal((16, C, K))
        dY = rng.standard_normal((B, H, W, K))
        dV, dW = oracle.conv_bwd(V, Wt, dY)
        lhs = (oracle.conv_fwd(V, Wt, H, W) * dY).sum()
        assert abs(lhs - (V * dV).sum()) < 1e-9 and abs(lhs - (Wt * dW).sum()) < 1e-9


def test_golden_vectors_from_upstream_cuda_kernels(oracle):
    """Fixtures produced by the reference's own CUDA kernels on a B200 (tests/golden/make_golden.py)."""
    files = sorted(glob.glob(os.path.join(GOLDEN, "ref_cuda_*.npz")))
    assert files, "golden fixtures missing"
    for f in files:
        z = np.load(f)
        X, Wt, dY = z["X"], z["Wt"], z["dY"]
        B, H, W, C = X.shape
        V = oracle.imtrans_fwd(X)
        assert oracle.max_rel(z["V"], V) < 1e-6, f
        Vr = np.maximum(z["V"], 0)
        assert oracle.max_rel(z["Y"], oracle.conv_fwd(Vr, Wt, H, W)) < 1e-5, f
        dV, dW = oracle.conv_bwd(Vr, Wt, dY)
        assert oracle.max_rel(z["dV"], dV) < 1e-5, f
        assert oracle.max_rel(z["dW"], dW) < 1e-5, f
        assert oracle.max_rel(z["dX"], oracle.imtrans_bwd(z["dV"], H, W, Vmask=Vr)) < 1e-5, f
        assert oracle.rel_l1(z["Y"], oracle.conv_fwd(Vr, Wt, H, W)) < 1e-6, f
