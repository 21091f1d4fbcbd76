"""Weight/mask interchange and the reference's magnitude pruning (CPU only)."""
import os
import pickle

import numpy as np
import torch

import wg_weights as ww

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "prune_masks.npz")


def test_gen_prune_mask_equals_reference_function():
    """Fixtures come from the reference's own gen_prune_mask (tests/golden/make_prune_golden.py)."""
    z = np.load(GOLDEN)
    n = sum(1 for k in z.files if k.startswith("w"))
    assert n >= 6
    for i in range(n):
        w = z["w%d" % i].copy()
        mask = ww.gen_prune_mask(w, float(z["density%d" % i]))
        assert np.array_equal(mask, z["mask%d" % i])
        assert np.array_equal(w, z["pruned%d" % i])           # pruned in place, like the reference
        again = (z["w%d" % i] * z["mask%d" % i]).astype(np.float32)
        assert np.array_equal(ww.gen_prune_mask(again, float(z["density%d" % i]) * 0.5), z["mask2_%d" % i])


def test_prune_layers_and_npz_round_trip(tmp_path):
    rng = np.random.default_rng(0)
    weights = {name: rng.standard_normal((16, 8, 8)).astype(np.float32) for name in ww.RESNET18_LAYER_NAMES[:3]}
    weights["conv1/W"] = rng.standard_normal((7, 7, 3, 64)).astype(np.float32)      # not a Winograd weight: untouched
    w1, m1 = ww.prune_layers(weights, 0.5)
    assert set(m1) == set(ww.RESNET18_LAYER_NAMES[:3]) and np.array_equal(w1["conv1/W"], weights["conv1/W"])
    for k, m in m1.items():
        assert abs(m.mean() - 0.5) < 1e-3 and np.array_equal(w1[k], weights[k] * m)
    w2, m2 = ww.prune_layers(w1, 0.25, existing_masks=m1)                              # the iterative ladder
    for k in m2:
        assert abs(m2[k].mean() - 0.25) < 1e-3 and np.all(m2[k] <= m1[k])
    p = str(tmp_path / "model.npz")
    ww.save_npz(p, w2, m2)
    w3, m3 = ww.load_npz(p)
    assert all(np.array_equal(w3[k], w2[k]) for k in w2) and all(np.array_equal(m3[k], m2[k]) for k in m2)
    pk = str(tmp_path / "prune_mask_0.25.pkl")
    with open(pk, "wb") as f:
        pickle.dump(m2, f, protocol=2)
    m4 = ww.load_mask_pickle(pk)
    assert all(np.array_equal(m4[k], m2[k]) for k in m2)


def test_kernel_transform_gives_the_direct_convolution(oracle):
    rng = np.random.default_rng(1)
    X = rng.standard_normal((2, 7, 6, 5))
    g = rng.standard_normal((3, 3, 5, 4))
    Wt = ww.kernel_transform(g)
    assert Wt.shape == (16, 5, 4) and np.allclose(Wt, oracle.kernel_transform(g))
    Y = oracle.conv_fwd(oracle.imtrans_fwd(X), Wt, 7, 6)
    ref = torch.nn.functional.conv2d(torch.from_numpy(X).permute(0, 3, 1, 2), torch.from_numpy(g).permute(3, 2, 0, 1),
                                     padding=1).permute(0, 2, 3, 1).numpy()
    assert np.abs(Y - ref).max() < 1e-12


def test_zero_block_fraction():
    m = np.ones((16, 64, 128), np.float32)
    assert ww.zero_block_fraction(m) == 0.0
    m[:, 32:, :64] = 0
    assert abs(ww.zero_block_fraction(m) - 0.25) < 1e-12
    rng = np.random.default_rng(0)
    assert ww.zero_block_fraction((rng.random((16, 256, 256)) < 0.3)) == 0.0    # unstructured masks leave no empty block
