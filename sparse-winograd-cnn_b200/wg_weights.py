"""Winograd-domain weights and pruning masks: interchange and the reference's magnitude pruning.

Layer names follow the reference graph: variables 'Winograd_W<stage><block>_<2a|2b>/W' of shape
(16, in_channel, out_channel) (ResNet-18-var/imagenet-resnet-transWino-prune.py:119-205), masks in a dict
keyed by the same names (ResNet-18-var/prune_script.py:63-82, read back at ...prune.py:388).
"""
import pickle

import numpy as np

# G of F(2x2,3x3), as expanded term by term in the reference tests' kernel_transform_num
# (winograd2x2_cublas/winograd2x2_imTrans/winograd2x2_imTrans_test.py:8-25)
G = np.array([[1, 0, 0], [0.5, 0.5, 0.5], [0.5, -0.5, 0.5], [0, 0, 1]], dtype=np.float64)


def kernel_transform(g_hwck):
    """Spatial 3x3 kernels (3,3,C,K) -> Winograd-domain weights (16,C,K) = G g G^T, position t = 4*row + col.
    With these weights and no nonlinearity the Winograd layer equals the 3x3 SAME convolution."""
    g = np.asarray(g_hwck, dtype=np.float64)
    if g.shape[:2] != (3, 3):
        raise ValueError("expected a (3,3,C,K) kernel")
    w = np.einsum("iy,yxck,jx->ijck", G, g, G)
    return w.reshape(16, g.shape[2], g.shape[3])


def gen_prune_mask(mat, density):
    """Keep the int(n*density) entries of largest magnitude, zero the rest IN PLACE, return the 0/1 mask.

    Same semantics as the reference function of this name (ResNet-18-var/prune_script.py:22-31), including
    its corner case: when int(n*density) is 0 the slice rank[:-0] is empty and nothing is pruned."""
    flat = mat.reshape(-1).copy()
    mask = np.ones_like(flat)
    rank = np.argsort(np.abs(flat))
    keep = int(rank.size * density)
    drop = rank[:-keep] if keep != 0 else rank[:0]
    flat[drop] = 0
    mask[drop] = 0
    np.copyto(mat, flat.reshape(mat.shape))
    return mask.reshape(mat.shape)


def is_winograd_weight(name):
    """The reference prunes exactly the variables whose name has 'Winograd_W' and '/W' (prune_script.py:68)."""
    return "Winograd_W" in name and "/W" in name


def prune_layers(weights, density, existing_masks=None):
    """One round of the reference's pruning loop (prune_script.py:63-78) over a dict of arrays: for each
    Winograd weight, the mask is computed on the weight times its existing mask, and the stored weight
    becomes weight * mask.  Returns (new weights dict, mask dict); other entries pass through."""
    out, masks = {}, {}
    for name, w in weights.items():
        if not is_winograd_weight(name):
            out[name] = w
            continue
        w = np.array(w, dtype=np.float32, copy=True)
        basis = w * existing_masks[name] if existing_masks is not None else w.copy()
        mask = gen_prune_mask(basis, float(density))
        masks[name] = mask.astype(np.float32)
        out[name] = w * mask
    return out, masks


def save_npz(path, weights, masks=None):
    """One .npz with '<layer>/W' weight arrays and, when given, '<layer>/W:mask' arrays."""
    blob = {k: np.asarray(v, dtype=np.float32) for k, v in weights.items()}
    for k, v in (masks or {}).items():
        blob[k + ":mask"] = np.asarray(v, dtype=np.float32)
    np.savez_compressed(path, **blob)


def load_npz(path):
    z = np.load(path)
    weights = {k: z[k] for k in z.files if not k.endswith(":mask")}
    masks = {k[:-5]: z[k] for k in z.files if k.endswith(":mask")}
    for k, w in weights.items():
        if is_winograd_weight(k) and (w.ndim != 3 or w.shape[0] != 16):
            raise ValueError("%s: expected (16, C, K), got %s" % (k, w.shape))
    return weights, masks


def load_mask_pickle(path):
    """The reference's prune_mask_<density>.pkl (prune_script.py:81-82): a pickled dict name -> ndarray,
    written by Python 2."""
    with open(path, "rb") as f:
        return pickle.load(f, encoding="latin1")


def zero_block_fraction(mask_or_weight, block_k=64, block_c=32):
    """Fraction of (block_c x block_k) blocks of a (16,C,K) array that are entirely zero: the share of
    weight blocks the tensor-core kernel skips.  An unstructured mask of density d leaves a block all zero
    with probability (1-d)^(block_c*block_k), i.e. practically never."""
    a = np.asarray(mask_or_weight)
    _, C, K = a.shape
    nc, nk = -(-C // block_c), -(-K // block_k)
    pad = np.zeros((16, nc * block_c, nk * block_k), dtype=bool)
    pad[:, :C, :K] = a != 0
    blocks = pad.reshape(16, nc, block_c, nk, block_k).any(axis=(2, 4))
    return float(1.0 - blocks.mean())


RESNET18_LAYER_NAMES = tuple("Winograd_W%d%s_%s/W" % (stage, blk, conv)
                             for stage in (2, 3, 4, 5) for blk in ("a", "b") for conv in ("2a", "2b"))
