"""ResNet-18-var forward graph around the Winograd-ReLU layers (inference form).

Topology as in the reference's Model._build_graph
(ResNet-18-var/imagenet-resnet-transWino-prune.py:113-220): 7x7/2 stem, 3x3/2 SAME max-pools, four
stages of two blocks; every 3x3 convolution is BatchNorm -> WinogradImTrans(relu) -> WinogradConv;
the `a` blocks carry a 1x1 shortcut convolution + BatchNorm, the `b` blocks an identity shortcut
after a ReLU.  The reference has `pool4` commented out (:191), so its stage 5 runs at 14x14;
`stage5_pool=True` restores the pool (7x7), which is the shape the benchmark configuration names.

The Winograd layers and (for NCHW activations) the max-pools run on this repository's kernels; the stem, 1x1
shortcuts and the classifier are stock torch ops.  With layout="NCHW" the layers of the two high-resolution stages (56x56 and 28x28) run
as one kernel each, BatchNorms and shortcut add included.  Weights are random (seeded): there is
no checkpoint to load here.
"""
import numpy as np
import torch
import torch.nn.functional as F

import wg2x2

STAGES = ((64, 64), (64, 128), (128, 256), (256, 512))       # (channels in, channels out) per stage
DENSITY = (0.6, 0.4, 0.3, 0.2)                               # Winograd-domain weight density per stage


def _same_pool(x):
    """MaxPooling(3, stride=2, padding='SAME') of TensorFlow without a padded copy.  For an even size TF pads one
    row/column at the bottom/right only (windows 2i..2i+2, the last one clipped): that is ceil_mode with no
    padding.  For an odd size it pads one on each side: padding=1."""
    H, W = x.shape[2], x.shape[3]
    return F.max_pool2d(x, 3, 2, padding=(H % 2, W % 2), ceil_mode=True)


class _BN(torch.nn.Module):
    """Inference BatchNorm as a per-channel affine map (scale, shift)."""

    def __init__(self, ch, gen):
        super().__init__()
        self.register_buffer("scale", 1.0 + 0.1 * torch.randn(ch, generator=gen))
        self.register_buffer("shift", 0.1 * torch.randn(ch, generator=gen))

    def forward(self, x):
        return x * self.scale.view(1, -1, 1, 1) + self.shift.view(1, -1, 1, 1)


class _Affine:
    """A (scale, shift) pair in the shape the layer calls take a BatchNorm."""

    def __init__(self, scale, shift):
        self.scale, self.shift = scale, shift


class _WinogradLayer(torch.nn.Module):
    """WinogradImTrans(relu) + WinogradConv with a fixed pruning mask."""

    def __init__(self, cin, cout, density, gen):
        super().__init__()
        std = (1.3 * (2.0 * 9.0 / 32.0) / (16 * cin)) ** 0.5       # the reference's default initialiser scale
        w = std * torch.randn((16, cin, cout), generator=gen)
        mask = (torch.rand((16, cin, cout), generator=gen) < density).float()
        self.register_buffer("W", (w * mask).contiguous())
        self.register_buffer("mask", mask)
        self.cout = cout
        self._prepared = None

    def prepared(self):
        if self._prepared is None or self._prepared.device != self.W.device:
            self._prepared = wg2x2.prepare_weights(self.W)
        return self._prepared

    @staticmethod
    def _to_kernel(x, layout):
        """(B,C,H,W)-shaped activation -> the contiguous tensor the kernels take: itself for NCHW, the (B,H,W,C)
        view of a channels-last tensor for NHWC (no copy when x already is channels-last)."""
        return x.contiguous() if layout == "NCHW" else x.permute(0, 2, 3, 1).contiguous()

    @staticmethod
    def _from_kernel(y, layout):
        return y if layout == "NCHW" else y.permute(0, 3, 1, 2)     # channels-last view of the (B,H,W,K) result

    def forward(self, x, math="tf32", layout="NCHW"):
        B, C, H, W = x.shape
        v = wg2x2.imtrans_fwd(self._to_kernel(x, layout), relu=True, layout=layout)
        if math == "tf32":
            y = wg2x2.conv_fwd_prepared(v, self.prepared(), self.cout, H, W, layout=layout)
        else:
            y = wg2x2.conv_fwd(v, self.W, H, W, layout=layout, math="fp32")
        return self._from_kernel(y, layout)

    def forward_fused(self, x, bn_in, bn_out=None, residual=None, layout="NCHW"):
        """BatchNorm -> transform + ReLU -> product [-> BatchNorm + shortcut add] in two kernels: bn_in folds
        into the transform's load, bn_out and the residual into the product's epilogue (tensor-core path)."""
        B, C, H, W = x.shape
        v = wg2x2.imtrans_fwd(self._to_kernel(x, layout), relu=True, layout=layout, in_scale=bn_in.scale, in_shift=bn_in.shift)
        y = wg2x2.conv_fwd_prepared(v, self.prepared(), self.cout, H, W, layout=layout,
                                    out_scale=None if bn_out is None else bn_out.scale,
                                    out_shift=None if bn_out is None else bn_out.shift,
                                    residual=None if residual is None else self._to_kernel(residual, layout))
        return self._from_kernel(y, layout)

    def onekernel_pays(self, x, layout):
        """True where the whole layer (both BatchNorms, ReLU, products, shortcut add) runs as the one-kernel path."""
        B, C, H, W = x.shape
        return (layout == "NCHW" and (self.cout <= 128 or (self.cout <= 256 and C <= 64))
                and wg2x2.fused_supported(B, H, W, C, self.cout, "NCHW"))

    def forward_onekernel(self, x, bn_in, bn_out=None, residual=None):
        """BatchNorm -> transform + ReLU -> product [-> BatchNorm + shortcut add] in one kernel (NCHW)."""
        res = None if residual is None else residual.contiguous()
        # the shortcut tensor is not used again: the kernel adds into it in place (no copy of it into a new output)
        return wg2x2.layer_fwd_fused(x.contiguous(), self.prepared(), self.cout, relu=True, out=res,
                                     in_scale=bn_in.scale, in_shift=bn_in.shift,
                                     out_scale=None if bn_out is None else bn_out.scale,
                                     out_shift=None if bn_out is None else bn_out.shift, residual=res)

    def forward_reference(self, x):
        """The same layer from the transform matrices with float64 einsums (for tests)."""
        BT = torch.tensor([[1, 0, -1, 0], [0, 1, 1, 0], [0, -1, 1, 0], [0, 1, 0, -1]], dtype=torch.float64, device=x.device)
        AT = torch.tensor([[1, 1, 1, 0], [0, 1, -1, -1]], dtype=torch.float64, device=x.device)
        B, C, H, W = x.shape
        nH, nW = (H + 1) // 2, (W + 1) // 2
        xp = F.pad(x.double(), (1, 2 * nW + 1 - W, 1, 2 * nH + 1 - H))
        d = torch.stack([torch.stack([xp[:, :, y:y + 2 * nH:2, s:s + 2 * nW:2] for s in range(4)], -1) for y in range(4)], -2)
        v = torch.relu(torch.einsum("iy,bchwyx,jx->ijbhwc", BT, d, BT))
        m = torch.einsum("ijbhwc,ijck->ijbhwk", v, self.W.double().view(4, 4, C, self.cout))
        y = torch.einsum("ai,ijbhwk,ej->bkhawe", AT, m, AT).reshape(B, self.cout, 2 * nH, 2 * nW)
        return y[:, :, :H, :W].float()


class ResNet18Var(torch.nn.Module):
    def __init__(self, num_classes=1000, stage5_pool=True, seed=0, math="tf32", fused=True, layout="NCHW"):
        super().__init__()
        gen = torch.Generator().manual_seed(seed)
        self.math = math
        # physical layout of the activations: "NCHW" (torch's default) lets the high-resolution layers run as one
        # kernel each; "NHWC" keeps them channels-last (the reference's layout) on the two-kernel path
        self.layout = layout
        self.fused = fused      # fold BatchNorms and shortcut additions into the Winograd kernels (tensor-core path)
        self.stage5_pool = stage5_pool
        self.stem = torch.nn.Parameter(torch.randn((64, 3, 7, 7), generator=gen) * (2.0 / (49 * 64)) ** 0.5, requires_grad=False)
        self.blocks = torch.nn.ModuleList()
        for s, (cin, cout) in enumerate(STAGES):
            blk_a = torch.nn.ModuleDict(dict(
                bn2a=_BN(cin, gen), w2a=_WinogradLayer(cin, cout, DENSITY[s], gen), bn2b=_BN(cout, gen),
                w2b=_WinogradLayer(cout, cout, DENSITY[s], gen), bn2c=_BN(cout, gen), bn1=_BN(cout, gen)))
            blk_a.short = torch.nn.Parameter(torch.randn((cout, cin, 1, 1), generator=gen) * (2.0 / cout) ** 0.5, requires_grad=False)
            if s == 0:
                blk_a["pre"] = _BN(cin, gen)          # res2a_1_relu is BNReLU in the reference, plain ReLU in later stages
            blk_b = torch.nn.ModuleDict(dict(
                bn2a=_BN(cout, gen), w2a=_WinogradLayer(cout, cout, DENSITY[s], gen), bn2b=_BN(cout, gen),
                w2b=_WinogradLayer(cout, cout, DENSITY[s], gen), bn2c=_BN(cout, gen)))
            self.blocks.append(torch.nn.ModuleList([blk_a, blk_b]))
        self.fc_w = torch.nn.Parameter(torch.randn((num_classes, 512), generator=gen) * (1.0 / 512) ** 0.5, requires_grad=False)
        self.fc_b = torch.nn.Parameter(torch.zeros(num_classes), requires_grad=False)

    def _block(self, blk, l, main, ref, main_bias=None):
        """main [+ main_bias] + bn2c(conv(bn2b(conv(bn2a(l))))) with the Winograd layers as `ref` says.  main_bias is a
        per-channel constant still owed to `main` (the folded BatchNorm shift of the 1x1 shortcut): on the fused path it
        rides on the last kernel's output shift instead of costing a pass over `main`."""
        if not ref and self.math == "tf32" and self.fused:
            wa, wb = blk["w2a"], blk["w2b"]
            t = (wa.forward_onekernel(l, blk["bn2a"]) if wa.onekernel_pays(l, self.layout)
                 else wa.forward_fused(l, blk["bn2a"], layout=self.layout))
            bn_out = blk["bn2c"]
            if main_bias is not None:
                if getattr(blk, "_out_folded", None) is None or blk._out_folded.shift.device != bn_out.shift.device:
                    blk._out_folded = _Affine(bn_out.scale, (bn_out.shift + main_bias).detach())
                bn_out = blk._out_folded
            if wb.onekernel_pays(t, self.layout):
                return wb.forward_onekernel(t, blk["bn2b"], bn_out=bn_out, residual=main)
            return wb.forward_fused(t, blk["bn2b"], bn_out=bn_out, residual=main, layout=self.layout)
        if main_bias is not None:
            main = main + main_bias.view(1, -1, 1, 1)
        conv = (lambda m, t: m.forward_reference(t)) if ref else (lambda m, t: m(t, self.math, self.layout))
        t = conv(blk["w2a"], blk["bn2a"](l))
        t = conv(blk["w2b"], blk["bn2b"](t))
        return main + blk["bn2c"](t)

    def forward(self, image, reference=False):
        """image: (B,3,H,W) float32, already normalised.  reference=True computes the Winograd layers with
        float64 einsums instead of this repository's kernels."""
        stem = self.stem
        # the pools between the stages: this library's kernel on NCHW activations (it also hands out relu(pooled), which
        # the next stage's shortcut branch starts from), torch's elsewhere
        own_pool = not reference and self.layout == "NCHW" and image.is_cuda
        own_stem = own_pool and self.math == "tf32" and wg2x2.stem_supported(image.shape[2], image.shape[3])
        pre = self.blocks[0][0]["pre"]
        l_relu = None
        if own_stem:      # conv1 + pool1 (+ the first shortcut's BNReLU) as one tensor-core kernel
            if getattr(self, "_stem_prep", None) is None or self._stem_prep.device != image.device:
                self._stem_prep = wg2x2.stem_prepare(stem.detach().contiguous())
            l, l_relu = wg2x2.stem7x7s2_pool(image.contiguous(), self._stem_prep, with_relu=True,
                                             relu_scale=pre.scale, relu_shift=pre.shift)
        elif (self.layout == "NHWC" or own_pool) and not reference:
            # the stem runs channels-last (cuDNN's faster form for it); for NCHW activations the first pool reads that
            # layout and writes NCHW.  7x7/2 with TensorFlow's SAME padding (2 before, 3 after), written straight
            # into a channels-last buffer
            B_, C_, H_, W_ = image.shape
            x = torch.empty((B_, C_, H_ + 5, W_ + 5), dtype=image.dtype, device=image.device, memory_format=torch.channels_last).zero_()
            x[:, :, 2:2 + H_, 2:2 + W_].copy_(image)
            if getattr(self, "_stem_cl", None) is None or self._stem_cl.device != stem.device:
                self._stem_cl = stem.detach().contiguous(memory_format=torch.channels_last)
            l = F.conv2d(x, self._stem_cl, stride=2)
        else:
            l = F.conv2d(F.pad(image, (2, 3, 2, 3)), stem, stride=2)
        if own_stem:
            pass
        elif own_pool:     # pool1, and relu(BN(pool1)) for the first stage's shortcut from the same pass
            l, l_relu = wg2x2.maxpool3x3s2_same(l, with_relu=True, relu_scale=pre.scale, relu_shift=pre.shift)
        else:
            l = _same_pool(l)
        for s, (blk_a, blk_b) in enumerate(self.blocks):
            if l_relu is not None:
                main = l_relu
            else:
                main = torch.relu(blk_a["pre"](l)) if s == 0 else torch.relu(l)
            if reference or not self.fused:
                main = blk_a["bn1"](F.conv2d(main, blk_a.short))
            else:   # the BatchNorm after the 1x1 shortcut folds into its weights (once) and bias
                if getattr(blk_a, "_short_folded", None) is None or blk_a._short_folded.device != blk_a.short.device:
                    blk_a._short_folded = (blk_a.short * blk_a["bn1"].scale.view(-1, 1, 1, 1)).detach()
                main = F.conv2d(main, blk_a._short_folded)      # its shift is added by the block's last kernel
            l = self._block(blk_a, l, main, reference, main_bias=None if (reference or not self.fused) else blk_a["bn1"].shift)
            l = self._block(blk_b, l, torch.relu(l), reference)
            l_relu = None
            if s < 2 or (s == 2 and self.stage5_pool):
                if own_pool:
                    l, l_relu = wg2x2.maxpool3x3s2_same(l.contiguous(), with_relu=True)
                else:
                    l = _same_pool(l)
        l = torch.relu(l).mean(dim=(2, 3))
        return F.linear(l, self.fc_w, self.fc_b)

    def winograd_layers(self):
        """name -> layer, with the reference's variable names 'Winograd_W<stage><block>_<2a|2b>/W'."""
        out = {}
        for s, (blk_a, blk_b) in enumerate(self.blocks):
            for tag, blk in (("a", blk_a), ("b", blk_b)):
                for conv in ("2a", "2b"):
                    out["Winograd_W%d%s_%s/W" % (s + 2, tag, conv)] = blk["w" + conv]
        return out

    def load_winograd_weights(self, weights, masks=None):
        """Install (16,C,K) weights (and masks) from dicts keyed like the reference checkpoint / mask pickle
        (see wg_weights.load_npz, wg_weights.load_mask_pickle).  Missing names keep their random values."""
        for name, layer in self.winograd_layers().items():
            if name not in weights:
                continue
            w = torch.as_tensor(np.asarray(weights[name]), dtype=torch.float32, device=layer.W.device)
            if tuple(w.shape) != tuple(layer.W.shape):
                raise ValueError("%s: expected %s, got %s" % (name, tuple(layer.W.shape), tuple(w.shape)))
            if masks is not None and name in masks:
                m = torch.as_tensor(np.asarray(masks[name]), dtype=torch.float32, device=layer.W.device)
                layer.mask.copy_(m)
                w = w * m
            layer.W.copy_(w)
            layer._prepared = None

    def winograd_flops(self, batch, size=224):
        """Dense Winograd-domain flops 2*16*P*C*K summed over the 16 layers (independent of the masks)."""
        sp = size // 4
        total = 0
        for s, (cin, cout) in enumerate(STAGES):
            P = batch * ((sp + 1) // 2) ** 2
            total += 2 * 16 * P * (cin * cout + 3 * cout * cout)
            if s < 2 or (s == 2 and self.stage5_pool):
                sp = (sp + 1) // 2
        return total
