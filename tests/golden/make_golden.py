"""Generate tests/golden/ref_cuda_*.npz from the reference's own CUDA kernels.

Needs a GPU and oracle/_ref/libwg_ref_cuda.so (make -C oracle ref: the upstream *.cu.cc files
compiled unmodified for sm_100a).  For each case it draws seeded inputs, runs the four upstream
launchers and stores inputs and outputs.  Shapes are the ones the reference's own test scripts
use (B=3, 6x6, (C,K) in (32,32), (32,64), (5,7); winograd2x2_imTrans_test.py:160-163,
winograd2x2_imTrans_grad_test.py:158-161, winograd2x2_conv_grad_test.py:160-163) plus two
larger even-sized ones.  Only even image sizes: the upstream gradient kernels read out of
bounds for odd ones.

    python tests/golden/make_golden.py [outdir]      (default: tests/golden/_new)
"""
import ctypes
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
CASES = [  # name, B, H, W, C, K
    ("b3_6x6_c32_k32", 3, 6, 6, 32, 32),
    ("b3_6x6_c32_k64", 3, 6, 6, 32, 64),
    ("b3_6x6_c5_k7", 3, 6, 6, 5, 7),
    ("b2_8x12_c16_k24", 2, 8, 12, 16, 24),
    ("b1_14x14_c64_k48", 1, 14, 14, 64, 48),
]


def main():
    out = sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden", "_new")
    os.makedirs(out, exist_ok=True)
    ref = ctypes.CDLL(os.path.join(ROOT, "oracle", "_ref", "libwg_ref_cuda.so"))
    dev = torch.device("cuda:0")
    P = ctypes.c_void_p
    for name, B, H, W, C, K in CASES:
        rng = np.random.default_rng(sum(map(ord, name)))
        nH, nW = H // 2, W // 2
        X = rng.standard_normal((B, H, W, C)).astype(np.float32)
        Wt = (0.05 * rng.standard_normal((16, C, K))).astype(np.float32)
        dY = rng.standard_normal((B, H, W, K)).astype(np.float32)
        x = torch.from_numpy(X).to(dev)
        wt = torch.from_numpy(Wt).to(dev)
        dy = torch.from_numpy(dY).to(dev)
        V = torch.empty((16, B, nH, nW, C), device=dev)
        ref.wgref_imtrans(P(x.data_ptr()), P(V.data_ptr()), C, B, H, W)
        Vr = torch.relu(V)  # the layer wrapper's nl=tf.nn.relu
        Y = torch.empty((B, H, W, K), device=dev)
        tmp = torch.empty(16 * B * nH * nW * K, device=dev)
        ptrs = torch.empty(80, dtype=torch.int64, device=dev)
        ref.wgref_conv(P(Vr.data_ptr()), P(wt.data_ptr()), P(Y.data_ptr()), P(tmp.data_ptr()), P(ptrs.data_ptr()), C, B, nH, nW, K)
        dV = torch.empty_like(V)
        dW = torch.empty_like(wt)
        ref.wgref_conv_grad(P(Vr.data_ptr()), P(wt.data_ptr()), P(dy.data_ptr()), P(dV.data_ptr()), P(dW.data_ptr()),
                            P(tmp.data_ptr()), P(ptrs.data_ptr()), C, B, H, W, K)
        dVm = (dV * (Vr > 0)).contiguous()  # ReluGrad, as autodiff inserts it
        dVc = dVm.clone()                   # the upstream launcher transforms its input in place
        dX = torch.empty_like(x)
        ref.wgref_imtrans_grad(P(dVc.data_ptr()), P(dX.data_ptr()), C, B, H, W)
        torch.cuda.synchronize()
        np.savez_compressed(os.path.join(out, "ref_cuda_%s.npz" % name), X=X, Wt=Wt, dY=dY, V=V.cpu().numpy(),
                            Y=Y.cpu().numpy(), dV=dV.cpu().numpy(), dW=dW.cpu().numpy(), dX=dX.cpu().numpy())
        print("wrote", name)


if __name__ == "__main__":
    main()
