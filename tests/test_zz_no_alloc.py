"""The weight-gradient entry point that allocates nothing (wg2x2_conv_bwd_dw_noalloc).

Some callers of this library may not allocate device memory: a framework hook that is handed
only the op's inputs and outputs, a process that forbids cudaMalloc once it is running, a
plug-in whose host application owns all of the GPU's memory.  For them the split-P partial
sums of dW go to a fixed array inside the library.  This file is collected last on purpose, and
must pass both alone in a fresh process and after every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = 1e-5  # the FP32-path tolerance of the other parity tests (max|a-b| / max|b|)


def _max_rel(a, b):
    return float((a.double() - b.double()).abs().max() / (b.double().abs().max() + 1e-300))


@pytest.mark.parametrize("layout,shape", [(0, (8, 28, 28, 64, 64)), (1, (6, 14, 14, 32, 48)), (0, (2, 7, 7, 20, 12))])
def test_noalloc_matches_workspace_entry_point_twice(layout, shape):
    from wg2x2._lib import lib
    B, H, W, C, K = shape
    nH, nW = (H + 1) // 2, (W + 1) // 2
    g = torch.Generator(device="cuda").manual_seed(5)
    V = torch.relu(torch.randn((16, B, nH, nW, C), device="cuda", generator=g))
    dY = torch.randn((B, H, W, K) if layout == 0 else (B, K, H, W), device="cuda", generator=g)
    mask = (torch.rand((16, C, K), device="cuda", generator=g) < 0.4).float()
    P = ctypes.c_void_p
    st = torch.cuda.current_stream().cuda_stream
    nws = lib.wg2x2_conv_bwd_workspace_bytes(B, H, W, C, K, 0, 1)
    assert nws > 0, "pick shapes whose dW contraction is split, so that scratch is really used"
    ws = torch.empty(nws, dtype=torch.uint8, device="cuda")
    want = torch.empty((16, C, K), device="cuda")
    assert lib.wg2x2_conv_bwd(P(V.data_ptr()), None, P(dY.data_ptr()), P(mask.data_ptr()), None, P(want.data_ptr()),
                              B, H, W, C, K, layout, 0, 0, P(ws.data_ptr()), nws, P(st)) == 0
    got = torch.empty((16, C, K), device="cuda")
    for call in range(2):   # two calls in a row share the built-in array
        got.fill_(float("nan"))
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]   # nothing but the C call runs between the two readings
        status = lib.wg2x2_conv_bwd_dw_noalloc(P(V.data_ptr()), P(dY.data_ptr()), P(mask.data_ptr()), P(got.data_ptr()),
                                               B, H, W, C, K, layout, P(st))
        torch.cuda.synchronize()
        free_after = torch.cuda.mem_get_info()[0]
        assert status == 0
        if call == 1:
            # the first call on a device may make the driver load the library's module, and with it
            # the built-in array; from then on free memory must not move
            assert free_after >= free_before - (1 << 20), "the entry point must not allocate device memory"
        assert torch.isfinite(got).all()
        assert _max_rel(got, want) <= TOL, "call %d" % call
        # same split count and the same order of additions as the workspace entry point: the very same bits
        assert torch.equal(got, want), "call %d" % call


def test_noalloc_rejects_sizes_beyond_the_builtin_scratch():
    from wg2x2._lib import lib
    cap = lib.wg2x2_conv_bwd_dw_noalloc_max_bytes()
    assert cap == 32 << 20
    # C=512, K=576: dW is 18.9 MB and the contraction is split in two -> 37.7 MB of partial sums
    B, H, W, C, K = 2, 8, 8, 512, 576
    assert lib.wg2x2_conv_bwd_workspace_bytes(B, H, W, C, K, 0, 1) > cap
    one = ctypes.c_void_p(256)
    assert lib.wg2x2_conv_bwd_dw_noalloc(one, one, None, one, B, H, W, C, K, 0, None) == -2
    assert lib.wg2x2_conv_bwd_dw_noalloc(None, one, None, one, B, H, W, 8, 8, 0, None) == -1
