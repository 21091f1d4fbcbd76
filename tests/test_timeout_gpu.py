"""The bounded device-side waits of the tensor-core kernels, made to run out on purpose.

Nothing here faults or hangs the GPU: a wait that runs out makes its role record where it was and leave, the
other roles follow, the kernel frees its tensor memory and returns, and the host reads WG2X2_ERR_TIMEOUT from
wg2x2_last_device_status.  The waits are made to run out by (a) a one-thread probe kernel that waits on a
barrier nobody arrives on, and (b) the test hook wg2x2_test_drop_load, with which CTA 0's weight producer stops
before one load -- so that nothing is in flight -- under a poll limit of a few thousand.  After each case a
normal call must give the right result again.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

TIMEOUT = -4
TOL_TF32 = 5e-3


@pytest.fixture()
def wg():
    import wg2x2
    from wg2x2._lib import lib
    yield wg2x2
    lib.wg2x2_test_drop_load(-1)
    lib.wg2x2_set_wait_limit(0)
    wg2x2.last_device_status()      # leave no stale status behind


def _layer_inputs(shape, seed=11):
    B, H, W, C, K = shape
    rng = np.random.default_rng(seed)
    X = rng.standard_normal((B, C, H, W)).astype(np.float32)
    Wt = (0.05 * rng.standard_normal((16, C, K))).astype(np.float32)
    return X, Wt


def test_wait_probe_reports_timeout_once(wg):
    from wg2x2._lib import lib
    assert wg.last_device_status()[0] == 0
    assert lib.wg2x2_test_wait_probe(10000, 0x1F42, None) == 0
    st, where = wg.last_device_status()
    assert st == TIMEOUT and where == 0x1F42
    st, _ = wg.last_device_status()              # reading cleared it
    assert st == 0
    assert lib.wg2x2_test_wait_probe(0, 1, None) == -1      # a limit of zero polls is refused


@pytest.mark.parametrize("nth", [0, 5])
def test_row_walk_kernel_times_out_and_recovers(wg, oracle, nth):
    from wg2x2._lib import lib
    shape = (2, 14, 14, 64, 64)
    B, H, W, C, K = shape
    X, Wt = _layer_inputs(shape)
    Xn = np.ascontiguousarray(np.transpose(X, (0, 2, 3, 1)))
    V = oracle.imtrans_fwd(Xn, relu=True, dtype=np.float32)
    Vd, prepared = torch.from_numpy(V).cuda(), wg.prepare_weights(torch.from_numpy(Wt).cuda())
    lib.wg2x2_set_wait_limit(20000)
    lib.wg2x2_test_drop_load(nth)
    wg.conv_fwd_prepared(Vd, prepared, K, H, W, wide=False)          # returns: the kernel gave up and left
    st, where = wg.last_device_status()
    assert st == TIMEOUT
    # the MMA issuer waiting for the stage that never came (0x3, low byte = stage index), or the epilogue, which
    # has been waiting for the accumulators since the kernel began and may run out first (0x4)
    assert (where >> 8) in (0x3, 0x4), "0x%x" % where
    if (where >> 8) == 0x3:
        assert (where & 0xFF) == nth % 8
    lib.wg2x2_set_wait_limit(0)
    Y = wg.conv_fwd_prepared(Vd, prepared, K, H, W, wide=False).cpu().numpy()
    assert wg.last_device_status()[0] == 0
    assert oracle.max_rel(Y, oracle.conv_fwd(V, Wt, H, W)) <= TOL_TF32


@pytest.mark.parametrize("nth", [0, 3])
def test_fused_layer_kernel_times_out_and_recovers(wg, oracle, nth):
    from wg2x2._lib import lib
    shape = (2, 16, 16, 64, 64)
    B, H, W, C, K = shape
    X, Wt = _layer_inputs(shape)
    Xd, prepared = torch.from_numpy(X).cuda(), wg.prepare_weights(torch.from_numpy(Wt).cuda())
    lib.wg2x2_set_wait_limit(20000)
    lib.wg2x2_test_drop_load(nth)
    wg.layer_fwd_fused(Xd, prepared, K, relu=True)
    st, where = wg.last_device_status()
    assert st == TIMEOUT
    # whichever role ran out first names itself: an MMA issuer waiting for the slot (0x10..0x13), a transform
    # team waiting for its input rows or its A group (0x0B, 0x0C), a producer waiting for a free buffer (0x09, 0x0A) or the epilogue (0x04, 0x05)
    assert (where >> 8) in (0x10, 0x11, 0x12, 0x13, 0x0C, 0x0B, 0x0A, 0x09, 0x04, 0x05), "0x%x" % where
    lib.wg2x2_set_wait_limit(0)
    Y = wg.layer_fwd_fused(Xd, prepared, K, relu=True).cpu().numpy()
    assert wg.last_device_status()[0] == 0
    Xn = np.ascontiguousarray(np.transpose(X, (0, 2, 3, 1)))
    want = oracle.conv_fwd(oracle.imtrans_fwd(Xn, relu=True, dtype=np.float32), Wt, H, W)
    assert oracle.max_rel(np.transpose(Y, (0, 2, 3, 1)), want) <= TOL_TF32
