"""Batch sharding over ranks (the N>1 path), exercised with two gloo processes on CPU; the per-shard
layer computation is played by the CPU oracle so that only the host-side logic is under test."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def test_shard_ranges_cover_the_batch():
    from wg2x2.shard import shard_range, shard_sizes
    for n in (1, 2, 7, 64, 255, 256):
        for world in (1, 2, 3, 4, 8):
            spans = [shard_range(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = shard_sizes(n, world)
            assert sum(sizes) == n and max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_range(4, 2, 2)


def _worker(rank, world, port, n_batch, result_dir):
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path[:0] = [root, os.path.join(root, "sparse-winograd-cnn_b200")]
    from oracle import wg_oracle as o
    from wg2x2 import shard
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(0)   # same seed on every rank: the full batch, as a loader would give it
        H, W, C, K = 6, 7, 8, 12
        X = rng.standard_normal((n_batch, H, W, C)).astype(np.float32)
        Wt = (0.1 * rng.standard_normal((16, C, K))).astype(np.float32)
        dY = rng.standard_normal((n_batch, H, W, K)).astype(np.float32)

        def layer(x, w):
            return torch.from_numpy(o.layer_fwd(x.numpy(), w.numpy(), relu=True, dtype=np.float32))

        y = shard.sharded_layer_fwd(torch.from_numpy(X), torch.from_numpy(Wt), layer, gather=True)
        want = o.layer_fwd(X, Wt, relu=True, dtype=np.float32)
        assert y.shape == want.shape and np.array_equal(y.numpy(), want)   # same code, same bits, any split
        # sharded backward: per-shard dW summed by one all-reduce equals the full-batch dW
        lo, hi = shard.shard_range(n_batch, world, rank)
        V = o.imtrans_fwd(X[lo:hi], relu=True)
        _, dW = o.conv_bwd(V, Wt, dY[lo:hi]) if hi > lo else (None, np.zeros((16, C, K)))
        dW = shard.allreduce_weight_grad(torch.from_numpy(np.ascontiguousarray(dW)))
        _, dW_full = o.conv_bwd(o.imtrans_fwd(X, relu=True), Wt, dY)
        assert np.allclose(dW.numpy(), dW_full, rtol=1e-10, atol=1e-10)
        open(os.path.join(result_dir, "ok%d" % rank), "w").close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n_batch", [5, 8])
def test_two_rank_sharded_layer_gloo(tmp_path, n_batch):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), n_batch, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / ("ok%d" % r)).exists() for r in range(world))
