"""Batch sharding of the Winograd-ReLU layer over the GPUs of one box.

Every tile of the layer depends only on its own image and on the (replicated) weights, so the
batch axis -- outermost in X, V and Y for both layouts -- splits into contiguous slabs with no
exchange on the forward path.  The reference reaches the same split through tensorpack's
SyncMultiGPUTrainerParameterServer, which gives each tower batch // n_gpu images
(ResNet-18-var/imagenet-resnet-transWino-prune.py:376,391).  A collective appears only when the
caller wants the whole output on every rank (`gather_batch`), or, for a sharded backward pass,
the one all-reduce of dW (`allreduce_weight_grad`).
"""
import torch
import torch.distributed as dist


def shard_range(n, world_size, rank):
    """Contiguous [start, stop) of rank's share of n items; the first n % world_size ranks get one more."""
    if not (0 <= rank < world_size):
        raise ValueError("rank %d outside world of %d" % (rank, world_size))
    base, extra = divmod(n, world_size)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_sizes(n, world_size):
    return [shard_range(n, world_size, r)[1] - shard_range(n, world_size, r)[0] for r in range(world_size)]


def gather_batch(y_local, n_total, group=None):
    """All-gather batch shards (dim 0) into the full batch on every rank; shards may differ by one image."""
    world = dist.get_world_size(group)
    sizes = shard_sizes(n_total, world)
    if y_local.shape[0] != sizes[dist.get_rank(group)]:
        raise ValueError("local shard has %d items, expected %d" % (y_local.shape[0], sizes[dist.get_rank(group)]))
    biggest = max(sizes)
    if y_local.shape[0] < biggest:   # pad to a common size; NCCL all_gather wants equal shapes
        pad = torch.zeros((biggest - y_local.shape[0],) + tuple(y_local.shape[1:]), dtype=y_local.dtype, device=y_local.device)
        y_send = torch.cat([y_local, pad], 0)
    else:
        y_send = y_local.contiguous()
    parts = [torch.empty_like(y_send) for _ in range(world)]
    dist.all_gather(parts, y_send, group=group)
    return torch.cat([p[:s] for p, s in zip(parts, sizes)], 0)


def allreduce_weight_grad(dW, group=None):
    """Sum of the per-shard weight gradients: the only exchange a sharded backward pass needs."""
    dist.all_reduce(dW, op=dist.ReduceOp.SUM, group=group)
    return dW


def sharded_layer_fwd(x_full, Wt, layer_fn, gather=True, group=None):
    """Run `layer_fn(x_shard, Wt)` on this rank's slab of x_full (dim 0 = batch) and optionally gather."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    lo, hi = shard_range(x_full.shape[0], world, rank)
    y_local = layer_fn(x_full[lo:hi].contiguous(), Wt)
    return gather_batch(y_local, x_full.shape[0], group) if gather else y_local
