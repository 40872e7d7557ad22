"""Data-parallel helpers: the op shards by clip, the only exchange is the weight-gradient all-reduce.

The reference trains under torch DDP (``src/eccv26_tad.py:288-300``): clips are split over ranks by a
``DistributedSampler`` and DDP all-reduces the adapter gradients.  Here the same two steps are explicit.
"""
import torch
import torch.distributed as dist


def shard_clips(n_clips, rank, world_size):
    """Contiguous block split of ``range(n_clips)``; the first ``n_clips % world_size`` ranks get one more."""
    base, extra = divmod(n_clips, world_size)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))


def allreduce_weight_grads(grad_weight, grad_bias=None, group=None, bucket=None):
    """Sum ``grad_weight`` (and ``grad_bias``) over ranks with ONE collective on a flat bucket.

    Returns views into the bucket shaped like the inputs.  ``bucket`` may be a preallocated flat tensor
    (``grad_weight.numel() + grad_bias.numel()`` elements) that the caller's kernels already wrote into.
    """
    n_w = grad_weight.numel()
    n_b = grad_bias.numel() if grad_bias is not None else 0
    if bucket is None:
        bucket = torch.empty(n_w + n_b, dtype=grad_weight.dtype, device=grad_weight.device)
        bucket[:n_w].copy_(grad_weight.reshape(-1))
        if n_b:
            bucket[n_w:].copy_(grad_bias.reshape(-1))
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(bucket, op=dist.ReduceOp.SUM, group=group)
    gw = bucket[:n_w].view(grad_weight.shape)
    gb = bucket[n_w:].view(grad_bias.shape) if n_b else None
    return gw, gb
