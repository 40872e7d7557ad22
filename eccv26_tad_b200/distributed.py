"""Data-parallel helpers: the op shards by clip, the only exchange is the weight-gradient all-reduce.

The reference trains under torch DDP (``src/eccv26_tad.py:288-300``): clips are split over ranks by a
``DistributedSampler`` and DDP all-reduces the adapter gradients.  Here the same two steps are explicit:
``shard_clips`` and a flat gradient bucket that every rank's kernels write into and one collective sums.
"""
import ctypes
import os

import torch
import torch.distributed as dist

from . import _lib


def shard_clips(n_clips, rank, world_size):
    """Contiguous block split of ``range(n_clips)``; the first ``n_clips % world_size`` ranks get one more."""
    base, extra = divmod(n_clips, world_size)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))


def slice_bounds(numel, rank, world_size):
    """The part of a bucket of ``numel`` 16-bit elements that ``rank`` sums in the two-shot exchange, as
    ``(first, last)`` element indices.  Mirrors the kernel (csrc/allreduce.cu): the bucket is cut into
    ``world_size`` slices of whole 16-byte units (8 elements)."""
    if numel % (8 * world_size):
        raise ValueError(f"a bucket of {numel} elements is not a multiple of 8 * {world_size}: pad it")
    per_rank = numel // world_size
    return rank * per_rank, (rank + 1) * per_rank


def padded_numel(numel, world_size):
    """Smallest bucket size >= numel whose slices are whole 128-byte lines (64 elements) on every rank."""
    q = 64 * world_size
    return -(-numel // q) * q


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


def _peer_exchange_possible(device, group):
    """This rank's own view: 16-bit bucket on a CUDA device of a single node where every GPU can address every
    other one, with torch's symmetric-memory allocator present.  No collective, no symmetric-memory call."""
    try:
        if device.type != "cuda":
            return False
        import torch.distributed._symmetric_memory as symm_mem   # noqa: F401
        world = dist.get_world_size(group)
        if world > 16 or torch.cuda.device_count() < world:
            return False
        if int(os.environ.get("LOCAL_WORLD_SIZE", world)) != world:      # more than one node
            return False
        me = device.index if device.index is not None else torch.cuda.current_device()
        return all(j == me or torch.cuda.can_device_access_peer(me, j) for j in range(torch.cuda.device_count()))
    except Exception:
        return False


class GradBucket:
    """Flat gradient bucket of ``numel`` elements that every rank's kernels write into and ``all_reduce()`` sums.

    ``exchange="collective"`` (default): an ordinary tensor, summed by ``dist.all_reduce`` (NCCL on CUDA, gloo on
    CPU).

    ``exchange="peer"``: the bucket is placed in memory that every rank of the node maps (torch's symmetric-memory
    allocator does the allocation and the handle exchange; multicast is not used) and summed by this library's own
    two-shot kernel (``svtad_allreduce_sum``: plain stores over NVLink that carry their own flags, bounded waits).  Whether that is
    possible is decided ONCE FOR ALL RANKS before any symmetric-memory call: every rank evaluates its own
    capabilities on the host and the minimum over the ranks is taken with one ordinary all-reduce on the default
    path.  If any rank says no, every rank uses the collective path.  After a unanimous yes, a failure of the
    set-up raises on the rank that saw it - it never falls back on its own, because a rank that left the set-up
    while its peers are still inside it would issue collectives the others never enter.

    ``kind`` says which exchange is in use.  Both can be captured into a CUDA graph; call ``all_reduce()`` once
    eagerly first.
    """

    def __init__(self, numel, dtype, device, group=None, exchange="collective"):
        if exchange not in ("collective", "peer"):
            raise ValueError("exchange must be 'collective' or 'peer'")
        self.group = group
        self.kind = "none"
        self.numel = numel
        device = torch.device(device)
        world = dist.get_world_size(group) if (dist.is_available() and dist.is_initialized()) else 1
        self._peer = None
        self.buffer = None
        use_peer = False
        if world > 1 and exchange == "peer":
            mine = 1 if (dtype in (torch.bfloat16, torch.float16) and _peer_exchange_possible(device, group)) else 0
            vote = torch.tensor([mine], dtype=torch.int32, device=device if device.type == "cuda" else "cpu")
            dist.all_reduce(vote, op=dist.ReduceOp.MIN, group=group)       # the one decision, taken by all ranks
            use_peer = bool(int(vote.item()))
            if not use_peer:
                self.fallback_reason = "not every rank can take part in the peer-memory exchange"
        if use_peer:
            self._setup_peer(numel, dtype, device, group, world)       # raises on failure, see the class docstring
        else:
            self.buffer = torch.zeros(numel, dtype=dtype, device=device)
            self.kind = "nccl" if device.type == "cuda" and world > 1 else ("gloo" if world > 1 else "none")

    def _setup_peer(self, numel, dtype, device, group, world):
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")      # plain peer memory only
        import torch.distributed._symmetric_memory as symm_mem
        lib = _lib.load()
        pg = group if group is not None else dist.group.WORLD
        n_pad = padded_numel(numel, world)
        stage_elems = lib.svtad_allreduce_stage_bytes(n_pad) // 2
        buf = symm_mem.empty(n_pad + stage_elems, dtype=dtype, device=device)
        hdl = symm_mem.rendezvous(buf, pg)
        buf.zero_()                                   # staging areas (and padding) start at zero on every rank ...
        torch.cuda.synchronize(device)
        dist.barrier(group=group)                     # ... before any rank's first exchange can write into them
        ptrs = [int(p) for p in hdl.buffer_ptrs]
        if len(ptrs) != world or int(hdl.rank) != dist.get_rank(group):
            raise RuntimeError("symmetric-memory handle does not match the process group")
        self._peer = {
            "hdl": hdl,
            "ptrs": (ctypes.c_void_p * world)(*ptrs),
            "rank": int(hdl.rank),
            "world": world,
            "n_pad": n_pad,
            "stage_off": n_pad * 2,
            "epoch": torch.zeros(lib.svtad_allreduce_epoch_bytes() // 4, dtype=torch.int32, device=device),
            "dtype": _lib.BF16 if dtype == torch.bfloat16 else _lib.F16,
            "limit": int(os.environ.get("SVTAD_ALLREDUCE_WAIT_CYCLES", "0")),
        }
        self._full = buf
        self.buffer = buf[:n_pad]
        self.kind = "svtad two-shot over peer memory"

    def view(self, offset, shape):
        n = 1
        for d in shape:
            n *= d
        return self.buffer[offset:offset + n].view(shape)

    def all_reduce(self):
        """Sums the bucket over the group in place (on the current stream); returns the bucket's first numel elements."""
        if self._peer is not None:
            p = self._peer
            stream = torch.cuda.current_stream(self.buffer.device).cuda_stream
            with torch.cuda.device(self.buffer.device):
                _lib.check(_lib.load().svtad_allreduce_sum(p["ptrs"], p["rank"], p["world"], p["n_pad"], p["dtype"],
                                                           p["stage_off"], p["epoch"].data_ptr(), p["limit"], stream))
        elif self.kind != "none":
            dist.all_reduce(self.buffer, op=dist.ReduceOp.SUM, group=self.group)
        return self.buffer[:self.numel]
