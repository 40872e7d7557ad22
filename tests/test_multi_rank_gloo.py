"""CPU tier: the N > 1 path on two gloo ranks.  Clips are independent, so summing the per-rank weight
gradients (one flat all-reduce) must equal the single-rank gradient of the whole batch; forward and
input-gradient rows of a rank's clips must equal the same rows of the whole-batch result."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from eccv26_tad_b200.distributed import GradBucket, allreduce_weight_grads, padded_numel, shard_clips, slice_bounds
from oracle import conv as oconv
from oracle import table as otab

CLIPS, T, H, W, C, K_KEEP = 5, 2, 6, 6, 8, 11


def _problem():
    rng = np.random.default_rng(17)
    scores = rng.standard_normal((CLIPS * T, H * W)).astype(np.float32)
    kept, table = otab.build_table(scores, K_KEEP, H, W, 3)
    n = table.shape[0]
    x = rng.standard_normal((n, C)).astype(np.float32)
    gy = rng.standard_normal((n, C)).astype(np.float32)
    w = rng.standard_normal((9, C, C)).astype(np.float32)
    return table, x, gy, w


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        table, x, gy, w = _problem()
        rows_per_clip = T * K_KEEP
        clips = shard_clips(CLIPS, rank, world)
        lo, hi = clips.start * rows_per_clip, clips.stop * rows_per_clip
        # a rank's table is rank-local: renumber its rows from zero
        tab = table[lo:hi].copy()
        tab[tab >= 0] -= lo
        y = oconv.fwd(x[lo:hi], tab, w, None)
        gx = oconv.dgrad(gy[lo:hi], tab, w)
        gw, gb = oconv.wgrad(gy[lo:hi], x[lo:hi], tab, 9)
        gw_t, gb_t = allreduce_weight_grads(torch.from_numpy(gw), torch.from_numpy(gb))
        # the same sum through the bucket object (on CPU / gloo it is an ordinary tensor + dist.all_reduce)
        bucket = GradBucket(gw.size + gb.size, torch.float64, "cpu")
        bucket.view(0, gw.shape).copy_(torch.from_numpy(gw))
        bucket.view(gw.size, gb.shape).copy_(torch.from_numpy(gb))
        flat = bucket.all_reduce()
        assert bucket.kind == "gloo"
        assert torch.equal(flat[:gw.size].view(gw.shape), gw_t) and torch.equal(flat[gw.size:], gb_t)
        # asking for the peer-memory exchange where it cannot work (CPU ranks): the decision is taken once for all
        # ranks by a collective BEFORE any set-up call, so both ranks land on the collective path together
        b16 = GradBucket(gw.size + gb.size, torch.bfloat16, "cpu", exchange="peer")
        assert b16.kind == "gloo" and "not every rank" in b16.fallback_reason
        b16.buffer.copy_(torch.arange(b16.numel, dtype=torch.float32).remainder(7).to(torch.bfloat16) * (rank + 1))
        s16 = b16.all_reduce()
        assert torch.equal(s16.float(), torch.arange(b16.numel, dtype=torch.float32).remainder(7) * 3)
        out[rank] = dict(lo=lo, hi=hi, y=y, gx=gx, gw=gw_t.numpy().copy(), gb=gb_t.numpy().copy())
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_match_single_rank():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(2, port, out), nprocs=2, join=True)
        out = dict(out)
    table, x, gy, w = _problem()
    y = oconv.fwd(x, table, w, None)
    gx = oconv.dgrad(gy, table, w)
    gw, gb = oconv.wgrad(gy, x, table, 9)
    covered = 0
    for r in (0, 1):
        o = out[r]
        np.testing.assert_allclose(o["y"], y[o["lo"]:o["hi"]], rtol=0, atol=1e-12)
        np.testing.assert_allclose(o["gx"], gx[o["lo"]:o["hi"]], rtol=0, atol=1e-12)
        np.testing.assert_allclose(o["gw"], gw, rtol=1e-12, atol=1e-12)
        np.testing.assert_allclose(o["gb"], gb, rtol=1e-12, atol=1e-12)
        covered += o["hi"] - o["lo"]
    assert covered == table.shape[0]


def test_two_shot_slices_partition_the_bucket():
    """The slices of the peer-memory exchange cover the bucket exactly once, in whole 16-byte units."""
    for numel, world in [(995904, 8), (995904, 2), (1024, 4), (64 * 3, 3), (padded_numel(1000, 8), 8)]:
        seen = np.zeros(numel, dtype=np.int32)
        for r in range(world):
            lo, hi = slice_bounds(numel, r, world)
            assert lo % 8 == 0 and hi % 8 == 0 and hi - lo == numel // world
            seen[lo:hi] += 1
        assert (seen == 1).all()
    assert padded_numel(995904, 8) % (64 * 8) == 0 and padded_numel(995904, 8) - 995904 < 64 * 8
    import pytest
    with pytest.raises(ValueError):
        slice_bounds(100, 0, 8)


def test_shard_clips_partitions():
    for n, world in [(8, 1), (8, 2), (8, 8), (5, 2), (3, 4)]:
        seen = []
        for r in range(world):
            seen += list(shard_clips(n, r, world))
        assert seen == list(range(n))
