"""CPU model of the index arithmetic of the two-shot exchange kernel (csrc/allreduce.cu: ``ar_rank_body``).

Every rank's threads walk the bucket's 16-byte units with the same stride; which unit goes to which slot of which
peer's staging area is pure arithmetic, restated here and checked for what the protocol relies on: every inbox and
outbox slot that is polled is written exactly once per call, nothing else is written, and the slices partition the
bucket - for the world sizes, bucket sizes and launch shapes the library uses.
"""
import itertools

import pytest

THREADS = 128          # AR_THREADS


def _ctas(n_unit, cap=128):
    return max(1, min(cap, (n_unit + 4 * THREADS - 1) // (4 * THREADS)))


def _model(world, n_unit, n_ctas):
    S = n_unit // world
    stride = n_ctas * THREADS
    inbox = [dict() for _ in range(world)]       # per destination rank: slot -> (source rank, unit)
    outbox = [dict() for _ in range(world)]
    polled_in = [set() for _ in range(world)]
    polled_out = [set() for _ in range(world)]
    reduced = [set() for _ in range(world)]
    for r in range(world):
        for t in range(stride):
            # 1. my copy of the other ranks' slices -> their inbox, row r
            for u in range(t, n_unit, stride):
                p = u // S
                if p == r:
                    continue
                slot = r * S + (u - p * S)
                assert slot not in inbox[p], "an inbox slot written twice"
                inbox[p][slot] = (r, u)
            # 2. my slice: poll the others' rows, push the sum to every other rank's outbox
            for j in range(t, S, stride):
                u = r * S + j
                for p in range(world):
                    if p != r:
                        polled_in[r].add(p * S + j)
                assert u not in reduced[r]
                reduced[r].add(u)
                for q in range(world):
                    if q != r:
                        assert u not in outbox[q], "an outbox slot written twice"
                        outbox[q][u] = r
            # 3. the other ranks' slices: from my outbox into my bucket
            for u in range(t, n_unit, stride):
                if u // S != r:
                    polled_out[r].add(u)
    return S, inbox, outbox, polled_in, polled_out, reduced


@pytest.mark.parametrize("world,n_unit,n_ctas", [(2, 8, 1), (2, 124488, 128), (3, 24, 1), (4, 124488, 128),
                                                 (8, 124488, 128), (8, 124488, 16), (8, 64, 1), (16, 1024, 2)])
def test_every_polled_slot_is_written_exactly_once(world, n_unit, n_ctas):
    S, inbox, outbox, polled_in, polled_out, reduced = _model(world, n_unit, n_ctas)
    assert S * world == n_unit
    for r in range(world):
        assert set(inbox[r]) == polled_in[r] and len(inbox[r]) == (world - 1) * S
        for slot, (src, u) in inbox[r].items():
            assert slot // S == src and u // S == r and u - r * S == slot - src * S      # row = source, same offset
        assert set(outbox[r]) == polled_out[r] == {u for u in range(n_unit) if u // S != r}
        assert all(owner == u // S for u, owner in outbox[r].items())                   # pushed by the slice's owner
        assert reduced[r] == set(range(r * S, (r + 1) * S))
    assert set(itertools.chain.from_iterable(reduced)) == set(range(n_unit))


def test_launch_shape_used_by_the_library():
    """The CTA count is a function of the bucket size alone, so every rank launches the same shape, and it stays the
    same from call to call for one bucket - which the per-CTA call counters (one per CTA, advanced once per call)
    rely on: a bucket's counters and staging areas must not be shared with a bucket of another size."""
    from eccv26_tad_b200.distributed import padded_numel
    n_pad = padded_numel(3 * (9 * 192 * 192 + 192), 8)
    assert n_pad % (64 * 8) == 0
    assert _ctas(n_pad // 8) == 128 and _ctas(8) == 1 and _ctas(4 * THREADS + 1) == 2
