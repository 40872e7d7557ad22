"""CPU tier: a model of the kernels' buffer ring (host logic only, no GPU code is exercised).

The tensor-core kernels hand 64-deep buffers from producer warps to the MMA thread through mbarriers that only
expose the PARITY of their phase.  Producer warp w owns the steps g with g % P == w and, before refilling buffer
g % S, waits until the buffer's "empty" barrier has completed (g // S) phases - which it can only test modulo 2.
The library therefore lets at most min(P, S) warps produce (``n_prod`` in csrc/conv_tc_hybrid.cu and
csrc/conv_tc_pair.cu).  This model replays random interleavings and checks the two facts behind that rule:
with P <= S no interleaving lets a producer overwrite a buffer the consumer has not read, and with P > S some
interleaving does."""
import random


def run(P, S, steps, seed, max_events=200000):
    """Returns True if some producer refilled a buffer that still held an unconsumed step."""
    rng = random.Random(seed)
    empty_phases = [0] * S          # completed phases of each buffer's "empty" barrier (one per consumed step)
    holds = [None] * S              # step currently stored in the buffer, None once consumed
    filled = set()                  # steps whose data has landed
    next_step = list(range(P))      # next step of each producer warp
    consumed = 0
    for _ in range(max_events):
        if consumed == steps:
            return False
        actors = [("p", w) for w in range(P) if next_step[w] < steps] + [("c", 0)]
        kind, w = rng.choice(actors)
        if kind == "p":
            g = next_step[w]
            b, use = g % S, g // S
            # parity wait: passes when the number of completed phases has the parity of `use`
            if empty_phases[b] % 2 != use % 2:
                continue
            if holds[b] is not None:
                return True         # the buffer still holds a step the consumer has not read
            holds[b] = g
            filled.add(g)
            next_step[w] += P
        else:
            g = consumed
            if g in filled and holds[g % S] == g:
                holds[g % S] = None
                empty_phases[g % S] += 1
                consumed += 1
    return False


def test_no_overwrite_when_producers_do_not_outnumber_buffers():
    for P, S in [(1, 2), (2, 2), (4, 4), (4, 5), (4, 8), (3, 3), (2, 6)]:
        for seed in range(60):
            assert not run(P, S, steps=40, seed=seed), (P, S, seed)


def test_overwrite_is_possible_with_more_producers_than_buffers():
    for P, S in [(4, 2), (4, 3), (6, 5), (8, 5)]:
        assert any(run(P, S, steps=40, seed=seed) for seed in range(400)), (P, S)
