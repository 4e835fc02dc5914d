"""CPU model of the flag / epoch protocol of the peer-memory all-reduce (muxserve_b200/csrc/tp_allreduce.cu).

The kernel's correctness argument is about ORDER, not arithmetic: CTA b of rank r only talks to CTA b of the other
ranks; its call counter in the exchange buffer is the epoch; flags carry the epoch; the data areas alternate with
the epoch's parity, and a rank can start epoch e + 2 only after every peer raised its flag of e + 1, i.e. finished
reading e.  This test runs that protocol — the same steps in the same order, one generator per (rank, CTA), every
remote store and every poll a scheduling point — under many random interleavings of several back-to-back calls and
checks that every value read carries the epoch it is read for and that all ranks end with the rank-order sum.  A
variant without the alternating areas must be caught by the same check (the test has teeth).

No GPU and no library call: the GPU tests (tests/test_gpu_tp_allreduce.py, tests/test_gpu_tp_multi.py) check the
kernel itself; this checks the reasoning the kernel rests on, on schedules no GPU run will ever produce on demand.
"""
import random

import pytest


class Buffer:
    """One rank's exchange buffer: per-CTA call counters, flags, and data areas by (parity, area, source/slice)."""

    def __init__(self, world, ctas):
        self.epoch = [0] * ctas
        self.ready = [[0] * ctas for _ in range(world)]
        self.done = [[0] * ctas for _ in range(world)]
        self.data = {}


class Violation(AssertionError):
    pass


def value(rank, cta, epoch):
    return (rank + 1) * 1000 + cta * 100 + epoch


def one_shot(bufs, r, c, calls, out, parity_areas=True):
    world = len(bufs)
    my = bufs[r]
    for _ in range(calls):
        e = my.epoch[c] + 1
        par = e & 1 if parity_areas else 0
        for q in range(world):                      # push my chunk into area [r] of every rank
            bufs[q].data[(par, "a", r, c)] = (e, value(r, c, e))
            yield
        for q in range(world):                      # release: the flag follows the data
            bufs[q].ready[r][c] = e
            yield
        while not all(my.ready[q][c] >= e for q in range(world)):
            yield
        total = 0
        for q in range(world):                      # local reduction in rank order
            tag, v = my.data[(par, "a", q, c)]
            if tag != e:
                raise Violation(f"rank {r} cta {c} epoch {e}: chunk of rank {q} carries epoch {tag}")
            total += v
            yield
        out[r][c].append(total)
        my.epoch[c] = e
        yield


def two_shot(bufs, r, c, calls, out, parity_areas=True):
    world = len(bufs)
    my = bufs[r]
    for _ in range(calls):
        e = my.epoch[c] + 1
        par = e & 1 if parity_areas else 0
        for s in range(world):                      # publish my input (all slices) in my own buffer
            my.data[(par, "a", s, c)] = (e, value(r, c, e) + s)
        yield
        for q in range(world):
            bufs[q].ready[r][c] = e
            yield
        while not all(my.ready[q][c] >= e for q in range(world)):
            yield
        total = 0
        for q in range(world):                      # my slice (index r) from every rank, over peer loads
            tag, v = bufs[q].data[(par, "a", r, c)]
            if tag != e:
                raise Violation(f"rank {r} cta {c} epoch {e}: slice of rank {q} carries epoch {tag}")
            total += v
            yield
        for q in range(world):                      # push the sum of slice r to everybody
            bufs[q].data[(par, "b", r, c)] = (e, total)
            yield
        for q in range(world):
            bufs[q].done[r][c] = e
            yield
        while not all(my.done[q][c] >= e for q in range(world)):
            yield
        got = []
        for s in range(world):
            tag, v = my.data[(par, "b", s, c)]
            if tag != e:
                raise Violation(f"rank {r} cta {c} epoch {e}: sum of slice {s} carries epoch {tag}")
            got.append(v)
            yield
        out[r][c].append(tuple(got))
        my.epoch[c] = e
        yield


def owners(bufs, r, c, calls, out, parity_areas=True):
    """The exchange of the fused o_proj kernel in its tile-owner form (muxserve_b200/csrc/oproj_allreduce.cu): `c` is
    the output tile, its owner rank is c mod world; the owner's flag array `done` has one entry per tile."""
    world = len(bufs)
    my = bufs[r]
    owner = c % world
    for _ in range(calls):
        e = my.epoch[c] + 1
        par = e & 1 if parity_areas else 0
        bufs[owner].data[(par, "a", r, c)] = (e, value(r, c, e))   # my partial tile -> the owner's area [r]
        yield
        bufs[owner].ready[r][c] = e
        yield
        if owner == r:
            while not all(my.ready[q][c] >= e for q in range(world)):
                yield
            total = 0
            for q in range(world):
                tag, v = my.data[(par, "a", q, c)]
                if tag != e:
                    raise Violation(f"owner {r} tile {c} epoch {e}: partial of rank {q} carries epoch {tag}")
                total += v
                yield
            for q in range(world):                                  # the sum goes where the owner's own partial lay
                bufs[q].data[(par, "a", r, c)] = (e, total)
                yield
            for q in range(world):
                bufs[q].done[0][c] = e
                yield
        while my.done[0][c] < e:
            yield
        tag, v = my.data[(par, "a", owner, c)]
        if tag != e:
            raise Violation(f"rank {r} tile {c} epoch {e}: the owner's sum carries epoch {tag}")
        out[r][c].append(v)
        my.epoch[c] = e
        yield


def run(proto, world, ctas, calls, seed, parity_areas=True, bias=None):
    rng = random.Random(seed)
    bufs = [Buffer(world, ctas) for _ in range(world)]
    out = [[[] for _ in range(ctas)] for _ in range(world)]
    procs = {(r, c): proto(bufs, r, c, calls, out, parity_areas) for r in range(world) for c in range(ctas)}
    # `bias`: a rank that runs far more often than the others (the fast rank that laps a slow one)
    weights = {k: (8.0 if bias is not None and k[0] == bias else 1.0) for k in procs}
    steps = 0
    while procs:
        keys = list(procs)
        k = rng.choices(keys, weights=[weights[x] for x in keys])[0]
        try:
            next(procs[k])
        except StopIteration:
            del procs[k]
        steps += 1
        assert steps < 2_000_000, "the protocol did not terminate (deadlock or livelock in the model)"
    return out


@pytest.mark.parametrize("world", [2, 3, 8])
def test_one_shot_every_read_sees_its_own_epoch_and_all_ranks_agree(world):
    calls, ctas = 5, 2
    for seed in range(40):
        out = run(one_shot, world, ctas, calls, seed, bias=seed % world if seed % 3 == 0 else None)
        for c in range(ctas):
            want = [sum(value(q, c, e) for q in range(world)) for e in range(1, calls + 1)]
            for r in range(world):
                assert out[r][c] == want


@pytest.mark.parametrize("world", [2, 4, 8])
def test_two_shot_every_read_sees_its_own_epoch_and_all_ranks_agree(world):
    calls, ctas = 4, 2
    for seed in range(30):
        out = run(two_shot, world, ctas, calls, seed, bias=seed % world if seed % 2 == 0 else None)
        for c in range(ctas):
            for e in range(1, calls + 1):
                want = tuple(sum(value(q, c, e) + s for q in range(world)) for s in range(world))
                for r in range(world):
                    assert out[r][c][e - 1] == want


def test_without_alternating_areas_the_same_check_catches_the_overwrite():
    """With ONE data area a fast rank's push of epoch e + 1 can land before a slow rank has read epoch e."""
    caught = 0
    for seed in range(200):
        try:
            run(one_shot, 2, 1, 4, seed, parity_areas=False, bias=0)
        except Violation:
            caught += 1
    assert caught > 0, "the model never produced the overwrite it is meant to detect"


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_o_proj_owner_exchange_every_read_sees_its_own_epoch(world):
    calls, tiles = 4, 5          # more tiles than some worlds have ranks, fewer than others: every owner pattern
    for seed in range(30):
        out = run(owners, world, tiles, calls, seed, bias=seed % world if seed % 2 == 0 else None)
        for c in range(tiles):
            want = [sum(value(q, c, e) for q in range(world)) for e in range(1, calls + 1)]
            for r in range(world):
                assert out[r][c] == want
