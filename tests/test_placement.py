"""Expert placement from routing statistics (host logic, no GPU): the planner's invariants, the balance it
reaches under the prefill workload's Zipf(1.1) popularity, the row rule that splits a copied expert's pairs,
and the routing average of the reference (src/model/routing_counts.h: ema = ema * keep + modular delta)."""
import numpy as np
import pytest

from fngine_b200 import placement as P


def zipf_load(seed, total=81920.0, s=1.1):
    rng = np.random.default_rng(seed)
    w = 1.0 / np.arange(1, 513) ** s
    load = np.zeros(512)
    load[rng.permutation(512)] = w / w.sum() * total
    return load


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_contiguous_placement_is_the_shard_rule(world):
    pl = P.Placement.contiguous(world)
    per = 512 // world
    assert pl.slots_needed() == per
    for r in range(world):
        assert pl.rank_experts[r] == list(range(r * per, (r + 1) * per))
        m = pl.slot_map(r)
        assert (m[r * per:(r + 1) * per] == np.arange(per)).all() and (np.delete(m, np.arange(r * per, (r + 1) * per)) == -1).all()
        sh = pl.share_table(r)
        assert (sh[r * per:(r + 1) * per] == (1 << 8)).all() and (sh >= 0).sum() == per


@pytest.mark.parametrize("world,extra", [(2, 0), (4, 4), (8, 0), (8, 4), (8, 8)])
def test_plan_invariants_and_balance(world, extra):
    load = zipf_load(3)
    slots = 512 // world + extra
    pl = P.plan_placement(load, world, slots)
    assert pl.slots_needed() <= slots
    assert all(1 <= len(c) <= world and len(set(c)) == len(c) for c in pl.copies)
    assert sum(len(x) for x in pl.rank_experts) == sum(len(c) for c in pl.copies)
    # every (row, expert) pair is kept by exactly one rank
    for e in (int(np.argmax(load)), 0, 511, int(np.argmin(load))):
        for row in range(23):
            assert sum(pl.keeps(r, e, row) for r in range(world)) == 1
    # the share tables state the same rule
    for r in range(world):
        sh = pl.share_table(r)
        for e in range(512):
            if r in pl.copies[e]:
                assert sh[e] >> 8 == len(pl.copies[e]) and sh[e] & 255 == pl.copies[e].index(r)
            else:
                assert sh[e] == -1
    # never worse than contiguous shards; with spare slots the ranks are level
    assert pl.imbalance(load) <= P.Placement.contiguous(world).imbalance(load) + 1e-12
    if extra >= 4:
        assert pl.imbalance(load) <= 1.02
    # same load, same plan
    assert P.plan_placement(load.copy(), world, slots).copies == pl.copies


def test_zipf_at_eight_ranks_needs_copies():
    """The hottest expert of Zipf(1.1) over 512 brings 0.42 of a rank's fair share at 8 ranks: spreading alone
    cannot level the ranks, copies can."""
    load = zipf_load(11)
    contiguous = P.Placement.contiguous(8).imbalance(load)
    spread = P.plan_placement(load, 8, 64).imbalance(load)
    copied = P.plan_placement(load, 8, 68)
    print("pair load, busiest rank / mean at 8 ranks: contiguous %.2f, spread %.2f, spread + copies %.3f (%d experts copied)"
          % (contiguous, spread, copied.imbalance(load), sum(len(c) > 1 for c in copied.copies)))
    assert contiguous > 1.3 and copied.imbalance(load) < 1.01
    assert P.should_replace(load, P.Placement.contiguous(8), copied)
    assert not P.should_replace(load, copied, copied)


def test_uniform_load_gets_no_copies():
    pl = P.plan_placement(np.ones(512), 8, 72)
    assert all(len(c) == 1 for c in pl.copies) and pl.slots_needed() == 64


def test_moves_between_placements():
    load = zipf_load(5)
    a, b = P.Placement.contiguous(4), P.plan_placement(load, 4, 132)
    moves = b.moves_from(a)
    assert all(r in b.copies[e] and r not in a.copies[e] for e, r in moves)
    assert b.moves_from(b) == []


def test_routing_average_follows_the_reference_rule():
    ema = P.RoutingEma(2, keep=0.5)
    c1 = np.zeros((2, 512), dtype=np.uint32)
    c1[0, 7], c1[1, 9] = 10, 4
    out = ema.update(c1)
    assert out[0, 7] == 10 and out[1, 9] == 4 and out.sum() == 14
    c2 = c1.copy()
    c2[0, 7] = 16
    out = ema.update(c2)
    assert out[0, 7] == 10 * 0.5 + 6 and out[1, 9] == 2
    # the counters are modular u32: a wrap still gives the true growth
    ema2 = P.RoutingEma(1, keep=1.0)
    a = np.zeros((1, 512), dtype=np.uint32)
    a[0, 0] = 0xFFFFFFF0
    ema2.update(a)
    b = a.copy()
    b[0, 0] = 0x10  # wrapped: grew by 0x20
    assert ema2.update(b)[0, 0] == np.float32(0xFFFFFFF0) + 0x20


def test_bad_plans_are_refused():
    with pytest.raises(ValueError):
        P.plan_placement(np.ones(512), 3)
    with pytest.raises(ValueError):
        P.plan_placement(np.ones(512), 8, 63)
    with pytest.raises(ValueError):
        P.Placement(2, [[0]] * 511 + [[0, 0]])
