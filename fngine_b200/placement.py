"""Expert placement across the GPUs of one node from routing statistics.

The reference engine keeps the hottest experts of a layer on its one GPU and the rest in host memory,
ranks them by an exponential moving average of the decode routing counts (src/model/routing_counts.h:
ema = ema * keep + (counts - last) on modular u32 counters, keep 0.999, README "Adaptive replacement")
and swaps a pair when the newcomer's average is twice the resident's. On a box of B200s every expert is
resident somewhere, so the same statistic answers a different question: WHICH GPU holds an expert, and
how many copies of it exist. With a skewed router (the prefill workload's Zipf bias) contiguous shards
leave one rank with a multiple of the mean pair load and every other rank waiting for it in the
combine exchange.

plan_placement spreads the experts over the ranks by longest-processing-time-first on their load and
gives the hottest experts extra copies where spreading alone cannot level the ranks; the copies of an expert split its
pairs by row number (row r goes to copy r % n), which every rank can evaluate alone as long as all
ranks see the same rows in the same order (the dense exchange of ep_prefill). Everything here is host
logic on numpy arrays and is exercised without a GPU by tests/test_placement.py.
"""
import numpy as np

EXPERTS = 512


class RoutingEma:
    """Host mirror of the reference's routing average: update(counts) folds the growth of the modular
    u32 counters [layers][512] since the previous call into ema = ema * keep + delta."""

    def __init__(self, layers, keep=0.999, start=None):
        self.keep = float(keep)
        self.ema = np.zeros((layers, EXPERTS), dtype=np.float32) if start is None else np.array(start, dtype=np.float32)
        self.last = np.zeros((layers, EXPERTS), dtype=np.uint32)

    def update(self, counts):
        counts = np.asarray(counts, dtype=np.uint32).reshape(self.last.shape)
        delta = (counts - self.last).astype(np.uint32)  # modular, as the device kernel's subtraction
        self.ema = (self.ema * np.float32(self.keep) + delta.astype(np.float32)).astype(np.float32)
        self.last = counts.copy()
        return self.ema


class Placement:
    """copies[e] = the ranks that hold expert e (at least one), in copy order; rank_experts[r] = the
    experts rank r holds, in slot order."""

    def __init__(self, world, copies):
        self.world = int(world)
        self.copies = [list(c) for c in copies]
        if len(self.copies) != EXPERTS or any(len(c) < 1 or len(c) > 255 or len(set(c)) != len(c) for c in self.copies):
            raise ValueError("every expert needs between 1 and 255 copies on different ranks")
        if any(r < 0 or r >= world for c in self.copies for r in c):
            raise ValueError("a copy names a rank outside the world")
        self.rank_experts = [[] for _ in range(world)]
        for e, c in enumerate(self.copies):
            for r in c:
                self.rank_experts[r].append(e)

    @staticmethod
    def contiguous(world):
        per = EXPERTS // world
        return Placement(world, [[e // per] for e in range(EXPERTS)])

    def slots_needed(self):
        return max(len(x) for x in self.rank_experts)

    def share_table(self, rank):
        """int32 [512] for fb_moe_route_placed: -1, or (copies << 8) | index of this rank's copy."""
        t = np.full(EXPERTS, -1, dtype=np.int32)
        for e, c in enumerate(self.copies):
            if rank in c:
                t[e] = (len(c) << 8) | c.index(rank)
        return t

    def slot_map(self, rank):
        """int32 [512]: expert -> slot in this rank's slot array, -1 when the rank does not hold it (the
        slot_of table of the decode kernels)."""
        t = np.full(EXPERTS, -1, dtype=np.int32)
        for s, e in enumerate(self.rank_experts[rank]):
            t[e] = s
        return t

    def keeps(self, rank, expert, row):
        c = self.copies[expert]
        return rank in c and row % len(c) == c.index(rank)

    def rank_loads(self, load):
        """Expected pairs per rank when expert e brings load[e] pairs, split evenly over its copies."""
        out = np.zeros(self.world, dtype=np.float64)
        for e, c in enumerate(self.copies):
            for r in c:
                out[r] += float(load[e]) / len(c)
        return out

    def imbalance(self, load):
        l = self.rank_loads(load)
        return float(l.max() / l.mean()) if l.mean() > 0 else 1.0

    def moves_from(self, other):
        """(expert, rank) copies this placement has and `other` has not: what a re-placement uploads."""
        return [(e, r) for e in range(EXPERTS) for r in self.copies[e] if r not in other.copies[e]]


def _spread(load, n, world, slots_per_rank):
    """Longest processing time first: the (expert, copy) shares, heaviest first (ties: lower expert id), each
    go to the least loaded rank that has a free slot and no copy of that expert yet (ties: lower rank)."""
    shares = [(-(load[e] / n[e]), e, c) for e in range(EXPERTS) for c in range(n[e])]
    shares.sort()
    rank_load = np.zeros(world, dtype=np.float64)
    rank_free = np.full(world, slots_per_rank, dtype=np.int64)
    copies = [[] for _ in range(EXPERTS)]
    for neg, e, _c in shares:
        best = -1
        for r in range(world):
            if rank_free[r] > 0 and r not in copies[e] and (best < 0 or rank_load[r] < rank_load[best]):
                best = r
        if best < 0:  # no rank left that lacks this expert: the extra copy is dropped
            continue
        copies[e].append(best)
        rank_load[best] += -neg
        rank_free[best] -= 1
    return copies, rank_load


def plan_placement(load, world, slots_per_rank=None, max_copies=None, tolerance=0.01):
    """Spread 512 experts with the given load (pairs, or a routing average) over `world` ranks.

    The experts are spread by longest-processing-time-first on their load. While the busiest rank then
    still exceeds the mean by more than `tolerance` and spare slots remain (world * slots_per_rank - 512),
    the expert with the largest load per copy gets one more copy (at most max_copies, default: one per
    rank) and the spread is redone: copies appear only where spreading alone cannot level the ranks, i.e.
    for experts whose own load is a large part of a rank's fair share. Deterministic: every rank computes
    the same plan from the same load."""
    load = np.asarray(load, dtype=np.float64).reshape(EXPERTS)
    if EXPERTS % world:
        raise ValueError("world size must divide 512")
    per = EXPERTS // world
    slots_per_rank = per if slots_per_rank is None else int(slots_per_rank)
    if slots_per_rank < per:
        raise ValueError("fewer slots than experts")
    max_copies = min(world, 255) if max_copies is None else max(1, min(int(max_copies), world, 255))
    n = np.ones(EXPERTS, dtype=np.int64)
    copies, rank_load = _spread(load, n, world, slots_per_rank)
    for _ in range(world * slots_per_rank - EXPERTS):
        mean = rank_load.mean()
        if mean <= 0 or rank_load.max() <= mean * (1.0 + tolerance):
            break
        share = np.where(n < max_copies, load / n, -1.0)
        e = int(np.argmax(share))  # first maximum: lower id wins ties
        if share[e] <= 0:
            break
        n[e] += 1
        copies, rank_load = _spread(load, n, world, slots_per_rank)
    return Placement(world, copies)


def should_replace(load, current, candidate, ratio=2.0):
    """The reference swaps a pair of experts only when the newcomer's average is `ratio` times the
    resident's; the analogue for a whole placement: re-place only when the busiest rank's excess over
    the mean shrinks by that factor."""
    cur, new = current.imbalance(load) - 1.0, candidate.imbalance(load) - 1.0
    return cur > 0 and new * ratio <= cur
