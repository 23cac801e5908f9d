"""Randomised interleaving check of the expert-parallel exchange protocol (``parallel/fused_ep.py``).

The kernels synchronise ranks only through epoch-valued flags in peer memory. This test replays the exact sequence of
buffer accesses and flag operations of every rank (forward and backward of several layers and steps) under thousands of
random schedules and asserts the two properties the buffer plan relies on:

* no rank ever writes a buffer while a read of its previous contents is still outstanding, and
* no rank ever reads a buffer before all writes of the current exchange have landed,

in particular for the two gradient buffers that all layers share. A deliberately broken variant (a wait removed) must
be caught, which shows the checker can see such races.
"""
import random

import pytest

FLAG_COUNTS, FLAG_OFFSETS, FLAG_ROWS, FLAG_Y, FLAG_DY, FLAG_DX = range(6)


class Hazard(AssertionError):
    pass


class World:
    def __init__(self, n):
        self.n = n
        self.flags = {}            # (owner, slot, src) -> epoch value
        self.writers = {}          # (owner, buf) -> set of (rank, tag) writes in flight
        self.readers = {}          # (owner, buf) -> set of (rank, tag) reads in flight
        self.version = {}          # (owner, buf) -> {writer rank: tag of its last completed write}

    def flag(self, owner, slot, src):
        return self.flags.get((owner, slot, src), 0)

    # a write / read is split into begin and end so that other ranks can be scheduled in between
    def begin_write(self, rank, owner, buf, tag):
        key = (owner, buf)
        for r, t in self.readers.get(key, ()):
            if t != tag:
                raise Hazard(f"rank {rank} writes {key} for {tag} while rank {r} still reads {t}")
        for r, t in self.writers.get(key, ()):
            if t != tag:
                raise Hazard(f"rank {rank} writes {key} for {tag} while rank {r} still writes {t}")
        self.writers.setdefault(key, set()).add((rank, tag))

    def end_write(self, rank, owner, buf, tag):
        self.writers[(owner, buf)].discard((rank, tag))
        if tag[0] == "zero":           # a fill of the whole buffer destroys what every writer had put there
            self.version[(owner, buf)] = {}
        else:
            self.version.setdefault((owner, buf), {})[rank] = tag

    def begin_read(self, rank, owner, buf, tag, writers):
        key = (owner, buf)
        if self.writers.get(key):
            raise Hazard(f"rank {rank} reads {key} for {tag} while {self.writers[key]} still write")
        for w in writers:
            have = self.version.get(key, {}).get(w)
            if have != tag:
                raise Hazard(f"rank {rank} reads {key} expecting {tag} from writer {w}, found {have}")
        self.readers.setdefault(key, set()).add((rank, tag))

    def end_read(self, rank, owner, buf, tag):
        self.readers[(owner, buf)].discard((rank, tag))


def rank_program(w: World, me: int, layers: int, steps: int, broken: str = ""):
    """Generator of one rank's operations; yields ("wait", predicate) or ("op", None) after every atomic action."""
    n = w.n
    peers = range(n)
    fwd_epoch = bwd_epoch = 0

    def write(owner, buf, tag):
        w.begin_write(me, owner, buf, tag)
        yield ("op", None)
        w.end_write(me, owner, buf, tag)
        yield ("op", None)

    def read(owner, buf, tag, writers):
        w.begin_read(me, owner, buf, tag, writers)
        yield ("op", None)
        w.end_read(me, owner, buf, tag)
        yield ("op", None)

    def signal(slot, epoch):
        for p in peers:
            w.flags[(p, slot, me)] = epoch
        yield ("op", None)

    def wait(slot, epoch):
        yield ("wait", lambda: all(w.flag(me, slot, s) >= epoch for s in peers))

    for step in range(steps):
        for L in range(layers):                                   # ---------------- forward
            fwd_epoch += 1
            tag = ("f", step, L)
            for p in peers:                                       # ep_exchange: counts out
                yield from write(p, "counts", tag)
            yield from signal(FLAG_COUNTS, fwd_epoch)
            yield from wait(FLAG_COUNTS, fwd_epoch)
            yield from read(me, "counts", tag, peers)
            for p in peers:                                       # offsets back to the sources
                yield from write(p, "offsets", tag)
            yield from signal(FLAG_OFFSETS, fwd_epoch)
            yield from wait(FLAG_OFFSETS, fwd_epoch)
            yield from read(me, "offsets", tag, peers)            # ep_push_rows reads its offsets ...
            for p in peers:                                       # ... and stores rows into every destination
                yield from write(p, f"x_recv{L}", tag)
            yield from signal(FLAG_ROWS, fwd_epoch)
            yield from wait(FLAG_ROWS, fwd_epoch)
            yield from read(me, f"x_recv{L}", tag, peers)         # expert GEMMs
            yield from write(me, f"y{L}", tag)
            yield from signal(FLAG_Y, fwd_epoch)
            if broken != "no_wait_y":
                yield from wait(FLAG_Y, fwd_epoch)
            for p in peers:                                       # ep_pull_rows (combine)
                yield from read(p, f"y{L}", tag, [p])
        for L in reversed(range(layers)):                         # ---------------- backward
            bwd_epoch += 1
            ftag, btag = ("f", step, L), ("b", step, L)
            for p in peers:                                       # combine backward: w * dout rows to the experts' ranks
                yield from write(p, "dy", btag)
            yield from signal(FLAG_DY, bwd_epoch)
            for p in peers:                                       # routing-weight gradient reads the expert outputs again
                yield from read(p, f"y{L}", ftag, [p])
            yield from wait(FLAG_DY, bwd_epoch)
            yield from read(me, "dy", btag, peers)                # expert backward
            yield from read(me, f"x_recv{L}", ftag, peers)
            yield from write(me, "dxr", btag)
            if broken != "no_zero_order":
                yield from write(me, "dy", ("zero", step, L))     # zero-fill precedes the signal
            yield from signal(FLAG_DX, bwd_epoch)
            if broken == "no_zero_order":
                yield from write(me, "dy", ("zero", step, L))     # broken: zero-fill after peers may already push again
            if broken != "no_wait_dx":
                yield from wait(FLAG_DX, bwd_epoch)
            for p in peers:                                       # dispatch backward pulls the input gradients
                yield from read(p, "dxr", btag, [p])


def run(n, layers, steps, seed, broken=""):
    rng = random.Random(seed)
    w = World(n)
    progs = [rank_program(w, r, layers, steps, broken) for r in range(n)]
    blocked = [None] * n
    alive = set(range(n))
    ticks = 0
    while alive:
        runnable = [r for r in alive if blocked[r] is None or blocked[r]()]
        if not runnable:
            raise AssertionError(f"deadlock: ranks {sorted(alive)} all wait")
        r = rng.choice(runnable)
        blocked[r] = None
        try:
            kind, pred = next(progs[r])
        except StopIteration:
            alive.discard(r)
            continue
        if kind == "wait" and not pred():
            blocked[r] = pred
        ticks += 1
    return ticks


@pytest.mark.parametrize("n", [2, 3, 4])
def test_exchange_protocol_has_no_races_under_random_schedules(n):
    for seed in range(300):
        run(n, layers=3, steps=2, seed=seed)


def test_dy_zero_fill_of_shared_buffer_is_ordered_before_the_next_push():
    """The zero-fill write uses its own tag: a peer's push for the next layer must not overlap it."""
    for seed in range(200):
        run(2, layers=2, steps=2, seed=seed)


@pytest.mark.parametrize("broken", ["no_wait_y", "no_wait_dx", "no_zero_order"])
def test_checker_detects_a_removed_synchronisation(broken):
    caught = 0
    for seed in range(300):
        try:
            run(3, layers=3, steps=2, seed=seed, broken=broken)
        except Hazard:
            caught += 1
    assert caught > 0
