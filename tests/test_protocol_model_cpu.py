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

FLAG_COUNTS, FLAG_OFFSETS, FLAG_ROWS, FLAG_Y, FLAG_DY, FLAG_DX, FLAG_RD = range(7)


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
            # this layer's padding rows of the shared gradient buffer are cleared by their owner; peers write received rows
            # only, so the two may overlap (modelled as a buffer of its own)
            yield from write(me, "dy_pad", btag)
            for p in peers:                                       # combine backward: w * dout rows to the experts' ranks
                yield from write(p, "dy", btag)
            yield from signal(FLAG_DY, bwd_epoch)
            if broken == "remote_dots":
                for p in peers:                                   # older variant: re-read the expert outputs remotely
                    yield from read(p, f"y{L}", ftag, [p])
                yield from wait(FLAG_DY, bwd_epoch)
            else:
                # routing-weight gradient on the expert's side: row dots of (y, dy) into a shared scalar buffer, a flag,
                # then every source fetches its pairs' scalars
                yield from wait(FLAG_DY, bwd_epoch)
                yield from read(me, f"y{L}", ftag, [me])
                yield from read(me, "dy", btag, peers)
                yield from write(me, "rowdots", btag)
                yield from signal(FLAG_RD, bwd_epoch)
                if broken != "no_wait_rd":
                    yield from wait(FLAG_RD, bwd_epoch)
                for p in peers:
                    yield from read(p, "rowdots", btag, [p])
            yield from read(me, "dy", btag, peers)                # expert backward
            yield from read(me, "dy_pad", btag, [me])
            yield from read(me, f"x_recv{L}", ftag, peers)
            yield from write(me, "dxr", btag)
            yield from signal(FLAG_DX, bwd_epoch)
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


@pytest.mark.parametrize("broken", ["no_wait_y", "no_wait_dx", "no_wait_rd"])
def test_checker_detects_a_removed_synchronisation(broken):
    caught = 0
    for seed in range(300):
        try:
            run(3, layers=3, steps=2, seed=seed, broken=broken)
        except Hazard:
            caught += 1
    assert caught > 0


# ---------------------------------------------------------------------------------------------------------------
# tensor-parallel fused collectives: all-gather -> GEMM (pull from peers' gather buffers) and GEMM -> reduce-scatter
# (partial tiles stay in the producer's staging and the owner pulls them, or are pushed into the owner's staging slots),
# parallel/fused_collectives.py. The gathered buffers are read again
# by the weight-gradient GEMMs of the backward pass; the next write of a buffer (by its owner) and the peers' pulls of
# the new contents may only happen after those reads, which the call order (weight gradient BEFORE the layer's next
# fused call) guarantees.
# ---------------------------------------------------------------------------------------------------------------
def tp_rank_program(w: World, me: int, layers: int, steps: int, staging_buffers: int = 2, bwd_gather_buffers: int = 2,
                    back_to_back: bool = False, wgrad_late: bool = False, rs_pull: bool = True):
    n = w.n
    peers = range(n)
    epochs = {}
    rs_calls = 0
    ag_bwd_calls = 0

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

    def ag_gemm(buf, tag):
        epochs[buf] = epochs.get(buf, 0) + 1
        e = epochs[buf]
        yield from write(me, buf, tag)                           # own token slice into the gather buffer
        for p in peers:
            w.flags[(p, ("ready", buf), me)] = e
        yield ("op", None)
        for p in peers:                                          # copy CTAs: wait for the peer's slice, then pull it
            if p == me:
                continue
            yield ("wait", lambda p=p: w.flag(me, ("ready", buf), p) >= e)
            yield from read(p, buf, tag, [p])

    def gemm_rs(tag):
        nonlocal rs_calls
        par = rs_calls % staging_buffers
        rs_calls += 1
        buf = f"stage{par}"
        epochs[buf] = epochs.get(buf, 0) + 1
        e = epochs[buf]
        if rs_pull:
            # partial tiles of every owner into this rank's own staging, a counter at the owner per finished share; the
            # owner then reads its slot of every producer's staging (peer loads) and sums in rank order
            for p in peers:                                      # slot p of my staging holds owner p's rows
                yield from write(me, (buf, p), tag)
                w.flags[(p, ("cnt", buf), me)] = e
                yield ("op", None)
            yield ("wait", lambda: all(w.flag(me, ("cnt", buf), s) >= e for s in peers))
            for p in peers:
                yield from read(p, (buf, me), tag, [p])
            return
        for p in peers:                                          # partial tiles into the owner's slot, then its counter
            yield from write(p, buf, tag)
            w.flags[(p, ("cnt", buf), me)] = e
            yield ("op", None)
        yield ("wait", lambda: all(w.flag(me, ("cnt", buf), s) >= e for s in peers))
        yield from read(me, buf, tag, peers)                     # owner sums the slots in rank order

    for step in range(steps):
        for L in range(layers):
            yield from ag_gemm(f"G_attn{L}", ("f", step, L, "qkv"))
            yield from gemm_rs(("f", step, L, "o"))
            if back_to_back:          # two row-parallel products in a row (no gather in between to order the ranks)
                yield from gemm_rs(("f", step, L, "o2"))
                yield from gemm_rs(("f", step, L, "o3"))
            yield from ag_gemm(f"G_mlp{L}", ("f", step, L, "gate_up"))
            yield from gemm_rs(("f", step, L, "down"))
        for L in reversed(range(layers)):
            for name in ("down", "o"):
                par = ag_bwd_calls % bwd_gather_buffers          # row-parallel backward: gather dy, shared buffers
                ag_bwd_calls += 1
                yield from ag_gemm(f"G_bwd{par}", ("b", step, L, name))
                yield from read(me, f"G_bwd{par}", ("b", step, L, name), [me])    # its weight gradient reads the gathered dy
                if back_to_back:
                    par = ag_bwd_calls % bwd_gather_buffers
                    ag_bwd_calls += 1
                    yield from ag_gemm(f"G_bwd{par}", ("b", step, L, name + "2"))
                    yield from read(me, f"G_bwd{par}", ("b", step, L, name + "2"), [me])
                # column-parallel backward: weight gradient from the gathered forward input, then dgrad + reduce-scatter
                gbuf, gname = (f"G_mlp{L}", "gate_up") if name == "down" else (f"G_attn{L}", "qkv")
                if not wgrad_late:
                    yield from read(me, gbuf, ("f", step, L, gname), [me])
                yield from gemm_rs(("b", step, L, name + "_dx"))
                if wgrad_late:     # broken order: a peer that has finished this reduce-scatter may push the next step's rows
                    yield from read(me, gbuf, ("f", step, L, gname), [me])


def run_tp(n, layers, steps, seed, **kw):
    rng = random.Random(seed)
    w = World(n)
    progs = [tp_rank_program(w, r, layers, steps, **kw) for r in range(n)]
    blocked = [None] * n
    alive = set(range(n))
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


@pytest.mark.parametrize("n", [2, 4, 8])
@pytest.mark.parametrize("back_to_back", [False, True])
@pytest.mark.parametrize("rs_pull", [True, False])
def test_tensor_parallel_fused_collectives_have_no_races(n, back_to_back, rs_pull):
    for seed in range(100):
        run_tp(n, layers=2, steps=2, seed=seed, back_to_back=back_to_back, rs_pull=rs_pull)


@pytest.mark.parametrize("kw", [dict(staging_buffers=1), dict(bwd_gather_buffers=1), dict(staging_buffers=1, rs_pull=False)])
def test_single_buffering_of_shared_tp_buffers_is_caught(kw):
    """Why the shared buffers alternate: when two calls of the same kind follow each other directly, a fast rank would
    overwrite, in a single buffer, data that a slow peer still reads. (With a call of the other kind in between, which
    needs a signal from every peer, one buffer would do; two cover every call order.)"""
    caught = 0
    for seed in range(300):
        try:
            run_tp(4, layers=2, steps=2, seed=seed, back_to_back=True, **kw)
        except Hazard:
            caught += 1
    assert caught > 0
