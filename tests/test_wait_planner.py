"""The wait decisions of the fused all-gather (nihilus_b200/csrc/deliveries.h, the code the library itself runs), checked
without a GPU: programs of launches are planned once and then replayed on a model of G ranks that run at different
speeds, with remote stores that land late.  The model knows what every read must see and reports a stale row (a read
before the delivery landed), a row from the future (a peer ran ahead and overwrote what this rank had not read yet) and
a deadlock (every rank waiting)."""
import random

import pytest

BUF = 4096  # bytes per model buffer


class Prog:
    """A sequence of launches over numbered buffers.  Symmetric buffers live at fake addresses inside one region."""

    def __init__(self, capi, n_buffers, window):
        self.capi = capi
        self.base = 0x10000000
        self.n_buffers = n_buffers
        self.planner = capi.WaitPlanner(window)
        self.planner.add_region(self.base, n_buffers * BUF)
        self.steps = []  # ("launch", reads, writes, delivers, waits, lag) | ("sync", need)

    def addr(self, b):
        return (self.base + b * BUF, BUF)

    def launch(self, reads, writes, delivers):
        waits, lag = self.planner.launch([self.addr(b) for b in reads], [self.addr(b) for b in writes], delivers)
        self.steps.append(("launch", tuple(reads), tuple(writes), delivers, waits, lag))
        return waits, lag

    def sync(self):
        self.steps.append(("sync", self.planner.wait_all()))

    def close(self):
        self.planner.close()


def replay(prog, world, seed, late=0.7):
    """Runs the planned program on `world` model ranks under a random schedule.  Returns None or a description of what
    went wrong."""
    rng = random.Random(seed)
    steps = prog.steps
    # what a read of buffer b by step i must see: the index of the last earlier step that wrote b (-1: initial contents)
    last_write, expect = {}, []
    for i, st in enumerate(steps):
        if st[0] == "launch":
            expect.append({b: last_write.get(b, -1) for b in st[1]})
            for b in st[2]:
                last_write[b] = i
        else:
            expect.append({})
    pc = [0] * world
    done = [0] * world  # completed delivering launches
    announced = [0] * world
    inflight = [[] for _ in range(world)]  # per source rank: (dst, buffer, version)
    copy = [[[-1] * world for _ in range(prog.n_buffers)] for _ in range(world)]  # copy[rank][buffer][slice]

    def land(src, everything):
        keep = []
        for dst, b, v in inflight[src]:
            if everything or rng.random() > late:
                copy[dst][b][src] = v
            else:
                keep.append((dst, b, v))
        inflight[src] = keep

    stalled = 0
    while any(p < len(steps) for p in pc):
        r = rng.randrange(world)
        if pc[r] >= len(steps):
            continue
        for s in range(world):
            land(s, False)
        st = steps[pc[r]]
        # start of any launch (or of the wait kernel): the previous kernels' stores are complete, then the announcement
        land(r, True)
        announced[r] = done[r]
        waits, lag = (st[4], st[5]) if st[0] == "launch" else (st[1], 0)
        if waits and any(announced[p] < done[r] - lag for p in range(world) if p != r):
            stalled += 1
            if stalled > 20000:
                return "deadlock at step %d of rank %d" % (pc[r], r)
            continue
        stalled = 0
        if st[0] == "launch":
            i = pc[r]
            for b, want in expect[i].items():
                for s in range(world):
                    got = copy[r][b][s]
                    if got != want:
                        kind = "stale" if got < want else "from the future"
                        return "rank %d step %d reads buffer %d slice %d: version %d, wanted %d (%s)" % (r, i, b, s, got, want, kind)
            for b in st[2]:
                if st[3]:  # delivers: own slice now, the peers' copies some time before this rank's next announcement
                    copy[r][b][r] = i
                    for p in range(world):
                        if p != r:
                            inflight[r].append((p, b, i))
                else:  # computed whole on every rank
                    for s in range(world):
                        copy[r][b][s] = i
            if st[3]:
                done[r] += 1
        pc[r] += 1
    for r in range(1, world):
        if copy[r] != copy[0]:
            return "ranks end with different buffers"
    return None


def test_independent_launches_do_not_wait_and_dependent_ones_wait_for_exactly_their_producer(capi):
    p = Prog(capi, 8, window=4)
    assert p.launch([], [0], True) == (False, 0)  # nothing delivered yet
    assert p.launch([], [1], True) == (False, 0)  # independent of the first: runs on while its rows are in flight
    assert p.launch([0], [2], True) == (True, 1)  # reads what delivering launch 1 delivered; 2 launches enqueued so far -> lag 1
    assert p.launch([5], [6], False) == (False, 0)  # reads rows nobody delivers, delivers nothing
    assert p.launch([2], [3], False) == (True, 0)  # reads the rows of the latest delivering launch (number 3)
    assert p.planner.seq == 3
    assert p.launch([1], [4], False) == (False, 0)  # launch 2 was confirmed by the wait for launch 3: nothing left to wait for
    p.sync()
    assert p.steps[-1] == ("sync", False)  # and nothing is pending any more
    p.close()
    # window 0: every launch waits for every earlier delivery
    p = Prog(capi, 8, window=0)
    assert p.launch([], [0], True) == (False, 0)
    assert p.launch([], [1], True) == (True, 0)
    assert p.launch([7], [2], False) == (True, 0)
    p.close()


def test_the_window_bounds_how_far_a_rank_runs_ahead(capi):
    p = Prog(capi, 64, window=4)
    lags = [p.launch([], [i], True) for i in range(20)]
    p.close()
    # the check falls on every second delivering launch and asks for (enqueued so far - 4)
    assert lags[:5] == [(False, 0)] * 5
    assert [w for w, _ in lags[5:]] == [False, True] * 7 + [False]
    assert all(lag == 4 for w, lag in lags if w)


@pytest.mark.parametrize("world", [2, 3, 8])
@pytest.mark.parametrize("window", [0, 1, 4])
def test_a_chain_of_dependent_stages_over_two_buffers(capi, world, window):
    p = Prog(capi, 4, window)
    p.launch([], [0], True)
    for k in range(1, 40):
        p.launch([(k - 1) % 2], [k % 2], True)  # reads the other buffer, rewrites the one the launch before it read
    p.sync()
    for seed in range(30):
        assert replay(p, world, seed) is None
    p.close()


@pytest.mark.parametrize("world", [2, 4])
def test_the_benchmarked_step_replayed_like_a_graph(capi, world):
    """Independent stage inputs; q/k/v and attn_output computed whole on every rank, gate+up and down delivered; every step
    rewrites the buffers of the step before and ends with a wait for everything."""
    layers = 6
    p = Prog(capi, 4 * layers, window=4)
    for _ in range(4):
        for layer in range(layers):
            p.launch([], [4 * layer], False)
            p.launch([], [4 * layer + 1], False)
            p.launch([], [4 * layer + 2], True)
            p.launch([], [4 * layer + 3], True)
        p.sync()
    n_wait = sum(1 for s in p.steps if s[0] == "launch" and s[4])
    assert n_wait <= 4 * layers  # at most every second delivering launch polls the peers
    for seed in range(30):
        assert replay(p, world, seed) is None
    p.close()


@pytest.mark.parametrize("window", [0, 2, 4])
def test_random_programs_within_the_documented_rule(capi, window):
    """Random reads, writes and deliveries.  The one rule a caller must keep: after a launch that delivers nothing, some
    other delivering launch has to come before a delivering launch rewrites what it read or wrote."""
    for trial in range(40):
        rng = random.Random(1000 + trial)
        nb = 6
        p = Prog(capi, nb, window)
        blocked = {}  # buffer -> True while its last reader delivered nothing and no delivering launch has followed
        for _ in range(60):
            if rng.random() < 0.05:
                p.sync()  # a wait for every delivery is not a meeting of the ranks: the rule still holds across it
                continue
            delivers = rng.random() < 0.6
            reads = rng.sample(range(nb), rng.randrange(0, 3))
            choices = [b for b in range(nb) if b not in reads and not (delivers and blocked.get(b))]
            if not choices:
                continue
            w = rng.choice(choices)
            p.launch(reads, [w], delivers)
            if delivers:
                blocked = {b: False for b in blocked}
                for b in reads:
                    blocked[b] = False  # a delivering reader may be followed directly by the rewrite
            else:
                for b in reads + [w]:
                    blocked[b] = True
        p.sync()
        for seed in range(10):
            for world in (2, 3):
                err = replay(p, world, seed)
                assert err is None, (trial, seed, world, err)
        p.close()


def test_the_model_catches_a_missing_wait(capi):
    """The replay is only worth something if it fails when a wait is taken away."""
    p = Prog(capi, 4, window=4)
    p.launch([], [0], True)
    for k in range(1, 20):
        p.launch([(k - 1) % 2], [k % 2], True)
    p.sync()
    broken = [(s[0], s[1], s[2], s[3], False, 0) if s[0] == "launch" else s for s in p.steps]
    p.steps = broken
    assert any(replay(p, 2, seed) is not None for seed in range(20))
    p.close()


def _record(p, body):
    """Plans `body` (a list of (reads, writes, delivers) or "sync") between capture_begin and capture_end; returns the recording's
    number and the planned steps, whose answers are frozen."""
    p.planner.capture_begin()
    first = len(p.steps)
    for item in body:
        if item == "sync":
            p.sync()
        else:
            p.launch(*item)
    return p.planner.capture_end(), p.steps[first:]


@pytest.mark.parametrize("world", [2, 3])
@pytest.mark.parametrize("window", [0, 4])
def test_a_recorded_step_replayed_after_any_history(capi, world, window):
    """What nhb_graph_begin / _end / _launch do: the recorded launches keep the waits they were planned with, whatever ran
    before a replay -- eager launches that deliver into the recording's buffers, other recordings, nothing at all."""
    for trial in range(12):
        rng = random.Random(4000 + trial)
        nb = 6
        p = Prog(capi, nb, window)
        # some history before the first capture, ending with a delivering launch that nobody has waited for
        p.launch([], [0], True)
        p.launch([0], [1], True)
        # recording A: a dependent chain that rewrites buffers 0..2; recording B: reads A's results, delivers into 3..5
        rec_a, steps_a = _record(p, [([], [0], True), ([0], [1], True), ([1], [2], True), ([2], [0], True)])
        rec_b, steps_b = _record(p, [([0], [3], True), ([3, 1], [4], False), ([], [5], True), ([5], [3], True), "sync"])
        for _ in range(10):
            kind = rng.choice(["a", "b", "eager", "sync"])
            if kind == "a":
                p.steps.extend(steps_a)
                p.planner.replayed(rec_a)
            elif kind == "b":
                p.steps.extend(steps_b)
                p.planner.replayed(rec_b)
            elif kind == "eager":
                # (a launch that delivers nothing is followed by a delivering one before anything it touched is delivered into)
                w = rng.randrange(3, nb)
                p.launch([rng.choice([b for b in range(nb) if b != w])], [w], True)  # (a mul_mat never reads what it writes)
                p.launch([rng.randrange(5)], [5], True)
            else:
                p.sync()
        p.sync()
        for seed in range(10):
            err = replay(p, world, seed)
            assert err is None, (trial, seed, err)
        p.close()
