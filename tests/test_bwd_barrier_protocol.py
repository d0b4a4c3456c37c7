"""A model of the mbarrier protocol of the persistent tcgen05 backward (csrc/bwd_tc5_d64.cu), run
under random interleavings on the CPU.

The kernel's roles (TMA producer, four score-issuing threads, one or two second-stage issuing
threads, two elementwise warpgroups) talk only through mbarriers that are waited on by phase
parity.  A parity wait is right only if the waiter sees every phase of the barrier in order: a
waiter that skips a phase passes too early, one that falls two phases behind never passes.  Both
mistakes are easy to make when a role has no work in some item of the persistent loop, so the
protocol is written down once more here, small enough to be searched: every role is a generator
that yields at each wait, asynchronous completions (TMA arrivals, tcgen05.commit arrivals) are
delivered at random later points, and every wait names the event it stands for, which must have
happened when the wait passes.

What is modelled, with the kernel's names: loop_full / loop_empty per ring stage; s_full indexed by
g % 6 (same accumulator buffer g % 3 and same elementwise group g & 1); p_full per accumulator
buffer; own_staged / own_free per staging half (the score threads arrive on own_free too); done and
out_free per output buffer (two for the own-queries launch, one for the own-keys launch); the item
epilogue deferred behind the group's first sub-tile of the next item.
"""
import random

import pytest

NBUF = 3  # score accumulator buffers (sub-tiles in flight)
NSF = 6   # s_full barriers


class Bar:
    def __init__(self, count):
        self.count = count
        self.pending = count
        self.phase = 0

    def arrive(self):
        self.pending -= 1
        if self.pending == 0:
            self.pending = self.count
            self.phase += 1

    def passed(self, parity):
        """mbarrier.try_wait.parity: true when the phase with this parity has completed, i.e. the
        current (incomplete) phase has the other parity."""
        return (self.phase & 1) != parity


def run(stages, n_subs, own_keys, seed):
    """One random interleaving for a CTA whose item list has n_subs[i] sub-tiles in item i.
    Returns "ok", or a description of the deadlock; raises AssertionError on a premature pass."""
    rnd = random.Random(seed)
    n_out = 2 if own_keys else 1      # second-stage issuing threads
    n_out_buf = 1 if own_keys else 2  # output accumulator buffers
    loop_full = [Bar(1) for _ in range(stages)]
    loop_empty = [Bar(n_out) for _ in range(stages)]
    s_full = [Bar(2) for _ in range(NSF)]   # the two score threads of a sub-tile
    p_full = [Bar(1) for _ in range(NBUF)]  # one elementwise group (modelled as one agent)
    own_staged = [Bar(1), Bar(1)]
    own_free = [Bar(2 + 4) for _ in range(2)]  # two elementwise groups + four score threads
    done = [Bar(n_out), Bar(n_out)]
    out_free = [Bar(2), Bar(2)]
    bars = loop_full + loop_empty + s_full + p_full + own_staged + own_free + done + out_free
    events = set()  # what has really happened
    pending = []    # asynchronous completions not yet delivered
    count = {}

    def later(fn):
        pending.append(fn)

    def wait(bar, parity, need):
        while not bar.passed(parity):
            yield ("wait", need, parity, bar.phase)
        assert need is None or need in events, f"wait passed before {need}"

    def tally(key, n, event):
        count[key] = count.get(key, 0) + 1
        if count[key] == n:
            events.add(event)

    def producer():
        def load_own(j):  # own tiles of item j -> staging half j & 1
            h, use = j & 1, j >> 1
            if use > 0:
                yield from wait(own_free[h], (use - 1) & 1, ("item_done", j - 2))
            later(lambda: (events.add(("own_staged", j)), own_staged[h].arrive()))

        yield from load_own(0)
        gbase = 0
        for kact, n in enumerate(n_subs):
            loaded = kact + 1 >= len(n_subs)
            for s in range(n):
                if s == stages and not loaded:
                    yield from load_own(kact + 1)
                    loaded = True
                g = gbase + s
                yield from wait(loop_empty[g % stages], ((g // stages) & 1) ^ 1,
                                ("out_done", g - stages) if g >= stages else None)
                later(lambda g=g: (events.add(("tile", g)), loop_full[g % stages].arrive()))
                yield
            if not loaded:
                yield from load_own(kact + 1)
            gbase += n

    def score_thread(r):  # sub-tiles g = r, r + 2, ...
        g, gbase = r, 0
        for kact, n in enumerate(n_subs):
            yield from wait(own_staged[kact & 1], (kact >> 1) & 1, ("own_staged", kact))  # also without work here
            while g < gbase + n:
                if g >= NBUF:
                    f = g - NBUF
                    yield from wait(loop_empty[f % stages], (f // stages) & 1, ("out_done", f))
                yield from wait(loop_full[g % stages], (g // stages) & 1, ("tile", g))
                later(lambda g=g: (tally(("sc", g), 2, ("scores", g)), s_full[g % NSF].arrive()))
                yield
                g += 2
            own_free[kact & 1].arrive()
            yield
            gbase += n

    def out_thread():
        g = 0
        for kact, n in enumerate(n_subs):
            for s in range(n):
                yield from wait(p_full[g % NBUF], (g // NBUF) & 1, ("operands", g))
                if s == 0 and kact >= n_out_buf:
                    yield from wait(out_free[kact % n_out_buf], (kact // n_out_buf - 1) & 1,
                                    ("out_read", kact - n_out_buf))
                later(lambda g=g: (tally(("out", g), n_out, ("out_done", g)), loop_empty[g % stages].arrive()))
                yield
                g += 1
            later(lambda kact=kact: (tally(("done", kact), n_out, ("item_mma_done", kact)),
                                     done[kact % n_out_buf].arrive()))
            yield

    def elementwise(wg):  # sub-tiles with g & 1 == wg
        def epilogue(kact):
            yield from wait(done[kact % n_out_buf], (kact // n_out_buf) & 1, ("item_mma_done", kact))
            tally(("ep", kact), 2, ("out_read", kact))
            tally(("ep2", kact), 2, ("item_done", kact))
            out_free[kact % n_out_buf].arrive()
            own_free[kact & 1].arrive()
            yield

        gbase, pend = 0, None
        for kact, n in enumerate(n_subs):
            s = (wg - gbase) & 1
            while s < n:
                g = gbase + s
                if own_keys:
                    yield from wait(loop_full[g % stages], (g // stages) & 1, ("tile", g))  # stat_full in the kernel
                yield from wait(s_full[g % NSF], (g // NSF) & 1, ("scores", g))
                events.add(("operands", g))
                p_full[g % NBUF].arrive()
                yield
                if pend is not None:
                    yield from epilogue(pend)
                    pend = None
                s += 2
            if pend is not None:
                yield from epilogue(pend)
            pend = kact
            gbase += n
        if pend is not None:
            yield from epilogue(pend)

    agents = [producer(), score_thread(0), score_thread(1), score_thread(0), score_thread(1), out_thread(),
              elementwise(0), elementwise(1)] + ([out_thread()] if own_keys else [])
    names = ["producer", "scoreA0", "scoreA1", "scoreB0", "scoreB1", "out0", "elem0", "elem1", "out1"]
    alive = [True] * len(agents)
    last = [None] * len(agents)
    idle = 0

    def state():
        return (len(events), tuple(b.phase for b in bars), tuple(b.pending for b in bars), len(pending))

    while any(alive):
        if pending and rnd.random() < 0.3:
            pending.pop(rnd.randrange(len(pending)))()
            idle = 0
            continue
        i = rnd.randrange(len(agents))
        if not alive[i]:
            continue
        before = state()
        try:
            last[i] = next(agents[i])
        except StopIteration:
            alive[i] = False
            idle = 0
            continue
        idle = 0 if state() != before else idle + 1
        if idle > 20000 and not pending:
            return "deadlock: " + str([(n, w) for n, w, a in zip(names, last, alive) if a])
    return "ok"


def _item_lists():
    rr = random.Random(5)
    lists = [(6, [64, 60, 8, 4]), (5, [32, 32, 32]), (6, [17, 23, 31]), (6, [1, 1, 2, 1, 3, 1, 1]),
             (5, [1, 1, 2, 1, 3, 1, 1]), (6, [1]), (5, [2, 1])]
    for _ in range(13):
        lists.append((rr.choice([5, 6]), [rr.choice([1, 1, 2, 3, 4, 5, 7, 16, 33]) for _ in range(rr.randint(1, 7))]))
    return lists


@pytest.mark.parametrize("own_keys", [False, True], ids=["own_queries", "own_keys"])
def test_protocol_has_no_deadlock_and_no_premature_pass(own_keys):
    for stages, n_subs in _item_lists():
        for seed in range(6):
            assert run(stages, n_subs, own_keys, seed) == "ok", (stages, n_subs, seed)


def test_model_detects_a_waiter_that_skips_phases():
    """The mistake the model is there to catch: two elementwise groups sharing one s_full barrier per
    accumulator buffer (g % 3) see only every other phase of it, and a wait can pass before its
    scores exist."""
    global NSF
    saved = NSF
    NSF = NBUF
    try:
        with pytest.raises(AssertionError):
            for seed in range(40):
                run(6, [16, 16], False, seed)
    finally:
        NSF = saved
