"""Models of the mbarrier protocols of the pipelined head-dimension-128 kernels (csrc/fwd_tc5_pipe128.cu,
csrc/bwd_tc5_pipe128.cu), run under random interleavings on the CPU.

The roles of a CTA talk only through mbarriers that are waited on by phase parity.  Such a wait is right only if the
waiter can be neither a whole phase ahead of what it asks about nor two phases behind it: in the first case it passes
before the event has happened, in the second it cannot tell the phase it waits for from a later one of the same
parity.  Each role is a generator that yields at every wait; asynchronous completions (TMA arrivals, tcgen05.commit
arrivals) are delivered at random later points; every wait names the event it stands for, which must have happened
when the wait passes, and a run in which nobody can move any more is a deadlock.

Forward: K ring and V ring of two stages each, two score buffers (s_full / p_full per buffer), pv_done with one phase
per key tile (waited on by the softmax threads only when they rescale), o_full for the epilogue.
Backward: ring X of three stages, ring Y of one stage (launch that owns queries), two issuing threads that both commit
on s_full, one or more elementwise groups that arrive on p_full, `done` for the epilogue.
"""
import random

import pytest


class Bar:
    def __init__(self, count):
        self.count, self.pending, self.phase = count, count, 0

    def arrive(self):
        self.pending -= 1
        if self.pending == 0:
            self.pending = self.count
            self.phase += 1

    def passed(self, parity):
        """mbarrier.try_wait.parity: the phase with this parity has completed."""
        return (self.phase & 1) != parity


class World:
    def __init__(self, seed):
        self.rnd = random.Random(seed)
        self.events, self.pending, self.bars, self.tallies = set(), [], [], {}

    def bar(self, count):
        b = Bar(count)
        self.bars.append(b)
        return b

    def later(self, fn):
        self.pending.append(fn)

    def wait(self, bar, parity, need):
        while not bar.passed(parity):
            yield ("wait", need)
        assert need is None or need in self.events, f"wait passed before {need}"

    def tally(self, key, n, event):
        self.tallies[key] = self.tallies.get(key, 0) + 1
        if self.tallies[key] == n:
            self.events.add(event)

    def run(self, agents, names):
        alive, last, idle = [True] * len(agents), [None] * len(agents), 0

        def state():
            return (len(self.events), tuple(b.phase for b in self.bars), tuple(b.pending for b in self.bars),
                    len(self.pending))

        while any(alive):
            if self.pending and self.rnd.random() < 0.3:
                self.pending.pop(self.rnd.randrange(len(self.pending)))()
                idle = 0
                continue
            i = self.rnd.randrange(len(agents))
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
            if idle > 20000 and not self.pending:
                return "deadlock: " + str([(n, w) for n, w, a in zip(names, last, alive) if a])
        return "ok"


# ------------------------------------------------------------------------------------------------
# forward
# ------------------------------------------------------------------------------------------------
def run_forward(n_tiles, seed, epilogue_on_pv_done=False, rescale_prob=0.3):
    w = World(seed)
    k_full, k_empty = [w.bar(1), w.bar(1)], [w.bar(1), w.bar(1)]
    v_full, v_empty = [w.bar(1), w.bar(1)], [w.bar(1), w.bar(1)]
    s_full, p_full = [w.bar(1), w.bar(1)], [w.bar(1), w.bar(1)]
    pv_done, o_full = w.bar(1), w.bar(1)

    def producer():
        def load_k(t):
            yield from w.wait(k_empty[t & 1], ((t >> 1) & 1) ^ 1, ("s_done", t - 2) if t >= 2 else None)
            w.later(lambda: (w.events.add(("k", t)), k_full[t & 1].arrive()))

        def load_v(t):
            yield from w.wait(v_empty[t & 1], ((t >> 1) & 1) ^ 1, ("pv_done", t - 2) if t >= 2 else None)
            w.later(lambda: (w.events.add(("v", t)), v_full[t & 1].arrive()))

        yield from load_k(0)
        if n_tiles > 1:
            yield from load_k(1)
        for t in range(n_tiles):
            yield from load_v(t)
            if t + 2 < n_tiles:
                yield from load_k(t + 2)

    def issuer():
        def issue_s(t):
            yield from w.wait(k_full[t & 1], (t >> 1) & 1, ("k", t))
            # the commits arrive when the MMAs, and every MMA issued before them, have completed
            w.later(lambda: (w.events.add(("s_done", t)), s_full[t & 1].arrive(), k_empty[t & 1].arrive()))
            yield

        yield from issue_s(0)
        for t in range(n_tiles):
            if t + 1 < n_tiles:
                yield from issue_s(t + 1)
            yield from w.wait(p_full[t & 1], (t >> 1) & 1, ("p", t))
            yield from w.wait(v_full[t & 1], (t >> 1) & 1, ("v", t))
            w.later(lambda t=t: (w.events.add(("pv_done", t)), v_empty[t & 1].arrive(), pv_done.arrive()))
            yield
        w.later(lambda: (w.events.add("all_done"), o_full.arrive()))
        yield

    def softmax():
        for t in range(n_tiles):
            yield from w.wait(s_full[t & 1], (t >> 1) & 1, ("s_done", t))
            if t > 0 and w.rnd.random() < rescale_prob:
                yield from w.wait(pv_done, (t - 1) & 1, ("pv_done", t - 1))
            w.events.add(("p", t))
            p_full[t & 1].arrive()
            yield
        if epilogue_on_pv_done:
            yield from w.wait(pv_done, (n_tiles - 1) & 1, ("pv_done", n_tiles - 1))
        else:
            yield from w.wait(o_full, 0, "all_done")

    # tcgen05.commit arrivals of one issuing thread are delivered in issue order: model that by making each later()
    # of the issuer depend on the previous one having been delivered
    order = {"next": 0, "count": 0}
    raw_later = w.later

    def ordered_later(fn):
        me = order["count"]
        order["count"] += 1

        def attempt():
            if order["next"] == me:
                order["next"] += 1
                fn()
            else:
                raw_later(attempt)

        raw_later(attempt)

    issuer_gen = issuer()

    def issuer_wrapped():
        # route the issuer's completions through the in-order queue, everybody else's directly
        nonlocal issuer_gen
        while True:
            w.later = ordered_later
            try:
                x = next(issuer_gen)
            except StopIteration:
                w.later = raw_later
                return
            w.later = raw_later
            yield x

    return w.run([producer(), issuer_wrapped(), softmax()], ["producer", "issuer", "softmax"])


@pytest.mark.parametrize("n_tiles", [1, 2, 3, 4, 7, 16, 33])
def test_forward_protocol_has_no_deadlock_and_no_premature_pass(n_tiles):
    for seed in range(12):
        assert run_forward(n_tiles, seed) == "ok", (n_tiles, seed)


def test_forward_model_detects_an_epilogue_that_waits_on_the_per_tile_barrier():
    """A softmax thread that leaves the tile loop may be two phases of pv_done behind, where a parity wait cannot tell
    the last tile's phase from an earlier one: the epilogue has a barrier of its own (o_full) for that reason."""
    with pytest.raises(AssertionError):
        for seed in range(60):
            run_forward(8, seed, epilogue_on_pv_done=True, rescale_prob=0.0)


# ------------------------------------------------------------------------------------------------
# backward
# ------------------------------------------------------------------------------------------------
def run_backward(n_tiles, own_keys, groups, seed, second_skips_p_full=False):
    w = World(seed)
    STAGES = 3
    x_full = [w.bar(2 if own_keys else 1) for _ in range(STAGES)]  # own keys: TMA bytes + the row statistics
    x_empty = [w.bar(2 if own_keys else 1) for _ in range(STAGES)]  # own keys: both issuing threads read the stage
    y_full, y_empty = w.bar(1), w.bar(1)
    s_full, p_full = [w.bar(2), w.bar(2)], [w.bar(groups), w.bar(groups)]
    done = w.bar(1)

    def producer():
        for t in range(n_tiles):
            st = t % STAGES
            yield from w.wait(x_empty[st], ((t // STAGES) & 1) ^ 1, ("x_free", t - STAGES) if t >= STAGES else None)
            w.later(lambda t=t, st=st: (w.tally(("x", t), 2 if own_keys else 1, ("x", t)), x_full[st].arrive()))
            if own_keys:
                w.tally(("x", t), 2, ("x", t))
                x_full[st].arrive()  # the statistics
            else:
                yield from w.wait(y_empty, (t & 1) ^ 1, ("e_done", t - 1) if t >= 1 else None)
                w.later(lambda t=t: (w.events.add(("y", t)), y_full.arrive()))
            yield

    def in_order(gen):
        """tcgen05.commit arrivals of one issuing thread are delivered in issue order."""
        order = {"next": 0, "count": 0}
        raw = w.later

        def ordered(fn):
            me = order["count"]
            order["count"] += 1

            def attempt():
                if order["next"] == me:
                    order["next"] += 1
                    fn()
                else:
                    raw(attempt)

            raw(attempt)

        while True:
            w.later = ordered
            try:
                x = next(gen)
            except StopIteration:
                w.later = raw
                return
            w.later = raw
            yield x

    def first():
        def issue_s(t):
            yield from w.wait(x_full[t % STAGES], (t // STAGES) & 1, ("x", t))
            # [S | TS] of tile t overwrite the buffer whose operands the outputs of tile t - 2 read: same thread, in order
            assert t < 2 or ("out_issued", t - 2) in w.events
            w.later(lambda: (w.tally(("s", t), 2, ("scores", t)), s_full[t & 1].arrive()))
            yield

        yield from issue_s(0)
        for t in range(n_tiles):
            if t + 1 < n_tiles:
                yield from issue_s(t + 1)
            yield from w.wait(p_full[t & 1], (t >> 1) & 1, ("operands", t))
            w.events.add(("out_issued", t))
            w.later(lambda t=t: (w.tally(("xf", t), 2 if own_keys else 1, ("x_free", t)), x_empty[t % STAGES].arrive()))
            yield
        w.later(lambda: (w.events.add("all_done"), done.arrive()))
        yield

    def second():
        def issue_e(t):
            if own_keys:
                yield from w.wait(x_full[t % STAGES], (t // STAGES) & 1, ("x", t))
            else:
                yield from w.wait(y_full, t & 1, ("y", t))
            # [E | FP] of tile t overwrite what the elementwise threads read for tile t - 2
            assert t < 2 or ("operands", t - 2) in w.events, f"E/FP of tile {t} overwritten before tile {t - 2} was read"

            def complete():
                w.tally(("s", t), 2, ("scores", t))
                s_full[t & 1].arrive()
                w.events.add(("e_done", t))
                if own_keys:
                    w.tally(("xf", t), 2, ("x_free", t))
                    x_empty[t % STAGES].arrive()
                else:
                    y_empty.arrive()

            w.later(complete)
            yield

        yield from issue_e(0)
        for t in range(n_tiles - 1):
            yield from issue_e(t + 1)
            if not second_skips_p_full:
                yield from w.wait(p_full[t & 1], (t >> 1) & 1, ("operands", t))

    def elementwise(grp):
        for t in range(n_tiles):
            if own_keys:
                yield from w.wait(x_full[t % STAGES], (t // STAGES) & 1, ("x", t))
            yield from w.wait(s_full[t & 1], (t >> 1) & 1, ("scores", t))
            w.tally(("p", t), groups, ("operands", t))
            p_full[t & 1].arrive()
            yield
        yield from w.wait(done, 0, "all_done")

    agents = [producer(), in_order(first()), in_order(second())] + [elementwise(g) for g in range(groups)]
    return w.run(agents, ["producer", "issuer1", "issuer2"] + [f"elem{g}" for g in range(groups)])


@pytest.mark.parametrize("own_keys,groups", [(True, 2), (False, 3)], ids=["own_keys", "own_queries"])
def test_backward_protocol_has_no_deadlock_and_no_premature_pass(own_keys, groups):
    for n_tiles in (1, 2, 3, 4, 5, 9, 32):
        for seed in range(10):
            assert run_backward(n_tiles, own_keys, groups, seed) == "ok", (n_tiles, seed)


def test_backward_model_detects_a_second_issuer_that_does_not_wait_for_the_readers():
    """The second issuing thread issues no output products, but it still has to wait for p_full(t): that is what tells
    it that E and FP of tile t have been read before it forms those of tile t + 2 in the same buffer."""
    with pytest.raises(AssertionError):
        for seed in range(60):
            run_backward(12, False, 3, seed, second_skips_p_full=True)
