"""A model of the mbarrier protocol of the single-pass head-dimension-64 backward (csrc/bwd_tc5_fused64.cu), run under
random interleavings on the CPU.

Roles of a CTA: the TMA producer (own tiles once per item, streamed tiles and row statistics per sub-tile), three
issuing threads (scores; dK and dV; dQ), two elementwise groups and the dQ read-back group.  They talk only through
mbarriers waited on by phase parity, so every waiter has to stay within one phase of what it waits for.  The engine
(World) is the one of the head-dimension-128 models: each role is a generator that yields at every wait, asynchronous
completions are delivered at random later points (those of one issuing thread in issue order), every wait names the
event it stands for, and a run in which nobody can move is reported as a deadlock.

The barrier that needs care is p_full.  Sub-tile g + 1 of the elementwise groups depends on the dV products of g
(av_free) and on the products of g - 1 (out_free), but not on the dQ product of g.  The groups can therefore complete
p_full(g + 1) before the dQ issuer has looked at p_full(g); with a single barrier that issuer is then two phases
behind and its parity wait never passes.  The kernel has one p_full per result buffer (g & 1) for that reason, and
the model shows both the stall of the single barrier and the absence of one with the pair.
"""
import pytest

from tests.test_pipe128_barrier_protocol import World

GROUPS = 2  # elementwise groups (128 threads each in the kernel; one agent each here)


def in_order(w, gen):
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


def run_fused64(n_subs, stages, seed, single_p_full=False, slow_dq=0.0, own_bufs=1):
    """One random interleaving for a CTA whose item k has n_subs[k] sub-tiles (0: an item of padding only, which every
    role skips).  slow_dq: probability with which the dQ issuer lets a turn pass without doing anything.  own_bufs: sets
    of own tiles (2 in the variant without tangents: the next item's are loaded while this item still runs)."""
    w = World(seed)
    own_full = [w.bar(1) for _ in range(own_bufs)]
    own_free = [w.bar(2) for _ in range(own_bufs)]
    loop_full = [w.bar(1) for _ in range(stages)]
    loop_empty = [w.bar(2) for _ in range(stages)]
    stat_full = [w.bar(1) for _ in range(stages)]
    s_full, s_free = w.bar(1), w.bar(GROUPS)
    p_full = [w.bar(GROUPS)] if single_p_full else [w.bar(GROUPS), w.bar(GROUPS)]
    out_free = [w.bar(2), w.bar(2)]
    av_free, dq_full, dq_free = w.bar(1), w.bar(1), w.bar(1)
    done, acc_free = w.bar(1), w.bar(GROUPS)
    items = [(k, n) for k, n in enumerate(n_subs) if n > 0]

    def wait_p_full(g):
        if single_p_full:
            return w.wait(p_full[0], g & 1, ("operands", g))
        return w.wait(p_full[g & 1], (g >> 1) & 1, ("operands", g))

    def producer():
        g = 0
        for kact, (k, n) in enumerate(items):
            oset, ouse = kact % own_bufs, kact // own_bufs
            if ouse > 0:
                yield from w.wait(own_free[oset], (ouse - 1) & 1, ("own_released", kact - own_bufs))
            w.later(lambda kact=kact, oset=oset: (w.events.add(("own", kact)), own_full[oset].arrive()))
            for _ in range(n):
                st = g % stages
                yield from w.wait(loop_empty[st], ((g // stages) & 1) ^ 1, ("ring_free", g - stages) if g >= stages else None)
                w.later(lambda g=g, st=st: (w.events.add(("loop", g)), loop_full[st].arrive()))
                # the statistics of the stage are overwritten here: their readers must be through
                assert g < stages or ("operands", g - stages) in w.events
                w.events.add(("stat", g))
                stat_full[st].arrive()
                g += 1
                yield

    def scores():
        g = 0
        for kact, (k, n) in enumerate(items):
            yield from w.wait(own_full[kact % own_bufs], (kact // own_bufs) & 1, ("own", kact))
            for _ in range(n):
                st = g % stages
                yield from w.wait(loop_full[st], (g // stages) & 1, ("loop", g))
                if g > 0:
                    yield from w.wait(s_free, (g - 1) & 1, ("scores_read", g - 1))
                w.later(lambda g=g, st=st: (w.events.add(("scores", g)), s_full.arrive(),
                                            w.tally(("rf", g), 2, ("ring_free", g)), loop_empty[st].arrive()))
                g += 1
                yield
            w.later(lambda kact=kact: (w.tally(("or", kact), 2, ("own_released", kact)), own_free[kact % own_bufs].arrive()))

    def dkdv():
        g = 0
        for kact, (k, n) in enumerate(items):
            for s in range(n):
                st, ob = g % stages, g & 1
                yield from wait_p_full(g)
                if s == 0 and kact > 0:
                    yield from w.wait(acc_free, (kact - 1) & 1, ("acc_read", kact - 1))
                w.later(lambda g=g, st=st, ob=ob: (w.tally(("rf", g), 2, ("ring_free", g)), loop_empty[st].arrive(),
                                                   w.tally(("of", g), 2, ("out_read", g)), out_free[ob].arrive(),
                                                   w.events.add(("av_read", g)), av_free.arrive()))
                g += 1
                yield
            w.later(lambda kact=kact: (w.events.add(("done", kact)), done.arrive()))

    def dq():
        g = 0
        for kact, (k, n) in enumerate(items):
            for _ in range(n):
                while w.rnd.random() < slow_dq:
                    yield ("dawdle", g)
                ob = g & 1
                yield from wait_p_full(g)
                if g >= 1:
                    yield from w.wait(dq_free, (g - 1) & 1, ("dq_read", g - 1))
                w.later(lambda g=g, ob=ob: (w.events.add(("dq", g)), dq_full.arrive(),
                                            w.tally(("of", g), 2, ("out_read", g)), out_free[ob].arrive()))
                g += 1
                yield
            w.later(lambda kact=kact: (w.tally(("or", kact), 2, ("own_released", kact)), own_free[kact % own_bufs].arrive()))

    def elementwise(grp):
        g = 0
        for kact, (k, n) in enumerate(items):
            for _ in range(n):
                st, ob, use = g % stages, g & 1, g >> 1
                yield from w.wait(stat_full[st], (g // stages) & 1, ("stat", g))
                yield from w.wait(s_full, g & 1, ("scores", g))
                w.tally(("sr", g), GROUPS, ("scores_read", g))
                s_free.arrive()
                yield
                if use > 0:
                    yield from w.wait(out_free[ob], (use - 1) & 1, ("out_read", g - 2))
                if g > 0:
                    yield from w.wait(av_free, (g - 1) & 1, ("av_read", g - 1))
                w.tally(("p", g), GROUPS, ("operands", g))
                p_full[0 if single_p_full else ob].arrive()
                g += 1
                yield
            yield from w.wait(done, kact & 1, ("done", kact))
            w.tally(("ar", kact), GROUPS, ("acc_read", kact))
            acc_free.arrive()
            yield

    def read_back():
        g = 0
        for kact, (k, n) in enumerate(items):
            for _ in range(n):
                yield from w.wait(dq_full, g & 1, ("dq", g))
                w.events.add(("dq_read", g))
                dq_free.arrive()
                g += 1
                yield

    agents = [producer(), in_order(w, scores()), in_order(w, dkdv()), in_order(w, dq())]
    agents += [elementwise(i) for i in range(GROUPS)] + [read_back()]
    names = ["producer", "scores", "dkdv", "dq"] + [f"elem{i}" for i in range(GROUPS)] + ["read_back"]
    return w.run(agents, names)


@pytest.mark.parametrize("stages", [2, 3])
@pytest.mark.parametrize("n_subs", [[1], [2], [5], [1, 1, 1], [3, 0, 4], [16, 8, 1], [32]], ids=str)
def test_fused64_protocol_has_no_deadlock_and_no_premature_pass(n_subs, stages):
    for seed in range(8):
        assert run_fused64(n_subs, stages, seed) == "ok", (n_subs, stages, seed)
        assert run_fused64(n_subs, stages, seed, slow_dq=0.9) == "ok", (n_subs, stages, seed, "slow dQ issuer")
        assert run_fused64(n_subs, stages, seed, own_bufs=2) == "ok", (n_subs, stages, seed, "two sets of own tiles")
        assert run_fused64(n_subs, stages, seed, slow_dq=0.9, own_bufs=2) == "ok", (n_subs, stages, seed, "two sets, slow dQ")


def test_fused64_model_shows_the_stall_of_a_single_p_full_barrier():
    """With one p_full barrier and a dQ issuer that is late, the elementwise groups complete two phases before the
    issuer has seen the first one, and its wait never passes."""
    results = [run_fused64([24], 3, seed, single_p_full=True, slow_dq=0.97) for seed in range(10)]
    assert any(r.startswith("deadlock") and "'dq'" in r for r in results), results
