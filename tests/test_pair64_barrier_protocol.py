"""A model of the mbarrier protocol of the head-dimension-64 forward (csrc/fwd_tc5_pair64.cu), run under random
interleavings on the CPU.

One persistent CTA serves items of two 128-row query tiles X = 0, 1 that share every key stage.  Roles: the TMA producer
(the item's Q tiles once, then the key tiles some query tile uses, through a three-stage ring), one issuing thread per
query tile, one softmax warpgroup per query tile.  With a boolean mask and its tile bitmap a key tile may be used by
both query tiles, by one of them, or by none (then nobody loads it); an issuing thread releases a stage it does not use
by a plain arrival, after flushing a pending output product that still reads an older stage.

Barriers, with the kernel's names: q_full / q_empty (both issuing threads arrive once per item, used or not);
kv_full / kv_empty per stage (two arrivals); per query tile s_full, s_free, p_full, pv_done (one phase per used tile)
and o_free (one phase per item in which the query tile used a tile).  The engine is the one of the other models
(tests/test_pipe128_barrier_protocol.py): every wait names the event it stands for, asynchronous completions arrive
later (those of one issuing thread in issue order), and a state in which nobody can move is a deadlock.  Data hazards
are asserted where the kernel relies on an ordering: the scores of tile t+1 overwrite the score accumulator only after
the softmax threads have read tile t; P and W of tile t are written only after the output products of tile t-1 have
read the shared-memory tiles; the first output product of an item overwrites O only after the previous epilogue.
"""
import pytest

from tests.test_fused64_barrier_protocol import in_order
from tests.test_pipe128_barrier_protocol import World

STAGES = 3


def run_pair64(items, seed, grow_prob=0.3, skip_flush=False):
    """items: list of lists; items[k][j] in {0, 1, 2, 3} says which query tiles use key tile j of item k (bit X).
    skip_flush: the issuing thread releases a stage it does not use without first issuing its pending output product
    (the mistake the kernel's comment warns about)."""
    w = World(seed)
    q_full, q_empty = w.bar(1), w.bar(2)
    kv_full = [w.bar(1) for _ in range(STAGES)]
    kv_empty = [w.bar(2) for _ in range(STAGES)]
    s_full, s_free = [w.bar(1), w.bar(1)], [w.bar(1), w.bar(1)]
    p_full, pv_done, o_free = [w.bar(1), w.bar(1)], [w.bar(1), w.bar(1)], [w.bar(1), w.bar(1)]
    live = [(k, use) for k, use in enumerate(items) if any(use)]  # items with n_load > 0

    def last(use, X):
        js = [j for j, m in enumerate(use) if m & (1 << X)]
        return js[-1] if js else -1

    def producer():
        g = 0
        for kact, (k, use) in enumerate(live):
            if kact > 0:
                yield from w.wait(q_empty, (kact - 1) & 1, ("q_released", kact - 1))
            w.later(lambda kact=kact: (w.events.add(("q", kact)), q_full.arrive()))
            for m in use:
                if m == 0:
                    continue
                st = g % STAGES
                yield from w.wait(kv_empty[st], ((g // STAGES) & 1) ^ 1, ("kv_free", g - STAGES) if g >= STAGES else None)
                w.later(lambda g=g, st=st: (w.events.add(("kv", g)), kv_full[st].arrive()))
                g += 1
                yield

    def issuer(X):
        g, T, kx = 0, 0, 0  # loaded tiles seen, tiles used by this query tile, items in which it used a tile
        for kact, (k, use) in enumerate(live):
            yield from w.wait(q_full, kact & 1, ("q", kact))
            my_last = last(use, X)
            pend, first = None, True

            def issue_pv(p):
                pg, pT, pfirst = p
                yield from w.wait(p_full[X], pT & 1, ("p", X, pT))
                if pfirst and kx > 0:
                    yield from w.wait(o_free[X], (kx - 1) & 1, ("o_read", X, kx - 1))
                w.later(lambda: (w.tally(("kvf", pg), 2, ("kv_free", pg)), kv_empty[pg % STAGES].arrive(),
                                 w.events.add(("pv", X, pT)), pv_done[X].arrive()))
                yield

            for j, m in enumerate(use):
                if m == 0:
                    continue
                st = g % STAGES
                yield from w.wait(kv_full[st], (g // STAGES) & 1, ("kv", g))
                if m & (1 << X):
                    if T > 0:
                        yield from w.wait(s_free[X], (T - 1) & 1, ("s_read", X, T - 1))

                    def scores_done(T=T, last_one=(j == my_last), kact=kact):
                        w.events.add(("s", X, T))
                        s_full[X].arrive()
                        if last_one:
                            w.tally(("qr", kact), 2, ("q_released", kact))
                            q_empty.arrive()

                    w.later(scores_done)
                    yield
                    if pend is not None:
                        yield from issue_pv(pend)
                    pend, first = (g, T, first), False
                    T += 1
                else:
                    if pend is not None and not skip_flush:
                        yield from issue_pv(pend)
                        pend = None
                    w.tally(("kvf", g), 2, ("kv_free", g))
                    kv_empty[st].arrive()
                    yield
                g += 1
            if pend is not None:
                yield from issue_pv(pend)
            if not first:
                kx += 1
            else:
                w.tally(("qr", kact), 2, ("q_released", kact))
                q_empty.arrive()
            yield

    def softmax(X):
        T, kx = 0, 0
        for k, use in enumerate(items):
            n_used = sum(1 for m in use if m & (1 << X))
            if n_used == 0:
                yield  # zeros and lse = +inf: no barrier of the protocol is touched
                continue
            for u in range(n_used):
                yield from w.wait(s_full[X], T & 1, ("s", X, T))
                w.events.add(("s_read", X, T))
                s_free[X].arrive()
                yield
                seen = False
                if u > 0 and w.rnd.random() < grow_prob:  # the running maximum grew: O is rescaled in place
                    yield from w.wait(pv_done[X], (T - 1) & 1, ("pv", X, T - 1))
                    seen = True
                if T > 0 and not seen:
                    yield from w.wait(pv_done[X], (T - 1) & 1, ("pv", X, T - 1))
                assert T == 0 or ("pv", X, T - 1) in w.events  # P / W are single-buffered
                w.events.add(("p", X, T))
                p_full[X].arrive()
                T += 1
                yield
            yield from w.wait(pv_done[X], (T - 1) & 1, ("pv", X, T - 1))
            w.events.add(("o_read", X, kx))
            o_free[X].arrive()
            kx += 1
            yield

    agents = [producer(), in_order(w, issuer(0)), in_order(w, issuer(1)), softmax(0), softmax(1)]
    return w.run(agents, ["producer", "issuer0", "issuer1", "softmax0", "softmax1"])


def causal_items(n_pairs):
    """Item p: query tiles 2p and 2p+1 of 128 rows, 64-key tiles; tile X uses keys below its last row."""
    out = []
    for p in range(n_pairs):
        n0, n1 = 2 * (2 * p + 1), 2 * (2 * p + 2)
        out.append([(1 if j < n0 else 0) | (2 if j < n1 else 0) for j in range(n1)])
    return out


@pytest.mark.parametrize("items", [
    [[3]], [[3, 3, 3, 3, 3, 3, 3]], [[3] * 5, [3] * 2, [3]], causal_items(3), [[1, 1], [2, 2], [3]],
    [[3, 1, 2, 0, 3, 2, 2, 1, 1, 3], [0, 0], [2, 0, 1], [1, 1, 1, 1, 2]], [[0, 0, 0], [2], [1], [3, 3]],
], ids=lambda x: "-".join("".join(map(str, it)) for it in x)[:40])
def test_pair64_protocol_has_no_deadlock_and_no_premature_pass(items):
    for seed in range(10):
        assert run_pair64(items, seed) == "ok", (items, seed)
    assert run_pair64(items, 99, grow_prob=0.0) == "ok"
    assert run_pair64(items, 98, grow_prob=1.0) == "ok"


def test_pair64_protocol_random_tile_maps():
    import random

    rnd = random.Random(7)
    for trial in range(25):
        items = [[rnd.choice([0, 1, 2, 3, 3]) for _ in range(rnd.randint(1, 9))] for _ in range(rnd.randint(1, 5))]
        assert run_pair64(items, trial) == "ok", items


def test_pair64_model_shows_why_a_pending_product_is_flushed_before_a_plain_release():
    """An issuing thread that releases the stages it does not use while an output product of an older stage is still
    pending lets the producer run into that older stage: the producer waits for the stage, the thread for the producer."""
    items = [[3, 2, 2, 2, 2, 2, 2, 3, 3]]
    results = [run_pair64(items, seed, skip_flush=True) for seed in range(20)]
    assert any(r.startswith("deadlock") for r in results), results
