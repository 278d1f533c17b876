"""CPU model of the barrier protocol of the tensor-core forward kernel (csrc/tc_fwd.cuh).

The kernel's producer, its two product-issuing threads and its two row groups are modelled as
coroutines that wait on parity barriers exactly as the CUDA code does (same slot / phase arithmetic,
same barrier counts per role); copies and tensor products complete asynchronously, products in issue
order per issuing thread.  A random scheduler interleaves everything.  The model checks that

  * nothing deadlocks and every agent runs to its end,
  * every product reads the ring slot content it expects and every row group reads the score buffer
    it expects (a parity wait passed by a thread that had not seen the barrier's previous phase
    shows up here as stale content),
  * the P.V products of the last pass see their own tile's probabilities, in order.

With an odd ring depth and the issuers on alternate tiles the model fails (that configuration once
faulted on the device); the kernel's even depths pass.  The second test checks the arrival counts
of the named-barrier turn taking between the two row groups.

Both forms of the kernel are modelled: one query tile per thread block (Lazy Attention, the
candidate-list solver, FLA_FLAG_ONE_TILE_CTAS) and two (pair=True: issuer and row group g own query
tile g and work on every key tile, with the running tile index 2t + g in the slot and phase
arithmetic; a ring slot is released by both issuers; in the last pass each issuer runs its own
S -> P -> P.V chain with the probabilities written over the scores).
"""
import random

import pytest


class Bar:
    def __init__(s, count): s.count = count; s.pending = count; s.phase = 0
    def arrive(s):
        s.pending -= 1
        assert s.pending >= 0
        if s.pending == 0: s.phase += 1; s.pending = s.count
    def done(s, parity): return (s.phase & 1) != parity

def run(nkt, actives, seed, stages=4, verbose=False, pair=False):
    # actives: list of tile lists, one per score pass (pass 0 = all), plus the last pass's list
    # pair: the form with two query tiles per thread block (issuer / row group g owns query tile g)
    rnd = random.Random(seed)
    npass = len(actives) - 1            # score passes
    nuse = 2 if pair else 1             # issuers that read a ring slot before it is released
    B = dict(ring_full=[Bar(2) for _ in range(stages)], ring_empty=[Bar(nuse) for _ in range(stages)],
             s_full=[Bar(1) for _ in range(4)], s_free=[Bar(1) for _ in range(4)],
             f_full=[Bar(1) for _ in range(2)], p_full=[Bar(1) for _ in range(2)], pv_done=[Bar(1) for _ in range(2)],
             pass_done=Bar(1), pass_ack=Bar(3), o_full=Bar(nuse), grp=Bar(2))
    state = dict(cont=None, ring=[None] * stages, sbuf=[None] * 4, P=[None] * 2, o=[], o2=([], []),
                 readers=[0] * stages)
    def release(st):
        # a slot's content is gone once every issuer that reads it has done so
        state["readers"][st] += 1
        if state["readers"][st] == nuse:
            state["readers"][st] = 0; state["ring"][st] = None
    events = []   # async completions: (fn)
    log = []
    def adv(rp):
        rp[0] += 1
        if rp[0] == stages: rp[0] = 0; rp[1] ^= 1

    def producer():
        rp = [0, 0]; ps = 0
        def load(tag):
            yield ("wait", B["ring_empty"][rp[0]], rp[1] ^ 1, "prod ring_empty")
            st = rp[0]
            B["ring_full"][st].arrive()
            def land(st=st, tag=tag):
                state["ring"][st] = tag; B["ring_full"][st].arrive()
            events.append(land)
            adv(rp)
        while True:
            for kt in actives[ps]:
                yield from load(("K", ps, kt))
            yield ("wait", B["pass_done"], ps & 1, "prod pass_done")
            ps += 1
            go = state["cont"]
            B["pass_ack"].arrive()
            if not go: break
        assert ps == npass, ("producer pass count", ps, npass)
        prev = None
        for kt in actives[ps]:
            yield from load(("K", "fin", kt))
            if prev is not None: yield from load(("V", "fin", prev))
            prev = kt
        if prev is not None: yield from load(("V", "fin", prev))

    def issuer(me):
        rp = [0, 0]; sn = 0; ps = 0
        queue = []   # in-order async completion per issuer
        def commit(fn): queue.append(fn)
        def flush_event():
            if queue:
                fn = queue.pop(0); fn()
        issuer_queues[me] = queue
        while True:
            for kt in actives[ps]:
                if pair or (sn & 1) == me:
                    vs = 2 * sn + me if pair else sn
                    sb = vs & 3
                    yield ("wait", B["ring_full"][rp[0]], rp[1], f"iss{me} ring_full")
                    yield ("wait", B["s_free"][sb], ((vs >> 2) & 1) ^ 1, f"iss{me} s_free")
                    st = rp[0]
                    assert state["ring"][st] == ("K", ps, kt), ("wrong ring content", state["ring"][st], ps, kt)
                    def done(st=st, sb=sb, tag=(ps, kt)):
                        state["sbuf"][sb] = tag; release(st)
                        B["ring_empty"][st].arrive(); B["s_full"][sb].arrive()
                    commit(done)
                adv(rp); sn += 1
            yield ("wait", B["pass_done"], ps & 1, f"iss{me} pass_done")
            ps += 1
            go = state["cont"]
            B["pass_ack"].arrive()
            if not go: break
        assert ps == npass, ("issuer pass count", me, ps, npass)
        fin = actives[ps]
        s_role = (sn & 1) == me
        pos0 = sn      # tiles that went through the ring so far (one slot per tile in the score passes)
        nf = len(fin)
        if pair:
            # issuer `me` runs the chain S -> P -> P.V of query tile `me`: score buffer `me`, accumulator `me`
            for t, kt in enumerate(fin):
                k_ofs = 0 if t == 0 else 2 * t - 1
                v_ofs = 2 * nf - 1 if t == nf - 1 else 2 * t + 2
                stk = (pos0 + k_ofs) % stages; phk = ((pos0 + k_ofs) // stages) & 1
                stv = (pos0 + v_ofs) % stages; phv = ((pos0 + v_ofs) // stages) & 1
                yield ("wait", B["ring_full"][stk], phk, f"iss{me} fin K ring_full")
                if t >= 1: yield ("wait", B["pv_done"][me], (t - 1) & 1, f"iss{me} pv_done")
                assert state["ring"][stk] == ("K", "fin", kt), ("fin wrong K", state["ring"][stk], kt)
                assert t == 0 or state["o2"][me][-1:] == [fin[t - 1]], "S over P before P.V read it"
                def done_s(st=stk, kt=kt):
                    state["sbuf"][me] = ("fin", kt); release(st)
                    B["ring_empty"][st].arrive(); B["f_full"][me].arrive()
                commit(done_s)
                yield ("wait", B["p_full"][me], t & 1, f"iss{me} p_full")
                yield ("wait", B["ring_full"][stv], phv, f"iss{me} fin V ring_full")
                assert state["ring"][stv] == ("V", "fin", kt), ("fin wrong V", state["ring"][stv], kt)
                assert state["P"][me] == kt, ("wrong P", state["P"][me], kt)
                def done_pv(st=stv, kt=kt):
                    state["o2"][me].append(kt); release(st)
                    B["ring_empty"][st].arrive(); B["pv_done"][me].arrive()
                commit(done_pv)
            commit(lambda: B["o_full"].arrive())
            return
        for t, kt in enumerate(fin):
            sb = t & 1
            ofs = (0 if t == 0 else 2 * t - 1) if s_role else (2 * nf - 1 if t == nf - 1 else 2 * t + 2)
            st = (pos0 + ofs) % stages; ph = ((pos0 + ofs) // stages) & 1
            yield ("wait", B["ring_full"][st], ph, f"iss{me} fin ring_full")
            if s_role:
                if t >= 2: yield ("wait", B["p_full"][sb], ((t - 2) >> 1) & 1, "issS p_full")
                assert state["ring"][st] == ("K", "fin", kt), ("fin wrong K", state["ring"][st], kt)
                def done(st=st, sb=sb, kt=kt):
                    state["sbuf"][sb] = ("fin", kt); release(st)
                    B["ring_empty"][st].arrive(); B["f_full"][sb].arrive()
                commit(done)
            else:
                yield ("wait", B["p_full"][sb], (t >> 1) & 1, "issPV p_full")
                assert state["ring"][st] == ("V", "fin", kt), ("fin wrong V", state["ring"][st], kt)
                assert state["P"][sb] == kt, ("wrong P", state["P"][sb], kt)
                def done(st=st, sb=sb, kt=kt):
                    state["o"].append(kt); release(st)
                    B["ring_empty"][st].arrive(); B["pv_done"][sb].arrive()
                commit(done)
        if not s_role: commit(lambda: B["o_full"].arrive())

    def rows(g):
        sn = 0; rpass = 0; signalled = 0
        for ps in range(npass):
            run_i = sn
            for kt in actives[ps]:
                cs = run_i; run_i += 1
                if pair: cs = 2 * cs + g      # every tile, for this group's query tile
                elif (cs & 1) != g: continue
                buf = cs & 3
                yield ("wait", B["s_full"][buf], (cs >> 2) & 1, f"rows{g} s_full")
                assert state["sbuf"][buf] == (ps, kt), ("rows read wrong buffer", state["sbuf"][buf], ps, kt)
                B["s_free"][buf].arrive()
            sn = run_i
            # named barrier between the groups (two phases: all arrive, then proceed)
            ph = B["grp"].phase & 1
            B["grp"].arrive()
            yield ("wait", B["grp"], ph, f"rows{g} group barrier")
            if g == 0:
                if signalled > 0: yield ("wait", B["pass_ack"], (signalled - 1) & 1, "tid0 pass_ack")
                signalled += 1
                state["cont"] = ps + 1 < npass
                B["pass_done"].arrive()
        fin = actives[npass]
        if pair:
            for u, kt in enumerate(fin):
                yield ("wait", B["f_full"][g], u & 1, f"rows{g} f_full")
                assert state["sbuf"][g] == ("fin", kt), ("rows fin wrong", state["sbuf"][g], kt)
                state["sbuf"][g] = None          # the probabilities go over the scores
                state["P"][g] = kt
                B["p_full"][g].arrive()
            yield ("wait", B["o_full"], 0, f"rows{g} o_full")
            assert state["o2"][g] == fin, ("O order", g, state["o2"][g], fin)
            return
        for u, kt in enumerate(fin):
            if (u & 1) != g: continue
            yield ("wait", B["f_full"][g], (u >> 1) & 1, f"rows{g} f_full")
            assert state["sbuf"][g] == ("fin", kt), ("rows fin wrong", state["sbuf"][g], kt)
            if u >= 2:
                yield ("wait", B["pv_done"][g], ((u - 2) >> 1) & 1, f"rows{g} pv_done")
                assert state["o"] and fin[u - 2] in state["o"], "P overwritten before use"
            state["P"][g] = kt
            B["p_full"][g].arrive()
        yield ("wait", B["o_full"], 0, f"rows{g} o_full")
        assert state["o"] == fin, ("O order", state["o"], fin)

    issuer_queues = {}
    agents = {"prod": producer(), "iss0": issuer(0), "iss1": issuer(1), "rows0": rows(0), "rows1": rows(1)}
    waiting = {}
    for name, gen in list(agents.items()):
        try: waiting[name] = next(gen)
        except StopIteration: del agents[name]
    steps = 0
    while agents:
        steps += 1
        choices = []
        for name in agents:
            w = waiting[name]
            if w[1].done(w[2]): choices.append(("agent", name))
        for i in range(len(events)): choices.append(("event", i))
        for me, qu in issuer_queues.items():
            if qu: choices.append(("mma", me))
        if not choices:
            return "DEADLOCK: " + "; ".join(f"{n} at {waiting[n][3]}" for n in agents)
        kind, x = rnd.choice(choices)
        if kind == "agent":
            try: waiting[x] = next(agents[x])
            except StopIteration: del agents[x]
        elif kind == "event":
            events.pop(x)()
        else:
            issuer_queues[x].pop(0)()
        if steps > 10**6: return "LIVELOCK"
    return None

def shrink(nkt, npass, rnd):
    acts = [list(range(nkt)), list(range(nkt))]
    cur = list(range(nkt))
    for _ in range(npass - 1):
        keep = [k for k in cur if rnd.random() < 0.7] or [rnd.choice(cur)]
        cur = keep; acts.append(cur)
    acts = acts[:npass]
    acts.append(cur if npass > 1 else list(range(nkt)))   # last pass: the final bitmap
    return acts



def _cases(rnd, n):
    for _ in range(n):
        nkt = rnd.randint(1, 9)
        npass = rnd.randint(1, 6)
        yield nkt, shrink(nkt, npass, rnd)


@pytest.mark.parametrize("stages", [4, 8])
def test_forward_protocol_has_no_deadlock_or_stale_operand(stages):
    rnd = random.Random(stages)
    for trial, (nkt, acts) in enumerate(_cases(rnd, 1500)):
        assert run(nkt, acts, trial, stages=stages) is None, (nkt, acts)


@pytest.mark.parametrize("stages", [4, 8])
def test_two_tile_form_has_no_deadlock_or_stale_operand(stages):
    """Two query tiles per block: a ring slot is read by both issuers, each issuer and row group runs its own
    S -> P -> P.V chain in the last pass, the output barrier takes one arrival per issuer."""
    rnd = random.Random(100 + stages)
    for trial, (nkt, acts) in enumerate(_cases(rnd, 1500)):
        assert run(nkt, acts, trial, stages=stages, pair=True) is None, (nkt, acts)


def test_odd_ring_depth_is_caught_by_the_model():
    rnd = random.Random(5)
    failures = 0
    for trial, (nkt, acts) in enumerate(_cases(rnd, 1500)):
        try:
            failures += run(nkt, acts, trial, stages=5) is not None
        except AssertionError:
            failures += 1
    assert failures > 0


def _turns(first, nact, seed):
    """Row groups g = 0, 1; barrier 4+g = "group g's turn" (one unit = one whole group arriving)."""
    rnd = random.Random(seed)
    bars = {0: 0, 1: 0}

    def agent(g):
        mine = [k for k in range(nact) if (first + k) % 2 == g]
        if g != first:
            yield ("arrive", first)
        for _ in mine:
            yield ("sync", g)
            yield ("arrive", g ^ 1)
        last = (first + nact + 1) % 2
        if (nact > 0 and g != last) or (nact == 0 and g == first):
            yield ("sync", g)

    ags = {0: agent(0), 1: agent(1)}
    cur = {}
    for g in (0, 1):
        try:
            cur[g] = next(ags[g])
        except StopIteration:
            pass
    while cur:
        runnable = [g for g, op in cur.items() if op[0] == "arrive" or bars[op[1]] > 0]
        if not runnable:
            return "deadlock"
        g = rnd.choice(runnable)
        op = cur[g]
        if op[0] == "arrive":
            bars[op[1]] += 1
            if bars[op[1]] > 1:
                return "double arrival"
        else:
            bars[op[1]] -= 1
        try:
            cur[g] = next(ags[g])
        except StopIteration:
            del cur[g]
    return "leftover" if bars[0] or bars[1] else None


def test_turn_taking_counts_balance_for_every_pass_shape():
    for first in (0, 1):
        for nact in range(0, 14):
            for seed in range(30):
                assert _turns(first, nact, seed) is None, (first, nact)
