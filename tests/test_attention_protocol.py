"""A host model of the barrier protocol of the persistent attention kernel (monoserve_b200/csrc/attention.cu,
attention_core.cuh): one CTA's producer, MMA warp and two softmax groups working through a chain of items with
no CTA-wide barrier between them, under random interleavings.  The model carries the same mbarriers with the same
arrival counts and phase arithmetic (uses of a stage counted across items), the two kinds of item (quad-replicated
decode items done by group 0; items whose key tiles alternate between the groups, S of tile j + 2 issued before
P V of tile j, K requested ahead of V) and tags every buffer with the (item, tile) it holds, so that a read of the
wrong tile, an overwrite of an unread buffer or a deadlock shows.  Two rules of the device code are then checked
by breaking them: a warp without rows must delay its P arrival like a working warp, and every softmax thread
passes one barrier between reading the accumulators and the next item.  A second model covers the failure path:
the abort flag goes up at an arbitrary moment and every role must still reach the end of the kernel.
"""
import random

import pytest


class Phase:
    """An mbarrier: `count` arrivals complete a phase; a wait names the parity of the phase it waits for."""

    def __init__(self, count):
        self.count, self.pending, self.phase = count, count, 0

    def arrive(self):
        self.pending -= 1
        assert self.pending >= 0
        if self.pending == 0:
            self.phase += 1
            self.pending = self.count

    def done(self, parity):
        return (self.phase & 1) != parity


class Meet:
    """A named barrier of n threads."""

    def __init__(self, n):
        self.n, self.count, self.gen = n, 0, 0

    def wait(self, who):
        g = self.gen
        self.count += 1
        if self.count == self.n:
            self.count, self.gen = 0, self.gen + 1
        while self.gen == g:
            yield who


THREADS = 3   # softmax threads modelled per group; the last one stands for a warp without rows in alternating items


def run_chain(items, seed, rowless_waits=True, final_barrier=True):
    """items: [(kind, tiles)], kind 'alt' or 'rep'.  Returns None, or a description of the first problem."""
    rnd = random.Random(seed)
    bar = {n: [Phase(1), Phase(1)] for n in ("k_full", "v_full", "k_empty", "v_empty", "s_full", "o_full")}
    bar["p_full"] = [Phase(THREADS), Phase(THREADS)]     # P of a tile comes from one group
    bar["s_free"] = [Phase(THREADS), Phase(THREADS)]
    q_full, q_empty = Phase(1), Phase(1)
    S, K, V, O, Q = [None, None], [None, None], [None, None], [None, None], [None]
    P_rows = [{}, {}]
    unread_s = [set(), set()]
    errors = []
    all_softmax, quadrant = Meet(2 * THREADS), Meet(2 * THREADS)

    def parity(base, j):
        return (base[j & 1] + (j >> 1)) & 1

    def advance(n, st):
        st[0] += 1
        st[1][0] += (n + 1) >> 1
        st[1][1] += n >> 1

    def wait(b, par, who):
        while not b.done(par):
            yield who

    def producer():
        st = [0, [0, 0]]
        for rec, (kind, n) in enumerate(items):
            base = list(st[1])
            if st[0] > 0:
                yield from wait(q_empty, (st[0] - 1) & 1, f"producer: Q of item {rec}")
            Q[0] = rec
            q_full.arrive()
            lead = 2 if kind == "alt" else 1
            for step in range(n + lead):
                if step < n:
                    j, s = step, step & 1
                    uses = base[s] + (j >> 1)
                    if uses > 0:
                        yield from wait(bar["k_empty"][s], (uses - 1) & 1, f"producer: K stage, item {rec} tile {j}")
                    K[s] = (rec, j)
                    bar["k_full"][s].arrive()
                if step >= lead:
                    j = step - lead
                    s = j & 1
                    uses = base[s] + (j >> 1)
                    if uses > 0:
                        yield from wait(bar["v_empty"][s], (uses - 1) & 1, f"producer: V stage, item {rec} tile {j}")
                    V[s] = (rec, j)
                    bar["v_full"][s].arrive()
                yield None
            advance(n, st)

    def mma():
        st = [0, [0, 0]]
        for rec, (kind, n) in enumerate(items):
            base, alt = list(st[1]), kind == "alt"
            yield from wait(q_full, st[0] & 1, f"mma: Q of item {rec}")

            def mma_s(j):
                s = j & 1
                yield from wait(bar["k_full"][s], parity(base, j), f"mma: K, item {rec} tile {j}")
                uses = base[s] + (j >> 1)
                if uses > 0:
                    yield from wait(bar["s_free" if alt else "p_full"][s], (uses - 1) & 1, f"mma: S free, item {rec} tile {j}")
                if K[s] != (rec, j) or Q[0] != rec:
                    errors.append(f"S of item {rec} tile {j} reads K {K[s]}, Q {Q[0]}")
                if unread_s[s]:
                    errors.append(f"S[{s}] overwritten by item {rec} tile {j} before {sorted(unread_s[s])} read it")
                S[s] = (rec, j)
                unread_s[s] = set(range(THREADS))
                bar["s_full"][s].arrive()
                bar["k_empty"][s].arrive()
                if j == n - 1:
                    q_empty.arrive()

            if n == 0:
                q_empty.arrive()
            for j in range(min(n, 2)):
                yield from mma_s(j)
            for j in range(n):
                s = j & 1
                if alt and j + 2 < n:
                    yield from mma_s(j + 2)
                yield from wait(bar["v_full"][s], parity(base, j), f"mma: V, item {rec} tile {j}")
                yield from wait(bar["p_full"][s], parity(base, j), f"mma: P, item {rec} tile {j}")
                if V[s] != (rec, j):
                    errors.append(f"P V of item {rec} tile {j} reads V {V[s]}")
                for t in range(THREADS - 1 if alt else THREADS):
                    if P_rows[s].get(t) != (rec, j):
                        errors.append(f"P V of item {rec} tile {j} reads rows of thread {t}: {P_rows[s].get(t)}")
                O[s if alt else 0] = (rec, j)
                bar["o_full"][s].arrive()
                bar["v_empty"][s].arrive()
                if not alt and j + 2 < n:
                    yield from mma_s(j + 2)
                yield None
            for j in range(max(0, n - 2), n):
                yield from wait(bar["k_empty"][j & 1], parity(base, j), f"mma: tail K, item {rec}")
                yield from wait(bar["v_empty"][j & 1], parity(base, j), f"mma: tail V, item {rec}")
            advance(n, st)

    def softmax(wg, tid):
        st = [0, [0, 0]]
        me = f"softmax {wg}.{tid}"
        for rec, (kind, n) in enumerate(items):
            base = list(st[1])
            if kind == "rep":
                if wg == 0:
                    for j in range(n):
                        s = j & 1
                        yield from wait(bar["s_full"][s], parity(base, j), f"{me}: S, item {rec} tile {j}")
                        if S[s] != (rec, j):
                            errors.append(f"{me} reads S {S[s]}, wants item {rec} tile {j}")
                        unread_s[s].discard(tid)
                        if j >= 2:
                            yield from wait(bar["o_full"][j & 1], parity(base, j - 2), f"{me}: P free, item {rec} tile {j}")
                        P_rows[j & 1][tid] = (rec, j)
                        bar["p_full"][s].arrive()
                        bar["s_free"][s].arrive()
                        yield None
                    if n > 0:
                        yield from wait(bar["o_full"][(n - 1) & 1], parity(base, n - 1), f"{me}: last P V, item {rec}")
                        if O[0] != (rec, n - 1):
                            errors.append(f"{me} merges O {O[0]}, wants item {rec} tile {n - 1}")
                yield from all_softmax.wait(f"{me}: barrier, item {rec}")
            else:
                s = wg
                for j in range(wg, n, 2):
                    yield from wait(bar["s_full"][s], parity(base, j), f"{me}: S, item {rec} tile {j}")
                    if tid == THREADS - 1:   # a warp without rows keeps the protocol only
                        unread_s[s].discard(tid)
                        bar["s_free"][s].arrive()
                        if rowless_waits and j >= 2:
                            yield from wait(bar["o_full"][s], parity(base, j - 2), f"{me}: rowless, item {rec} tile {j}")
                        bar["p_full"][s].arrive()
                        continue
                    if S[s] != (rec, j):
                        errors.append(f"{me} reads S {S[s]}, wants item {rec} tile {j}")
                    for _ in range(rnd.randrange(1, 4)):
                        yield None                                   # the maximum pass
                    if j >= 2:
                        yield from wait(bar["o_full"][s], parity(base, j - 2), f"{me}: P free, item {rec} tile {j}")
                    if S[s] != (rec, j):
                        errors.append(f"{me} re-reads S {S[s]}, wants item {rec} tile {j}")
                    unread_s[s].discard(tid)
                    bar["s_free"][s].arrive()
                    for _ in range(rnd.randrange(1, 7)):
                        yield None                                   # the exponentials
                    P_rows[s][tid] = (rec, j)
                    bar["p_full"][s].arrive()
                    yield None
                for j in range(max(0, n - 2), n):
                    yield from wait(bar["o_full"][j & 1], parity(base, j), f"{me}: last P V, item {rec}")
                yield from quadrant.wait(f"{me}: exchange, item {rec}")
                for _ in range(rnd.randrange(0, 3)):
                    yield None
                for j in range(max(0, n - 2), n):
                    if O[j & 1] != (rec, j):
                        errors.append(f"{me} merges O[{j & 1}] {O[j & 1]}, wants item {rec} tile {j}")
                if final_barrier:
                    yield from all_softmax.wait(f"{me}: barrier, item {rec}")
            advance(n, st)

    procs = {"producer": producer(), "mma": mma()}
    for wg in range(2):
        for t in range(THREADS):
            procs[f"softmax {wg}.{t}"] = softmax(wg, t)
    blocked, idle = {}, 0
    while procs:
        name = rnd.choice(list(procs))
        try:
            r = next(procs[name])
        except StopIteration:
            del procs[name]
            blocked.pop(name, None)
            idle = 0
            continue
        if r is None:
            blocked.pop(name, None)
            idle = 0
        else:
            blocked[name] = r
            idle += 1
        if idle > 20000:
            return f"deadlock: {blocked}"
    return errors[0] if errors else None


def chains():
    out = [[("alt", n)] * 4 for n in range(9)] + [[("rep", n)] * 3 for n in (0, 1, 2, 5)]
    rnd = random.Random(1)
    for _ in range(40):
        out.append([(rnd.choice(["alt", "rep"]), rnd.choice([0, 1, 2, 3, 4, 5, 7])) for _ in range(6)])
    return out


def first_problem(**rules):
    for items in chains():
        for seed in range(20):
            res = run_chain(items, seed, **rules)
            if res:
                return items, seed, res
    return None


def test_protocol_has_no_deadlock_and_no_hazard():
    assert first_problem() is None


def test_model_sees_an_early_arrival_of_a_rowless_warp():
    """The rule: S of tile j goes out before P of tile j - 2 is complete, so a warp without rows must not arrive
    for tile j's P right after S(j), or its arrival completes the phase of tile j - 2 early."""
    found = first_problem(rowless_waits=False)
    assert found is not None and "P V" in found[2], found


def test_model_sees_a_missing_barrier_after_the_merge():
    """The rule: nobody starts the next item (whose first P V overwrites an accumulator) before every thread has
    read both accumulators of this one."""
    found = first_problem(final_barrier=False)
    assert found is not None and "merges O" in found[2], found


@pytest.mark.parametrize("n", [1, 2, 3, 8])
def test_every_tile_is_multiplied_once(n):
    """Phase counts stay aligned over a long chain of equal items."""
    assert run_chain([("alt", n), ("rep", n)] * 6, seed=n) is None


# ----------------------------------------------------------------------------------------------------------
# The failure path.  On the device every mbarrier wait is bounded and fails at once after the abort flag has been
# raised; the named barriers between softmax threads are not bounded, so what has to hold is that no softmax thread
# is ever left at one.  The model below raises the flag at an arbitrary moment of an arbitrary interleaving and
# requires every role to reach the end of the kernel.

class Vote(Meet):
    """A named barrier that also tells every participant whether any of them passed a set flag (bar.red.or)."""

    def __init__(self, n):
        super().__init__(n)
        self.acc, self.result = False, False

    def wait(self, who, flag=False):
        g = self.gen
        self.acc = self.acc or flag
        self.count += 1
        if self.count == self.n:
            self.result, self.acc = self.acc, False
            self.count, self.gen = 0, self.gen + 1
        while self.gen == g:
            yield who
        return self.result


def run_failure(items, seed, abort_step, one_decision=True):
    """Returns None when every role leaves, else the roles that are stuck."""
    rnd = random.Random(seed)
    state = {"abort": False, "step": 0}
    bar = {n: [Phase(1), Phase(1)] for n in ("k_full", "v_full", "k_empty", "v_empty", "s_full", "o_full")}
    bar["p_full"] = [Phase(THREADS), Phase(THREADS)]
    bar["s_free"] = [Phase(THREADS), Phase(THREADS)]
    q_full, q_empty = Phase(1), Phase(1)
    claim_full, claim_empty = [Phase(1), Phase(1)], [Phase(1 + 2 * THREADS), Phase(1 + 2 * THREADS)]
    claim = [None, None]
    all_softmax, quadrant, group0, leave = Meet(2 * THREADS), Meet(2 * THREADS), Meet(THREADS), Vote(2 * THREADS)

    def parity(base, j):
        return (base[j & 1] + (j >> 1)) & 1

    def advance(n, st):
        st[0] += 1
        st[1][0] += (n + 1) >> 1
        st[1][1] += n >> 1

    def wait(b, par, who):
        """A bounded wait: True when the phase completes, False once the abort flag is up."""
        while not b.done(par):
            if state["abort"]:
                return False
            yield who
        return True

    def producer():
        st = [0, [0, 0]]
        for it in range(len(items) + 1):
            slot = it & 1
            if it >= 2 and not (yield from wait(claim_empty[slot], ((it >> 1) - 1) & 1, "producer: claim slot")):
                return
            claim[slot] = it if it < len(items) else -1
            claim_full[slot].arrive()
            if claim[slot] < 0:
                return
            kind, n = items[it]
            base = list(st[1])
            ok = True
            if st[0] > 0:
                ok = yield from wait(q_empty, (st[0] - 1) & 1, "producer: Q")
            if ok:
                q_full.arrive()
                lead = 2 if kind == "alt" else 1
                for step in range(n + lead):
                    if step < n:
                        s, uses = step & 1, base[step & 1] + (step >> 1)
                        if uses > 0 and not (yield from wait(bar["k_empty"][s], (uses - 1) & 1, "producer: K stage")):
                            break
                        bar["k_full"][s].arrive()
                    if step >= lead:
                        j = step - lead
                        s, uses = j & 1, base[j & 1] + (j >> 1)
                        if uses > 0 and not (yield from wait(bar["v_empty"][s], (uses - 1) & 1, "producer: V stage")):
                            break
                        bar["v_full"][s].arrive()
                    yield None
            advance(n, st)
            if state["abort"]:
                return

    def mma():
        st = [0, [0, 0]]
        for it in range(len(items) + 1):
            slot = it & 1
            if not (yield from wait(claim_full[slot], (it >> 1) & 1, "mma: claim")):
                return
            i = claim[slot]
            claim_empty[slot].arrive()
            if i < 0:
                return
            kind, n = items[i]
            base, alt = list(st[1]), kind == "alt"

            def mma_s(j):
                s = j & 1
                if not (yield from wait(bar["k_full"][s], parity(base, j), "mma: K")):
                    return False
                uses = base[s] + (j >> 1)
                if uses > 0 and not (yield from wait(bar["s_free" if alt else "p_full"][s], (uses - 1) & 1, "mma: S free")):
                    return False
                bar["s_full"][s].arrive()
                bar["k_empty"][s].arrive()
                if j == n - 1:
                    q_empty.arrive()
                return True

            ok = yield from wait(q_full, st[0] & 1, "mma: Q")
            if ok and n == 0:
                q_empty.arrive()
            for j in range(min(n, 2)):
                ok = ok and (yield from mma_s(j))
            for j in range(n):
                if not ok:
                    break
                s = j & 1
                if alt and j + 2 < n and not (yield from mma_s(j + 2)):
                    break
                if not (yield from wait(bar["v_full"][s], parity(base, j), "mma: V")):
                    break
                if not (yield from wait(bar["p_full"][s], parity(base, j), "mma: P")):
                    break
                bar["o_full"][s].arrive()
                bar["v_empty"][s].arrive()
                if not alt and j + 2 < n and not (yield from mma_s(j + 2)):
                    break
                yield None
            advance(n, st)
            if state["abort"]:
                return

    def softmax(wg, tid):
        st = [0, [0, 0]]
        me = f"softmax {wg}.{tid}"
        for it in range(len(items) + 1):
            slot = it & 1
            got = yield from wait(claim_full[slot], (it >> 1) & 1, f"{me}: claim")
            i = claim[slot] if got else -1
            if got:
                claim_empty[slot].arrive()
            if one_decision:
                if (yield from leave.wait(f"{me}: exit vote", flag=(not got) or state["abort"])):
                    return
            elif not got:
                return
            if i < 0:
                return
            kind, n = items[i]
            base = list(st[1])
            ok = True
            if kind == "rep":
                if wg == 0:
                    for j in range(n):
                        s = j & 1
                        if ok:
                            ok = yield from wait(bar["s_full"][s], parity(base, j), f"{me}: S")
                        if ok and j >= 2:
                            ok = yield from wait(bar["o_full"][j & 1], parity(base, j - 2), f"{me}: P free")
                        if ok:
                            bar["p_full"][s].arrive()
                            bar["s_free"][s].arrive()
                        yield None
                    if ok and n > 0:
                        ok = yield from wait(bar["o_full"][(n - 1) & 1], parity(base, n - 1), f"{me}: last P V")
                    yield from group0.wait(f"{me}: merge barrier")
                    yield from group0.wait(f"{me}: merge barrier")
                yield from all_softmax.wait(f"{me}: closing barrier")
            else:
                s = wg
                for j in range(wg, n, 2):
                    if not (yield from wait(bar["s_full"][s], parity(base, j), f"{me}: S")):
                        ok = False
                        break
                    bar["s_free"][s].arrive()
                    if j >= 2 and not (yield from wait(bar["o_full"][s], parity(base, j - 2), f"{me}: P free")):
                        ok = False
                        break
                    for _ in range(rnd.randrange(0, 4)):
                        yield None
                    bar["p_full"][s].arrive()
                for j in range(max(0, n - 2), n):
                    ok = ok and (yield from wait(bar["o_full"][j & 1], parity(base, j), f"{me}: last P V"))
                yield from quadrant.wait(f"{me}: exchange")
                yield from all_softmax.wait(f"{me}: closing barrier")
            advance(n, st)
            if not one_decision and state["abort"]:
                return

    procs = {"producer": producer(), "mma": mma()}
    for wg in range(2):
        for t in range(THREADS):
            procs[f"softmax {wg}.{t}"] = softmax(wg, t)
    blocked, idle = {}, 0
    while procs:
        state["step"] += 1
        if state["step"] == abort_step:
            state["abort"] = True
        name = rnd.choice(list(procs))
        try:
            r = next(procs[name])
        except StopIteration:
            del procs[name]
            blocked.pop(name, None)
            idle = 0
            continue
        if r is None:
            blocked.pop(name, None)
            idle = 0
        else:
            blocked[name] = r
            idle += 1
        if idle > 20000:
            return blocked
    return None


def stuck_somewhere(one_decision):
    rnd = random.Random(7)
    for trial in range(1500):
        items = [(rnd.choice(["alt", "rep"]), rnd.choice([0, 1, 2, 3, 5])) for _ in range(rnd.randrange(1, 6))]
        res = run_failure(items, seed=trial, abort_step=rnd.randrange(1, 1500), one_decision=one_decision)
        if res:
            return items, trial, res
    return None


def test_every_role_leaves_after_an_abort_at_any_moment():
    assert stuck_somewhere(one_decision=True) is None


def test_without_the_common_exit_decision_a_thread_can_be_left_at_a_barrier():
    """Each softmax thread reading the abort flag for itself between two items: some leave, the others wait for
    them at the next item's barriers."""
    found = stuck_somewhere(one_decision=False)
    assert found is not None and any("barrier" in w or "exchange" in w for w in found[2].values()), found


def test_failure_model_runs_clean_chains_to_the_end():
    for seed in range(20):
        assert run_failure([("alt", 5), ("rep", 3), ("alt", 2), ("rep", 0), ("alt", 0)], seed, abort_step=-1) is None
