"""The serving loop's host logic (monoserve_b200/engine.py: admission under slots / pages / token budget,
the two-buffer decode switch, when pages, slots and program handles are given back) against a model of
the fabric that runs here: lanes that adopt a published program at an iteration boundary, finite
programs that stop after their iterations, handles that must not be released while published or
running.  The model's decode program gives every slot of its batch one token per iteration, its prefill
program the first token; nothing here needs a GPU.  The behaviour mirrors the reference's loop
(monoserve/engine.py:303-527: requests join the decode batch after their prefill pass, the batch changes
only at iteration boundaries, KV pages are freed once no running program can touch them).
"""
import types

import numpy as np
import pytest

from monoserve_b200 import engine as eng_mod
from monoserve_b200.engine import DECODE, PREFILL, Engine, PagePool


class ModelFabric:
    """What Engine uses of Fabric, with the lane semantics of the device scheduler."""
    num_workers = 16

    def __init__(self):
        self.programs, self.next_handle, self.next_gen = {}, 1, 1
        self.published = [0, 0]
        self.lanes = [dict(gen=0, iterations=0, running=0, handle=0, in_prog=0) for _ in range(2)]
        self.maps = []

    def make(self, kind, slots, iterations):
        h, self.next_handle = self.next_handle, self.next_handle + 1
        self.programs[h] = dict(kind=kind, slots=list(slots), iterations=iterations, gen=self.next_gen)
        self.next_gen += 1
        return h

    def upload(self, tiles, stages, succ, first, reset, iterations):
        return self.make("idle", [], iterations)

    def generation(self, h):
        return self.programs[h]["gen"]

    def publish(self, map, caps, order, programs, forms=None):
        assert len(map) == self.num_workers and set(map) <= {DECODE, PREFILL}
        assert DECODE in map and PREFILL in map, "each lane keeps at least one worker"
        for h in programs:
            assert h == 0 or h in self.programs, f"published handle {h} was released"
        self.published = list(programs)
        self.maps.append(map.count(DECODE))

    def release(self, h):
        assert h in self.programs, f"handle {h} released twice"
        assert h not in self.published, f"handle {h} released while published"
        for lane in self.lanes:
            assert not (lane["running"] and lane["handle"] == h), f"handle {h} released while it runs"
        del self.programs[h]

    def progress(self):
        return dict(error=0, lanes=[dict(gen=l["gen"], iterations=l["iterations"], running=l["running"]) for l in self.lanes])

    def _adopt(self, lane, h):
        lane.update(handle=h, gen=self.programs[h]["gen"], in_prog=0, running=1)

    def tick(self, effect):
        """One iteration of every running lane, then the boundary: switch to a newer published program, stop after
        a finite program's last iteration, or go round again.  An idle lane adopts a newer published program."""
        for n, lane in enumerate(self.lanes):
            wanted = self.published[n]
            newer = wanted and self.programs[wanted]["gen"] != lane["gen"]
            if not lane["running"]:
                if newer:
                    self._adopt(lane, wanted)
                continue
            prog = self.programs[lane["handle"]]
            effect(prog)
            lane["iterations"] += 1
            lane["in_prog"] += 1
            if newer:
                self._adopt(lane, wanted)
            elif prog["iterations"] and lane["in_prog"] >= prog["iterations"]:
                lane["running"] = 0


class ModelTable:
    """RequestTable without a device: the pages of each slot and the host token rings."""

    def __init__(self, slots, bt_stride, ring=64):
        self.slots, self.bt_stride, self.ring = slots, bt_stride, ring
        self.pages = {}
        self.host_steps = np.zeros(slots, dtype=np.int64)
        self.host_tokens = np.zeros((slots, ring), dtype=np.int32)

    def set_pages(self, slot, pages):
        assert len(pages) <= self.bt_stride
        self.pages[slot] = list(pages)

    def open(self, slot, seq_len, temperature=0.0):
        self.host_steps[slot] = 0

    def produced(self, slot):
        return int(self.host_steps[slot])

    def tokens(self, slot, first, last):
        return [int(self.host_tokens[slot, i % self.ring]) for i in range(first, last)]


class WatchedPool(PagePool):
    def __init__(self, n):
        super().__init__(n)
        self.given_back = set()

    def take(self, n):
        out = super().take(n)
        self.given_back -= set(out)
        return out

    def give(self, pages):
        assert not (set(pages) & self.given_back), "a page given back twice"
        self.given_back |= set(pages)
        super().give(pages)


class ModelLaneStub:
    """ModelLane's builder calls, recorded as programs of the model fabric."""

    def __init__(self, fab, lane_id, cfg, weights, kv, max_tokens, max_slots, logit_rows, bt_stride, requests):
        self.fab, self.lane_id, self.max_tokens, self._keep = fab, lane_id, max_tokens, []
        self.built = []

    def build_prefill(self, reqs, iterations=1):
        assert sum(len(prompt) for _, prompt, _ in reqs) <= self.max_tokens, "a pass above the token budget"
        assert len({slot for slot, _, _ in reqs}) == len(reqs)
        self._keep.append(object())
        self.built.append([slot for slot, _, _ in reqs])
        return self.fab.make("prefill", [slot for slot, _, _ in reqs], iterations)

    def build_decode(self, slots, iterations=0):
        assert 0 < len(slots) <= self.max_tokens and len(set(slots)) == len(slots), "a decode batch above max_decode"
        self._keep.append(object())
        return self.fab.make("decode", slots, iterations)


class Harness:
    def __init__(self, monkeypatch, slots=12, pages=64, max_decode=4, token_budget=96, page=16, planner=None):
        monkeypatch.setattr(eng_mod, "ModelLane", ModelLaneStub)
        monkeypatch.setattr(eng_mod.torch.cuda, "synchronize", lambda *a, **k: None)
        self.fab, self.pool = ModelFabric(), WatchedPool(pages)
        self.table = ModelTable(slots, bt_stride=16)
        kv = types.SimpleNamespace(page=page)
        self.eng = Engine(self.fab, None, None, kv, self.table, self.pool, max_decode=max_decode,
                          token_budget=token_budget, planner=planner)
        self.clock = 0.0
        self.eng.now = lambda: self.clock   # the loop's clock counts rounds

    def effect(self, prog):
        """What one iteration of a program does to the request table; checks that it touches live state only."""
        for slot in prog["slots"]:
            assert not (set(self.table.pages[slot]) & self.pool.given_back), \
                f"a running {prog['kind']} program writes KV pages that went back to the pool (slot {slot})"
            step = int(self.table.host_steps[slot])
            if prog["kind"] == "prefill":
                assert step == 0
            self.table.host_tokens[slot, step % self.table.ring] = step
            self.table.host_steps[slot] = step + 1

    def check_state(self):
        held = [r for r in self.eng.reqs.values() if r.slot is not None]
        slots = [r.slot for r in held]
        assert len(set(slots)) == len(slots), "two requests in one slot"
        assert not (set(slots) & set(self.eng.free_slots)), "a slot both held and free"
        pages = [p for r in held for p in r.pages]
        assert len(set(pages)) == len(pages), "a KV page held by two requests"
        assert 0 not in pages, "the sink page handed out"

    def run(self, requests, rounds=4000):
        """requests: [(round of arrival, rid, prompt length, max_tokens)]."""
        pending = sorted(requests, key=lambda q: q[0])   # stable: the order given within a round
        finished = []
        for n in range(rounds):
            self.clock = float(n)
            while pending and pending[0][0] <= n:
                _, rid, plen, out = pending.pop(0)
                self.eng.submit(rid, list(range(plen)), out, arrival=float(n))
            finished += self.eng.step()
            self.check_state()
            self.fab.tick(self.effect)
            if not pending and not self.eng.busy():
                return finished, n
        raise AssertionError(f"not finished after {rounds} rounds: {self.eng.stats}, queue {len(self.eng.queue)}")


def requests_of(seed, n, max_prompt=60, max_out=40, spread=200):
    rng = np.random.default_rng(seed)
    return [(int(rng.integers(0, spread)), f"q{i}", int(rng.integers(1, max_prompt)), int(rng.integers(1, max_out)))
            for i in range(n)]


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_every_request_gets_its_tokens_in_order_and_everything_comes_back(monkeypatch, seed):
    h = Harness(monkeypatch)
    reqs = requests_of(seed, 40)
    finished, _ = h.run(reqs)
    assert sorted(r.rid for r in finished) == sorted(rid for _, rid, _, _ in reqs)
    for _, rid, _, out in reqs:
        r = h.eng.reqs[rid]
        assert r.tokens == list(range(out)), f"{rid}: tokens lost, repeated or from another request"
        assert r.first_time is not None and r.finish_time >= r.first_time >= r.arrival
        assert r.slot is None and r.pages == []
    # first come first served: first tokens in the order of submission
    firsts = [r.first_time for r in h.eng.reqs.values()]   # a dict keeps the order of submission
    assert firsts == sorted(firsts)
    assert h.fab.programs == {}, "program handles left behind"
    assert h.pool.available() == 63 and sorted(h.eng.free_slots) == list(range(12))
    assert h.eng.stats["decode_programs"] > 0 and h.eng.stats["prefill_passes"] > 0


def test_decode_batch_and_pass_stay_within_their_limits(monkeypatch):
    """Many requests at once: the decode batch never exceeds max_decode (the lane stub asserts it), a prefill pass
    never exceeds the token budget, and the queue drains in several passes."""
    h = Harness(monkeypatch, max_decode=3, token_budget=64)
    reqs = [(0, f"q{i}", 30, 5) for i in range(10)]
    finished, _ = h.run(reqs)
    assert len(finished) == 10
    assert all(len(slots) <= 2 for slots in h.eng.pre.built), "two 30-token prompts fit a 64-token pass, three do not"
    assert h.eng.stats["prefill_passes"] >= 5


def test_admission_waits_for_pages(monkeypatch):
    """A pool that holds one request at a time: the second is admitted only after the first one's pages are back,
    which is after the decode lane has left the program that served it."""
    h = Harness(monkeypatch, pages=8)   # 7 usable pages; a 50-token prompt needs ceil(51 / 16) + 2 = 6
    finished, _ = h.run([(0, "q0", 50, 6), (0, "q1", 50, 6)])
    assert [r.rid for r in finished] == ["q0", "q1"]
    a, b = h.eng.reqs["q0"], h.eng.reqs["q1"]
    assert b.first_time > a.finish_time
    assert h.pool.available() == 7


def test_oversized_requests_are_refused_at_submission(monkeypatch):
    h = Harness(monkeypatch)
    with pytest.raises(ValueError, match="exceed max_len"):
        h.eng.submit("long", list(range(200)), 100)
    with pytest.raises(ValueError, match="pass budget"):
        h.eng.submit("wide", list(range(97)), 4)
    assert not h.eng.busy()


def test_planner_split_is_published_while_both_lanes_run(monkeypatch):
    """With a planner the published map follows its answer whenever both lanes have work, and keeps the last
    split otherwise."""
    calls = []

    class Planner:
        stats = {}

        def split(self, contexts, prompts, workers):
            calls.append((list(contexts), list(prompts), workers))
            if not contexts or not prompts:
                return None
            return min(workers - 1, 3 + len(contexts))

    h = Harness(monkeypatch, planner=Planner())
    finished, _ = h.run([(0, "q0", 20, 30), (6, "q1", 40, 10), (9, "q2", 10, 10)])
    assert len(finished) == 3
    both = [(c, p) for c, p, _ in calls if c and p]
    assert both, "no publish with both lanes busy"
    assert all(w == 16 for _, _, w in calls)
    for contexts, prompts in both:
        assert all(c >= 10 for c in contexts) and set(prompts) <= {20, 40, 10}
    assert h.fab.maps[0] == 8 and any(m == 4 for m in h.fab.maps), "the decode lane's share follows the planner"


def test_an_eos_token_ends_the_request_and_later_tokens_are_dropped(monkeypatch):
    """The model's lanes sample token n at step n: with eos {5} the request ends after six tokens with reason
    "stop", whatever the lane went on to sample before the loop saw it; the others run to their lengths."""
    h = Harness(monkeypatch)
    h.eng.submit("stops", list(range(20)), 30, arrival=0.0, eos={5})
    h.eng.submit("runs", list(range(20)), 12, arrival=0.0)
    finished, _ = h.run([])
    assert sorted(r.rid for r in finished) == ["runs", "stops"]
    a, b = h.eng.reqs["stops"], h.eng.reqs["runs"]
    assert a.tokens == [0, 1, 2, 3, 4, 5] and a.reason == "stop"
    assert b.tokens == list(range(12)) and b.reason == "length"
    assert h.pool.available() == 63 and h.fab.programs == {}


def test_a_request_ends_when_the_cache_has_no_page_left_to_grow_into(monkeypatch):
    """Two long generations in a pool too small for both: one of them ends early with reason "length" once no page is
    left and less than a page of room remains ahead of it, before any of its tokens could land outside its
    pages; its pages then let the other one run to the end."""
    h = Harness(monkeypatch, pages=10)   # 9 usable pages of 16 tokens; each request starts with 3
    reqs = [(0, "q0", 10, 100), (0, "q1", 10, 100)]
    finished, _ = h.run(reqs)
    assert len(finished) == 2
    lengths = sorted(len(h.eng.reqs[rid].tokens) for _, rid, _, _ in reqs)
    assert lengths[1] == 100 and lengths[0] < 100   # 110 tokens need 9 pages with the look-ahead: the whole pool
    for _, rid, _, _ in reqs:
        r = h.eng.reqs[rid]
        assert r.tokens == list(range(len(r.tokens))) and r.reason == "length"
    assert h.pool.available() == 9
