"""The serving loop over the fabric: continuous batching with one prefill lane and a
double-buffered decode lane, driven from the host while the persistent kernel runs.

What the reference's engine does around its fabric (monoserve/engine.py:303-527): requests
arrive, prompts are batched into a prefill pass under a token budget, a request whose
prompt is done joins the decode batch, the decode lane's program is rebuilt in the buffer
that is not running and replaces the running one at an iteration boundary, KV pages are
kept ahead of the sequences, and new tokens are collected from pinned rings.  This module
is that loop for this library's lanes (`ModelLane`), without the reference's admission
control: requests are admitted first come first served while slots, pages and the token
budget allow, and the published plan is a fixed SM split (the plan search of
monoserve_b200.control can supply another one).

The fabric is given a few SMs fewer than the GPU has: programs are built while the kernel
is resident, and the small host-driven copies and fills of a build need somewhere to run.
Request state that the device reads (block-table rows, lengths, last tokens) is written
through Fabric.write, which never launches a kernel.

    table = RequestTable(fab, slots, bt_stride)
    eng = Engine(fab, cfg, weights, kv, table, max_decode=64, token_budget=2048)
    eng.submit(rid, prompt_tokens, max_tokens)
    while eng.busy(): finished = eng.step()
"""
import struct
import time

import numpy as np
import torch

from monoserve_b200.fabric import Program, Tile
from monoserve_b200.model import ModelLane

DECODE, PREFILL = 0, 1      # fabric lanes
LOOKAHEAD_PAGES = 2         # KV pages kept ahead of a decoding sequence


def arrival_times(rate, seed, num):
    """Poisson arrivals, the first at 0: unit exponentials from the seed, divided by the rate, so
    that the points of a rate sweep share one arrival pattern (eval/loadgen.py:54-70)."""
    gaps = np.random.default_rng(seed).standard_exponential(max(0, num - 1))
    return np.concatenate([[0.0], np.cumsum(gaps)])[:num] / rate


def lognormal_lengths(num, median, sigma, lo, hi, seed):
    """Integer lengths drawn from a log-normal with the given median and sigma, clipped to [lo, hi]."""
    v = np.random.default_rng(seed).lognormal(np.log(median), sigma, num)
    return np.clip(np.rint(v), lo, hi).astype(np.int64)


class PagePool:
    """KV pages by number; page 0 is the sink every unused block-table entry points at."""

    def __init__(self, n_pages):
        self.free = list(range(n_pages - 1, 0, -1))

    def available(self):
        return len(self.free)

    def take(self, n):
        if n > len(self.free):
            raise MemoryError(f"{n} KV pages wanted, {len(self.free)} free")
        out = self.free[-n:][::-1]
        del self.free[-n:]
        return out

    def give(self, pages):
        self.free.extend(reversed(pages))


class RequestTable:
    """Slot-indexed request state shared by every lane (monoserve/runtime/requests.py): the block
    table, sequence lengths, last tokens and step counts on the device, and the token rings in pinned
    host memory.  Writes go through Fabric.write, so they are safe beside a running fabric."""

    def __init__(self, fab, slots, bt_stride, ring=64):
        self.fab, self.slots, self.bt_stride, self.ring = fab, slots, bt_stride, ring
        z = lambda *shape, dt=torch.int32: torch.zeros(*shape, dtype=dt, device="cuda")  # noqa: E731
        self.bt = z(slots, bt_stride)
        self.seq_len, self.last_token, self.steps = z(slots), z(slots), z(slots)
        self.temperature = z(slots, dt=torch.float32)
        self.host_tokens = torch.zeros(slots, ring, dtype=torch.int32).pin_memory()
        self.host_steps = torch.zeros(slots, dtype=torch.int64).pin_memory()
        torch.cuda.synchronize()

    def set_pages(self, slot, pages):
        row = np.zeros(self.bt_stride, dtype=np.int32)
        row[:len(pages)] = pages
        self.fab.write(self.bt.data_ptr() + 4 * slot * self.bt_stride, row.tobytes())

    def open(self, slot, seq_len, temperature=0.0):
        """A request takes the slot: its length after the prompt, no tokens produced yet."""
        self.host_steps[slot] = 0
        self.fab.write(self.seq_len.data_ptr() + 4 * slot, struct.pack("<i", seq_len))
        self.fab.write(self.steps.data_ptr() + 4 * slot, struct.pack("<i", 0))
        self.fab.write(self.temperature.data_ptr() + 4 * slot, struct.pack("<f", temperature))

    def produced(self, slot):
        return int(self.host_steps[slot])

    def tokens(self, slot, first, last):
        return [int(self.host_tokens[slot, i % self.ring]) for i in range(first, last)]


class _Req:
    def __init__(self, rid, prompt, max_tokens, arrival, eos=()):
        self.rid, self.prompt, self.max_tokens, self.arrival = rid, list(prompt), max_tokens, arrival
        self.eos, self.reason = frozenset(eos), None   # reason: "stop" (an eos token), "length" (max_tokens, or no KV page left)
        self.slot, self.pages, self.delivered = None, [], 0
        self.tokens, self.token_times, self.first_time, self.finish_time = [], [], None, None


class SearchPlanner:
    """The SM split of the two lanes from the control plane's plan search (monoserve_b200/control.py: the time
    estimator over a calibration, Algorithm 1), asked whenever both lanes have a program: the decode lane's work is
    the contexts of its batch with the deadline `tpot_s` per step, the prefill lane's its pass with the deadline
    `ttft_s`; expected expert activations come from uniform routing shares and the hot sets.  The reference's
    engine takes its plans from the same search through its admission policy (monoserve/engine.py:303-527); here
    only the split is taken, the queue stays first come first served."""

    def __init__(self, cfg, hot, tpot_s=0.05, ttft_s=0.5, calibration=None, fp8=False):
        import os
        import types
        from monoserve_b200 import control
        path = calibration or os.path.join(os.path.dirname(os.path.abspath(__file__)), "calibration", "b200.json")
        self.control, self.cfg, self.tpot_s, self.ttft_s = control, cfg, tpot_s, ttft_s
        self.est = control.Estimator(control.model_shape(types.SimpleNamespace(**vars(cfg), fp8=fp8)),
                                     control.load_calibration(path))
        shares = np.full((cfg.num_layers, cfg.num_experts), 1.0 / cfg.num_experts)
        self.view = control.profile_view(shares, shares, hot)
        self.search = control.PlanSearch(self.est)
        self.dense = getattr(cfg, "dense_layers", 0)
        self.stats = dict(searches=0, infeasible=0, micros=0.0)

    def _work(self, decode, seqs, deadline, rows):
        w = self.control.LaneWork()
        w.decode, w.deadline = decode, deadline
        w.passes = [[self.control.Seq(t, c) for t, c in seqs]]
        on = [self.view.expected(decode, l, rows * self.cfg.top_k) if l >= self.dense else (0.0, 0.0)
              for l in range(self.cfg.num_layers)]
        w.active, w.miss = [a for a, _ in on], [m for _, m in on]
        return w

    def split(self, contexts, prompts, workers):
        """Workers of the decode lane out of `workers`, for a decode batch with these context lengths beside a
        prefill pass with these prompt lengths; None when either lane is empty."""
        if not contexts or not prompts:
            return None
        lanes = [self.est.load(self._work(True, [(1, c) for c in contexts], self.tpot_s, len(contexts))),
                 self.est.load(self._work(False, [(n, 0) for n in prompts], self.ttft_s, sum(prompts)))]
        plan = self.search.solve(lanes)
        self.stats["searches"] += 1
        self.stats["micros"] += plan.micros
        if not plan.feasible:
            self.stats["infeasible"] += 1   # the search's fallback split is still the best it found
        sms = [l.sms for l in plan.lanes]
        return min(workers - 1, max(1, round(sms[0] * workers / max(1, sum(sms)))))


class Engine:
    """One GPU, one prefill lane, one decode lane with two program buffers."""

    def __init__(self, fab, cfg, weights, kv, table, pool, max_decode=64, token_budget=2048, max_len=None,
                 sm_decode=None, caps=(8, 8), forms=(64, 0), planner=None):
        self.fab, self.cfg, self.kv, self.table, self.pool = fab, cfg, kv, table, pool
        self.max_decode, self.token_budget = max_decode, token_budget
        self.max_len = max_len or table.bt_stride * kv.page
        shared = dict(bt_stride=table.bt_stride, requests=table)
        self.pre = ModelLane(fab, PREFILL, cfg, weights, kv, max_tokens=token_budget, max_slots=table.slots,
                             logit_rows=table.slots, **shared)
        self.dec = [ModelLane(fab, DECODE, cfg, weights, kv, max_tokens=max_decode, max_slots=table.slots,
                              logit_rows=max_decode, **shared) for _ in range(2)]
        for lane in [self.pre] + self.dec:
            lane.keep_base = len(lane._keep)   # operand blocks made at construction stay; those of a build go with its program
        n = fab.num_workers
        self.sm_decode = sm_decode if sm_decode is not None else n // 2
        self.map = [DECODE] * self.sm_decode + [PREFILL] * (n - self.sm_decode)
        self.caps, self.forms = list(caps), list(forms)
        self.planner = planner   # a SearchPlanner: the split follows the lanes' work instead of staying at sm_decode
        idle = Program()
        idle.stage([Tile(0)])
        self.idle_program = idle   # a one-tile program that ends a lane: published when the decode batch is empty
        self.reqs, self.queue, self.free_slots = {}, [], list(range(table.slots - 1, -1, -1))
        self.prefilling, self.pre_handle, self.pre_iter0 = [], None, 0
        self.joining = []
        self.dec_batch, self.dec_handle, self.dec_buf = [], None, 0     # what the decode lane runs now
        self.dec_pending = None                                            # (handle, gen, buffer, batch, old handle)
        self.retired = []                                                  # (requests to free once the switch is through)
        self.t0 = time.perf_counter()
        self.stats = dict(published=0, decode_programs=0, prefill_passes=0, switch_waits=0, prefill_build_s=0.0,
                          decode_build_s=0.0)   # *_build_s: host time spent building programs
        torch.cuda.synchronize()

    # ------------------------------------------------------------------ requests
    def now(self):
        return time.perf_counter() - self.t0

    def submit(self, rid, prompt, max_tokens, arrival=None, eos=()):
        if len(prompt) + max_tokens > self.max_len:
            raise ValueError(f"request {rid}: {len(prompt)} + {max_tokens} tokens exceed max_len {self.max_len}")
        if len(prompt) > self.token_budget:
            raise ValueError(f"request {rid}: a prompt of {len(prompt)} tokens exceeds the pass budget {self.token_budget}")
        r = _Req(rid, prompt, max_tokens, self.now() if arrival is None else arrival, eos)
        self.reqs[rid] = r
        self.queue.append(r)

    def busy(self):
        return bool(self.queue or self.prefilling or self.joining or self.dec_batch or self.dec_pending)

    # ------------------------------------------------------------------ one round
    def step(self):
        """One round of the loop; returns the requests that finished in it."""
        now = self.now()
        done = []
        self._finish_switch()
        self._finish_prefill(now)
        done += self._collect(now)
        self._rebuild_decode()
        self._start_prefill()
        return done

    def _publish(self):
        programs = [self.dec_pending[0] if self.dec_pending else (self.dec_handle or 0), self.pre_handle or 0]
        if self.planner is not None:
            batch = self.dec_pending[3] if self.dec_pending else self.dec_batch
            contexts = [len(r.prompt) + r.delivered for r in batch if r.finish_time is None]
            prompts = [len(r.prompt) for r in self.prefilling] if self.pre_handle else []
            n = self.fab.num_workers
            dec = self.planner.split(contexts, prompts, n)
            if dec is not None:
                self.map = [DECODE] * dec + [PREFILL] * (n - dec)
        self.fab.publish(map=self.map, caps=self.caps, order=[DECODE, PREFILL], programs=programs, forms=self.forms)
        self.stats["published"] += 1

    def _lane_state(self, lane):
        return self.fab.progress()["lanes"][lane]

    def _start_prefill(self):
        if self.prefilling or not self.queue:
            return
        page = self.kv.page
        batch, tokens = [], 0
        # rows the decode lane will need: the batch it runs (or is switching to) that has not finished, and the joiners
        current = self.dec_pending[3] if self.dec_pending else self.dec_batch
        in_flight = sum(1 for r in current if r.finish_time is None) + len(self.joining)
        while self.queue and self.free_slots and in_flight + len(batch) < self.max_decode:
            r = self.queue[0]
            need = -(-(len(r.prompt) + 1) // page) + LOOKAHEAD_PAGES
            if tokens + len(r.prompt) > self.token_budget or need > self.pool.available():
                break
            self.queue.pop(0)
            r.slot, r.pages = self.free_slots.pop(), self.pool.take(need)
            self.table.set_pages(r.slot, r.pages)
            self.table.open(r.slot, len(r.prompt))
            batch.append(r)
            tokens += len(r.prompt)
        if not batch:
            return
        del self.pre._keep[self.pre.keep_base:]   # the operand blocks of the lane's previous pass: that program has ended
        self.pre_iter0 = self._lane_state(PREFILL)["iterations"]
        t_build = time.perf_counter()
        self.pre_handle = self.pre.build_prefill([(r.slot, r.prompt, 0) for r in batch], iterations=1)
        self.stats["prefill_build_s"] += time.perf_counter() - t_build
        self.prefilling = batch
        self.stats["prefill_passes"] += 1
        self._publish()

    def _finish_prefill(self, now):
        if not self.prefilling:
            return
        st = self._lane_state(PREFILL)
        if st["iterations"] <= self.pre_iter0 or st["running"]:
            return
        for r in self.prefilling:   # the pass sampled each request's first token into its ring
            r.first_time = now
            self.joining.append(r)
        self.prefilling = []
        ended, self.pre_handle = self.pre_handle, None
        self._publish()            # the lane's published program goes first: a published handle cannot be released
        self.fab.release(ended)

    def _rebuild_decode(self):
        if self.dec_pending is not None:
            return   # one switch at a time: the idle buffer is only free once the last switch is through
        target = [r for r in self.dec_batch if r.finish_time is None] + self.joining
        if [r.rid for r in target] == [r.rid for r in self.dec_batch]:
            return
        buf = 1 - self.dec_buf
        if target:
            lane = self.dec[buf]
            del lane._keep[lane.keep_base:]   # this buffer's previous program was replaced a switch ago
            t_build = time.perf_counter()
            h = lane.build_decode([r.slot for r in target], iterations=0)
            self.stats["decode_build_s"] += time.perf_counter() - t_build
            self.stats["decode_programs"] += 1
        else:
            h = self.idle_program.upload(self.fab, first=0, iterations=1)
        gone = [r for r in self.dec_batch if r.finish_time is not None]
        self.dec_pending = (h, self.fab.generation(h), buf, target, self.dec_handle, gone)
        self.joining = []
        self._publish()

    def _finish_switch(self):
        if self.dec_pending is None:
            return
        h, gen, buf, batch, old, gone = self.dec_pending
        st = self._lane_state(DECODE)
        if st["gen"] != gen:
            self.stats["switch_waits"] += 1
            return
        if not batch and st["running"]:
            return   # the idle program has not ended yet
        # the old program has left at its iteration boundary: its handle, and the pages and slots of the
        # requests that finished under it, are free
        if old:
            self.fab.release(old)
        for r in gone:
            self.pool.give(r.pages)
            self.free_slots.append(r.slot)
            r.pages, r.slot = [], None
        self.dec_batch, self.dec_buf = batch, buf
        self.dec_handle = h if batch else None
        self.dec_pending = None
        if not batch:   # the idle program has ended: take it off the lane, then free it
            self._publish()
            self.fab.release(h)

    def _collect(self, now):
        done = []
        watched = self.dec_batch + self.joining + (self.dec_pending[3] if self.dec_pending else [])
        seen = set()
        for r in watched:
            if r.rid in seen or r.slot is None or r.finish_time is not None:
                continue
            seen.add(r.rid)
            n = min(self.table.produced(r.slot), r.max_tokens)
            if n > r.delivered:
                new = self.table.tokens(r.slot, r.delivered, n)
                stop = next((i for i, t in enumerate(new) if t in r.eos), None)
                if stop is not None:   # the tokens the lane sampled after an eos are dropped
                    new, r.reason = new[:stop + 1], "stop"
                r.tokens += new
                r.token_times += [now] * len(new)
                r.delivered += len(new)
            if r.reason is None and r.delivered >= r.max_tokens:
                r.reason = "length"
            if r.reason is None and not self._ensure_pages(r, len(r.prompt) + r.delivered):
                r.reason = "length"   # the cache has no page left for the sequence to grow into
            if r.reason is not None:
                r.finish_time = now
                done.append(r)
        return done

    def _ensure_pages(self, r, length):
        """Keeps LOOKAHEAD_PAGES pages ahead of a decoding sequence of `length` tokens.  False when the pool has none
        left and less than a page of room remains ahead of the sequence (monoserve/engine.py:509-516 ends the request
        with "length" then): the lane may run a page's worth of steps before the host sees the tokens."""
        page = self.kv.page
        need = min(-(-(length + 1) // page) + LOOKAHEAD_PAGES, self.table.bt_stride)
        if need <= len(r.pages):
            return True
        if need - len(r.pages) > self.pool.available():
            return length + page <= len(r.pages) * page
        r.pages += self.pool.take(need - len(r.pages))
        self.table.set_pages(r.slot, r.pages)   # entries in use keep their values; new ones lie ahead of the sequence
        return True

    # ------------------------------------------------------------------ a whole run
    def serve(self, requests, poll_s=2e-4, timeout_s=600.0):
        """requests: [(arrival seconds, rid, prompt tokens, max_tokens)].  Submits each at its arrival
        time on the wall clock and runs the loop until all have finished.  Returns {rid: record}."""
        pending = sorted(requests, key=lambda q: q[0])
        self.t0 = time.perf_counter()
        n_done, total = 0, len(pending)
        while n_done < total:
            now = self.now()
            if now > timeout_s:
                prog = self.fab.progress()
                raise TimeoutError(f"{total - n_done} requests unfinished after {timeout_s} s: error word "
                                   f"{prog['error']:#x}, lanes {prog['lanes'][:2]}, stats {self.stats}, queued "
                                   f"{len(self.queue)}, prefilling {len(self.prefilling)}, joining {len(self.joining)}, "
                                   f"decoding {len(self.dec_batch)}, pending switch {self.dec_pending is not None}")
            while pending and pending[0][0] <= now:
                t, rid, prompt, max_tokens = pending.pop(0)
                self.submit(rid, prompt, max_tokens, arrival=t)
            n_done += len(self.step())
            time.sleep(poll_s)
        while self.busy():   # let the last switch (to the idle program) go through
            self.step()
            time.sleep(poll_s)
        return {r.rid: dict(arrival=r.arrival, first_token=r.first_time, finish=r.finish_time, tokens=r.tokens,
                            token_times=r.token_times, prompt_len=len(r.prompt), reason=r.reason)
                for r in self.reqs.values()}


def summarize(records):
    """TTFT and time per output token over finished requests: mean / p50 / p99 in milliseconds, and
    the output-token throughput over the span of the run."""
    ttft = np.array([r["first_token"] - r["arrival"] for r in records.values()]) * 1e3
    tpot = np.array([(r["finish"] - r["first_token"]) / max(1, len(r["tokens"]) - 1) for r in records.values()
                     if len(r["tokens"]) > 1]) * 1e3
    span = max(r["finish"] for r in records.values()) - min(r["arrival"] for r in records.values())
    out_tokens = sum(len(r["tokens"]) for r in records.values())
    q = lambda a, p: float(np.percentile(a, p)) if len(a) else None  # noqa: E731
    return dict(requests=len(records), output_tokens=out_tokens, span_s=span, output_tokens_per_s=out_tokens / span,
                ttft_ms=dict(mean=float(ttft.mean()), p50=q(ttft, 50), p99=q(ttft, 99)),
                tpot_ms=dict(mean=float(tpot.mean()) if len(tpot) else None, p50=q(tpot, 50), p99=q(tpot, 99)))
