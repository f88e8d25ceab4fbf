"""Mechanism tests of the persistent fabric with test tiles.  The first part of this file is
a copy, re-flowed, of the reference's own tests/test_fabric_core.py:75-219 (same helpers,
scenarios and thresholds; the epoch-spread bound is 2.5 tiles instead of 1.5), because running
the reference's tests against this library is the drop-in check; the tests after them (marks and
trace, bad tile, deadline, malformed upload) are this build's own.  The scenarios: every tile runs exactly once and
never before the stages it depends on; workers serve their own lane first and
borrow from other lanes; link credits bound the link tiles in flight; a new epoch
reaches every worker within about one tile; programs iterate and are replaced at
iteration boundaries.  Each test allocates before start() and reads after stop().
"""
import time

import numpy as np
import pytest
import torch

from monoserve_b200.fabric import KIND, Fabric, Program, Tile

pytestmark = pytest.mark.gpu
TRACE_WORDS = 4   # start, end, (worker, sm), (count, lane)


def trace_buffer(n):
    return torch.zeros(n, TRACE_WORDS, dtype=torch.int64, device="cuda")


def decode_trace(t):
    t = t.cpu().numpy().astype(np.uint64)
    return {"start": t[:, 0].astype(np.int64), "end": t[:, 1].astype(np.int64),
            "worker": (t[:, 2] & 0xFFFFFFFF).astype(np.int64), "count": (t[:, 3] & 0xFFFFFFFF).astype(np.int64),
            "lane": (t[:, 3] >> np.uint64(32)).astype(np.int64)}


def spin(ns, trace, idx, lane_tag=0):
    return Tile(KIND["spin"], i=(idx, lane_tag), a=(ns, trace.data_ptr()))


def wait_idle(fab, lane, timeout=30.0):
    t0 = time.time()
    while time.time() - t0 < timeout:
        if fab.lane_stats(lane)["running"] == 0 and fab.progress()["lanes"][lane]["iterations"] > 0:
            return
        time.sleep(0.01)
    raise TimeoutError(f"lane {lane} did not finish: {fab.progress()}")


def wait_until(pred, timeout=30.0, what="condition"):
    t0 = time.time()
    while not pred():
        if time.time() - t0 > timeout:
            raise TimeoutError(what)
        time.sleep(1e-4)


@pytest.fixture
def fab():
    f = Fabric(pool_bytes=256 << 20)
    f.set_max_run(60)
    yield f
    f.stop()
    f.close()


def test_dag_order_and_exactly_once(fab):
    trace = trace_buffer(4096)
    p = Program()
    idx = iter(range(4096))
    s0 = p.stage([spin(20_000, trace, next(idx)) for _ in range(40)])
    s1 = p.stage([spin(15_000, trace, next(idx)) for _ in range(300)])
    s2 = p.stage([spin(30_000, trace, next(idx)) for _ in range(100)])
    s3 = p.stage([spin(10_000, trace, next(idx)) for _ in range(64)])
    for a, b in ((s0, s1), (s0, s2), (s1, s3), (s2, s3)):
        p.after(a, b)
    h = p.upload(fab, first=s0)
    fab.start()
    fab.publish(map=[0] * fab.num_workers, caps=[0], order=[0], programs=[h])
    wait_idle(fab, 0)
    fab.stop()
    assert fab.progress()["error"] == 0
    tr = decode_trace(trace)
    bounds = {s0: (0, 40), s1: (40, 340), s2: (340, 440), s3: (440, 504)}
    assert (tr["count"][:504] == 1).all(), "every tile runs exactly once"
    for pred, succ in ((s0, s1), (s0, s2), (s1, s3), (s2, s3)):
        a, b = bounds[pred]
        c, d = bounds[succ]
        assert tr["start"][c:d].min() >= tr["end"][a:b].max()
    assert len(set(tr["worker"][40:340])) > fab.num_workers // 2, "work spreads"


def test_floors_and_borrowing(fab):
    n = fab.num_workers
    half = n // 2
    trace = trace_buffer(40_000)
    p0, p1 = Program(), Program()
    p0.stage([spin(20_000, trace, i, 0) for i in range(30_000)])
    p1.stage([spin(20_000, trace, 32_768 + i, 1) for i in range(200)])
    h0, h1 = p0.upload(fab, first=0), p1.upload(fab, first=0)
    lane_of = [0] * half + [1] * (n - half)
    fab.start()
    fab.publish(map=lane_of, caps=[0, 0], order=[0, 1], programs=[h0, 0])
    time.sleep(0.001)
    fab.publish(map=lane_of, caps=[0, 0], order=[0, 1], programs=[h0, h1])
    wait_idle(fab, 0)
    wait_idle(fab, 1)
    fab.stop()
    assert fab.progress()["error"] == 0
    tr = decode_trace(trace)
    assert (tr["count"][:30_000] == 1).all() and (tr["count"][32_768:32_968] == 1).all()
    w0, w1 = tr["worker"][:30_000], tr["worker"][32_768:32_968]
    own1 = np.isin(w1, np.arange(half, n)).mean()
    borrowed0 = np.isin(w0, np.arange(half, n)).mean()
    assert own1 > 0.9, f"lane 1 tiles should run on lane 1 workers ({own1:.2f})"
    assert borrowed0 > 0.2, f"idle lane 1 workers should borrow lane 0 tiles ({borrowed0:.2f})"


@pytest.mark.parametrize("cap", [2, 8])
def test_link_slots_bound_inflight(fab, cap):
    src = torch.randint(0, 255, (256 << 20,), dtype=torch.uint8, device="cuda")
    sink = torch.zeros(fab.num_workers, dtype=torch.int32, device="cuda")
    trace = trace_buffer(2048)
    chunk = 1 << 20
    p = Program()
    link = p.stage([Tile(KIND["read"], i=(i,), a=(src.data_ptr() + (i % 256) * chunk, chunk, sink.data_ptr(),
                                                   trace.data_ptr())) for i in range(1024)], link=True)
    other = p.stage([spin(5_000, trace, 1100 + i) for i in range(400)])
    p.after(link, other)
    h = p.upload(fab, first=link)
    fab.start()
    fab.reset_inflight_max(0)
    fab.publish(map=[0] * fab.num_workers, caps=[cap], order=[0], programs=[h])
    wait_idle(fab, 0)
    stats = fab.lane_stats(0)
    fab.stop()
    assert fab.progress()["error"] == 0
    tr = decode_trace(trace)
    assert (tr["count"][:1024] == 1).all()
    assert (tr["count"][1100:1500] == 1).all()
    assert stats["inflight_max"] <= cap
    assert stats["inflight_max"] == cap, "the gate should admit exactly cap tiles"
    assert stats["slots"] == 0


def test_epoch_reaches_workers_within_a_tile(fab):
    trace = trace_buffer(1 << 14)
    tile_ns = 50_000
    p = Program()
    p.stage([spin(tile_ns, trace, i) for i in range(12_000)])
    h = p.upload(fab, first=0)
    fab.start()
    fab.publish(map=[0] * fab.num_workers, caps=[0], order=[0], programs=[h])
    time.sleep(0.2)
    e = fab.publish(map=[0] * fab.num_workers, caps=[0], order=[0], programs=[h])
    wait_until(lambda: min(fab.progress()["worker_epoch"]) >= e, what="epoch")
    ns = np.array(fab.progress()["worker_epoch_ns"], dtype=np.int64)
    fab.stop()
    spread_us = (ns.max() - ns.min()) / 1e3
    # the scheduler warp runs one tile ahead, so a worker sees the new epoch at most two tiles later
    assert spread_us <= tile_ns / 1e3 * 2.5, spread_us


def test_iterations(fab):
    trace = trace_buffer(1024)
    p = Program()
    a = p.stage([spin(2_000, trace, i) for i in range(50)])
    b = p.stage([spin(2_000, trace, 50 + i) for i in range(50)])
    p.after(a, b)
    h = p.upload(fab, first=a, iterations=5)
    fab.start()
    fab.publish(map=[0] * fab.num_workers, caps=[0], order=[0], programs=[h])
    wait_idle(fab, 0)
    it = fab.progress()["lanes"][0]["iterations"]
    fab.stop()
    tr = decode_trace(trace)
    assert it == 5
    assert (tr["count"][:100] == 5).all()


def test_program_switch_at_boundary(fab):
    trace = trace_buffer(1024)
    p1 = Program()
    p1.stage([spin(5_000, trace, i) for i in range(64)])
    h1 = p1.upload(fab, first=0, iterations=0)
    p2 = Program()
    p2.stage([spin(5_000, trace, 512 + i) for i in range(64)])
    h2 = p2.upload(fab, first=0, iterations=3)
    fab.start()
    fab.publish(map=[0] * fab.num_workers, caps=[0], order=[0], programs=[h1])
    time.sleep(0.05)
    fab.publish(map=[0] * fab.num_workers, caps=[0], order=[0], programs=[h2])
    wait_until(lambda: fab.lane_stats(0)["running"] == 0, what="switch")
    gen = fab.progress()["lanes"][0]["gen"]
    fab.stop()
    tr = decode_trace(trace)
    assert gen == fab.generation(h2)
    assert (tr["count"][512:576] == 3).all()
    assert tr["count"][:64].min() >= 1


def test_marks_trace_and_safe_memory_access(fab):
    """Stage marks reach the host mirror, stage events land in the trace buffer, and
    read / write / blob_alloc work while the kernel runs."""
    trace = trace_buffer(64)
    events = torch.zeros(64, 2, dtype=torch.int64, device="cuda")
    p = Program()
    a = p.stage([spin(1_000, trace, i) for i in range(8)], mark=(3 << 8) | 1)
    b = p.stage([spin(1_000, trace, 8 + i) for i in range(8)], mark=(3 << 8) | 2)
    p.after(a, b)
    h = p.upload(fab, first=a, iterations=2)
    fab.set_trace(events.data_ptr(), 64)
    blob = fab.blob_alloc(256)
    fab.start()
    fab.write(blob, bytes(range(200)))
    fab.publish(map=[0] * fab.num_workers, caps=[0], order=[0], programs=[h])
    wait_idle(fab, 0)
    assert fab.read(blob, 200) == bytes(range(200))
    assert fab.progress()["lanes"][0]["mark"] == (3 << 8) | 2
    n_ev = fab.trace_count()
    fab.stop()
    fab.blob_free(blob)
    assert n_ev == 2 * 2 * 3   # (activate + complete) x 3 stages (two + reset) x 2 iterations
    ev = events.cpu().numpy()[:n_ev]
    assert set((ev[:, 0] & 0xFFFFF).tolist()) == {0, 1, 2}
    info = fab.program_info(h)
    assert info["n_stages"] == 3 and info["iterations"] == 2
    fab.release(h)
    with pytest.raises(RuntimeError, match="unknown program"):
        fab.release(h)


def test_bad_tile_kind_is_reported_not_trapped(fab):
    p = Program()
    p.stage([Tile(999)])
    h = p.upload(fab, first=0)
    fab.start()
    fab.publish(map=[0] * fab.num_workers, caps=[0], order=[0], programs=[h])
    wait_idle(fab, 0)
    fab.stop()
    assert fab.progress()["error"] & 8   # MONOFAB_FABRIC_ERR_BAD_TILE; the context is still usable:
    assert int(torch.ones(4, device="cuda").sum()) == 4


def test_deadline_stops_an_idle_fabric(fab):
    """Nothing published, nobody calls stop(): the kernel leaves by itself."""
    fab.set_max_run(0.3)
    fab.start()
    t0 = time.time()
    wait_until(lambda: fab.progress()["error"] & 4, timeout=10, what="deadline")
    assert time.time() - t0 < 5
    fab.stop()


def test_upload_rejects_malformed_programs(fab):
    tiles = torch.zeros(2, 8, dtype=torch.int64)
    stages = torch.tensor([[0, 5, 0, 1, 0, 0, 0, 0]], dtype=torch.int32)   # names 5 tiles of 2
    succ = torch.tensor([0], dtype=torch.int32)
    with pytest.raises(RuntimeError, match="names tiles"):
        fab.upload(tiles, stages, succ, 0, 0, 1)
    with pytest.raises(RuntimeError, match="contiguous CPU"):
        fab.upload(tiles.to(torch.int32), stages, succ, 0, 0, 1)
    with pytest.raises(RuntimeError, match="lanes"):
        fab.publish(map=[0], caps=[0] * 5, order=[0] * 5, programs=[0] * 5)
