"""Stage traces of a running fabric (the role of the reference's
monoserve/fabric/trace.py:25-90, whose names StageTrace / spans / summary this module keeps).

    trace = StageTrace(capacity=1 << 20)     # device buffer; allocate it before the fabric starts
    trace.start(fab); ...run programs...; records = trace.stop(fab)
    print(summary(records, labels, lane=0))

The kernel writes one record of two u64 per stage event: (stage | lane << 32 | event << 40 |
tag << 48, device ns); event 0 = the stage was activated (its last predecessor completed),
1 = its last tile completed.  A stage's span runs from activation to completion and so
includes the time it waited for workers; stages that run side by side overlap, so spans do
not add up to wall time.  `labels[stage]` is a name or a (name, layer) pair.
"""
import numpy as np

ACTIVATE, COMPLETE = 0, 1


class StageTrace:
    def __init__(self, capacity=1 << 20, device="cuda"):
        import torch
        self.capacity = capacity
        self.buf = torch.zeros(capacity, 2, dtype=torch.int64, device=device)

    def start(self, fab):
        fab.set_trace(self.buf.data_ptr(), self.capacity)

    def stop(self, fab):
        """int64 [n, 5] = stage, lane, event, tag, device ns, ordered by time."""
        n = min(fab.trace_count(), self.capacity)
        fab.set_trace(0, 0)
        raw = np.frombuffer(fab.read(self.buf.data_ptr(), 16 * n), dtype="<u8").reshape(n, 2)
        word = raw[:, 0]
        rec = np.empty((n, 5), dtype=np.int64)
        rec[:, 0] = word & np.uint64(0xFFFFFFFF)
        rec[:, 1] = (word >> np.uint64(32)) & np.uint64(0xFF)
        rec[:, 2] = (word >> np.uint64(40)) & np.uint64(0xFF)
        rec[:, 3] = (word >> np.uint64(48)) & np.uint64(0xFFF)
        rec[:, 4] = raw[:, 1]
        return rec[np.argsort(rec[:, 4], kind="stable")]


def _label(labels, stage):
    lab = labels[stage] if stage < len(labels) and labels[stage] is not None else f"stage{stage}"
    return lab if isinstance(lab, tuple) else (lab, -1)


def spans(records, labels, lane=None):
    """[(name, layer, tag, activation ns, completion ns)] of every stage that was both activated
    and completed inside the trace, in completion order."""
    rec = records if lane is None else records[records[:, 1] == lane]
    opened, out = {}, []
    for stage, _, event, tag, t in rec.tolist():
        if event == ACTIVATE:
            opened[(stage, tag)] = t
        else:
            t0 = opened.pop((stage, tag), None)
            if t0 is not None:
                name, layer = _label(labels, stage)
                out.append((name, layer, tag, t0, t))
    return out


def _extent(items, key):
    """{key(item): (earliest activation, latest completion)}"""
    ext = {}
    for item in items:
        k = key(item)
        lo, hi = ext.get(k, (item[3], item[4]))
        ext[k] = (min(lo, item[3]), max(hi, item[4]))
    return ext


def summary(records, labels, lane=None, experts=("w13", "red", "w2", "fetch")):
    """Text table: per stage name the count and span statistics (largest total first); the extent of
    every layer's expert stages per iteration; the wall time of the first iterations."""
    sp = spans(records, labels, lane)
    if not sp:
        return "no complete stages in the trace"
    by_name = {}
    for name, _, _, t0, t1 in sp:
        by_name.setdefault(name, []).append((t1 - t0) / 1e3)
    rows = [f"{'stage':14s} {'n':>6s} {'mean us':>9s} {'p50 us':>9s} {'max us':>9s} {'sum ms':>9s}"]
    for name, us in sorted(by_name.items(), key=lambda kv: -sum(kv[1])):
        us = np.asarray(us)
        rows.append(f"{name:14s} {us.size:6d} {us.mean():9.1f} {np.median(us):9.1f} {us.max():9.1f} {us.sum() / 1e3:9.3f}")
    layer_ext = _extent([s for s in sp if s[0] in experts], key=lambda s: (s[2], s[1]))
    if layer_ext:
        us = np.asarray([hi - lo for lo, hi in layer_ext.values()]) / 1e3
        rows.append(f"experts of a layer: mean {us.mean():.1f} us, max {us.max():.1f} us ({us.size} layer iterations)")
    iter_ext = _extent(sp, key=lambda s: s[2])
    ms = sorted((hi - lo) / 1e6 for lo, hi in iter_ext.values())
    rows.append("iterations (ms): " + ", ".join(f"{x:.2f}" for x in ms[:8]))
    return "\n".join(rows)
