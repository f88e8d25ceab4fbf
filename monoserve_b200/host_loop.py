"""Python side of the host loop (include/monofab.h, csrc/host_loop.cu): staging, by the copy
engine, of the host-resident experts a prefill lane is about to use into the lane's HBM staging
buffer.  Mirrors the reference's monoserve/runtime/host_loop.py:1-47 (`staging_order`,
`HostLoop(fab, weights)`, `add_prefill_lane`, `start`, `stop`, `stats`)."""
import ctypes

import numpy as np

from monoserve_b200 import _C

REGION_HOST, REGION_STAGE0 = 0, 2   # region ids of the (region, slot) tables (monoserve/runtime/kinds.py:16-18)


def staging_order(profile, weights, layer):
    """Experts to stage for a layer, best first: prefill activation frequency, skipping the experts
    the hot tier already holds (monoserve/runtime/host_loop.py:11-17)."""
    p = profile[layer] if profile is not None else np.ones(weights.cfg.num_experts)
    hot = set(weights.hot[layer])
    return [int(e) for e in np.argsort(-np.asarray(p), kind="stable") if int(e) not in hot]


class RawHostLoop:
    """The C-ABI object.  fab = None makes a loop that issues no CUDA call: marks are injected with
    `inject`, `step` runs one poll, `log` returns what it decided (tests of the policy)."""

    def __init__(self, fab, layers, experts, w13_bytes, w2_bytes, host_w13=None, host_w2=None, host_region=REGION_HOST):
        self._lib = _C.lib
        self._h = ctypes.c_void_p()
        self.layers = layers
        a13 = (ctypes.c_uint64 * layers)(*(host_w13 or [0] * layers))
        a2 = (ctypes.c_uint64 * layers)(*(host_w2 or [0] * layers))
        _C.check(self._lib.monofab_host_loop_create(fab._h if fab is not None else None, layers, experts, w13_bytes,
                                                    w2_bytes, a13, a2, host_region, ctypes.byref(self._h)))

    def add_lane(self, lane, region, w13_dst, w2_dst, slots, tables, order):
        """order: per layer, the experts to stage, best first."""
        assert len(order) == self.layers
        flat = [e for layer in order for e in layer]
        offs = np.cumsum([0] + [len(layer) for layer in order]).astype(np.int32)
        arr = (ctypes.c_int32 * max(1, len(flat)))(*flat)
        off = (ctypes.c_int32 * len(offs))(*offs.tolist())
        _C.check(self._lib.monofab_host_loop_add_lane(self._h, lane, region, w13_dst, w2_dst, slots, tables, arr, off))

    def start(self, poll_us=5):
        _C.check(self._lib.monofab_host_loop_start(self._h, poll_us))

    def stop(self):
        _C.check(self._lib.monofab_host_loop_stop(self._h))

    def stats(self):
        out = (ctypes.c_uint64 * 5)()
        _C.check(self._lib.monofab_host_loop_stats(self._h, out))
        return dict(zip(("copies", "bytes", "flips", "restores", "polls"), list(out)))

    def inject(self, lane_index, mark, gen=1, running=1):
        _C.check(self._lib.monofab_host_loop_inject(self._h, lane_index, mark, gen, running))

    def step(self, n=1):
        for _ in range(n):
            _C.check(self._lib.monofab_host_loop_step(self._h))

    def log(self):
        """[(kind, lane, layer, expert, slot)]: kind "copy" | "flip" | "restore"."""
        n = ctypes.c_int32()
        _C.check(self._lib.monofab_host_loop_log(self._h, None, 0, ctypes.byref(n)))
        buf = (ctypes.c_int32 * max(1, 5 * n.value))()
        _C.check(self._lib.monofab_host_loop_log(self._h, buf, n.value, ctypes.byref(n)))
        names = ("copy", "flip", "restore")
        return [(names[buf[5 * i]],) + tuple(buf[5 * i + 1:5 * i + 5]) for i in range(n.value)]

    def close(self):
        if getattr(self, "_h", None) and self._h.value:
            self._lib.monofab_host_loop_destroy(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        self.close()


class HostLoop:
    """loop = HostLoop(fab, weights); loop.add_prefill_lane(lane, staging_index, profile); loop.start()
    (monoserve/runtime/host_loop.py:20-47).  `weights` is a ModelWeights with staging buffers
    (`alloc_staging`), `lane` a ModelLane built with the same `staging_index`."""

    def __init__(self, fab, weights):
        cfg = weights.cfg
        w13_bytes, w2_bytes = weights.expert_bytes()
        # the copy engine reads the pinned host stacks directly (dense layers have none)
        host13 = [0 if t is None else t.data_ptr() for t in weights.host_w13]
        host2 = [0 if t is None else t.data_ptr() for t in weights.host_w2]
        self.impl = RawHostLoop(fab, cfg.num_layers, cfg.num_experts, w13_bytes, w2_bytes, host13, host2, REGION_HOST)
        self.weights = weights

    def add_prefill_lane(self, lane, staging_index, profile=None):
        """Stage for `lane` into staging buffer `staging_index`; each half of the buffer holds one
        layer's worth of experts."""
        w = self.weights
        slots = w.staging_slots // 2
        order = [staging_order(profile, w, l) if w.host_w13[l] is not None else [] for l in range(w.cfg.num_layers)]
        # every lane has its own tables and weight maps, and region 2 of a lane's maps is the staging buffer
        # it was built with (the reference numbers the buffers REGION_STAGE0 + staging_index in shared maps)
        assert lane.staging_index == staging_index
        self.impl.add_lane(lane.lane_id, REGION_STAGE0, w.stage_w13[staging_index].data_ptr(),
                           w.stage_w2[staging_index].data_ptr(), slots, lane.tables.data_ptr(), order)

    def start(self, poll_us=5):
        self.impl.start(poll_us)

    def stop(self):
        self.impl.stop()

    def stats(self):
        return self.impl.stats()

    def close(self):
        self.impl.close()
