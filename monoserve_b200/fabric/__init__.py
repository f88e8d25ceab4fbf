"""Python surface of the fabric: `Fabric` (the persistent kernel on one GPU),
lane programs (`Program`, `Tile`, `tile_array`), and operand-block packing by
queried layouts (`args`).  Same names and calling conventions as the reference's
monoserve/fabric package and its native Fabric class (csrc/bindings.cpp:184-296)."""
import ctypes

import numpy as np

from monoserve_b200.fabric.program import KIND, STAGE_LINK, STAGE_MARK, STAGE_RESET, Program, Tile, tile_array

__all__ = ["KIND", "STAGE_LINK", "STAGE_MARK", "STAGE_RESET", "Program", "Tile", "tile_array", "Fabric"]


class Fabric:
    """The persistent fabric on one GPU.

    fab = Fabric(); h = program.upload(fab, first=0); fab.start()
    fab.publish(map=[0] * fab.num_workers, caps=[0], order=[0], programs=[h]); ...; fab.stop()
    """

    def __init__(self, num_workers=0, smem_bytes=200 * 1024, device=0, pool_bytes=1 << 30):
        from monoserve_b200 import _C
        self._C, self._lib = _C, _C.lib
        self._h = ctypes.c_void_p()
        _C.check(self._lib.monofab_fabric_create(num_workers, device, pool_bytes, ctypes.byref(self._h)))

    def __del__(self):
        self.close()

    def close(self):
        if getattr(self, "_h", None) and self._h.value and self._lib is not None:
            self._lib.monofab_fabric_destroy(self._h)
            self._h = ctypes.c_void_p()

    def _info(self):
        nw, ns, run = ctypes.c_int32(), ctypes.c_int32(), ctypes.c_int32()
        ep = ctypes.c_uint64()
        self._C.check(self._lib.monofab_fabric_info(self._h, ctypes.byref(nw), ctypes.byref(ns), ctypes.byref(run),
                                                    ctypes.byref(ep)))
        return nw.value, ns.value, bool(run.value), ep.value

    num_workers = property(lambda self: self._info()[0])
    num_sms = property(lambda self: self._info()[1])
    running = property(lambda self: self._info()[2])
    epoch = property(lambda self: self._info()[3])

    def start(self):
        self._C.check(self._lib.monofab_fabric_start(self._h))

    def stop(self):
        if self._h.value:
            self._C.check(self._lib.monofab_fabric_stop(self._h))

    def set_idle_cap(self, ns):
        self._C.check(self._lib.monofab_fabric_set_limits(self._h, int(ns), 120 * 10 ** 9))

    def set_max_run(self, seconds):
        """The kernel leaves on its own after this long (0 = no limit)."""
        self._C.check(self._lib.monofab_fabric_set_limits(self._h, 0, int(seconds * 1e9)))

    def upload(self, tiles, stages, succ, first_stage, reset_stage, iterations):
        """tiles int64 [n, 8], stages int32 [m, 8], succ int32 [k]: CPU tensors."""
        import torch
        for t, dt, cols in ((tiles, torch.int64, 8), (stages, torch.int32, 8)):
            if t.device.type != "cpu" or t.dtype != dt or t.dim() != 2 or t.shape[1] != cols or not t.is_contiguous():
                raise RuntimeError(f"monofab: upload wants contiguous CPU tensors of shape [n, {cols}] and dtype {dt}")
        if succ.device.type != "cpu" or succ.dtype != torch.int32 or not succ.is_contiguous():
            raise RuntimeError("monofab: upload wants succ as a contiguous CPU int32 tensor")
        h = ctypes.c_uint64()
        self._C.check(self._lib.monofab_fabric_upload(self._h, tiles.data_ptr(), tiles.shape[0], stages.data_ptr(),
                                                      stages.shape[0], succ.data_ptr(), succ.numel(), first_stage,
                                                      reset_stage, iterations, ctypes.byref(h)))
        return h.value

    def release(self, handle):
        self._C.check(self._lib.monofab_fabric_release(self._h, handle))

    def program_info(self, handle):
        info = (ctypes.c_uint32 * 6)()
        self._C.check(self._lib.monofab_fabric_program_info(self._h, handle, ctypes.byref(info)))
        return dict(zip(("gen", "n_tiles", "n_stages", "first_stage", "reset_stage", "iterations"), list(info)))

    def generation(self, handle):
        return self.program_info(handle)["gen"]

    def publish(self, map, caps, order, programs, forms=()):
        n = len(programs)
        m = (ctypes.c_int32 * len(map))(*map)
        c = (ctypes.c_uint32 * n)(*caps)
        o = (ctypes.c_int32 * n)(*order)
        p = (ctypes.c_uint64 * n)(*programs)
        f = (ctypes.c_uint32 * n)(*forms) if len(forms) else None
        e = ctypes.c_uint64()
        self._C.check(self._lib.monofab_fabric_publish(self._h, m, len(map), c, o, p, n, f, ctypes.byref(e)))
        return e.value

    def progress(self):
        lanes = (ctypes.c_uint64 * 20)()
        we, wn = (ctypes.c_uint64 * 256)(), (ctypes.c_uint64 * 256)()
        err = ctypes.c_uint64()
        self._C.check(self._lib.monofab_fabric_progress(self._h, lanes, we, wn, ctypes.byref(err)))
        nw = self.num_workers
        keys = ("iterations", "gen", "running", "mark", "mark_ns")
        return {"lanes": [dict(zip(keys, lanes[5 * l:5 * l + 5])) for l in range(4)],
                "worker_epoch": list(we)[:nw], "worker_epoch_ns": list(wn)[:nw], "error": err.value}

    def lane_stats(self, lane):
        s = (ctypes.c_uint32 * 7)()
        self._C.check(self._lib.monofab_fabric_lane_stats(self._h, lane, ctypes.byref(s)))
        return dict(zip(("slots", "inflight", "inflight_max", "running", "tag", "iter_in_prog", "gen"), list(s)))

    def reset_inflight_max(self, lane):
        self._C.check(self._lib.monofab_fabric_reset_inflight_max(self._h, lane))

    def iterations(self, lane):
        return self.progress()["lanes"][lane]["iterations"]

    def iteration_times(self, lane, start, count, timeout=60.0):
        out = (ctypes.c_uint64 * count)()
        self._C.check(self._lib.monofab_fabric_iteration_times(self._h, lane, start, count, float(timeout), out))
        return list(out)

    def read(self, src, nbytes):
        buf = ctypes.create_string_buffer(nbytes)
        self._C.check(self._lib.monofab_fabric_read(self._h, src, buf, nbytes))
        return buf.raw

    def write(self, dst, data):
        data = bytes(data)
        self._C.check(self._lib.monofab_fabric_write(self._h, dst, data, len(data)))

    def blob_alloc(self, nbytes):
        a = ctypes.c_uint64()
        self._C.check(self._lib.monofab_fabric_blob_alloc(self._h, nbytes, ctypes.byref(a)))
        return a.value

    def blob_free(self, addr):
        self._C.check(self._lib.monofab_fabric_blob_free(self._h, addr))

    def set_trace(self, ptr, capacity):
        self._C.check(self._lib.monofab_fabric_set_trace(self._h, ptr, capacity))

    def trace_count(self):
        n = ctypes.c_uint32()
        self._C.check(self._lib.monofab_fabric_trace_count(self._h, ctypes.byref(n)))
        return n.value

    def worker_tiles(self):
        words, since = (ctypes.c_uint64 * 256)(), (ctypes.c_uint64 * 256)()
        self._C.check(self._lib.monofab_fabric_worker_tiles(self._h, words, since))
        out = []
        for w, t in list(zip(words, since))[:self.num_workers]:
            out.append(dict(running=bool(w >> 63), completing=bool((w >> 62) & 1), lane=(w >> 56) & 0x3f,
                            kind=(w >> 44) & 0xfff, stage=(w >> 24) & 0xfffff, tile=w & 0xffffff, since_ns=t))
        return out

    def wait_notes(self):
        """Per worker that left after a bounded wait ran out: where its producer, MMA and first
        exec warp were waiting (record, phase counts, tile, site) and the records finished."""
        words = (ctypes.c_uint64 * 1024)()
        self._C.check(self._lib.monofab_fabric_wait_notes(self._h, words))
        out = {}
        for i in range(self.num_workers):
            w = list(words[4 * i:4 * i + 4])
            if any(w):
                f = lambda v: dict(record=v >> 48, q=(v >> 40) & 0xff, ph0=(v >> 32) & 0xff, ph1=(v >> 24) & 0xff,  # noqa: E731
                                   tile=(v >> 8) & 0xff, site=v & 0xff)
                out[i] = dict(producer=f(w[0]), mma=f(w[1]), exec=f(w[2]), exec_done=w[3] & 0xffffffff,
                              mma_done=w[3] >> 32)
        return out

    def tensor_map(self, base, dims, strides_bytes, box, dtype=0, swizzle=128, packed=False):
        rank = len(dims)
        d = (ctypes.c_uint64 * rank)(*dims)
        s = (ctypes.c_uint64 * max(1, rank - 1))(*strides_bytes)
        b = (ctypes.c_uint32 * rank)(*box)
        h = ctypes.c_uint64()
        self._C.check(self._lib.monofab_fabric_tensor_map(self._h, base, d, s, b, rank, dtype, swizzle, ctypes.byref(h)))
        if packed:
            self._C.check(self._lib.monofab_fabric_tensor_map_packed(self._h, h.value, 1))
        return h.value
