"""Drop-in for the reference's native extension module `monoserve._C`
(csrc/bindings.cpp:171-384): the same module-level functions, the same classes with
the same method names, argument order, defaults, return shapes and error type
(RuntimeError("monofab: ...")), implemented over libmonofab's C ABI.

What differs, and why, is listed in the docstrings below and in one place:
`DEVIATIONS`.  Raw 64-bit device addresses cross this boundary exactly as they do
in the reference (monoserve/fabric/args.py:28-29).
"""
import ctypes
import types

from monoserve_b200 import _C as _native
from monoserve_b200.fabric import Fabric as _Fabric
from monoserve_b200.fabric import args as _args

DEVIATIONS = {
    "tile kinds 45 / 46": "taken, with one difference in how they run: a K-split tile of kind 45 is executed as one "
                          "symmetric K-range record per block of bm rows, so the weight slice is read once per row "
                          "block, not once per tile (from L2 when it is in HBM); results are the same sums. This "
                          "library's own builders use 256-row blocks and the staged form (kind 49) instead.",
    "attention tiles": "kinds 33 / 34 take this library's work items (monoserve_b200.attention.fabric_tiles), not "
                       "AttnArgs blocks; attn_args() still packs the reference's struct for callers that only "
                       "inspect it.",
    "smem_bytes": "accepted and ignored: the worker's shared-memory size is fixed by the kernel.",
    "GreenPartitions": "a stub (an ablation in the reference); create() raises.",
    "wait_note_address": "per fabric in this library; the module-level function returns the address for the most "
                         "recently created Fabric, 0 if there is none.",
}

struct_layouts = _native.struct_layouts
host_device_pointer = _native.host_device_pointer
_latest_fabric = None


def wait_note_address():
    """Device address of the fabric's long-wait records (csrc/bindings.cpp:182)."""
    f = _latest_fabric() if _latest_fabric is not None else None
    return f.wait_note_address() if f is not None else 0


def gemm_args(out, ld_out, k_tiles, epi, bm, n_limit, pair_token=0, pair_weight=0, residual=0, ld_res=0, bias=0,
              up_offset=0, w_fp8=0):
    """Packed GemmArgs block (csrc/bindings.cpp:332-356)."""
    return _args.pack("GemmArgs", out=out, ld_out=ld_out, k_tiles=k_tiles, epi=epi, bm=bm, n_limit=n_limit,
                      pair_token=pair_token, pair_weight=pair_weight, residual=residual, ld_res=ld_res, bias=bias,
                      up_offset=up_offset, w_fp8=w_fp8)


def attn_args(q_map, k_map, v_map, out, ws_o, ws_m, ws_l, block_table, req_info, scale_log2, bt_stride, hq, hkv,
              chunk_blocks, max_chunks):
    """Packed AttnArgs block (csrc/bindings.cpp:357-383); group = hq / hkv is filled in."""
    return _args.pack("AttnArgs", q_map=q_map, k_map=k_map, v_map=v_map, out=out, ws_o=ws_o, ws_m=ws_m, ws_l=ws_l,
                      block_table=block_table, req_info=req_info, scale_log2=scale_log2, bt_stride=bt_stride, hq=hq,
                      hkv=hkv, group=hq // hkv, chunk_blocks=chunk_blocks, max_chunks=max_chunks)


class Fabric(_Fabric):
    """class Fabric of csrc/bindings.cpp:184-296 over monofab_fabric_*."""

    def __init__(self, num_workers=0, smem_bytes=200 * 1024, device=0, pool_bytes=1 << 30):
        import weakref
        super().__init__(num_workers, smem_bytes, device, pool_bytes)
        global _latest_fabric
        _latest_fabric = weakref.ref(self)

    def start_on(self, stream, context, workers, first_worker=0):
        """Launch workers [first_worker, first_worker + workers) on the caller's stream (a raw
        cudaStream_t value), inside `context` if it is non-zero (csrc/host/fabric.cpp:204-227)."""
        self._C.check(self._lib.monofab_fabric_start_on(self._h, int(stream), int(context), workers, first_worker))

    def program_info(self, handle):
        """{tiles, stages, runtime (device addresses), n_tiles, n_stages} as csrc/bindings.cpp:243-253; the
        handle is the device address of the program descriptor, whose first three words are those addresses."""
        import struct
        tiles, stages, runtime = struct.unpack("<3Q", self.read(handle, 24))
        info = super().program_info(handle)
        return {"tiles": tiles, "stages": stages, "runtime": runtime, "n_tiles": info["n_tiles"],
                "n_stages": info["n_stages"]}

    def generation(self, handle):
        return super().program_info(handle)["gen"]

    def lane_ring(self, lane, link=False, max_entries=4096):
        """{head, tail, reserve, entries} of a lane's stage ring (csrc/bindings.cpp:255-265)."""
        counters = (ctypes.c_uint64 * 3)()
        entries = (ctypes.c_uint32 * max(1, max_entries))()
        n = ctypes.c_int32()
        self._C.check(self._lib.monofab_fabric_lane_ring(self._h, lane, int(bool(link)), max_entries,
                                                         ctypes.byref(counters), entries, ctypes.byref(n)))
        return {"head": counters[0], "tail": counters[1], "reserve": counters[2], "entries": list(entries[:n.value])}

    def worker_tiles(self):
        """[{running, completing, lane, kind, stage, index, ns}] (csrc/bindings.cpp:266-281)."""
        return [dict(running=int(t["running"]), completing=int(t["completing"]), lane=t["lane"], kind=t["kind"],
                     stage=t["stage"], index=t["tile"], ns=t["since_ns"]) for t in super().worker_tiles()]

    def progress(self):
        """{lanes, worker_epoch, worker_epoch_ns} (csrc/bindings.cpp:26-62), plus this library's `error`."""
        return super().progress()

    def wait_note_address(self):
        a = ctypes.c_uint64()
        self._C.check(self._lib.monofab_fabric_wait_note_address(self._h, ctypes.byref(a)))
        return a.value


class GreenPartitions:
    """csrc/bindings.cpp:298-304.  Green-context SM partitions are an ablation in the reference
    (monoserve/ablations.py); this library divides SMs by the published worker map instead, so the
    class exists for import compatibility and refuses to create partitions."""

    size = 0

    def create(self, counts):
        raise RuntimeError("monofab: green-context partitions are not built in this library; divide the SMs "
                           "with Fabric.publish(map=...) or start_on(workers=..., first_worker=...)")

    def destroy(self):
        return None

    def stream(self, index):
        raise RuntimeError("monofab: no partitions")

    def context(self, index):
        raise RuntimeError("monofab: no partitions")


class HostLoop:
    """class HostLoop of csrc/bindings.cpp:306-330 over monofab_host_loop_*: same constructor
    and add_lane signatures (order is a list of per-layer expert lists)."""

    def __init__(self, fab, layers, experts, w13_bytes, w2_bytes, host_w13, host_w2, host_region):
        self._fab = fab   # keeps the fabric alive, as py::keep_alive<1, 2> does
        self._layers = layers
        self._h = ctypes.c_void_p()
        a13 = (ctypes.c_uint64 * layers)(*host_w13)
        a2 = (ctypes.c_uint64 * layers)(*host_w2)
        _native.check(_native.lib.monofab_host_loop_create(fab._h, layers, experts, w13_bytes, w2_bytes, a13, a2,
                                                           host_region, ctypes.byref(self._h)))

    def add_lane(self, lane, region, w13_dst, w2_dst, slots, tables, order):
        flat, offsets = [], [0]
        for layer in range(self._layers):
            flat += list(order[layer]) if layer < len(order) else []
            offsets.append(len(flat))
        o = (ctypes.c_int32 * max(1, len(flat)))(*flat)
        off = (ctypes.c_int32 * len(offsets))(*offsets)
        _native.check(_native.lib.monofab_host_loop_add_lane(self._h, lane, region, w13_dst, w2_dst, slots, tables, o, off))

    def start(self, poll_us=5):
        _native.check(_native.lib.monofab_host_loop_start(self._h, poll_us))

    def stop(self):
        if self._h.value:
            _native.check(_native.lib.monofab_host_loop_stop(self._h))

    def stats(self):
        out = (ctypes.c_uint64 * 5)()
        _native.check(_native.lib.monofab_host_loop_stats(self._h, out))
        return dict(zip(("copies", "bytes", "flips", "restores", "polls"), list(out)))

    def __del__(self):
        if getattr(self, "_h", None) and self._h.value and _native.lib is not None:
            _native.lib.monofab_host_loop_destroy(self._h)
            self._h = ctypes.c_void_p()


def _control_module():
    try:
        from monoserve_b200 import control as built
        return built.as_native_module()
    except ImportError:
        m = types.ModuleType("monoserve._C.control")
        m.__doc__ = "Time estimator, plan search and admission: not built in this library."
        return m


control = _control_module()
