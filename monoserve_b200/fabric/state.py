"""Read-only views of a fabric's bookkeeping for tests and tools: the stage table and
run-time counters of an uploaded program, its tile descriptors, and what waits in a lane's
rings (the role of the reference's monoserve/fabric/state.py:11-40).  Every read goes
through Fabric.read, i.e. the control stream, so it is safe beside a running kernel; values
may be caught mid-update.

`fab` is any object with the reference's Fabric methods `program_info` (returning the
device addresses "tiles", "stages", "runtime" and the counts) , `read` and `lane_ring`:
monoserve_b200.compat._C.Fabric."""
import numpy as np

STAGE_BITS = 20          # a ring entry is tag << 20 | stage
TAG_MASK = 0xFFF
_STATIC = ("first", "count", "succ_first", "succ_count", "deps_init", "flags", "mark")


def program_state(fab, handle):
    """dict of per-stage uint32 arrays: the seven StageStatic columns, and next / tag / done /
    deps of StageRuntime (tag_next holds next in its low word and the tag in its high word)."""
    info = fab.program_info(handle)
    n = info["n_stages"]
    static = np.frombuffer(fab.read(info["stages"], 32 * n), dtype="<u4").reshape(n, 8)
    run = np.frombuffer(fab.read(info["runtime"], 16 * n), dtype="<u4").reshape(n, 4)
    state = {name: static[:, col].copy() for col, name in enumerate(_STATIC)}
    state["next"], state["tag"] = run[:, 0].copy(), run[:, 1] & TAG_MASK
    state["done"], state["deps"] = run[:, 2].copy(), run[:, 3].copy()
    return state


def program_tiles(fab, handle, first=0, count=None):
    """uint64 [n, 8]: tile descriptors first .. first + count - 1 (all from `first` if count is None)."""
    info = fab.program_info(handle)
    n = info["n_tiles"] - first if count is None else count
    return np.frombuffer(fab.read(info["tiles"] + 64 * first, 64 * n), dtype="<u8").reshape(n, 8)


def ring_entries(fab, lane, link=False):
    """(head, tail, [(stage, tag), ...]) of a lane's ring, oldest entry first."""
    view = fab.lane_ring(lane, link)
    words = np.asarray(view["entries"], dtype=np.uint32)
    pairs = list(zip((words & ((1 << STAGE_BITS) - 1)).tolist(), (words >> STAGE_BITS).tolist()))
    return view["head"], view["tail"], pairs
