"""Lane programs: DAGs of stages of tiles, packed for upload to the fabric.

The same builder interface as the reference's monoserve/fabric/program.py
(Program.stage / after / reserve / dynamic_first / pack / upload, Tile,
tile_array, KIND, STAGE_*), producing the same wire format:

  tiles   int64 [n, 8]   word 0 = kind | lane << 16 | flags << 24 | stage << 32,
                         word 1 = i0 | i1 << 32, word 2 = i2 | i3 << 32, words 3..7 = a[0..4]
  stages  int32 [m, 8]   first tile, tile count, first successor, successor count,
                         predecessor count, flags, mark, 0
  succ    int32 [k]      successor stage ids

A program ends with a reset stage that the builder adds: it depends on every
sink stage, its tiles re-arm the bookkeeping of all other stages, and its
completion ends one iteration.  Tiles reserved for run-time generation sit
after the user tiles and BEFORE the reset tiles.
"""
import numpy as np
import torch

KIND = {"nop": 0, "spin": 1, "read": 2, "probe": 3, "zero_runtime": 4}
STAGE_LINK, STAGE_RESET, STAGE_MARK = 1, 2, 4
_LOW32 = np.uint64(0xFFFFFFFF)


class Tile:
    """One tile: kind, four 32-bit operands i, five 64-bit operands a."""
    __slots__ = ("kind", "i", "a", "flags")

    def __init__(self, kind, i=(0, 0, 0, 0), a=(0, 0, 0, 0, 0), flags=0):
        self.kind, self.i, self.a, self.flags = kind, tuple(i), tuple(a), flags


def _column(value, shape):
    """One operand as a flat uint64 column of prod(shape) entries, or a scalar when it is one."""
    a = np.asarray(value)
    if a.ndim == 0:
        return np.uint64(int(a) & 0xFFFFFFFFFFFFFFFF)
    return np.broadcast_to(a.astype(np.int64, copy=False), shape).reshape(-1).astype(np.uint64)


def tile_array(kind, i0=0, i1=0, i2=0, i3=0, a0=0, a1=0, a2=0, a3=0, a4=0):
    """(n, 8) uint64 tiles from broadcastable operand arrays."""
    ops = (i0, i1, i2, i3, a0, a1, a2, a3, a4)
    shape = np.broadcast_shapes(*[np.shape(v) for v in ops])
    c = [_column(v, shape) for v in ops]
    out = np.zeros((int(np.prod(shape, dtype=np.int64)), 8), dtype=np.uint64)
    out[:, 0] = np.uint64(kind & 0xFFFF)
    out[:, 1] = (c[0] & _LOW32) | ((c[1] & _LOW32) << np.uint64(32))
    out[:, 2] = (c[2] & _LOW32) | ((c[3] & _LOW32) << np.uint64(32))
    for j in range(5):
        out[:, 3 + j] = c[4 + j]
    return out


_NO_TILES = np.zeros((0, 8), dtype=np.uint64)
_NO_TILES.setflags(write=False)


def _as_tile_rows(tiles):
    if isinstance(tiles, np.ndarray):
        return tiles.astype(np.uint64, copy=False)
    if len(tiles) == 0:
        return _NO_TILES
    rows = np.zeros((len(tiles), 8), dtype=np.uint64)
    for n, t in enumerate(tiles):
        i = (list(t.i) + [0] * 4)[:4]
        a = (list(t.a) + [0] * 5)[:5]
        rows[n] = tile_array(t.kind, *i, *a)[0]
        rows[n, 0] |= np.uint64((t.flags & 0xFF) << 24)
    return rows


class Program:
    def __init__(self):
        self._tiles, self._counts, self._flags, self._marks, self._labels = [], [], [], [], []
        self._edge_from, self._edge_to = [], []   # the DAG's edges in the order they were added
        self.reserved = 0

    def stage(self, tiles=(), link=False, mark=None, label=None):
        """Add a stage; returns its id.  link: its tiles read host memory (gated by
        link credits); mark: value reported to the host when the stage completes."""
        rows = _as_tile_rows(tiles)
        self._tiles.append(rows)
        self._counts.append(len(rows))
        self._flags.append((STAGE_LINK if link else 0) | (STAGE_MARK if mark is not None else 0))
        self._marks.append(mark or 0)
        self._labels.append(label)
        return len(self._tiles) - 1

    def stages(self, n, link=False, label=None):
        """n empty stages (their tiles are written at run time) with consecutive ids; returns the first id."""
        first = len(self._tiles)
        self._tiles.extend([_NO_TILES] * n)
        self._counts.extend([0] * n)
        self._flags.extend([STAGE_LINK if link else 0] * n)
        self._marks.extend([0] * n)
        self._labels.extend([label] * n)
        return first

    def after(self, pred, succ):
        """succ becomes ready only after pred has completed."""
        self._edge_from.append(pred)
        self._edge_to.append(succ)

    def fan_out(self, pred, first, n):
        """pred -> each of the stages first .. first + n - 1."""
        self._edge_from.extend([pred] * n)
        self._edge_to.extend(range(first, first + n))

    def pairwise(self, first_a, first_b, n):
        """first_a + i -> first_b + i for i < n."""
        self._edge_from.extend(range(first_a, first_a + n))
        self._edge_to.extend(range(first_b, first_b + n))

    def fan_in(self, first, n, succ):
        """each of the stages first .. first + n - 1 -> succ."""
        self._edge_from.extend(range(first, first + n))
        self._edge_to.extend([succ] * n)

    def labels(self):
        return list(self._labels) + [("reset", -1)]

    def reserve(self, n):
        """Reserve n tiles that device tiles fill at run time (see dynamic_first)."""
        self.reserved += n

    @property
    def dynamic_first(self):
        return sum(self._counts)

    def pack(self, first, iterations=1, reset_tiles=8):
        """(tiles int64 [n, 8], stages int32 [m, 8], succ int32 [k], first, reset, iterations)."""
        n_user = len(self._tiles)
        reset = n_user
        n_all = n_user + 1
        e_from = np.asarray(self._edge_from, dtype=np.int64)
        e_to = np.asarray(self._edge_to, dtype=np.int64)
        preds_user = np.bincount(e_to, minlength=n_user)
        orphan = np.flatnonzero(preds_user == 0)
        orphan = orphan[orphan != first]
        if orphan.size:
            raise ValueError(f"stage {int(orphan[0])} has no predecessor and is not the first stage, "
                             f"so it would never become ready")
        # every sink gets the reset stage as its only successor; a stage's successors keep the order they were added in
        sinks = np.flatnonzero(np.bincount(e_from, minlength=n_user) == 0)
        e_from = np.concatenate((e_from, sinks))
        e_to = np.concatenate((e_to, np.full(sinks.size, reset, dtype=np.int64)))
        flat = e_to[np.argsort(e_from, kind="stable")]
        n_succ = np.bincount(e_from, minlength=n_all)
        preds = np.concatenate((preds_user, [sinks.size]))
        per = -(-n_all // max(1, reset_tiles))
        zero = [Tile(KIND["zero_runtime"], i=(b, min(n_all, b + per), reset, 0)) for b in range(0, n_all, per)]
        tiles = self._tiles + [_as_tile_rows(zero)]
        flags = self._flags + [STAGE_RESET]
        marks = self._marks + [0]
        # tile blocks in stage order (the dynamic region before the reset stage's), every tile stamped with its stage
        counts = np.asarray(self._counts + [len(zero)], dtype=np.int64)
        firsts = np.concatenate(([0], np.cumsum(counts)[:-1]))
        firsts[reset] += self.reserved
        live = np.flatnonzero(counts)
        blocks = [tiles[sid] for sid in live.tolist()]
        stamp = np.repeat(live.astype(np.uint64), counts[live])
        if self.reserved:   # the dynamic region: zero tiles in front of the reset stage's
            at = int(np.searchsorted(live, reset))
            blocks.insert(at, np.zeros((self.reserved, 8), dtype=np.uint64))
            stamp = np.insert(stamp, int(counts[live[:at]].sum()), np.zeros(self.reserved, dtype=np.uint64))
        packed = np.concatenate(blocks) if blocks else np.zeros((0, 8), dtype=np.uint64)
        packed[:, 0] = (packed[:, 0] & _LOW32) | (stamp << np.uint64(32))
        rows = np.zeros((n_all, 8), dtype=np.int64)
        rows[:, 0], rows[:, 1] = firsts, counts
        rows[:, 2] = np.concatenate(([0], np.cumsum(n_succ)[:-1]))
        rows[:, 3], rows[:, 4], rows[:, 5], rows[:, 6] = n_succ, preds, flags, marks
        succ = torch.from_numpy(flat).to(torch.int32) if flat.size else torch.tensor([0], dtype=torch.int32)
        return (torch.from_numpy(packed.view(np.int64)), torch.from_numpy(rows).to(torch.int32), succ, first, reset,
                iterations)

    def upload(self, fabric, first, iterations=1, reset_tiles=8):
        return fabric.upload(*self.pack(first, iterations, reset_tiles))
