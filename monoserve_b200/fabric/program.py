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


def tile_array(kind, i0=0, i1=0, i2=0, i3=0, a0=0, a1=0, a2=0, a3=0, a4=0):
    """(n, 8) uint64 tiles from broadcastable operand arrays."""
    ops = np.broadcast_arrays(*[np.asarray(v, dtype=np.int64) for v in (i0, i1, i2, i3, a0, a1, a2, a3, a4)])
    cols = [np.ascontiguousarray(o).reshape(-1).astype(np.uint64) for o in ops]
    out = np.zeros((cols[0].size, 8), dtype=np.uint64)
    out[:, 0] = np.uint64(kind & 0xFFFF)
    out[:, 1] = (cols[0] & _LOW32) | ((cols[1] & _LOW32) << np.uint64(32))
    out[:, 2] = (cols[2] & _LOW32) | ((cols[3] & _LOW32) << np.uint64(32))
    out[:, 3:8] = np.stack(cols[4:9], axis=1)
    return out


def _as_tile_rows(tiles):
    if isinstance(tiles, np.ndarray):
        return tiles.astype(np.uint64, copy=False)
    rows = np.zeros((len(tiles), 8), dtype=np.uint64)
    for n, t in enumerate(tiles):
        i = (list(t.i) + [0] * 4)[:4]
        a = (list(t.a) + [0] * 5)[:5]
        rows[n] = tile_array(t.kind, *i, *a)[0]
        rows[n, 0] |= np.uint64((t.flags & 0xFF) << 24)
    return rows


class Program:
    def __init__(self):
        self._tiles, self._flags, self._marks, self._succ, self._preds, self._labels = [], [], [], [], [], []
        self.reserved = 0

    def stage(self, tiles=(), link=False, mark=None, label=None):
        """Add a stage; returns its id.  link: its tiles read host memory (gated by
        link credits); mark: value reported to the host when the stage completes."""
        self._tiles.append(_as_tile_rows(tiles))
        self._flags.append((STAGE_LINK if link else 0) | (STAGE_MARK if mark is not None else 0))
        self._marks.append(mark or 0)
        self._succ.append([])
        self._preds.append(0)
        self._labels.append(label)
        return len(self._tiles) - 1

    def labels(self):
        return list(self._labels) + [("reset", -1)]

    def after(self, pred, succ):
        """succ becomes ready only after pred has completed."""
        self._succ[pred].append(succ)
        self._preds[succ] += 1

    def reserve(self, n):
        """Reserve n tiles that device tiles fill at run time (see dynamic_first)."""
        self.reserved += n

    @property
    def dynamic_first(self):
        return sum(len(t) for t in self._tiles)

    def pack(self, first, iterations=1, reset_tiles=8):
        """(tiles int64 [n, 8], stages int32 [m, 8], succ int32 [k], first, reset, iterations)."""
        n_user = len(self._tiles)
        for sid in range(n_user):
            if sid != first and self._preds[sid] == 0:
                raise ValueError(f"stage {sid} has no predecessor and is not the first stage, "
                                 f"so it would never become ready")
        reset = n_user
        n_all = n_user + 1
        sinks = [s for s in range(n_user) if not self._succ[s]]
        per = -(-n_all // max(1, reset_tiles))
        zero = [Tile(KIND["zero_runtime"], i=(b, min(n_all, b + per), reset, 0)) for b in range(0, n_all, per)]
        tiles = self._tiles + [_as_tile_rows(zero)]
        flags = self._flags + [STAGE_RESET]
        marks = self._marks + [0]
        preds = self._preds + [len(sinks)]
        succ = [list(s) for s in self._succ] + [[]]
        for s in sinks:
            succ[s].append(reset)
        blocks, rows, flat = [], [], []
        at = 0
        for sid, t in enumerate(tiles):
            if sid == reset and self.reserved:
                blocks.append(np.zeros((self.reserved, 8), dtype=np.uint64))   # the dynamic region
                at += self.reserved
            t = t.copy()
            if len(t):
                t[:, 0] = (t[:, 0] & _LOW32) | (np.uint64(sid) << np.uint64(32))
            blocks.append(t)
            rows.append([at, len(t), len(flat), len(succ[sid]), preds[sid], flags[sid], marks[sid], 0])
            flat.extend(succ[sid])
            at += len(t)
        packed = np.concatenate(blocks) if blocks else np.zeros((0, 8), dtype=np.uint64)
        return (torch.from_numpy(packed.view(np.int64).copy()), torch.tensor(rows, dtype=torch.int64).to(torch.int32),
                torch.tensor(flat if flat else [0], dtype=torch.int32), first, reset, iterations)

    def upload(self, fabric, first, iterations=1, reset_tiles=8):
        return fabric.upload(*self.pack(first, iterations, reset_tiles))
