"""Host-side pieces of the decoder lanes that need no GPU: the rotary table the qk_rope tile reads must
hold exactly the cos / sin values the reference's oracle computes, for full and partial rotary."""
import torch

from oracle import torch_path as tp


def test_rope_table_matches_oracle_rope():
    from monoserve_b200.model import rope_table
    g = torch.Generator().manual_seed(0)
    for theta, rot in [(1e6, 128), (1e4, 64)]:
        table = rope_table(theta, rot, 300)              # [pos][rot / 2][cos, sin]
        x = torch.randn(7, 3, 128, generator=g)
        pos = torch.tensor([0, 1, 5, 17, 64, 255, 299])
        half = rot // 2
        c, s = table[pos, :, 0][:, None, :], table[pos, :, 1][:, None, :]
        x1, x2 = x[..., :half], x[..., half:rot]
        mine = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s, x[..., rot:]], -1)
        assert torch.equal(mine, tp.rope(x, pos, theta, rot))


def test_logits_tiles_cover_rows_and_experts_once():
    import numpy as np
    from monoserve_b200.lane import LOGIT_EXPERTS, LOGIT_ROWS, logits_tiles
    for T, E in [(1, 16), (37, 128), (256, 160)]:
        tiles = logits_tiles(0x1000, T, E)
        seen = np.zeros((T, E), dtype=np.int32)
        for t in tiles:
            r0, rows = int(t[1] & 0xffffffff), int(t[1] >> 32)
            e0, ne = int(t[2] & 0xffffffff), int(t[2] >> 32)
            assert rows <= LOGIT_ROWS and ne <= LOGIT_EXPERTS and int(t[0] & 0xffff) == 48
            seen[r0:r0 + rows, e0:e0 + ne] += 1
        assert (seen == 1).all()


def test_rows_per_tile_keep_a_stage_to_whole_rounds():
    """The lane picks the rows per tile of its row-wise stages so that a stage does not spill a few tiles into
    another round over the workers, and the router projection's tile height by rounds x rows; every choice must
    still cover all rows (the tile builder takes care of the last, shorter tile)."""
    import types
    import numpy as np
    from monoserve_b200.lane import logits_tiles
    from monoserve_b200.model import ModelLane, _retarget
    lane = types.SimpleNamespace(fab=types.SimpleNamespace(num_workers=148))
    for T in (1, 8, 148, 149, 300, 592, 593, 4096):
        per = ModelLane._per(lane, T)
        tiles = -(-T // per)
        assert per >= 1 and (tiles <= 148 or per % 4 == 0)
        assert tiles <= 148 or tiles <= 2 * 148 + 148          # beyond one round: about two
        rows = ModelLane._logit_rows(lane, T, 128)
        assert 8 <= rows <= 32
        seen = np.zeros((T, 128), dtype=np.int32)
        for t in logits_tiles(0, T, 128, rows=rows):
            r0, n = int(t[1] & 0xffffffff), int(t[1] >> 32)
            e0, ne = int(t[2] & 0xffffffff), int(t[2] >> 32)
            seen[r0:r0 + n, e0:e0 + ne] += 1
        assert (seen == 1).all()
    assert ModelLane._per(lane, 300) == 3 and ModelLane._logit_rows(lane, 300, 128) == 18   # 100 and 136 tiles
    a = logits_tiles(777, 20, 128)
    assert (a == _retarget(logits_tiles(0, 20, 128), a0=777)).all()   # a template re-addressed = built with the address


def test_operand_arena_batches_its_writes():
    """A build puts hundreds of operand blocks; they reach the device in one write per flush, blocks put earlier in
    the build can still be patched, and a block of an earlier build cannot."""
    import pytest
    from monoserve_b200.model import _Arena

    class FakeFabric:
        def __init__(self):
            self.writes = []

        def write(self, dst, data):
            self.writes.append((dst, bytes(data)))

    arena = _Arena.__new__(_Arena)            # no device buffer here: only the bookkeeping is under test
    arena.fab, arena.at, arena.flushed, arena.host = FakeFabric(), 0, 0, bytearray(4096)
    arena.buf = type("Buf", (), {"data_ptr": lambda self: 0x10000, "numel": lambda self: 4096})()
    a = arena.put(b"\x01" * 100)
    b = arena.put(b"\x02" * 300)
    assert (a.data_ptr(), b.data_ptr()) == (0x10000, 0x10000 + 256) and arena.fab.writes == []
    arena.patch(a, b"\x07" * 100)
    arena.flush()
    (dst, data), = arena.fab.writes
    assert dst == 0x10000 and len(data) == 256 + 512 and data[:100] == b"\x07" * 100 and data[256:556] == b"\x02" * 300
    c = arena.put(b"\x03" * 16)
    with pytest.raises(AssertionError):
        arena.patch(a, b"\x00")               # already flushed: the device copy would not follow
    arena.flush()
    assert arena.fab.writes[1] == (0x10000 + 768, b"\x03" * 16 + bytes(240))
    arena.flush()
    assert len(arena.fab.writes) == 2         # nothing new, nothing written
    with pytest.raises(RuntimeError):
        arena.put(bytes(4096))
    arena.reset()
    assert arena.put(b"x").data_ptr() == 0x10000 and c.data_ptr() == 0x10000 + 768
