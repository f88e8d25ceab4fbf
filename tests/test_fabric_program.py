"""Program packing (CPU): the wire format, the reset stage, and the position of
the dynamic region (the reference pins it in tests/test_fabric_core.py:222-239)."""
import numpy as np
import pytest

from monoserve_b200.fabric.program import KIND, STAGE_LINK, STAGE_MARK, STAGE_RESET, Program, Tile, tile_array


def test_dynamic_region_precedes_reset_tiles():
    p = Program()
    a = p.stage([Tile(KIND["nop"])] * 3)
    b = p.stage()
    p.after(a, b)
    p.reserve(5)
    dyn = p.dynamic_first
    tiles, stages, _, _, reset, _ = p.pack(a, iterations=4)
    st = stages.numpy()
    r_first, r_count = int(st[reset, 0]), int(st[reset, 1])
    assert dyn == 3 and r_count > 0
    assert r_first >= dyn + 5
    assert tiles.shape[0] == r_first + r_count
    kinds = tiles.numpy()[r_first:r_first + r_count, 0] & 0xFFFF
    assert (kinds == KIND["zero_runtime"]).all()


def test_wire_format_and_reset_stage():
    p = Program()
    s0 = p.stage([Tile(7, i=(1, 2, 3, 4), a=(10, 11, 12, 13, 14), flags=5)], mark=9)
    s1 = p.stage(tile_array(33, i0=np.arange(4), a0=100), link=True)
    s2 = p.stage([Tile(KIND["nop"])])
    p.after(s0, s1)
    p.after(s0, s2)
    tiles, stages, succ, first, reset, it = p.pack(s0, iterations=2, reset_tiles=2)
    t, st = tiles.numpy().view(np.uint64), stages.numpy()
    assert (first, reset, it) == (0, 3, 2) and st.shape == (4, 8)
    w0 = int(t[0, 0])
    assert w0 & 0xFFFF == 7 and (w0 >> 24) & 0xFF == 5 and w0 >> 32 == 0
    assert int(t[0, 1]) == 1 | (2 << 32) and int(t[0, 2]) == 3 | (4 << 32) and t[0, 3:8].tolist() == [10, 11, 12, 13, 14]
    assert [int(x) >> 32 for x in t[1:5, 0]] == [1] * 4 and [int(x) & 0xFFFFFFFF for x in t[1:5, 1]] == [0, 1, 2, 3]
    assert st[0].tolist()[:7] == [0, 1, 0, 2, 0, STAGE_MARK, 9]
    assert st[1].tolist()[:7] == [1, 4, 2, 1, 1, STAGE_LINK, 0]       # a sink: its only successor is the reset stage
    assert st[2].tolist()[:7] == [5, 1, 3, 1, 1, 0, 0]
    assert st[3, 4] == 2 and st[3, 5] == STAGE_RESET and st[3, 1] == 2  # waits for both sinks; two re-arm tiles
    assert succ.tolist() == [1, 2, 3, 3]
    z = t[6:8]
    assert [(int(r[1]) & 0xFFFFFFFF, int(r[1]) >> 32, int(r[2]) & 0xFFFFFFFF) for r in z] == [(0, 2, 3), (2, 4, 3)]


def test_unreachable_stage_is_rejected():
    p = Program()
    p.stage([Tile(KIND["nop"])])
    p.stage([Tile(KIND["nop"])])
    with pytest.raises(ValueError, match="never become ready"):
        p.pack(0)


def test_pack_matches_the_reference_builder():
    """Fixture: the same programs packed by the reference's monoserve/fabric/program.py
    (tests/golden/make_golden.py:program_fixture)."""
    import importlib.util
    import os
    gold = os.path.join(os.path.dirname(__file__), "golden")
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(gold, "make_golden.py"))
    mg = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mg)
    import monoserve_b200.fabric.program as mine
    g = np.load(os.path.join(gold, "program_pack_reference.npz"))
    for name, (tiles, stages, succ, first, reset, it) in mg.program_spec(mine).items():
        assert np.array_equal(tiles.numpy(), g[name + "_tiles"]), name
        assert np.array_equal(stages.numpy(), g[name + "_stages"]), name
        assert np.array_equal(succ.numpy(), g[name + "_succ"]), name
        assert [first, reset, it] == g[name + "_meta"].tolist()


def test_bulk_stage_calls_build_the_same_program():
    """stages / fan_out / pairwise / fan_in (what a lane uses for a layer's 2 x E expert stages) against the
    same DAG built stage by stage."""
    one, bulk = Program(), Program()
    a = one.stage([Tile(KIND["nop"])])
    w = [one.stage() for _ in range(5)]
    v = [one.stage(link=True) for _ in range(5)]
    c = one.stage([Tile(KIND["nop"])], mark=3)
    for e in range(5):
        one.after(a, w[e])
        one.after(w[e], v[e])
        one.after(v[e], c)
    a2 = bulk.stage([Tile(KIND["nop"])])
    w0, v0 = bulk.stages(5), bulk.stages(5, link=True)
    c2 = bulk.stage([Tile(KIND["nop"])], mark=3)
    bulk.fan_out(a2, w0, 5)
    bulk.pairwise(w0, v0, 5)
    bulk.fan_in(v0, 5, c2)
    for x, y in zip(one.pack(a), bulk.pack(a2)):
        if hasattr(x, "numpy"):
            assert x.dtype == y.dtype and (x.numpy() == y.numpy()).all()
        else:
            assert x == y
