"""The attention work list (host logic, no GPU): every (request, block of query tokens,
KV head) is covered exactly once over its visible keys, parts start on 128-key
boundaries, and the merge list addresses the workspace rows the parts write."""
import numpy as np

from monoserve_b200.attention import plan_items


def _check(req_info, hq, hkv, part_tiles):
    group = hq // hkv
    items, merge, ws_rows = plan_items(req_info, hq, hkv, part_tiles=part_tiles)
    items, merge = items.numpy(), merge.numpy()
    cover = {}
    used = np.zeros(max(ws_rows, 1), dtype=np.int32)
    for req, h, row0, n, pos0, kv_len, k0, k1, ws, *_ in items:
        assert n * group <= 128 and k0 % 128 == 0
        vis = min(kv_len, pos0 + n)
        if ws < 0:
            assert k0 == 0 and k1 == 0
            cover.setdefault((req, h, row0), []).append((0, vis))
        else:
            assert k1 > k0 and k0 < vis
            cover.setdefault((req, h, row0), []).append((k0, min(k1, vis)))
            used[ws:ws + n * group] += 1
    assert ws_rows == 0 or (used == 1).all()
    for (req, h, row0), spans in cover.items():
        spans.sort()
        assert spans[0][0] == 0
        for a, b in zip(spans, spans[1:]):
            assert a[1] == b[0]
    for row0, n, h, ws, parts, stride, *_ in merge:
        assert parts >= 2 and stride == n * group and ws + parts * stride <= ws_rows
    # every query row of every request appears for every KV head
    for req, (row0, pos0, rows, kv_len) in enumerate(req_info):
        for h in range(hkv):
            got = sorted((r0, n) for (rq, hh, r0), _ in cover.items() if rq == req and hh == h
                         for n in [next(it[3] for it in items if it[0] == req and it[1] == h and it[2] == r0)])
            at = row0
            for r0, n in got:
                assert r0 == at
                at += n
            assert at == row0 + rows
    return items, merge


def test_plan_covers_every_key_once():
    req_info = [(0, 2999, 1, 3000), (1, 99, 1, 100), (2, 0, 700, 700), (702, 4000, 300, 4300)]
    for hq, hkv in [(32, 4), (12, 4), (96, 8)]:
        for part_tiles in [None, 4, 9, 1 << 30]:
            _check(req_info, hq, hkv, part_tiles)


def test_plan_orders_longest_first_and_balances():
    req_info = [(i, 8191, 1, 8192) for i in range(8)]
    items, merge = _check(req_info, 32, 4, None)
    tiles = (np.maximum(np.where(items[:, 7] > 0, items[:, 7], items[:, 5]) - items[:, 6], 0) + 127) // 128
    assert (np.diff(tiles) <= 0).all()
    # 8 x 4 items of 64 tiles over 148 SMs: the plan must produce more items than requests x heads
    assert items.shape[0] > 32 and tiles.max() <= 16
