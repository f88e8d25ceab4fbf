"""Paged-KV GQA attention for mixed prefill / decode batches (head_dim 128).

Host mirror of the reference's attention stage (monoserve/runtime/lane.py:423-520
builds, per request, prefill tiles per (q head, 128-row block, KV chunk) and decode
tiles per (KV head, chunk); `req_info` rows are {first query row, position of that
row, query rows, keys visible}).  Here a work item is (request, KV head, block of
query tokens, key range); long items are split over key ranges for load balance and
merged by a second small kernel.
"""
import ctypes
import math

import torch

from monoserve_b200 import _C

SCALE_LOG2 = math.log2(math.e) / math.sqrt(128.0)   # monoserve/runtime/lane.py:238


SM_COUNT = 148          # CTAs that run at once: one work item per SM
MIN_PART_TILES = 4      # a part shorter than four 128-key tiles is not worth a merge


def plan_items(req_info, hq, hkv, sms=SM_COUNT, part_tiles=None):
    """The work list of one attention call, as the reference's lane builds prefill
    tiles per (block, KV chunk) and decode tiles per (KV head, chunk)
    (monoserve/runtime/lane.py:423-520), with the chunk length chosen for load balance.

    req_info: rows of (first query row, position of that row, query rows, keys visible),
    one per request (row index = block-table row).  Returns (items int32 [n, 12],
    merge int32 [m, 8], workspace rows).  Items are ordered longest first, so that the
    SMs that free up last take the shortest ones.
    """
    group = hq // hkv
    per_block = 128 // group
    blocks = []
    for req, (row0, pos0, rows, kv_len) in enumerate(req_info):
        for b in range(0, rows, per_block):
            n = min(per_block, rows - b)
            kv_end = min(kv_len, pos0 + b + n)
            blocks.append((req, row0 + b, n, pos0 + b, kv_len, -(-max(kv_end, 0) // 128)))
    total = sum(t for *_, t in blocks) * hkv
    if part_tiles is None:
        # aim at two rounds of equally long parts over the SMs
        part_tiles = max(MIN_PART_TILES, -(-total // (2 * sms)))
    items, merge, ws_rows = [], [], 0
    for req, row0, n, pos0, kv_len, tiles in blocks:
        parts = max(1, -(-tiles // part_tiles)) if tiles >= 2 * MIN_PART_TILES else 1
        per_part = -(-tiles // parts)
        parts = -(-tiles // per_part) if tiles else 1
        for h in range(hkv):
            if parts == 1:
                items.append((tiles, [req, h, row0, n, pos0, kv_len, 0, 0, -1, 0, 0, 0]))
                continue
            stride = n * group
            merge.append([row0, n, h, ws_rows, parts, stride, 0, 0])
            for part in range(parts):
                t0, t1 = part * per_part, min(tiles, (part + 1) * per_part)
                items.append((t1 - t0, [req, h, row0, n, pos0, kv_len, t0 * 128, t1 * 128, ws_rows, 0, 0, 0]))
                ws_rows += stride
    items.sort(key=lambda it: -it[0])
    return (torch.tensor([it for _, it in items], dtype=torch.int32).reshape(-1, 12),
            torch.tensor(merge, dtype=torch.int32).reshape(-1, 8), ws_rows)


def build_items(req_info, hq, hkv):
    """The unsplit work list: one item per (request, block of query tokens, KV head)."""
    return plan_items(req_info, hq, hkv, part_tiles=1 << 30)[0]


class AttentionPlan:
    """The work list of one batch shape, planned once and kept on the device with its
    split workspace; `run` only launches.  (The reference's lane rebuilds its attention
    tiles per step on the host too: monoserve/runtime/lane.py:423-520.)"""

    def __init__(self, req_info, hq, hkv, split=True, part_tiles=None, device="cuda"):
        self.hq, self.hkv = hq, hkv
        items, merge, self.ws_rows = plan_items(req_info, hq, hkv, part_tiles=part_tiles if split else 1 << 30)
        self.items, self.merge = items.to(device), merge.to(device)
        self.ws = torch.empty(self.ws_rows * 130, dtype=torch.float32, device=device) if self.ws_rows else None
        self.status = torch.zeros(1, dtype=torch.int32, device=device)

    def run(self, q, k_cache, v_cache, block_table, out=None, stream=None, check=True):
        T, hq, D = q.shape
        n_pages, page_size, hkv, _ = k_cache.shape
        assert D == 128 and (hq, hkv) == (self.hq, self.hkv)
        assert q.dtype == torch.bfloat16 and q.is_cuda and q.is_contiguous()
        assert k_cache.is_contiguous() and v_cache.is_contiguous() and k_cache.shape == v_cache.shape
        assert block_table.dtype == torch.int32 and block_table.is_cuda and block_table.is_contiguous()
        if out is None:
            out = torch.empty_like(q)
        st = stream if stream is not None else torch.cuda.current_stream()
        _C.check(_C.lib.monofab_attention(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
                                          block_table.data_ptr(), block_table.shape[1], self.items.data_ptr(),
                                          self.items.shape[0], T, hq, hkv, page_size, n_pages, SCALE_LOG2,
                                          self.ws.data_ptr() if self.ws is not None else None, self.ws_rows,
                                          self.merge.data_ptr() if self.merge.shape[0] else None, self.merge.shape[0],
                                          self.status.data_ptr(), ctypes.c_void_p(st.cuda_stream)))
        if check and int(self.status.item()):
            raise RuntimeError(f"monofab: attention kernel reported status {int(self.status.item())}")
        return out


def paged_attention(q, k_cache, v_cache, block_table, req_info, out=None, stream=None, split=True, part_tiles=None):
    """q bf16 [T, hq, 128]; k_cache / v_cache bf16 [pages, page_size, hkv, 128];
    block_table int32 [requests, stride]; req_info as in plan_items.  split=False keeps
    every (request, block, KV head) in one work item.  Returns bf16 [T, hq, 128]."""
    plan = AttentionPlan(req_info, q.shape[1], k_cache.shape[2], split=split, part_tiles=part_tiles)
    return plan.run(q, k_cache, v_cache, block_table, out=out, stream=stream)


K_ATTN_PREFILL, K_ATTN_DECODE, K_ATTN_MERGE = 33, 34, 35


def fabric_maps(fab, q, k_cache, v_cache):
    """Tensor maps of q and the paged caches in a fabric's table: (q_map, q_map_small or 0, k_map, v_map)."""
    T, hq, _ = q.shape
    n_pages, page, hkv, _ = k_cache.shape
    group = hq // hkv
    dims, strides = [128, hq, T], [256, hq * 256]
    q_map = fab.tensor_map(q.data_ptr(), dims, strides, [64, group, 128 // group])
    q_small = fab.tensor_map(q.data_ptr(), dims, strides, [64, group, 32 // group]) if 32 % group == 0 else 0
    # one box = one page's keys of one KV head, both halves of the head dimension, in groups of eight keys
    row = hkv * 256
    kd, ks, kb = [64, 8, 2 * hkv, page // 8, n_pages], [row, 128, 8 * row, page * row], [64, 8, 2, page // 8, 1]
    return q_map, q_small, fab.tensor_map(k_cache.data_ptr(), kd, ks, kb), fab.tensor_map(v_cache.data_ptr(), kd, ks, kb)


def fabric_tiles(items, merge, args_ptr, kind=K_ATTN_PREFILL):
    """The work list of plan_items as fabric tiles: (attention item tiles, merge tiles), each a
    uint64 [n, 8] array.  Tile fields: see make_attn_work / tile_attn_merge in csrc/fabric_seq_tiles.cuh."""
    import numpy as np
    from monoserve_b200.fabric import tile_array
    it = items.numpy().astype(np.int64).reshape(-1, 12)
    tiles = tile_array(kind, i0=it[:, 2], i1=it[:, 3] | (it[:, 1] << 16), i2=it[:, 6], i3=np.maximum(it[:, 7], 0),
                       a0=args_ptr, a1=it[:, 0] | ((it[:, 8] + 1) << 32), a2=it[:, 4] | (it[:, 5] << 32))
    mg = merge.numpy().astype(np.int64).reshape(-1, 8)
    merges = tile_array(K_ATTN_MERGE, i0=mg[:, 0], i1=mg[:, 1] | (mg[:, 2] << 16), i2=mg[:, 3],
                        i3=mg[:, 4] | (mg[:, 5] << 16), a0=args_ptr)
    return tiles, merges
