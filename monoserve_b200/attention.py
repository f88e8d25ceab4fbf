"""Paged-KV GQA attention for mixed prefill / decode batches (head_dim 128).

Host mirror of the reference's attention stage (monoserve/runtime/lane.py:423-520
builds, per request, prefill tiles per (q head, 128-row block, KV chunk) and decode
tiles per (KV head, chunk); `req_info` rows are {first query row, position of that
row, query rows, keys visible}).  Here a work item is (request, KV head, block of
query tokens) and the kernel walks all visible keys of the item.
"""
import ctypes
import math

import torch

from monoserve_b200 import _C

SCALE_LOG2 = math.log2(math.e) / math.sqrt(128.0)   # monoserve/runtime/lane.py:238


def build_items(req_info, hq, hkv):
    """req_info: rows of (first query row, position of that row, query rows, keys
    visible), one per request (row index = block-table row).  Returns int32 [n, 8]."""
    group = hq // hkv
    per_block = 128 // group
    items = []
    for req, (row0, pos0, rows, kv_len) in enumerate(req_info):
        for b in range(0, rows, per_block):
            n = min(per_block, rows - b)
            for h in range(hkv):
                items.append([req, h, row0 + b, n, pos0 + b, kv_len, 0, 0])
    return torch.tensor(items, dtype=torch.int32).reshape(-1, 8)


def paged_attention(q, k_cache, v_cache, block_table, req_info, out=None, stream=None):
    """q bf16 [T, hq, 128]; k_cache / v_cache bf16 [pages, page_size, hkv, 128];
    block_table int32 [requests, stride]; req_info as in build_items.  Returns bf16 [T, hq, 128]."""
    T, hq, D = q.shape
    n_pages, page_size, hkv, _ = k_cache.shape
    assert D == 128 and q.dtype == torch.bfloat16 and q.is_cuda and q.is_contiguous()
    assert k_cache.is_contiguous() and v_cache.is_contiguous() and k_cache.shape == v_cache.shape
    assert block_table.dtype == torch.int32 and block_table.is_cuda and block_table.is_contiguous()
    items = build_items(req_info, hq, hkv).cuda()
    if out is None:
        out = torch.empty_like(q)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    st = stream if stream is not None else torch.cuda.current_stream()
    _C.check(_C.lib.monofab_attention(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
                                      block_table.data_ptr(), block_table.shape[1], items.data_ptr(), items.shape[0],
                                      T, hq, hkv, page_size, n_pages, SCALE_LOG2, status.data_ptr(),
                                      ctypes.c_void_p(st.cuda_stream)))
    if int(status.item()):
        raise RuntimeError(f"monofab: attention kernel reported status {int(status.item())}")
    return out
