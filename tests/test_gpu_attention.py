"""Paged-KV GQA attention against dense torch softmax: the scenarios of the
reference's tests/test_fabric_attention.py:81-168 (prefill with (hq, hkv) in
{(32, 4), (12, 4)}, lengths 300 / 777, shuffled pages; decode lengths 100 / 513 /
1000), with the page size as a parameter (16 and 64) and the GLM head layout (96, 8).
Tolerance: the reference's, absolute error < 2e-2."""
import pytest
import torch

from oracle import torch_path as tp

pytestmark = pytest.mark.gpu
TOL = 2e-2


def make_cache(lens, hkv, page, seed):
    """Shuffled pages; returns k_cache, v_cache [pages, page, hkv, 128], block table, dense k/v per request."""
    g = torch.Generator().manual_seed(seed)
    need = [-(-n // page) for n in lens]
    n_pages = sum(need) + 3
    perm = torch.randperm(n_pages - 1, generator=g) + 1      # page 0 stays a sink
    kc = torch.randn(n_pages, page, hkv, 128, generator=g).to(torch.bfloat16)
    vc = torch.randn(n_pages, page, hkv, 128, generator=g).to(torch.bfloat16)
    bt = torch.zeros(len(lens), max(need), dtype=torch.int32)
    dense = []
    at = 0
    for r, n in enumerate(lens):
        pages = perm[at:at + need[r]]
        at += need[r]
        bt[r, :need[r]] = pages.to(torch.int32)
        k = kc[pages].reshape(-1, hkv, 128)[:n]
        v = vc[pages].reshape(-1, hkv, 128)[:n]
        dense.append((k.float(), v.float()))
    return kc, vc, bt, dense


def dense_reference(q, k, v, hq, hkv, pos0):
    """q [n, hq, 128] at positions pos0 .. pos0 + n - 1 over keys 0 .. len(k) - 1 (causal)."""
    n, L = q.shape[0], k.shape[0]
    kk, vv = k.repeat_interleave(hq // hkv, 1), v.repeat_interleave(hq // hkv, 1)
    s = torch.einsum("qhd,khd->hqk", q, kk) / 128 ** 0.5
    qpos = pos0 + torch.arange(n)
    mask = torch.arange(L)[None, :] > qpos[:, None]
    s = s.masked_fill(mask[None], float("-inf"))
    return tp.bf(torch.einsum("hqk,khd->qhd", s.softmax(-1), vv))


@pytest.mark.parametrize("page", [16, 64])
@pytest.mark.parametrize("hq,hkv", [(32, 4), (12, 4), (96, 8)])
def test_prefill(hq, hkv, page):
    from monoserve_b200.attention import paged_attention
    lens = [300, 777]
    kc, vc, bt, dense = make_cache(lens, hkv, page, seed=hq + page)
    g = torch.Generator().manual_seed(1)
    T = sum(lens)
    q = torch.randn(T, hq, 128, generator=g).to(torch.bfloat16)
    req_info, row = [], 0
    for n in lens:
        req_info.append((row, 0, n, n))
        row += n
    out = paged_attention(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), req_info).float().cpu()
    row = 0
    for r, n in enumerate(lens):
        ref = dense_reference(q[row:row + n].float(), dense[r][0], dense[r][1], hq, hkv, 0)
        err = (out[row:row + n] - ref).abs().max().item()
        assert err < TOL, (r, err)
        row += n


@pytest.mark.parametrize("page", [16, 64])
@pytest.mark.parametrize("hq,hkv", [(32, 4), (96, 8)])
def test_decode_and_chunked_prefill(hq, hkv, page):
    """Decode rows (one query token at the end of contexts of 100 / 513 / 1000 keys) mixed
    with a prefill chunk that continues a request at position 200."""
    from monoserve_b200.attention import paged_attention
    lens = [100, 513, 1000, 260]
    kc, vc, bt, dense = make_cache(lens, hkv, page, seed=7 + page)
    g = torch.Generator().manual_seed(2)
    rows = [1, 1, 1, 60]                      # the last request prefills positions 200 .. 259
    T = sum(rows)
    q = torch.randn(T, hq, 128, generator=g).to(torch.bfloat16)
    req_info, row = [], 0
    for n, L in zip(rows, lens):
        req_info.append((row, L - n, n, L))
        row += n
    out = paged_attention(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), req_info).float().cpu()
    row = 0
    for r, (n, L) in enumerate(zip(rows, lens)):
        ref = dense_reference(q[row:row + n].float(), dense[r][0], dense[r][1], hq, hkv, L - n)
        err = (out[row:row + n] - ref).abs().max().item()
        assert err < TOL, (r, err)
        row += n


def test_attention_rejects_bad_shapes():
    from monoserve_b200 import _C
    z = torch.zeros(8, device="cuda", dtype=torch.int32)
    rc = _C.lib.monofab_attention(z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), 1, z.data_ptr(),
                                  1, 1, 12, 5, 16, 1, 1.0, None, 0, None, 0, z.data_ptr(), None)
    assert rc == -1 and b"multiple of hkv" in _C.lib.monofab_last_error()
    rc = _C.lib.monofab_attention(z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), 1, z.data_ptr(),
                                  1, 1, 8, 4, 24, 1, 1.0, None, 0, None, 0, z.data_ptr(), None)
    assert rc == -1 and b"page_size" in _C.lib.monofab_last_error()
    rc = _C.lib.monofab_attention(z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), 1, z.data_ptr(),
                                  1, 1, 8, 4, 16, 1, 1.0, None, 0, z.data_ptr(), 1, z.data_ptr(), None)
    assert rc == -1 and b"workspace" in _C.lib.monofab_last_error()


@pytest.mark.parametrize("hq,hkv", [(32, 4), (12, 4), (96, 8)])
@pytest.mark.parametrize("part_tiles", [4, 7])
def test_split_kv_matches_dense_and_unsplit(hq, hkv, part_tiles):
    """Long contexts split over key ranges and merged: decode rows of 3000 / 1100 / 5000 keys
    (quad-replicated items where the group divides 32) and a 300-token prefill chunk at the
    end of a 2300-key request.  The split result must agree with dense softmax and, to
    rounding of the merge, with the unsplit run of the same kernel."""
    from monoserve_b200.attention import paged_attention, plan_items
    lens = [3000, 1100, 5000, 2300]
    rows = [1, 1, 1, 300]
    kc, vc, bt, dense = make_cache(lens, hkv, 16, seed=11 + hq)
    g = torch.Generator().manual_seed(3)
    q = torch.randn(sum(rows), hq, 128, generator=g).to(torch.bfloat16)
    req_info, row = [], 0
    for n, L in zip(rows, lens):
        req_info.append((row, L - n, n, L))
        row += n
    items, merge, ws_rows = plan_items(req_info, hq, hkv, part_tiles=part_tiles)
    assert merge.shape[0] > 0 and ws_rows > 0 and (items[:, 8] >= 0).sum() > merge.shape[0]
    args = (q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), req_info)
    out = paged_attention(*args, part_tiles=part_tiles).float().cpu()
    whole = paged_attention(*args, split=False).float().cpu()
    assert (out - whole).abs().max().item() < 4e-3
    row = 0
    for r, (n, L) in enumerate(zip(rows, lens)):
        ref = dense_reference(q[row:row + n].float(), dense[r][0], dense[r][1], hq, hkv, L - n)
        assert (out[row:row + n] - ref).abs().max().item() < TOL, r
        assert (whole[row:row + n] - ref).abs().max().item() < TOL, r
        row += n


@pytest.mark.parametrize("hq,hkv,lens,prompt", [(32, 4, [8192, 512, 6000], 2048), (96, 8, [16384, 1024], 4096)])
def test_full_size_contexts(hq, hkv, lens, prompt):
    """The context lengths and head layouts of the full-model benchmark configurations, page size
    16: decode rows at the longest contexts (8192 keys with 32 / 4 heads, 16384 with 96 / 8) and
    a whole prompt (2048 / 4096 tokens), planned as the benchmark plans them (split over key
    ranges, merged).  Prompt rows are checked on a sample of query blocks to bound the CPU time."""
    from monoserve_b200.attention import paged_attention
    all_lens = lens + [prompt]
    rows = [1] * len(lens) + [prompt]
    kc, vc, bt, dense = make_cache(all_lens, hkv, 16, seed=hq + 5)
    g = torch.Generator().manual_seed(4)
    q = torch.randn(sum(rows), hq, 128, generator=g).to(torch.bfloat16)
    req_info, row = [], 0
    for n, L in zip(rows, all_lens):
        req_info.append((row, L - n, n, L))
        row += n
    out = paged_attention(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), req_info).float().cpu()
    row = 0
    for r, (n, L) in enumerate(zip(rows, all_lens)):
        if n == 1:
            ref = dense_reference(q[row:row + 1].float(), dense[r][0], dense[r][1], hq, hkv, L - 1)
            assert (out[row:row + 1] - ref).abs().max().item() < TOL, r
        else:
            for lo in (0, n // 2 - 64, n - 128):     # first, middle and last query blocks of the prompt
                ref = dense_reference(q[row + lo:row + lo + 128].float(), dense[r][0][:lo + 128], dense[r][1][:lo + 128],
                                      hq, hkv, lo)
                assert (out[row + lo:row + lo + 128] - ref).abs().max().item() < TOL, (r, lo)
        row += n


def test_many_items_per_cta_mixed_kinds():
    """The kernel is persistent: with far more work items than SMs every CTA works through a chain of items,
    decode items (quad-replicated rows, merged through shared memory) and prefill blocks in turn, while its
    producer already loads the next item.  240 decode rows with contexts of 17 .. 700 keys and two prompts of
    300 and 150 tokens: about 1000 items on 148 CTAs."""
    from monoserve_b200.attention import paged_attention
    hq, hkv, page = 32, 4, 16
    g = torch.Generator().manual_seed(11)
    lens = torch.randint(17, 701, (240,), generator=g).tolist() + [300, 150]
    rows = [1] * 240 + [300, 150]
    kc, vc, bt, dense = make_cache(lens, hkv, page, seed=5)
    T = sum(rows)
    q = torch.randn(T, hq, 128, generator=g).to(torch.bfloat16)
    req_info, row = [], 0
    for n, L in zip(rows, lens):
        req_info.append((row, L - n, n, L))
        row += n
    out = paged_attention(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), req_info).float().cpu()
    row = 0
    for r, (n, L) in enumerate(zip(rows, lens)):
        ref = dense_reference(q[row:row + n].float(), dense[r][0], dense[r][1], hq, hkv, L - n)
        err = (out[row:row + n] - ref).abs().max().item()
        assert err < TOL, (r, err)
        row += n
