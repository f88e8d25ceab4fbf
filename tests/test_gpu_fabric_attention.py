"""Attention work items inside the persistent fabric (kinds 33 / 34 / 35): the scenarios of the
reference's tests/test_fabric_attention.py:81-168 (prefill over shuffled pages, decode rows,
a chunked prefill) run as a fabric program, mixed with GEMM-free row tiles on the same
workers, against dense torch softmax (absolute error < 2e-2) and against the stand-alone
kernel, whose results the fabric items must reproduce."""
import time

import pytest
import torch

from monoserve_b200.attention import SCALE_LOG2, fabric_maps, fabric_tiles, paged_attention, plan_items
from monoserve_b200.fabric import Fabric, Program
from monoserve_b200.fabric.args import pack
from tests.test_gpu_attention import TOL, dense_reference, make_cache

pytestmark = pytest.mark.gpu


@pytest.fixture
def fab():
    f = Fabric(pool_bytes=128 << 20)
    f.set_max_run(60)
    yield f
    f.stop()
    f.close()


def run(fab, program, first):
    h = program.upload(fab, first=first)
    fab.start()
    fab.publish(map=[0] * fab.num_workers, caps=[0], order=[0], programs=[h])
    t0 = time.time()
    while fab.progress()["lanes"][0]["iterations"] < 1:
        assert time.time() - t0 < 30, fab.progress()["error"]
        time.sleep(1e-3)
    fab.stop()
    assert fab.progress()["error"] == 0


@pytest.mark.parametrize("hq,hkv,page,part_tiles", [(32, 4, 16, None), (12, 4, 64, 4), (96, 8, 16, 4)])
def test_attention_items_in_fabric(fab, hq, hkv, page, part_tiles):
    lens = [300, 777, 1000, 2300, 1300]
    rows = [300, 777, 1, 1, 60]          # two prefills, two decode rows, one chunked prefill
    kc, vc, bt, dense = make_cache(lens, hkv, page, seed=hq + page)
    g = torch.Generator().manual_seed(5)
    T = sum(rows)
    q = torch.randn(T, hq, 128, generator=g).to(torch.bfloat16)
    req_info, row = [], 0
    for n, L in zip(rows, lens):
        req_info.append((row, L - n, n, L))
        row += n
    qd, kcd, vcd, btd = q.cuda(), kc.cuda(), vc.cuda(), bt.cuda()
    out = torch.zeros_like(qd)
    items, merge, ws_rows = plan_items(req_info, hq, hkv, part_tiles=part_tiles)
    assert merge.shape[0] > 0
    ws = torch.zeros(max(ws_rows, 1) * 130, dtype=torch.float32, device="cuda")
    q_map, q_small, k_map, v_map = fabric_maps(fab, qd, kcd, vcd)
    args = torch.frombuffer(bytearray(pack(
        "AttnArgs", q_map=q_map, k_map=k_map, v_map=v_map, out=out, ws_o=ws, ws_m=ws.data_ptr() + ws_rows * 512,
        block_table=btd, scale_log2=SCALE_LOG2, bt_stride=btd.shape[1], hq=hq, hkv=hkv, group=hq // hkv,
        page_size=page, q_map_small=q_small)), dtype=torch.uint8).cuda()
    tiles, merges = fabric_tiles(items, merge, args.data_ptr())
    p = Program()
    s_attn = p.stage(tiles)
    s_merge = p.stage(merges)
    p.after(s_attn, s_merge)
    run(fab, p, s_attn)
    got = out.float().cpu()
    alone = paged_attention(qd, kcd, vcd, btd, req_info, part_tiles=part_tiles).float().cpu()
    assert (got - alone).abs().max().item() < 4e-3
    row = 0
    for r, (n, L) in enumerate(zip(rows, lens)):
        ref = dense_reference(q[row:row + n].float(), dense[r][0], dense[r][1], hq, hkv, L - n)
        assert (got[row:row + n] - ref).abs().max().item() < TOL, r
        row += n


@pytest.mark.parametrize("hq,hkv,chunk_keys", [(32, 4, 0), (32, 4, 1024), (96, 8, 0)])
def test_decode_plan_tile(fab, hq, hkv, chunk_keys):
    """The per-step plan of the decode attention (kind 44): from req_info = {row, position, 1, keys}
    the tile writes one work item per (request, KV head, key range) and the merge tiles of split
    requests into the program's dynamic region; two iterations of the program give the same,
    correct result (the stages are re-planned every iteration)."""
    from monoserve_b200 import _C
    from monoserve_b200.fabric import tile_array
    lens = [3000, 1100, 5000, 700, 129]
    R, page, max_chunks = len(lens), 16, 8
    kc, vc, bt, dense = make_cache(lens, hkv, page, seed=3 + hq)
    g = torch.Generator().manual_seed(9)
    q = torch.randn(R, hq, 128, generator=g).to(torch.bfloat16)
    qd, kcd, vcd, btd = q.cuda(), kc.cuda(), vc.cuda(), bt.cuda()
    out = torch.zeros_like(qd)
    req_info = torch.tensor([(r, L - 1, 1, L) for r, L in enumerate(lens)], dtype=torch.int32).cuda()
    ws_rows = max_chunks * R * hq
    ws = torch.zeros(ws_rows * 130, dtype=torch.float32, device="cuda")
    q_map, q_small, k_map, v_map = fabric_maps(fab, qd, kcd, vcd)
    args = torch.frombuffer(bytearray(pack(
        "AttnArgs", q_map=q_map, k_map=k_map, v_map=v_map, out=out, ws_o=ws, ws_m=ws.data_ptr() + ws_rows * 512,
        block_table=btd, req_info=req_info, scale_log2=SCALE_LOG2, bt_stride=btd.shape[1], hq=hq, hkv=hkv,
        group=hq // hkv, max_chunks=max_chunks, page_size=page, q_map_small=q_small)), dtype=torch.uint8).cuda()
    blob = torch.zeros(_C.struct_layouts()["AttnPlanArgs"][0], dtype=torch.uint8, device="cuda")
    p = Program()
    s_plan = p.stage(tile_array(44, a0=blob.data_ptr()))
    s_attn = p.stage()
    s_merge = p.stage()
    p.after(s_plan, s_attn)
    p.after(s_attn, s_merge)
    dyn = R * hkv * (max_chunks + 1)
    p.reserve(dyn)
    blob.copy_(torch.frombuffer(bytearray(pack(
        "AttnPlanArgs", attn=args.data_ptr(), req_info=req_info.data_ptr(), rows=R, hkv=hkv, chunk_keys=chunk_keys,
        stage_attn=s_attn, stage_comb=s_merge, dyn_first=p.dynamic_first, dyn_cap=dyn, workers=fab.num_workers)),
        dtype=torch.uint8))
    torch.cuda.synchronize()
    h = p.upload(fab, first=s_plan, iterations=2)
    fab.start()
    fab.publish(map=[0] * fab.num_workers, caps=[0], order=[0], programs=[h])
    t0 = time.time()
    while fab.progress()["lanes"][0]["iterations"] < 2:
        assert time.time() - t0 < 30, (fab.progress()["error"], fab.wait_notes())
        time.sleep(1e-3)
    fab.stop()
    assert fab.progress()["error"] == 0
    got = out.float().cpu()
    for r, L in enumerate(lens):
        ref = dense_reference(q[r:r + 1].float(), dense[r][0], dense[r][1], hq, hkv, L - 1)
        assert (got[r:r + 1] - ref).abs().max().item() < TOL, r
