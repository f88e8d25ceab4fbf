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
