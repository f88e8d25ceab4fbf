"""The sequence-path tiles of the fabric one by one against torch: q/k head norm + rotary embedding +
KV append (kind 37; full and partial rotary, with and without the head norm), token embedding with the
first norm and the decode step's bookkeeping (kind 42), and next-token selection (kind 43: arg-max with the
lowest index on ties, and Gumbel-max sampling that is a pure function of seed, slot and step)."""
import time

import pytest
import torch

from monoserve_b200.fabric import Fabric, Program, Tile, tile_array
from monoserve_b200.fabric.args import pack
from monoserve_b200.model import rope_table
from oracle import torch_path as tp

pytestmark = pytest.mark.gpu


def block(name, **fields):
    return torch.frombuffer(bytearray(pack(name, **fields)), dtype=torch.uint8).cuda()


@pytest.fixture
def fab():
    f = Fabric(pool_bytes=64 << 20)
    f.set_max_run(60)
    yield f
    f.stop()
    f.close()


def run(fab, p, first):
    h = p.upload(fab, first=first)
    fab.start()
    fab.publish(map=[0] * fab.num_workers, caps=[0], order=[0], programs=[h])
    t0 = time.time()
    while fab.progress()["lanes"][0]["iterations"] < 1:
        assert time.time() - t0 < 30, fab.progress()["error"]
        time.sleep(1e-3)
    fab.stop()
    assert fab.progress()["error"] == 0


@pytest.mark.parametrize("rot,norm", [(128, True), (64, False), (64, True)])
def test_qk_rope_tile(fab, rot, norm):
    """tests/test_fabric_model.py:52-59 (Qwen: head norm, full rotary) and the GLM variant (no head norm,
    rotary on half of the head): q to its buffer, k and v to the paged caches at the rows' slots."""
    T, hq, hkv, page, theta, eps = 37, 8, 2, 16, 1e4, 1e-6
    g = torch.Generator().manual_seed(rot + norm)
    heads = hq + 2 * hkv
    qkv = torch.randn(T, heads * 128, generator=g).to(torch.bfloat16)
    qn = (1 + 0.1 * torch.randn(128, generator=g)).to(torch.bfloat16)
    kn = (1 + 0.1 * torch.randn(128, generator=g)).to(torch.bfloat16)
    pos = torch.randint(0, 200, (T,), generator=g).to(torch.int32)
    slot = (torch.randperm(20 * page, generator=g)[:T] + page).to(torch.int32)   # distinct cache rows, page 0 unused
    q_out = torch.zeros(T, hq, 128, dtype=torch.bfloat16, device="cuda")
    kc = torch.zeros(24, page, hkv, 128, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    cs = rope_table(theta, rot, 256).cuda()
    qd, qnd, knd, posd, slotd = qkv.cuda(), qn.cuda(), kn.cuda(), pos.cuda(), slot.cuda()
    args = block("QkArgs", qkv=qd, q_out=q_out, k_cache=kc, v_cache=vc, q_norm=qnd if norm else 0, k_norm=knd if norm else 0,
                 tok_pos=posd, tok_slot=slotd, cos_sin=cs, ld_qkv=heads * 128, hq=hq, hkv=hkv, rot_dim=rot, theta=theta,
                 eps=eps, max_pos=256)
    items = T * heads
    p = Program()
    s = p.stage(tile_array(37, i0=torch.arange(0, items, 48).numpy(),
                           i1=[min(48, items - i) for i in range(0, items, 48)], a0=args.data_ptr()))
    run(fab, p, s)
    x = qkv.float().view(T, heads, 128)
    q, k, v = x[:, :hq], x[:, hq:hq + hkv], x[:, hq + hkv:]
    if norm:
        q = tp.bf(q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True) + eps)) * qn.float()
        k = tp.bf(k * torch.rsqrt(k.pow(2).mean(-1, keepdim=True) + eps)) * kn.float()
    q_ref, k_ref = tp.bf(tp.rope(q, pos, theta, rot)), tp.bf(tp.rope(k, pos, theta, rot))
    got_q = q_out.float().cpu()
    got_k = kc.view(-1, hkv, 128)[slot.long().cuda()].float().cpu()
    got_v = vc.view(-1, hkv, 128)[slot.long().cuda()].float().cpu()
    # one bf16 ulp of slack: the row sum of squares is added in a different order than torch's mean
    assert (got_q - q_ref).abs().max().item() <= 2 ** -6 * q_ref.abs().max().item()
    assert (got_k - k_ref).abs().max().item() <= 2 ** -6 * k_ref.abs().max().item()
    assert float((got_q - q_ref).norm() / q_ref.norm()) < 2e-3
    assert torch.equal(got_v, v)
    untouched = torch.ones(24 * page, dtype=torch.bool)
    untouched[slot.long()] = False
    assert float(kc.view(-1, hkv * 128)[untouched.cuda()].abs().max()) == 0.0


def test_embed_tile_prefill_and_decode(fab):
    """Kind 42: x = embed[token], out = rmsnorm(x) * w; decode rows take the request's last token, advance its
    length and write position, cache slot and req_info (csrc/fabric/tiles/aux.cuh:199-218 with the page size
    a parameter)."""
    V, H, S, page, stride, eps = 300, 512, 6, 16, 5, 1e-6
    g = torch.Generator().manual_seed(4)
    embed = torch.randn(V, H, generator=g).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(H, generator=g)).to(torch.bfloat16)
    tokens = torch.randint(0, V, (21,), generator=g).to(torch.int32)
    ed, wd = embed.cuda(), w.cuda()
    x = torch.zeros(32, H, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros_like(x)
    pre = block("NormArgs", x=x, w=wd, out=out, embed=ed, tokens=tokens.cuda(), H=H, ld=H, eps=eps)
    p = Program()
    s = p.stage([Tile(42, i=(0, 16), a=(pre.data_ptr(),)), Tile(42, i=(16, 5), a=(pre.data_ptr(),))])
    run(fab, p, s)
    ref_x = embed[tokens.long()].float()
    assert torch.equal(x[:21].float().cpu(), ref_x)
    ref_n = tp.rms(ref_x, w, eps)
    assert (out[:21].float().cpu() - ref_n).abs().max().item() <= 2 ** -6 * ref_n.abs().max().item()
    # decode: rows 0..3 are requests in slots 4, 0, 5, 2
    row_req = torch.tensor([4, 0, 5, 2], dtype=torch.int32).cuda()
    last = torch.randint(0, V, (S,), generator=g).to(torch.int32).cuda()
    seq = torch.tensor([17, 3, 40, 0, 31, 79], dtype=torch.int32).cuda()     # slot 5 is at the table's end: 5 * 16 - 1
    bt = (torch.arange(S * stride, dtype=torch.int32).view(S, stride) + 7).cuda()
    tok_pos = torch.zeros(4, dtype=torch.int32, device="cuda")
    tok_slot = torch.zeros(4, dtype=torch.int32, device="cuda")
    info = torch.zeros(4, 4, dtype=torch.int32, device="cuda")
    step = block("StepArgs", row_req=row_req, last_token=last, seq_len=seq, block_table=bt, tok_pos=tok_pos,
                 tok_slot=tok_slot, req_info=info, bt_stride=stride, page_size=page)
    dec = block("NormArgs", x=x, w=wd, out=out, embed=ed, step=step, H=H, ld=H, eps=eps)
    seq0 = seq.cpu().clone()
    p = Program()
    s = p.stage([Tile(42, i=(0, 4), a=(dec.data_ptr(),))])
    run(fab, p, s)
    for r, sl in enumerate([4, 0, 5, 2]):
        pos = min(int(seq0[sl]), stride * page - 1)
        assert int(tok_pos[r]) == pos and int(seq[sl]) == pos + 1
        assert int(tok_slot[r]) == int(bt[sl, pos // page]) * page + pos % page
        assert info[r].tolist() == [r, pos, 1, pos + 1]
        assert torch.equal(x[r].cpu(), embed[int(last[sl])])
    assert int(seq[1]) == int(seq0[1]) and int(seq[3]) == int(seq0[3])       # untouched slots


def test_sample_tile(fab):
    """Kind 43: temperature 0 = arg-max with the lowest index on ties; temperature > 0 = Gumbel-max over
    logits / temperature with noise that depends only on (seed, slot, step, index)."""
    V, S, ring = 5000, 4, 8
    g = torch.Generator().manual_seed(8)
    logits = torch.randn(3, V, generator=g)
    logits[0, 4097] = logits[0, 911] = logits[0].max() + 1.0          # a tie: index 911 wins
    lg = logits.cuda()
    temp = torch.tensor([0.0, 0.0, 0.7, 0.7], device="cuda")
    last = torch.zeros(S, dtype=torch.int32, device="cuda")
    steps = torch.tensor([0, 5, 2, 2], dtype=torch.int32, device="cuda")
    host_tokens = torch.zeros(S, ring, dtype=torch.int32).pin_memory()
    host_steps = torch.zeros(S, dtype=torch.int64).pin_memory()
    from monoserve_b200 import _C
    args = block("SampleArgs", logits=lg, temperature=temp, last_token=last, steps=steps,
                 host_tokens=_C.host_device_pointer(host_tokens.data_ptr()),
                 host_steps=_C.host_device_pointer(host_steps.data_ptr()), seed=1234, V=V, ring=ring)
    p = Program()
    # rows 0 and 1 greedy (slots 0, 1); row 2 sampled twice with the same (slot, step) history in slots 2 and 3
    s = p.stage([Tile(43, i=(0, 0), a=(args.data_ptr(),)), Tile(43, i=(1, 1), a=(args.data_ptr(),)),
                 Tile(43, i=(2, 2), a=(args.data_ptr(),)), Tile(43, i=(2, 3), a=(args.data_ptr(),))])
    run(fab, p, s)
    assert int(last[0]) == 911
    assert int(last[1]) == int(logits[1].argmax())
    assert steps.tolist() == [1, 6, 3, 3]
    assert int(host_tokens[0, 0]) == 911 and int(host_tokens[1, 5]) == int(last[1]) and host_steps.tolist() == [1, 6, 3, 3]
    # the noise depends on the slot, so two slots sample independently; both tokens are plausible draws
    assert 0 <= int(last[2]) < V and 0 <= int(last[3]) < V
    probs = torch.softmax(logits[2] / 0.7, -1)
    assert probs[int(last[2])] > 1e-6 and probs[int(last[3])] > 1e-6
    # a second run from the same state reproduces the sampled tokens
    first = (int(last[2]), int(last[3]))
    steps.copy_(torch.tensor([0, 5, 2, 2], dtype=torch.int32))
    run(fab, p, s)
    assert (int(last[2]), int(last[3])) == first
