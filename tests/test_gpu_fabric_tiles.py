"""Row-wise model tiles inside the fabric (router, RMSNorm, AddNorm) against the
oracle, bit for bit, and two lanes running concurrently on disjoint SM floors with
link credits (the mixed prefill / decode arrangement of the reference's
tests/test_fabric_model.py:86-123, on GEMM tiles)."""
import time

import numpy as np
import pytest
import torch

import oracle
from monoserve_b200 import _C
from monoserve_b200.fabric import Fabric, Program, Tile
from monoserve_b200.fabric.args import pack

pytestmark = pytest.mark.gpu
KIND_GEMM, KIND_RMSNORM, KIND_ROUTER, KIND_ADDNORM = 32, 36, 38, 41


def block(name, **fields):
    return torch.frombuffer(bytearray(pack(name, **fields)), dtype=torch.uint8).cuda()


@pytest.fixture
def fab():
    f = Fabric(pool_bytes=128 << 20)
    f.set_max_run(60)
    yield f
    f.stop()
    f.close()


def run(fab, program, first, lanes=None, caps=(0,), iterations_wanted=1):
    h = program.upload(fab, first=first)
    fab.start()
    fab.publish(map=lanes or [0] * fab.num_workers, caps=list(caps), order=[0], programs=[h])
    t0 = time.time()
    while fab.progress()["lanes"][0]["iterations"] < iterations_wanted:
        assert time.time() - t0 < 30, fab.progress()["error"]
        time.sleep(1e-3)
    fab.stop()
    assert fab.progress()["error"] == 0


@pytest.mark.parametrize("T,E,K,scoring", [(100, 128, 8, 0), (37, 16, 4, 0), (70, 160, 6, 1)])
def test_router_tile_bit_exact(fab, T, E, K, scoring):
    g = torch.Generator().manual_seed(T)
    logits = torch.randn(T, E, generator=g) * 2
    bias = torch.randn(E, generator=g) * 0.1 if scoring else None
    lg = logits.cuda()
    ids = torch.zeros(T, K, dtype=torch.int32, device="cuda")
    w = torch.zeros(T, K, device="cuda")
    counts = torch.zeros(E, dtype=torch.int32, device="cuda")
    bd = bias.cuda() if bias is not None else None
    args = block("RouterArgs", logits=lg, topk_ids=ids, topk_w=w, counts=counts, bias=bd if bd is not None else 0,
                 E=E, K=K, scoring=scoring, renorm=1, scale=2.5 if scoring else 1.0)
    p = Program()
    s = p.stage([Tile(KIND_ROUTER, i=(r0, min(16, T - r0)), a=(args.data_ptr(),)) for r0 in range(0, T, 16)])
    run(fab, p, s)
    o_ids, o_w, o_counts = oracle.router_topk(logits.numpy(), K, bias=None if bias is None else bias.numpy(),
                                              scoring=scoring, renorm=1, scale=2.5 if scoring else 1.0)
    assert np.array_equal(ids.cpu().numpy(), o_ids)
    assert np.array_equal(w.cpu().numpy().view(np.int32), o_w.view(np.int32))
    assert np.array_equal(counts.cpu().numpy(), o_counts)
    assert float(lg.abs().max()) == 0.0


def test_norm_tiles_bit_exact(fab):
    T, H = 50, 512
    g = torch.Generator().manual_seed(3)
    x2 = torch.randn(T, H, generator=g).to(torch.bfloat16)
    acc = torch.randn(T, H, generator=g)
    wn = (1 + 0.1 * torch.randn(H, generator=g)).to(torch.bfloat16)
    gather = torch.full((T,), -1, dtype=torch.int32)
    gather[7], gather[20] = 0, 1
    x2d, accd, wd, gd = x2.cuda(), acc.cuda(), wn.cuda(), gather.cuda()
    x = torch.zeros(T, H, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(T, H, dtype=torch.bfloat16, device="cuda")
    out2 = torch.zeros(2, H, dtype=torch.bfloat16, device="cuda")
    plain_in = torch.randn(T, H, generator=g).to(torch.bfloat16).cuda()
    plain_out = torch.zeros(T, H, dtype=torch.bfloat16, device="cuda")
    a_add = block("NormArgs", x=x, x2=x2d, acc=accd, w=wd, out=out, gather=gd, out2=out2, H=H, ld=H, eps=1e-6)
    a_rms = block("NormArgs", x=plain_in, w=wd, out=plain_out, H=H, ld=H, eps=1e-6)
    p = Program()
    s0 = p.stage([Tile(KIND_ADDNORM, i=(r0, min(16, T - r0)), a=(a_add.data_ptr(),)) for r0 in range(0, T, 16)])
    s1 = p.stage([Tile(KIND_RMSNORM, i=(r0, min(16, T - r0)), a=(a_rms.data_ptr(),)) for r0 in range(0, T, 16)])
    p.after(s0, s1)
    run(fab, p, s0)
    ident = np.arange(T, dtype=np.int32).reshape(T, 1)
    ones = np.ones((T, 1), dtype=np.float32)
    want_x, want_n = oracle.combine(acc.numpy(), ident, ones, oracle.bf16_bits(x2), oracle.bf16_bits(wn), eps=1e-6)
    assert np.array_equal(oracle.bf16_bits(x), want_x)
    assert np.array_equal(oracle.bf16_bits(out), want_n)
    assert float(accd.abs().max()) == 0.0, "AddNorm zeroes the accumulator rows"
    assert np.array_equal(oracle.bf16_bits(out2), want_n[[7, 20]])
    zero = np.zeros((T, H), dtype=np.float32)
    _, want_p = oracle.combine(zero, ident, ones, oracle.bf16_bits(plain_in), oracle.bf16_bits(wn), eps=1e-6)
    assert np.array_equal(oracle.bf16_bits(plain_out), want_p)


def _gemm_stage_tiles(fab, w_base, w_shape, x, out, bm, e, keep):
    E, N, K = w_shape
    M = x.shape[0] - 256
    args = torch.frombuffer(bytearray(_C.gemm_args(out=out.data_ptr(), ld_out=N, k_tiles=K // 64, epi=0, bm=bm,
                                                   n_limit=N)), dtype=torch.uint8).cuda()
    keep.append(args)
    wm = fab.tensor_map(w_base, [K, N, E], [K * 2, N * K * 2], [64, 64, 1])
    xm = fab.tensor_map(x.data_ptr(), [K, x.shape[0]], [K * 2], [64, bm])
    return [Tile(KIND_GEMM, i=(n0, m0, min(bm, M - m0), e), a=(args.data_ptr(), wm, xm))
            for n0 in range(0, N, 128) for m0 in range(0, M, bm)]


def test_two_lanes_on_disjoint_floors_with_link_credits(fab):
    """A 'prefill' lane (tall tiles, HBM weights) and a repeating 'decode' lane (short
    tiles, weights in pinned host memory under 4 link credits) run at the same time on
    their own halves of the SMs; both produce the right results, the gate holds, and
    the decode lane's iteration timer ticks while the prefill lane is busy."""
    torch.manual_seed(7)
    keep = []
    E, N, K = 2, 1024, 1024
    w_hbm = (torch.randn(E, N, K, device="cuda") * 0.05).to(torch.bfloat16)
    w_host = (torch.randn(E, N, K) * 0.05).to(torch.bfloat16).pin_memory()
    xp = torch.randn(2048 + 256, K, device="cuda").to(torch.bfloat16)
    xd = torch.randn(24 + 256, K, device="cuda").to(torch.bfloat16)
    outp = torch.zeros(2048, N, dtype=torch.bfloat16, device="cuda")
    outd = torch.zeros(24, N, dtype=torch.bfloat16, device="cuda")
    pre, dec = Program(), Program()
    # the prefill lane repeats its stage chain 6 times to stay busy
    prev = None
    first_pre = None
    for _ in range(6):
        s = pre.stage(_gemm_stage_tiles(fab, w_hbm.data_ptr(), w_hbm.shape, xp, outp, 128, 1, keep))
        if prev is None:
            first_pre = s
        else:
            pre.after(prev, s)
        prev = s
    sd = dec.stage(_gemm_stage_tiles(fab, _C.host_device_pointer(w_host.data_ptr()), w_host.shape, xd, outd, 32, 0, keep),
                   link=True, mark=(0 << 8) | 3)
    hp = pre.upload(fab, first=first_pre, iterations=1)
    hd = dec.upload(fab, first=sd, iterations=0)
    n = fab.num_workers
    lanes = [0] * (n // 2) + [1] * (n - n // 2)
    fab.start()
    fab.reset_inflight_max(1)
    fab.publish(map=lanes, caps=[0, 4], order=[0, 1], programs=[hp, hd])
    ends = fab.iteration_times(1, 0, 5, timeout=30)
    t0 = time.time()
    while fab.progress()["lanes"][0]["iterations"] < 1:
        assert time.time() - t0 < 30
        time.sleep(1e-3)
    stats = fab.lane_stats(1)
    fab.stop()
    assert fab.progress()["error"] == 0
    assert stats["inflight_max"] <= 4
    assert all(b > a for a, b in zip(ends, ends[1:]))
    refp = xp[:2048].float() @ w_hbm[1].float().t()
    refd = xd[:24].float() @ w_host[0].cuda().float().t()
    assert float((outp.float() - refp).norm() / refp.norm()) < 1e-2
    assert float((outd.float() - refd).norm() / refd.norm()) < 1e-2
