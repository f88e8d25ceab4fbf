"""GEMM tiles inside the persistent fabric against torch, with the weights in HBM
and in pinned host memory read over the link: the scenarios of the reference's
tests/test_fabric_gemm.py:71-165,372-400 (dense store with residual for every tile
height, the expert FFN with the SiLU-and-multiply and weighted-add epilogues,
K-split partial sums), in the reference's tile operand convention."""
import time

import pytest
import torch

from monoserve_b200 import _C
from monoserve_b200.fabric import Fabric, Program, Tile

pytestmark = pytest.mark.gpu

KIND_GEMM = 32
KIND_GEMM_ASYM, KIND_ASYM_REDUCE = 45, 46
EPI_STORE, EPI_SILU_MUL, EPI_WADD, EPI_F32, EPI_ATOMIC = 0, 1, 2, 3, 4


def pinned_alias(t):
    """Pinned host copy of t and its device address (zero copy)."""
    pin = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
    pin.copy_(t)
    return pin, _C.host_device_pointer(pin.data_ptr())


def weight_map(fab, base, shape):   # (E, rows, K) bf16
    E, rows, K = shape
    return fab.tensor_map(base, [K, rows, E], [K * 2, rows * K * 2], [64, 64, 1])


def act_map(fab, x, bm):            # (M, K) bf16
    M, K = x.shape
    return fab.tensor_map(x.data_ptr(), [K, M], [x.stride(0) * 2], [64, bm])


def args_tensor(**kw):
    return torch.frombuffer(bytearray(_C.gemm_args(**kw)), dtype=torch.uint8).cuda()


@pytest.fixture
def fab():
    f = Fabric(pool_bytes=128 << 20)
    f.set_max_run(60)
    yield f
    f.stop()
    f.close()


def run_program(fab, p, first, caps=(0,)):
    h = p.upload(fab, first=first)
    fab.start()
    fab.publish(map=[0] * fab.num_workers, caps=list(caps), order=[0], programs=[h])
    t0 = time.time()
    while fab.progress()["lanes"][0]["iterations"] < 1:
        assert time.time() - t0 < 30, f"program did not finish: {fab.progress()['error']}"
        time.sleep(1e-3)
    fab.stop()
    assert fab.progress()["error"] == 0


@pytest.mark.parametrize("where", ["hbm", "cpu"])
@pytest.mark.parametrize("bm", [16, 32, 64, 128, 256])
def test_dense_store(fab, where, bm):
    torch.manual_seed(0)
    E, N, K, M = 2, 256, 512, 200
    w = (torch.randn(E, N, K, device="cuda") * 0.05).to(torch.bfloat16)
    x = torch.randn(M + 256, K, device="cuda").to(torch.bfloat16)[:M]
    res = torch.randn(M, N, device="cuda").to(torch.bfloat16)
    out = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16)
    keep, base = (None, w.data_ptr()) if where == "hbm" else pinned_alias(w)
    e = 1
    args = args_tensor(out=out.data_ptr(), ld_out=N, k_tiles=K // 64, epi=EPI_STORE, bm=bm, n_limit=N,
                       residual=res.data_ptr(), ld_res=N)
    wm, xm = weight_map(fab, base, w.shape), act_map(fab, x, bm)
    tiles = [Tile(KIND_GEMM, i=(n0, m0, min(bm, M - m0), e), a=(args.data_ptr(), wm, xm))
             for n0 in range(0, N, 128) for m0 in range(0, M, bm)]
    p = Program()
    s = p.stage(tiles, link=(where == "cpu"))
    run_program(fab, p, s, caps=(4,))
    ref = x.float() @ w[e].float().t() + res.float()
    err = (out.float() - ref).abs().max().item()
    assert err < 0.05 * ref.abs().max().item(), err
    rel = float((out.float() - ref).norm() / ref.norm())
    assert rel < 1e-2, rel
    del keep


@pytest.mark.parametrize("where", ["hbm", "cpu"])
def test_expert_ffn(fab, where):
    """w13 tiles with the SiLU-and-multiply epilogue, then w2 tiles that add
    routing-weighted outputs into the tokens' fp32 accumulators; the w2 stage
    depends on the w13 stage through the program's DAG."""
    torch.manual_seed(1)
    E, H, I, T, TOPK = 8, 512, 256, 64, 2
    w13 = (torch.randn(E, 2 * I, H, device="cuda") * 0.05).to(torch.bfloat16)
    w2 = (torch.randn(E, H, I, device="cuda") * 0.05).to(torch.bfloat16)
    x = torch.randn(T, H, device="cuda").to(torch.bfloat16)
    topk = torch.stack([torch.randperm(E, device="cuda")[:TOPK] for _ in range(T)])
    tw = torch.rand(T, TOPK, device="cuda")
    pairs = sorted((int(topk[t, k]), t, float(tw[t, k])) for t in range(T) for k in range(TOPK))
    xp = torch.zeros(len(pairs) + 64, H, device="cuda", dtype=torch.bfloat16)
    xp[:len(pairs)] = torch.stack([x[t] for _, t, _ in pairs])
    ptok = torch.tensor([t for _, t, _ in pairs], dtype=torch.int32, device="cuda")
    pw = torch.tensor([wt for _, _, wt in pairs], dtype=torch.float32, device="cuda")
    starts = {}
    for i, (e, _, _) in enumerate(pairs):
        starts.setdefault(e, [i, 0])[1] += 1
    hbuf = torch.zeros(len(pairs) + 64, I, device="cuda", dtype=torch.bfloat16)
    out32 = torch.zeros(T, H, device="cuda", dtype=torch.float32)
    if where == "cpu":
        k1, b13 = pinned_alias(w13)
        k2, b2 = pinned_alias(w2)
    else:
        k1 = k2 = None
        b13, b2 = w13.data_ptr(), w2.data_ptr()
    bm = 16
    a13 = args_tensor(out=hbuf.data_ptr(), ld_out=I, k_tiles=H // 64, epi=EPI_SILU_MUL, bm=bm, n_limit=I, up_offset=I)
    a2 = args_tensor(out=out32.data_ptr(), ld_out=H, k_tiles=I // 64, epi=EPI_WADD, bm=bm, n_limit=H,
                     pair_token=ptok.data_ptr(), pair_weight=pw.data_ptr())
    m13, m2 = weight_map(fab, b13, w13.shape), weight_map(fab, b2, w2.shape)
    mx, mh = act_map(fab, xp, bm), act_map(fab, hbuf, bm)
    t13, t2 = [], []
    for e, (s0, cnt) in starts.items():
        for m0 in range(s0, s0 + cnt, bm):
            mv = min(bm, s0 + cnt - m0)
            t13 += [Tile(KIND_GEMM, i=(f0, m0, mv, e), a=(a13.data_ptr(), m13, mx)) for f0 in range(0, I, 64)]
            t2 += [Tile(KIND_GEMM, i=(n0, m0, mv, e), a=(a2.data_ptr(), m2, mh)) for n0 in range(0, H, 128)]
    p = Program()
    s13 = p.stage(t13, link=(where == "cpu"))
    s2 = p.stage(t2, link=(where == "cpu"))
    p.after(s13, s2)
    run_program(fab, p, s13, caps=(8,))
    ref = torch.zeros(T, H, device="cuda")
    for t in range(T):
        for k in range(TOPK):
            e = int(topk[t, k])
            g = x[t].float() @ w13[e, :I].float().t()
            u = x[t].float() @ w13[e, I:].float().t()
            hh = (torch.nn.functional.silu(g) * u).to(torch.bfloat16).float()
            ref[t] += float(tw[t, k]) * (hh @ w2[e].float().t())
    err = (out32 - ref).abs().max().item()
    assert err < 0.03 * ref.abs().max().item(), err
    assert float((out32 - ref).norm() / ref.norm()) < 1e-2
    del k1, k2


@pytest.mark.parametrize("where", ["hbm", "cpu"])
@pytest.mark.parametrize("bm", [16, 64])
def test_k_split_expert_ffn(fab, where, bm):
    """The reference's K-split form (tests/test_fabric_gemm.py:177-250): w13 tiles of kind 45 add fp32 partial
    sums of gate and up rows over K ranges, for ALL rows of their expert; the reduce tiles (kind 46) turn them
    into h = silu(gate) * up and zero them; w2 tiles of kind 45 add routing-weighted outputs over K ranges."""
    from monoserve_b200.fabric.args import pack
    torch.manual_seed(2)
    E, H, I, T, TOPK = 4, 1024, 640, 48, 2   # experts get about 24 rows each: two row blocks at bm = 16
    w13 = (torch.randn(E, 2 * I, H, device="cuda") * 0.03).to(torch.bfloat16)
    w2 = (torch.randn(E, H, I, device="cuda") * 0.03).to(torch.bfloat16)
    x = torch.randn(T, H, device="cuda").to(torch.bfloat16)
    topk = torch.stack([torch.randperm(E, device="cuda")[:TOPK] for _ in range(T)])
    tw = torch.rand(T, TOPK, device="cuda")
    pairs = sorted((int(topk[t, k]), t, float(tw[t, k])) for t in range(T) for k in range(TOPK))
    xp = torch.zeros(len(pairs) + 64, H, device="cuda", dtype=torch.bfloat16)
    xp[:len(pairs)] = torch.stack([x[t] for _, t, _ in pairs])
    ptok = torch.tensor([t for _, t, _ in pairs], dtype=torch.int32, device="cuda")
    pw = torch.tensor([wt for _, _, wt in pairs], dtype=torch.float32, device="cuda")
    starts = {}
    for i, (e, _, _) in enumerate(pairs):
        starts.setdefault(e, [i, 0])[1] += 1
    ws = torch.zeros(len(pairs), 2 * I, device="cuda", dtype=torch.float32)
    hbuf = torch.zeros(len(pairs) + 64, I, device="cuda", dtype=torch.bfloat16)
    out32 = torch.zeros(T, H, device="cuda", dtype=torch.float32)
    if where == "cpu":
        k1, b13 = pinned_alias(w13)
        k2, b2 = pinned_alias(w2)
    else:
        k1 = k2 = None
        b13, b2 = w13.data_ptr(), w2.data_ptr()
    a13 = args_tensor(out=ws.data_ptr(), ld_out=2 * I, k_tiles=H // 64, epi=EPI_ATOMIC, bm=bm, n_limit=I, up_offset=I)
    a2 = args_tensor(out=out32.data_ptr(), ld_out=H, k_tiles=I // 64, epi=EPI_WADD, bm=bm, n_limit=H,
                     pair_token=ptok.data_ptr(), pair_weight=pw.data_ptr())
    red = torch.frombuffer(bytearray(pack("ReduceArgs", ws=ws, out=hbuf, I=I, ld_ws=2 * I, ld_out=I)), dtype=torch.uint8).cuda()
    m13, m2 = weight_map(fab, b13, w13.shape), weight_map(fab, b2, w2.shape)
    mx, mh = act_map(fab, xp, bm), act_map(fab, hbuf, bm)

    def splits(kt, most=8):   # K ranges of at most `most` K tiles
        return [(k0, min(most, kt - k0)) for k0 in range(0, kt, most)]
    t13, tr, t2 = [], [], []
    for e, (s0, cnt) in starts.items():
        t13 += [Tile(KIND_GEMM_ASYM, i=(f0, s0, cnt, e), a=(a13.data_ptr(), m13, mx, k0 | (kt << 16)))
                for f0 in range(0, I, 64) for k0, kt in splits(H // 64)]
        tr += [Tile(KIND_ASYM_REDUCE, i=(r0, min(64, s0 + cnt - r0)), a=(red.data_ptr(),)) for r0 in range(s0, s0 + cnt, 64)]
        t2 += [Tile(KIND_GEMM_ASYM, i=(n0, s0, cnt, e), a=(a2.data_ptr(), m2, mh, k0 | (kt << 16)))
               for n0 in range(0, H, 128) for k0, kt in splits(I // 64)]
    p = Program()
    s13, sr, s2 = p.stage(t13, link=(where == "cpu")), p.stage(tr), p.stage(t2, link=(where == "cpu"))
    p.after(s13, sr)
    p.after(sr, s2)
    run_program(fab, p, s13, caps=(8,))
    e_of = torch.tensor([e for e, _, _ in pairs], device="cuda")
    xr = xp[:len(pairs)].float()
    g = torch.einsum("mh,mih->mi", xr, w13[e_of, :I].float())
    u = torch.einsum("mh,mih->mi", xr, w13[e_of, I:].float())
    h_ref = torch.nn.functional.silu(g) * u
    assert (hbuf[:len(pairs)].float() - h_ref).abs().max().item() < 0.02 * h_ref.abs().max().item()
    assert ws.abs().max().item() == 0.0   # the reduce zeroed the partial sums
    y = torch.einsum("mi,mhi->mh", h_ref.to(torch.bfloat16).float(), w2[e_of].float()) * pw[:, None]
    ref = torch.zeros(T, H, device="cuda").index_add_(0, ptok.long(), y)
    assert (out32 - ref).abs().max().item() < 0.03 * ref.abs().max().item()
    assert float((out32 - ref).norm() / ref.norm()) < 1e-2
    del k1, k2


@pytest.mark.parametrize("bm", [16, 64])
def test_dense_split_k(fab, bm):
    """A K-split GEMM: every tile takes one K range and adds its partial sums into an
    fp32 output, the tile of the first range with the bias."""
    torch.manual_seed(5)
    E, N, K, M = 2, 256, 1024, 40
    w = (torch.randn(E, N, K, device="cuda") * 0.05).to(torch.bfloat16)
    x = torch.randn(M + 64, K, device="cuda").to(torch.bfloat16)[:M]
    bias = torch.randn(N, device="cuda").to(torch.bfloat16)
    out = torch.zeros(M, N, device="cuda", dtype=torch.float32)
    e = 1
    args = args_tensor(out=out.data_ptr(), ld_out=N, k_tiles=K // 64, epi=EPI_ATOMIC, bm=bm, n_limit=N,
                       bias=bias.data_ptr())
    wm, xm = weight_map(fab, w.data_ptr(), w.shape), act_map(fab, x, bm)
    ranges = [(0, 5), (5, 5), (10, 6)]   # uneven ranges over the 16 K tiles
    tiles = [Tile(KIND_GEMM, i=(n0, m0, min(bm, M - m0), e), a=(args.data_ptr(), wm, xm, k0 | (kn << 16)))
             for n0 in range(0, N, 128) for m0 in range(0, M, bm) for k0, kn in ranges]
    p = Program()
    s = p.stage(tiles)
    run_program(fab, p, s)
    ref = x.float() @ w[e].float().t() + bias.float()
    assert (out - ref).abs().max().item() < 0.02 * ref.abs().max().item()


@pytest.mark.parametrize("where", ["hbm", "cpu"])
def test_fp8_expert_ffn(fab, where):
    """FP8-e4m3 weights with per-output-channel fp32 scales (W8A16): the scenario of the reference's
    tests/test_fabric_gemm.py:246-283 — w13 tiles with the SiLU-and-multiply epilogue and w2 tiles with
    the weighted-add epilogue over quantised experts in HBM or in pinned host memory — against the
    de-quantised weights in fp32, mixed with bf16 tiles on the same workers."""
    from oracle import torch_path as tp
    torch.manual_seed(7)
    E, H, I, T, TOPK = 8, 512, 256, 64, 2
    w13 = torch.randn(E, 2 * I, H) * 0.05
    w2 = torch.randn(E, H, I) * 0.05
    q13, s13, d13 = tp.quantize_fp8(w13)
    q2, s2, d2 = tp.quantize_fp8(w2)
    x = torch.randn(T, H, device="cuda").to(torch.bfloat16)
    topk = torch.stack([torch.randperm(E, device="cuda")[:TOPK] for _ in range(T)])
    tw = torch.rand(T, TOPK, device="cuda")
    pairs = sorted((int(topk[t, k]), t, float(tw[t, k])) for t in range(T) for k in range(TOPK))
    xp = torch.zeros(len(pairs) + 64, H, device="cuda", dtype=torch.bfloat16)
    xp[:len(pairs)] = torch.stack([x[t] for _, t, _ in pairs])
    ptok = torch.tensor([t for _, t, _ in pairs], dtype=torch.int32, device="cuda")
    pw = torch.tensor([wt for _, _, wt in pairs], dtype=torch.float32, device="cuda")
    starts = {}
    for i, (e, _, _) in enumerate(pairs):
        starts.setdefault(e, [i, 0])[1] += 1
    hbuf = torch.zeros(len(pairs) + 64, I, device="cuda", dtype=torch.bfloat16)
    out32 = torch.zeros(T, H, device="cuda", dtype=torch.float32)
    if where == "cpu":
        k1, b13 = pinned_alias(q13)
        k2, b2 = pinned_alias(q2)
    else:
        k1, k2 = q13.cuda(), q2.cuda()
        b13, b2 = k1.data_ptr(), k2.data_ptr()
    sc13, sc2 = s13.cuda(), s2.cuda()
    bm = 16

    def fp8_map(base, shape):   # (E, rows, K) e4m3 bytes: byte strides, no swizzle (monoserve/runtime/weights.py:38-40)
        n_e, rows, k = shape
        return fab.tensor_map(base, [k, rows, n_e], [k, rows * k], [128, 64, 1], dtype=2, swizzle=0)

    a13 = args_tensor(out=hbuf.data_ptr(), ld_out=I, k_tiles=H // 64, epi=EPI_SILU_MUL, bm=bm, n_limit=I, up_offset=I,
                      w_fp8=1)
    a2 = args_tensor(out=out32.data_ptr(), ld_out=H, k_tiles=I // 64, epi=EPI_WADD, bm=bm, n_limit=H,
                     pair_token=ptok.data_ptr(), pair_weight=pw.data_ptr(), w_fp8=1)
    m13, m2 = fp8_map(b13, q13.shape), fp8_map(b2, q2.shape)
    mx, mh = act_map(fab, xp, bm), act_map(fab, hbuf, bm)
    t13, t2 = [], []
    for e, (s0, cnt) in starts.items():
        for m0 in range(s0, s0 + cnt, bm):
            mv = min(bm, s0 + cnt - m0)
            t13 += [Tile(KIND_GEMM, i=(f0, m0, mv, e), a=(a13.data_ptr(), m13, mx, 0, sc13.data_ptr() + e * 2 * I * 4))
                    for f0 in range(0, I, 64)]
            t2 += [Tile(KIND_GEMM, i=(n0, m0, mv, e), a=(a2.data_ptr(), m2, mh, 0, sc2.data_ptr() + e * H * 4))
                   for n0 in range(0, H, 128)]
    # a bf16 dense GEMM in a parallel stage, so that workers alternate between the two kinds of tiles
    wd = (torch.randn(1, 256, H, device="cuda") * 0.05).to(torch.bfloat16)
    od = torch.zeros(T, 256, device="cuda", dtype=torch.bfloat16)
    ad = args_tensor(out=od.data_ptr(), ld_out=256, k_tiles=H // 64, epi=EPI_STORE, bm=64, n_limit=256)
    md, mxd = weight_map(fab, wd.data_ptr(), wd.shape), act_map(fab, x, 64)
    td = [Tile(KIND_GEMM, i=(n0, 0, T, 0), a=(ad.data_ptr(), md, mxd)) for n0 in range(0, 256, 128)] * 8
    p = Program()
    s_first = p.stage([Tile(0)])
    s13_ = p.stage(t13, link=(where == "cpu"))
    s2_ = p.stage(t2, link=(where == "cpu"))
    sd = p.stage(td)
    p.after(s_first, s13_)
    p.after(s_first, sd)
    p.after(s13_, s2_)
    run_program(fab, p, s_first, caps=(8,))
    ref = torch.zeros(T, H)
    xc = x.float().cpu()
    for t in range(T):
        for k in range(TOPK):
            e = int(topk[t, k])
            ref[t] += float(tw[t, k]) * tp.ffn(xc[t:t + 1], d13[e], d2[e])[0]
    got = out32.cpu()
    rel = float((got - ref).norm() / ref.norm())
    assert rel < 3e-2, rel
    refd = xc @ wd[0].float().cpu().t()
    rel_d = float((od.float().cpu() - refd).norm() / refd.norm())
    assert rel_d < 1e-2, rel_d
    del k1, k2


def test_fetch_tiles_copy_host_memory_into_hbm(fab):
    """Fetch tiles (kind 49) bring pinned host bytes into an HBM buffer through the operand ring, in
    stages of 32 KB with a ragged last stage, interleaved on the same workers with GEMM tiles whose
    output depends on the fetched weights (a GEMM stage after the fetch stage reads the copy)."""
    torch.manual_seed(11)
    E, N, K, M = 3, 256, 512, 96
    w = (torch.randn(E, N, K) * 0.05).to(torch.bfloat16)
    pin, alias = pinned_alias(w)
    stage_buf = torch.zeros(E, N, K, dtype=torch.bfloat16, device="cuda")
    x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    out = torch.zeros(E, M, N, device="cuda", dtype=torch.bfloat16)
    total = w.numel() * 2
    chunk = 100 * 1024 + 48            # not a multiple of the 32 KB stage: ragged stages and a ragged last tile
    fetch = [Tile(49, i=(min(chunk, total - at),), a=(alias + at, stage_buf.data_ptr() + at))
             for at in range(0, total, chunk)]
    wm, xm = weight_map(fab, stage_buf.data_ptr(), stage_buf.shape), act_map(fab, x, 128)
    gemm = []
    keep = []
    for e in range(E):
        a = args_tensor(out=out[e].data_ptr(), ld_out=N, k_tiles=K // 64, epi=EPI_STORE, bm=128, n_limit=N)
        keep.append(a)
        gemm += [Tile(KIND_GEMM, i=(n0, 0, M, e), a=(a.data_ptr(), wm, xm)) for n0 in range(0, N, 128)]
    # a stage of GEMM tiles on weights that are already in HBM runs beside the fetch stage
    wd = (torch.randn(1, 256, K, device="cuda") * 0.05).to(torch.bfloat16)
    od = torch.zeros(M, 256, device="cuda", dtype=torch.bfloat16)
    ad = args_tensor(out=od.data_ptr(), ld_out=256, k_tiles=K // 64, epi=EPI_STORE, bm=128, n_limit=256)
    side = [Tile(KIND_GEMM, i=(n0, 0, M, 0), a=(ad.data_ptr(), weight_map(fab, wd.data_ptr(), wd.shape), xm))
            for n0 in range(0, 256, 128)] * 6
    p = Program()
    s0 = p.stage([Tile(0)])
    s_f = p.stage(fetch, link=True)
    s_g = p.stage(gemm)
    s_side = p.stage(side)
    p.after(s0, s_f)
    p.after(s0, s_side)
    p.after(s_f, s_g)
    run_program(fab, p, s0, caps=(4,))
    assert torch.equal(stage_buf.cpu(), w), "the staged copy is the host tensor, byte for byte"
    for e in range(E):
        ref = x.float() @ w[e].float().cuda().t()
        assert (out[e].float() - ref).abs().max().item() < 0.02 * ref.abs().max().item()
    refd = x.float() @ wd[0].float().t()
    assert (od.float() - refd).abs().max().item() < 0.02 * refd.abs().max().item()


def test_bad_fetch_tile_is_reported(fab):
    """A fetch tile whose size is not a multiple of 16 bytes is refused through the error word."""
    buf = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    pin = torch.zeros(4096, dtype=torch.uint8, pin_memory=True)
    p = Program()
    s = p.stage([Tile(49, i=(100,), a=(_C.host_device_pointer(pin.data_ptr()), buf.data_ptr()))])
    h = p.upload(fab, first=s)
    fab.start()
    fab.publish(map=[0] * fab.num_workers, caps=[0], order=[0], programs=[h])
    t0 = time.time()
    while fab.progress()["lanes"][0]["iterations"] < 1:
        assert time.time() - t0 < 30
        time.sleep(1e-3)
    fab.stop()
    assert fab.progress()["error"] & 8


def test_unsupported_gemm_tile_is_reported(fab):
    """A bad tile height is reported through the error word; the program still ends."""
    z = torch.zeros(64, 64, device="cuda", dtype=torch.bfloat16)
    args = args_tensor(out=z.data_ptr(), ld_out=64, k_tiles=1, epi=EPI_STORE, bm=24, n_limit=64)
    xm = act_map(fab, z, 16)
    p = Program()
    s = p.stage([Tile(KIND_GEMM, i=(0, 0, 16, 0), a=(args.data_ptr(), xm, xm))])
    h = p.upload(fab, first=s)
    fab.start()
    fab.publish(map=[0] * fab.num_workers, caps=[0], order=[0], programs=[h])
    t0 = time.time()
    while fab.progress()["lanes"][0]["iterations"] < 1:
        assert time.time() - t0 < 30
        time.sleep(1e-3)
    fab.stop()
    assert fab.progress()["error"] & 8
