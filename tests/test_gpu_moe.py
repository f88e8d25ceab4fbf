"""Parity of the CUDA MoE layer with the oracle, through the C ABI.

Integer / index work (routing ids, counts, prefix sums, pack lists, packed rows)
and the exactly-defined floating point (router logits, routing weights, the
combine given the expert outputs) must be BIT-EXACT.  The tensor-core GEMMs are
compared within the stated tolerance: rel-L2 <= 1e-2 per layer output in BF16.
"""
import numpy as np
import pytest
import torch

import oracle
from oracle import torch_path as tp

pytestmark = pytest.mark.gpu

TOL_BF16 = 1e-2   # rel-L2 of a layer output, BF16 weights


def rel_l2(a, b):
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def make_weights(H, I, E, seed, router_scale=None):
    g = torch.Generator().manual_seed(seed)
    wr = (torch.randn(E, H, generator=g) * (router_scale or H ** -0.5)).to(torch.bfloat16)
    w13 = (torch.randn(E, 2 * I, H, generator=g) * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(E, H, I, generator=g) * 0.02).to(torch.bfloat16)
    return wr, w13, w2


def make_layer(T_max, H, I, E, K, hot, seed=0, **kw):
    from monoserve_b200.moe import MoELayer
    wr, w13, w2 = make_weights(H, I, E, seed, kw.pop("router_scale", None))
    m = MoELayer(H, I, E, K, T_max, **kw)
    m.set_router(wr.cuda())
    m.set_experts(w13, w2, hot)
    return m, wr, w13, w2


def acts(T, H, seed):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(T, H, generator=g).to(torch.bfloat16), torch.randn(T, H, generator=g).to(torch.bfloat16))


def bits(t):
    return oracle.bf16_bits(t)


# --------------------------------------------------------------------- routing
@pytest.mark.parametrize("T,H,E", [(1, 256, 8), (37, 512, 16), (64, 2048, 128), (5, 4096, 128), (9, 768, 24)])
def test_router_logits_bit_exact(T, H, E):
    from monoserve_b200 import _C
    g = torch.Generator().manual_seed(T + H)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    wr = (torch.randn(E, H, generator=g) * H ** -0.5).to(torch.bfloat16)
    out = torch.zeros(T, E, device="cuda")
    xd, wd = x.cuda(), wr.cuda()
    _C.check(_C.lib.monofab_router_logits(xd.data_ptr(), wd.data_ptr(), out.data_ptr(), T, H, E, None))
    torch.cuda.synchronize()
    want = oracle.router_logits(bits(x), bits(wr))
    assert np.array_equal(out.cpu().numpy().view(np.int32), want.view(np.int32))


@pytest.mark.parametrize("T,E,K,scoring", [(64, 128, 8, 0), (33, 16, 4, 0), (5, 256, 16, 0), (1, 8, 1, 0),
                                           (100, 160, 6, 1), (70, 128, 8, 1)])
def test_router_topk_bit_exact(T, E, K, scoring):
    from monoserve_b200 import _C
    g = torch.Generator().manual_seed(7 * T + E)
    logits = torch.randn(T, E, generator=g) * 2
    bias = torch.randn(E, generator=g) * 0.1 if scoring else None
    scale = 2.5 if scoring else 1.0
    lg = logits.cuda()
    ids = torch.zeros(T, K, dtype=torch.int32, device="cuda")
    w = torch.zeros(T, K, device="cuda")
    counts = torch.zeros(E, dtype=torch.int32, device="cuda")
    bd = bias.cuda() if bias is not None else None
    _C.check(_C.lib.monofab_router_topk(lg.data_ptr(), bd.data_ptr() if bd is not None else None, ids.data_ptr(),
                                        w.data_ptr(), counts.data_ptr(), None, None, T, E, K, scoring, 1, scale, 1,
                                        None))
    torch.cuda.synchronize()
    o_ids, o_w, o_counts = oracle.router_topk(logits.numpy(), K, bias=None if bias is None else bias.numpy(),
                                              scoring=scoring, renorm=1, scale=scale)
    assert np.array_equal(ids.cpu().numpy(), o_ids)
    assert np.array_equal(w.cpu().numpy().view(np.int32), o_w.view(np.int32))
    assert np.array_equal(counts.cpu().numpy(), o_counts)
    assert float(lg.abs().max()) == 0.0   # the tile zeroes the logits it read (aux.cuh:341-343)


def test_router_ties_lowest_index_wins():
    from monoserve_b200 import _C
    logits = torch.zeros(3, 16)
    logits[1, [3, 7, 9]] = 1.0
    lg = logits.cuda()
    ids = torch.zeros(3, 4, dtype=torch.int32, device="cuda")
    w = torch.zeros(3, 4, device="cuda")
    _C.check(_C.lib.monofab_router_topk(lg.data_ptr(), None, ids.data_ptr(), w.data_ptr(), None, None, None, 3, 16, 4,
                                        0, 1, 1.0, 0, None))
    assert ids.cpu().tolist() == [[0, 1, 2, 3], [3, 7, 9, 0], [0, 1, 2, 3]]


# ------------------------------------------------------------------ whole layer
def check_layer_against_c_oracle(m, wr, w13, w2, xn, x2, K):
    T, H = xn.shape
    out = m.forward(xn.cuda(), x2.cuda() if x2 is not None else None)
    torch.cuda.synchronize()
    assert m.status() == 0
    r = oracle.moe_layer(bits(xn), None if x2 is None else bits(x2), bits(wr), bits(w13), bits(w2), K)
    P = T * K
    ws = {n: m.workspace(n) for n in ("logits", "topk_ids", "topk_w", "counts", "starts", "pair_token",
                                      "pair_weight", "pair_pos", "xp", "h", "y")}
    E, I = wr.shape[0], w13.shape[1] // 2
    assert np.array_equal(ws["logits"][:T * E].cpu().numpy().view(np.int32), r["logits"].ravel().view(np.int32))
    assert np.array_equal(ws["topk_ids"][:P].cpu().numpy(), r["topk_ids"].ravel())
    assert np.array_equal(ws["topk_w"][:P].cpu().numpy().view(np.int32), r["topk_w"].ravel().view(np.int32))
    assert np.array_equal(ws["counts"][:E].cpu().numpy(), r["counts"])
    assert np.array_equal(ws["starts"][:E + 1].cpu().numpy(), r["starts"])
    assert np.array_equal(ws["pair_token"][:P].cpu().numpy(), r["pair_token"])
    assert np.array_equal(ws["pair_weight"][:P].cpu().numpy().view(np.int32), r["pair_weight"].view(np.int32))
    assert np.array_equal(ws["pair_pos"][:P].cpu().numpy(), r["pair_pos"].ravel())
    assert np.array_equal(bits(ws["xp"][:P * H]), r["xp"].ravel())
    h_gpu = ws["h"][:P * I].float().cpu().view(P, I)
    h_ref = torch.from_numpy(oracle.bits_to_f32(r["h"]))
    assert rel_l2(h_gpu, h_ref) < TOL_BF16
    y_gpu = ws["y"][:P * H].cpu().view(P, H)
    assert rel_l2(y_gpu, torch.from_numpy(r["y"])) < TOL_BF16
    assert rel_l2(out.float().cpu(), torch.from_numpy(oracle.bits_to_f32(r["out"]))) < TOL_BF16
    # the combine is exactly defined given y: bit-exact against the oracle run on the GPU's own y
    x_c = oracle.combine(y_gpu.numpy(), r["pair_pos"], r["topk_w"], None if x2 is None else bits(x2))
    assert np.array_equal(bits(out), x_c)
    return out


@pytest.mark.parametrize("T,H,I,E,K", [(37, 256, 128, 8, 2), (1, 256, 64, 8, 2), (33, 512, 256, 16, 4),
                                       (130, 256, 192, 4, 2)])
def test_layer_small_all_intermediates(T, H, I, E, K):
    m, wr, w13, w2 = make_layer(max(T, 64), H, I, E, K, hot=list(range(0, E, 2)), seed=T)
    xn, x2 = acts(T, H, 100 + T)
    check_layer_against_c_oracle(m, wr, w13, w2, xn, x2, K)
    check_layer_against_c_oracle(m, wr, w13, w2, xn, None, K)
    m.close()


def test_layer_empty_batch_and_bounds():
    m, wr, w13, w2 = make_layer(16, 256, 128, 8, 2, hot=[0, 1])
    xn, _ = acts(4, 256, 1)
    assert m.forward(xn[:0].cuda()).shape == (0, 256)
    with pytest.raises(RuntimeError, match="max_tokens"):
        m.forward(acts(17, 256, 2)[0].cuda())
    with pytest.raises(RuntimeError, match="form"):
        m.set_plan(0, 8, 48)
    m.close()


def test_skewed_routing_many_rows_per_expert():
    """Almost every token picks the same experts: segments longer than one row
    block, and many experts with no rows at all."""
    T, H, I, E, K = 400, 256, 128, 16, 2
    m, wr, w13, w2 = make_layer(T, H, I, E, K, hot=[0, 5], seed=3)
    wr = wr.clone()
    wr[3] = 0
    wr[9] = 0
    xn, x2 = acts(T, H, 4)
    xn = (xn.float().abs() * 0.5).to(torch.bfloat16)   # positive activations
    wr[3] = 0.25   # experts 3 and 9 win almost everywhere
    wr[9] = 0.2
    m.set_router(wr.cuda())
    for form in (64, 128, 0):   # 0: one 256-row pass over a host-resident expert
        m.set_plan(0, 4, form)
        check_layer_against_c_oracle(m, wr, w13, w2, xn, x2, K)
    counts = m.workspace("counts")[:E].cpu()
    assert counts[3] > 256 and (counts == 0).sum() >= 1
    m.close()


@pytest.mark.parametrize("form", [16, 32, 64, 128, 0])
@pytest.mark.parametrize("credits", [1, 4, 1 << 20])
def test_forms_and_credits_give_the_same_layer(form, credits):
    T, H, I, E, K = 96, 512, 256, 16, 4
    m, wr, w13, w2 = make_layer(T, H, I, E, K, hot=list(range(4)), seed=5)
    xn, x2 = acts(T, H, 6)
    m.set_plan(0, 1 << 20, 128)
    base = m.forward(xn.cuda(), x2.cuda()).clone()
    m.set_plan(0, credits, form)
    out = m.forward(xn.cuda(), x2.cuda())
    torch.cuda.synchronize()
    assert m.status() == 0
    ref, _, _ = tp.moe_layer(xn.float(), x2.float(), wr, w13, w2, K)
    assert rel_l2(out.float().cpu(), ref) < TOL_BF16
    assert rel_l2(out.float(), base.float()) < 2e-3
    m.close()


def test_placement_does_not_change_results():
    """All experts hot, half hot, none hot: the same arithmetic wherever the weights are."""
    T, H, I, E, K = 64, 512, 256, 16, 4
    xn, x2 = acts(T, H, 8)
    outs = []
    for hot in (list(range(E)), list(range(0, E, 2)), []):
        m, wr, w13, w2 = make_layer(T, H, I, E, K, hot=hot, seed=9)
        m.set_plan(0, 8, 128)
        outs.append(m.forward(xn.cuda(), x2.cuda()).clone())
        torch.cuda.synchronize()
        assert m.status() == 0
        m.close()
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])


def test_zero_credits_runs_only_hbm_experts_safely():
    """credits = 0 means no CTA may read host memory (the reference publishes
    caps=[0] for programs without link stages): the kernel must still finish."""
    T, H, I, E, K = 32, 256, 128, 8, 2
    m, wr, w13, w2 = make_layer(T, H, I, E, K, hot=list(range(E)), seed=10)
    m.set_plan(0, 0, 64)
    xn, x2 = acts(T, H, 11)
    out = m.forward(xn.cuda(), x2.cuda())
    torch.cuda.synchronize()
    assert m.status() == 0
    ref, _, _ = tp.moe_layer(xn.float(), x2.float(), wr, w13, w2, K)
    assert rel_l2(out.float().cpu(), ref) < TOL_BF16
    m.close()


def test_fewer_ctas_same_result():
    T, H, I, E, K = 64, 512, 256, 16, 4
    m, wr, w13, w2 = make_layer(T, H, I, E, K, hot=list(range(8)), seed=12)
    xn, x2 = acts(T, H, 13)
    a = m.forward(xn.cuda(), x2.cuda()).clone()
    m.set_plan(5, 2, 64)
    b = m.forward(xn.cuda(), x2.cuda())
    torch.cuda.synchronize()
    assert m.status() == 0
    assert rel_l2(a.float(), b.float()) < 2e-3
    m.close()


def test_host_buffer_entry_point_matches_device_entry_point():
    T, H, I, E, K = 48, 512, 256, 16, 4
    m, wr, w13, w2 = make_layer(T, H, I, E, K, hot=list(range(8)), seed=14)
    xn, x2 = acts(T, H, 15)
    dev = m.forward(xn.cuda(), x2.cuda()).cpu()
    out_h = torch.empty(T, H, dtype=torch.bfloat16, pin_memory=True)
    m.forward_host(xn.pin_memory(), x2.pin_memory(), out_h)
    assert torch.equal(out_h, dev)
    m.close()


# ------------------------------------------------- the reference's own shapes
def test_qwen3_layer_config1_ragged_batch():
    """Benchmark configuration 1: Qwen3-30B-A3B layer (E 128, top-8, H 2048, I 768), weights
    N(0, 0.02) seed 0, activations N(0,1) seed 1, 64 decode tokens + one 512-token
    prefill.  Routing exact vs the C oracle, output vs the reference's torch path."""
    T, H, I, E, K = 576, 2048, 768, 128, 8
    g = torch.Generator().manual_seed(0)
    wr = (torch.randn(E, H, generator=g) * 0.02).to(torch.bfloat16)
    w13 = (torch.randn(E, 2 * I, H, generator=g) * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(E, H, I, generator=g) * 0.02).to(torch.bfloat16)
    g1 = torch.Generator().manual_seed(1)
    xn = torch.randn(T, H, generator=g1).to(torch.bfloat16)
    from monoserve_b200.moe import MoELayer
    m = MoELayer(H, I, E, K, T)
    m.set_router(wr.cuda())
    m.set_experts(w13, w2, hot=list(range(64)))
    out = m.forward(xn.cuda())
    torch.cuda.synchronize()
    assert m.status() == 0
    logits = oracle.router_logits(bits(xn), bits(wr))
    ids, w, counts = oracle.router_topk(logits, K)
    P = T * K
    assert np.array_equal(m.workspace("topk_ids")[:P].cpu().numpy(), ids.ravel())
    assert np.array_equal(m.workspace("topk_w")[:P].cpu().numpy().view(np.int32), w.ravel().view(np.int32))
    starts = oracle.scan(counts)
    pt, pw, pp = oracle.pack(ids, w, starts)
    assert np.array_equal(m.workspace("starts")[:E + 1].cpu().numpy(), starts)
    assert np.array_equal(m.workspace("pair_token")[:P].cpu().numpy(), pt)
    assert np.array_equal(m.workspace("pair_pos")[:P].cpu().numpy(), pp.ravel())
    torch.set_num_threads(max(1, torch.get_num_threads()))
    routing = (torch.from_numpy(w), torch.from_numpy(ids.astype(np.int64)))
    ref, _, _ = tp.moe_layer(xn.float(), None, wr, w13, w2, K, routing=routing)
    assert rel_l2(out.float().cpu(), ref) < TOL_BF16
    # size-independent property: the layer is permutation-equivariant over tokens, bit for bit
    perm = torch.randperm(T, generator=g1)
    out_p = m.forward(xn[perm].contiguous().cuda())
    assert torch.equal(out_p.cpu(), out.cpu()[perm])
    m.close()


# ------------------------------------------------------ pack from given routing
def random_routing(T, E, K, seed):
    g = torch.Generator().manual_seed(seed)
    ids = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).to(torch.int32) if T else \
        torch.zeros(0, K, dtype=torch.int32)
    w = torch.rand(T, K, generator=g)
    return ids, w


def run_pack_pairs(fn_name, ids, w, E, x=None, with_scratch=True):
    from monoserve_b200 import _C
    T, K = ids.shape
    P = T * K
    d = dict(counts=torch.full((E,), -1, dtype=torch.int32, device="cuda"),
             starts=torch.full((E + 1,), -1, dtype=torch.int32, device="cuda"),
             pair_token=torch.full((max(P, 1),), -1, dtype=torch.int32, device="cuda"),
             pair_weight=torch.zeros(max(P, 1), device="cuda"),
             pair_pos=torch.full((max(P, 1),), -1, dtype=torch.int32, device="cuda"))
    ids_d, w_d = ids.cuda(), w.cuda()
    H = x.shape[1] if x is not None else 0
    x_d = x.cuda() if x is not None else None
    xp = torch.zeros(max(P, 1), H, dtype=torch.bfloat16, device="cuda") if x is not None else None
    args = [ids_d.data_ptr(), w_d.data_ptr(), T, E, K, H, x_d.data_ptr() if x is not None else None,
            xp.data_ptr() if x is not None else None, d["counts"].data_ptr(), d["starts"].data_ptr(),
            d["pair_token"].data_ptr(), d["pair_weight"].data_ptr(), d["pair_pos"].data_ptr()]
    if with_scratch:
        nbytes = _C.lib.monofab_pack_scratch_bytes(T, E, K)
        scratch = torch.empty(max(nbytes, 4), dtype=torch.uint8, device="cuda")
        args += [scratch.data_ptr(), nbytes]
    _C.check(getattr(_C.lib, fn_name)(*args, None))
    torch.cuda.synchronize()
    d["xp"] = xp
    return {k: (v.cpu() if v is not None else None) for k, v in d.items()}


def check_pack_against_oracle(r, ids, w, E, x=None):
    T, K = ids.shape
    P = T * K
    counts = np.bincount(ids.numpy().ravel(), minlength=E).astype(np.int32)
    starts = oracle.scan(counts)
    pt, pw, pp = oracle.pack(ids.numpy(), w.numpy(), starts)
    assert np.array_equal(r["counts"].numpy(), counts)
    assert np.array_equal(r["starts"].numpy(), starts)
    assert np.array_equal(r["pair_token"].numpy()[:P], pt)
    assert np.array_equal(r["pair_weight"].numpy()[:P].view(np.int32), pw.view(np.int32))
    assert np.array_equal(r["pair_pos"].numpy()[:P], pp.ravel())
    if x is not None and P:
        assert np.array_equal(bits(r["xp"][:P]), oracle.permute_rows(bits(x), pt))


@pytest.mark.parametrize("T,E,K,H", [(1, 8, 2, 0), (33, 16, 4, 256), (300, 128, 8, 512), (64, 256, 16, 0),
                                     (0, 8, 2, 0), (1000, 24, 3, 64)])
def test_pack_pairs_bit_exact(T, E, K, H):
    ids, w = random_routing(T, E, K, seed=T + E)
    x = torch.randn(T, H).to(torch.bfloat16) if H else None
    r = run_pack_pairs("monofab_pack_pairs", ids, w, E, x)
    check_pack_against_oracle(r, ids, w, E, x)


def test_pack_pairs_rejects_small_scratch():
    from monoserve_b200 import _C
    ids, w = random_routing(40, 8, 2, 0)
    z = torch.zeros(256, dtype=torch.int32, device="cuda")
    rc = _C.lib.monofab_pack_pairs(ids.cuda().data_ptr(), w.cuda().data_ptr(), 40, 8, 2, 0, None, None, z.data_ptr(),
                                   z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), 16, None)
    assert rc == -1 and b"scratch" in _C.lib.monofab_last_error()


# --------------------------------------------------------------- FP8 (W8A16)
TOL_FP8 = 3e-2   # rel-L2 of a layer output, FP8-e4m3 weights with per-output-channel scales


def make_fp8_layer(T, H, I, E, K, hot, seed, pack_hot=True):
    from monoserve_b200.moe import MoELayer
    wr, w13, w2 = make_weights(H, I, E, seed)
    q13, s13, d13 = tp.quantize_fp8(w13.float())
    q2, s2, d2 = tp.quantize_fp8(w2.float())
    m = MoELayer(H, I, E, K, T, fp8=True)
    m.set_router(wr.cuda())
    m.set_experts(q13, q2, hot, pack_hot=pack_hot, scales=(s13, s2))
    return m, wr, d13, d2


@pytest.mark.parametrize("hot,pack_hot,form", [("all", True, 64), ("half", True, 64), ("none", True, 0),
                                               ("all", False, 64), ("half", False, 128)])
def test_fp8_layer_against_dequantised_reference(hot, pack_hot, form):
    """FP8 experts in the hot tier (packed or reference row order) and in pinned
    host memory: output against the reference's path on the de-quantised weights
    (tests/test_fabric_model_glm.py:57-67, tests/test_fabric_gemm.py:246-251)."""
    T, H, I, E, K = 150, 512, 256, 16, 4
    hot_list = {"all": list(range(E)), "half": list(range(0, E, 2)), "none": []}[hot]
    m, wr, d13, d2 = make_fp8_layer(T, H, I, E, K, hot_list, seed=21, pack_hot=pack_hot)
    m.set_plan(0, 4, form)
    xn, x2 = acts(T, H, 22)
    out = m.forward(xn.cuda(), x2.cuda())
    torch.cuda.synchronize()
    assert m.status() == 0
    ids = m.workspace("topk_ids")[:T * K].cpu().view(T, K).long()
    w = m.workspace("topk_w")[:T * K].cpu().view(T, K)
    ref, _, _ = tp.moe_layer(xn.float(), x2.float(), wr, d13, d2, K, routing=(w, ids))
    assert rel_l2(out.float().cpu(), ref) < TOL_FP8
    # W8A16 is exact in the weights: the only differences are accumulation order and bf16 rounding of h
    assert rel_l2(out.float().cpu(), ref) < 2e-3
    m.close()


@pytest.mark.parametrize("I", [384, 320])
def test_fp8_qwen_shape_prefill_rows(I):
    """GLM-like FP8 at a larger shape with long expert segments (prefill-sized rows); I = 320 gives the
    down projection an odd number of 64-element K steps (the last e4m3 stage is half zero fill)."""
    T, H, E, K = 600, 1024, 8, 2
    m, wr, d13, d2 = make_fp8_layer(T, H, I, E, K, list(range(4)), seed=23)
    xn, x2 = acts(T, H, 24)
    out = m.forward(xn.cuda(), x2.cuda())
    torch.cuda.synchronize()
    assert m.status() == 0
    ids = m.workspace("topk_ids")[:T * K].cpu().view(T, K).long()
    w = m.workspace("topk_w")[:T * K].cpu().view(T, K)
    ref, _, _ = tp.moe_layer(xn.float(), x2.float(), wr, d13, d2, K, routing=(w, ids))
    assert rel_l2(out.float().cpu(), ref) < TOL_FP8
    m.close()
