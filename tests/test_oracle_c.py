"""The plain-C oracle: its exact-order arithmetic, its integer routing/packing
definitions, and its agreement with the restated torch path of the reference."""
import numpy as np
import pytest
import torch

import oracle
from oracle import torch_path as tp


def ulp_diff(a, b):
    a, b = np.asarray(a, np.float32), np.asarray(b, np.float32)
    ia, ib = a.view(np.int32).astype(np.int64), b.view(np.int32).astype(np.int64)
    return np.abs(ia - ib)


def test_expf_close_to_libm():
    x = np.concatenate([np.linspace(-100, 0, 20001), np.linspace(0, 88, 5001), [-103.5, -200.0, -1e30, 0.0]])
    got = oracle.expf(x.astype(np.float32))
    want = np.exp(x.astype(np.float32).astype(np.float64)).astype(np.float32)
    normal = want > 1e-37
    assert ulp_diff(got[normal], want[normal]).max() <= 2
    assert np.all(got[x < -103.0] == 0.0)
    assert oracle.expf(np.float32(0.0)) == 1.0


def test_router_matches_torch_on_tie_free_inputs():
    g = torch.Generator().manual_seed(0)
    for (T, E, K) in [(64, 128, 8), (33, 16, 4), (5, 256, 16), (1, 8, 1), (40, 160, 6)]:
        logits = torch.randn(T, E, generator=g)
        ids, w, counts = oracle.router_topk(logits.numpy(), K)
        p = logits.softmax(-1)
        tw, ti = p.topk(K, -1)
        tw = tw / tw.sum(-1, keepdim=True)
        assert np.array_equal(ids, ti.numpy().astype(np.int32))
        assert ulp_diff(w, tw.numpy()).max() <= 8
        assert np.array_equal(counts, np.bincount(ids.ravel(), minlength=E))
        assert np.allclose(w.sum(-1), 1.0, atol=1e-6)


def test_router_sigmoid_bias_scale():
    g = torch.Generator().manual_seed(1)
    T, E, K = 50, 64, 8
    logits, bias = torch.randn(T, E, generator=g), torch.randn(E, generator=g) * 0.1
    ids, w, _ = oracle.router_topk(logits.numpy(), K, bias=bias.numpy(), scoring=1, renorm=1, scale=2.5)
    p = torch.sigmoid(logits)
    _, ti = (p + bias).topk(K, -1)
    tw = p.gather(1, ti)
    tw = tw / tw.sum(-1, keepdim=True) * 2.5
    assert np.array_equal(ids, ti.numpy().astype(np.int32))
    assert np.allclose(w, tw.numpy(), rtol=2e-6)
    ids2, w2, _ = oracle.router_topk(logits.numpy(), K, bias=None, scoring=1, renorm=0, scale=1.0)
    assert np.allclose(w2, np.take_along_axis(p.numpy(), ids2.astype(np.int64), 1), rtol=2e-6)


def test_router_ties_take_lowest_index():
    logits = np.zeros((3, 16), dtype=np.float32)
    logits[1, [3, 7, 9]] = 1.0
    logits[2, :] = -5.0
    ids, w, counts = oracle.router_topk(logits, 4)
    assert ids[0].tolist() == [0, 1, 2, 3]
    assert ids[1].tolist() == [3, 7, 9, 0]
    assert ids[2].tolist() == [0, 1, 2, 3]
    assert np.all(w[0] == 0.25)
    assert counts.sum() == 12


def test_router_rejects_bad_sizes():
    with pytest.raises(ValueError):
        oracle.router_topk(np.zeros((1, 300), np.float32), 4)
    with pytest.raises(ValueError):
        oracle.router_topk(np.zeros((1, 8), np.float32), 17)
    with pytest.raises(ValueError):
        oracle.router_topk(np.zeros((1, 4), np.float32), 8)


def test_scan_and_pack_are_stable():
    rng = np.random.default_rng(0)
    T, E, K = 77, 12, 3
    ids = np.stack([rng.permutation(E)[:K] for _ in range(T)]).astype(np.int32)
    w = rng.random((T, K), dtype=np.float32)
    counts = np.bincount(ids.ravel(), minlength=E).astype(np.int32)
    starts = oracle.scan(counts)
    assert starts[0] == 0 and starts[-1] == T * K and np.array_equal(np.diff(starts), counts)
    pt, pw, pp = oracle.pack(ids, w, starts)
    # the reference test builds its packed lists as sorted (expert, token) pairs
    # (tests/test_fabric_gemm.py:110-111): the same order
    pairs = sorted((int(ids[t, k]), t, k) for t in range(T) for k in range(K))
    assert pt.tolist() == [t for _, t, _ in pairs]
    assert np.array_equal(pw, np.array([w[t, k] for _, t, k in pairs], dtype=np.float32))
    for pos, (e, t, k) in enumerate(pairs):
        assert pp[t, k] == pos and starts[e] <= pos < starts[e + 1]
    # empty input and an expert nobody picked
    s0 = oracle.scan(np.zeros(4, np.int32))
    assert s0.tolist() == [0, 0, 0, 0, 0]


def test_router_logits_order_is_close_to_plain_dot():
    g = torch.Generator().manual_seed(2)
    x = torch.randn(9, 512, generator=g).to(torch.bfloat16)
    wr = (torch.randn(24, 512, generator=g) * 0.05).to(torch.bfloat16)
    lg = oracle.router_logits(oracle.bf16_bits(x), oracle.bf16_bits(wr))
    ref = (x.double() @ wr.double().t()).numpy()
    assert np.abs(lg - ref).max() < 1e-5 * np.abs(ref).max() + 1e-6


def test_c_layer_agrees_with_torch_path():
    """The C restatement and the restated torch path of the reference agree: same
    routing on a tie-free case, layer output within bf16 rounding."""
    g = torch.Generator().manual_seed(3)
    T, H, I, E, K = 37, 256, 128, 8, 2
    xn = torch.randn(T, H, generator=g).to(torch.bfloat16)
    x2 = torch.randn(T, H, generator=g).to(torch.bfloat16)
    wr = (torch.randn(E, H, generator=g) * H ** -0.5).to(torch.bfloat16)
    w13 = (torch.randn(E, 2 * I, H, generator=g) * H ** -0.5).to(torch.bfloat16)
    w2 = (torch.randn(E, H, I, generator=g) * I ** -0.5).to(torch.bfloat16)
    r = oracle.moe_layer(*(oracle.bf16_bits(t) for t in (xn, x2, wr, w13, w2)), K)
    out_t, tw, ti = tp.moe_layer(xn.float(), x2.float(), wr, w13, w2, K)
    assert np.array_equal(r["topk_ids"], ti.numpy().astype(np.int32))
    assert np.allclose(r["topk_w"], tw.numpy(), rtol=1e-5)
    out_c = torch.from_numpy(oracle.bits_to_f32(r["out"]))
    rel = (out_c - out_t).norm() / out_t.norm()
    assert rel < 3e-3, float(rel)
    # the pack really is a permutation of the rows
    xp = oracle.bits_to_f32(r["xp"])
    assert np.array_equal(xp, xn.float().numpy()[r["pair_token"]])


def test_combine_definition():
    rng = np.random.default_rng(1)
    T, K, H = 5, 3, 64
    y = rng.standard_normal((T * K, H)).astype(np.float32)
    pp = rng.permutation(T * K).reshape(T, K).astype(np.int32)
    w = rng.random((T, K)).astype(np.float32)
    x2 = torch.randn(T, H).to(torch.bfloat16)
    nw = (1 + 0.1 * torch.randn(H)).to(torch.bfloat16)
    x, normed = oracle.combine(y, pp, w, oracle.bf16_bits(x2), oracle.bf16_bits(nw), eps=1e-6)
    moe = np.zeros((T, H), np.float64)
    for k in range(K):
        moe += w[:, k:k + 1].astype(np.float64) * y[pp[:, k]]
    want = tp.bf(x2.float() + torch.from_numpy(moe).float())
    got = torch.from_numpy(oracle.bits_to_f32(x))
    assert (got - want).abs().max() <= 2 * want.abs().max() * 2 ** -8
    want_n = tp.rms(got, nw, 1e-6)
    got_n = torch.from_numpy(oracle.bits_to_f32(normed))
    assert (got_n - want_n).abs().max() <= 2 * want_n.abs().max() * 2 ** -8
