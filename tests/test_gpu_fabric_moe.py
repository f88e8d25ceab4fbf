"""One MoE layer as a fabric program (MoELane): routing / packing bit-exact against
the oracle, expert outputs within tolerance, the combine exact given y, with half of
the experts hot and half read from pinned host memory through link-gated stages; then
a prefill lane and a repeating decode lane side by side on disjoint SM floors
(the arrangement of the reference's tests/test_fabric_model.py:86-123)."""
import time

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


def weights(H, I, E, seed):
    g = torch.Generator().manual_seed(seed)
    wr = (torch.randn(E, H, generator=g) * H ** -0.5).to(torch.bfloat16)
    w13 = (torch.randn(E, 2 * I, H, generator=g) * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(E, H, I, generator=g) * 0.02).to(torch.bfloat16)
    return wr, w13, w2


def acts(T, H, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(T, H, generator=g).to(torch.bfloat16), torch.randn(T, H, generator=g).to(torch.bfloat16)


def wait_iterations(fab, lane, n, timeout=30):
    t0 = time.time()
    while fab.progress()["lanes"][lane]["iterations"] < n:
        assert time.time() - t0 < timeout, fab.progress()
        time.sleep(1e-3)


def check_lane(lane, wr, w13, w2, xn, x2, K):
    T, H = xn.shape
    P = T * K
    r = oracle.moe_layer(*(oracle.bf16_bits(t) for t in (xn, x2, wr, w13, w2)), K)
    E, I = wr.shape[0], w13.shape[1] // 2
    assert np.array_equal(lane.topk_ids[:T].cpu().numpy(), r["topk_ids"])
    assert np.array_equal(lane.topk_w[:T].cpu().numpy().view(np.int32), r["topk_w"].view(np.int32))
    assert np.array_equal(lane.starts.cpu().numpy(), r["starts"])
    assert np.array_equal(lane.pair_token[:P].cpu().numpy(), r["pair_token"])
    assert np.array_equal(lane.pair_weight[:P].cpu().numpy().view(np.int32), r["pair_weight"].view(np.int32))
    assert np.array_equal(lane.pair_pos[:T].cpu().numpy(), r["pair_pos"])
    assert np.array_equal(oracle.bf16_bits(lane.xp[:P]), r["xp"])
    y = lane.y[:P].cpu()
    rel = float((y - torch.from_numpy(r["y"])).norm() / torch.from_numpy(r["y"]).norm())
    assert rel < 1e-2, rel
    want = oracle.combine(y.numpy(), r["pair_pos"], r["topk_w"], oracle.bf16_bits(x2))
    assert np.array_equal(oracle.bf16_bits(lane.x[:T]), want)
    ref = torch.from_numpy(oracle.bits_to_f32(r["out"]))
    assert float((lane.x[:T].float().cpu() - ref).norm() / ref.norm()) < 1e-2
    assert int(lane.counts.abs().sum()) == 0, "the expander zeroes the counts for the next layer"


@pytest.mark.parametrize("form", [64, 0])
@pytest.mark.parametrize("pack_hot", [True, False])
def test_moe_layer_program(form, pack_hot):
    from monoserve_b200.fabric import Fabric
    from monoserve_b200.lane import MoELane
    T, H, I, E, K = 70, 512, 256, 16, 4
    wr, w13, w2 = weights(H, I, E, 1)
    xn, x2 = acts(T, H, 2)
    fab = Fabric(pool_bytes=128 << 20)
    fab.set_max_run(60)
    try:
        lane = MoELane(fab, 0, H, I, E, K, 96, wr, w13, w2, hot=list(range(0, E, 2)), pack_hot=pack_hot)
        lane.set_input(xn.cuda(), x2.cuda())
        h = lane.build(T, iterations=2)
        fab.start()
        fab.reset_inflight_max(0)
        fab.publish(map=[0] * fab.num_workers, caps=[4], order=[0], programs=[h], forms=[form])
        wait_iterations(fab, 0, 2)
        stats = fab.lane_stats(0)
        fab.stop()
        assert fab.progress()["error"] == 0
        assert 1 <= stats["inflight_max"] <= 4
        check_lane(lane, wr, w13, w2, xn, x2, K)
    finally:
        fab.stop()
        fab.close()


@pytest.mark.parametrize("hot", ["none", "half"])
def test_staged_form_reads_each_expert_once(hot):
    """Form 0 with a staging stack: host-resident experts with more rows than the threshold are
    copied into HBM by fetch tiles and computed from the copy.  The result is bit-identical to the
    unstaged form-0 run (same 256-row blocks over the same bytes), and routing and packing stay
    bit-exact against the oracle."""
    from monoserve_b200.fabric import Fabric
    from monoserve_b200.lane import MoELane
    T, H, I, E, K = 900, 512, 256, 8, 2     # ~225 rows per expert; threshold 200: most are staged, some not
    wr, w13, w2 = weights(H, I, E, 5)
    xn, x2 = acts(T, H, 6)
    hot_list = [] if hot == "none" else list(range(0, E, 2))
    outs = []
    for staged in (False, True):
        fab = Fabric(pool_bytes=128 << 20)
        fab.set_max_run(60)
        try:
            lane = MoELane(fab, 0, H, I, E, K, 1024, wr, w13, w2, hot=hot_list, staged=staged, staged_min_rows=200,
                           fetch_chunk=96 * 1024)
            lane.set_input(xn.cuda(), x2.cuda())
            h = lane.build(T, iterations=2)
            fab.start()
            fab.publish(map=[0] * fab.num_workers, caps=[4], order=[0], programs=[h], forms=[0])
            wait_iterations(fab, 0, 2)
            stats = fab.lane_stats(0)
            fab.stop()
            assert fab.progress()["error"] == 0
            assert stats["inflight_max"] <= 4
            if staged:
                check_lane(lane, wr, w13, w2, xn, x2, K)
                counts = np.diff(lane.starts.cpu().numpy())
                cold = [e for e in range(E) if e not in hot_list]
                assert any(counts[e] > 200 for e in cold) and any(counts[e] <= 200 for e in range(E))
                for e in cold:
                    if counts[e] > 200:   # the staged copy of an expert is its host tensor
                        assert torch.equal(lane.stage_w13[e].cpu(), w13[e])
                        assert torch.equal(lane.stage_w2[e].cpu(), w2[e])
            outs.append((lane.x[:T].cpu().clone(), lane.y[:T * K].cpu().clone()))
        finally:
            fab.stop()
            fab.close()
    assert torch.equal(outs[0][1], outs[1][1]), "expert outputs: staged == unstaged, bit for bit"
    assert torch.equal(outs[0][0], outs[1][0])


def test_qwen3_shape_layer_program_staged_and_permuted():
    """Benchmark configuration 1 shape in the fabric (E 128, top-8, H 2048, I 768; 64 decode tokens + one
    512-token prefill; half of the experts host-resident), form 0 with the staging stack and a threshold of
    32 rows, so the run mixes hot experts, host experts read in place and staged experts: routing and packing
    bit-exact against the C oracle, output against the reference's torch path; then the size-independent
    property: the layer is permutation-equivariant over tokens, bit for bit, although a permutation changes
    every expert's row order and which tiles run where."""
    from monoserve_b200.fabric import Fabric
    from monoserve_b200.lane import MoELane
    from oracle import torch_path as tp
    T, H, I, E, K = 576, 2048, 768, 128, 8
    g = torch.Generator().manual_seed(0)
    wr = (torch.randn(E, H, generator=g) * 0.02).to(torch.bfloat16)
    w13 = (torch.randn(E, 2 * I, H, generator=g) * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(E, H, I, generator=g) * 0.02).to(torch.bfloat16)
    g1 = torch.Generator().manual_seed(1)
    xn = torch.randn(T, H, generator=g1).to(torch.bfloat16)
    x2 = torch.zeros(T, H, dtype=torch.bfloat16)
    perm = torch.randperm(T, generator=g1)
    fab = Fabric(pool_bytes=512 << 20)
    fab.set_max_run(120)
    outs = []
    try:
        lane = MoELane(fab, 0, H, I, E, K, T, wr, w13, w2, hot=list(range(64)), staged=True, staged_min_rows=32)
        for x_in in (xn, xn[perm].contiguous()):
            lane.set_input(x_in.cuda(), x2.cuda())
            h = lane.build(T, iterations=1)
            fab.start()
            fab.publish(map=[0] * fab.num_workers, caps=[8], order=[0], programs=[h], forms=[0])
            wait_iterations(fab, 0, fab.progress()["lanes"][0]["iterations"] + 1, timeout=60)
            fab.stop()
            assert fab.progress()["error"] == 0
            outs.append(lane.x[:T].cpu().clone())
            if len(outs) == 1:
                logits = oracle.router_logits(oracle.bf16_bits(xn), oracle.bf16_bits(wr))
                ids, w, counts = oracle.router_topk(logits, K)
                starts = oracle.scan(counts)
                pt, pw, pp = oracle.pack(ids, w, starts)
                P = T * K
                assert np.array_equal(lane.topk_ids[:T].cpu().numpy().ravel(), ids.ravel())
                assert np.array_equal(lane.topk_w[:T].cpu().numpy().view(np.int32).ravel(), w.view(np.int32).ravel())
                assert np.array_equal(lane.starts.cpu().numpy(), starts)
                assert np.array_equal(lane.pair_token[:P].cpu().numpy(), pt)
                assert np.array_equal(lane.pair_pos[:T].cpu().numpy().ravel(), pp.ravel())
                assert (counts[64:] > 32).any() and (counts[64:] <= 32).any(), "staged and unstaged host experts"
                routing = (torch.from_numpy(w), torch.from_numpy(ids.astype(np.int64)))
                ref, _, _ = tp.moe_layer(xn.float(), x2.float(), wr, w13, w2, K, routing=routing)
                rel = float((outs[0].float() - ref).norm() / ref.norm())
                assert rel < 1e-2, rel
    finally:
        fab.stop()
        fab.close()
    assert torch.equal(outs[1], outs[0][perm])


def test_prefill_and_decode_lanes_side_by_side():
    from monoserve_b200.fabric import Fabric
    from monoserve_b200.lane import MoELane
    H, I, E, K = 512, 256, 16, 4
    wr, w13, w2 = weights(H, I, E, 3)
    xp_in, xp_res = acts(600, H, 4)
    xd_in, xd_res = acts(24, H, 5)
    fab = Fabric(pool_bytes=256 << 20)
    fab.set_max_run(60)
    try:
        hot = list(range(8))
        pre = MoELane(fab, 0, H, I, E, K, 600, wr, w13, w2, hot=hot)
        dec = MoELane(fab, 1, H, I, E, K, 32, wr, w13, w2, hot=hot)
        pre.set_input(xp_in.cuda(), xp_res.cuda())
        dec.set_input(xd_in.cuda(), xd_res.cuda())
        hp = pre.build(600, iterations=3)
        hd = dec.build(24, iterations=0)      # the decode lane repeats until replaced
        n = fab.num_workers
        lanes = [0] * (n // 2) + [1] * (n - n // 2)
        fab.start()
        fab.publish(map=lanes, caps=[8, 4], order=[0, 1], programs=[hp, hd], forms=[64, 64])
        ends = fab.iteration_times(1, 0, 6, timeout=30)
        wait_iterations(fab, 0, 3)
        fab.stop()
        assert fab.progress()["error"] == 0
        assert all(b > a for a, b in zip(ends, ends[1:]))
        check_lane(pre, wr, w13, w2, xp_in, xp_res, K)
        # the decode lane stopped mid-iteration; its last complete results are still those of its batch
        r = oracle.moe_layer(*(oracle.bf16_bits(t) for t in (xd_in, xd_res, wr, w13, w2)), K)
        assert np.array_equal(dec.topk_ids[:24].cpu().numpy(), r["topk_ids"])
    finally:
        fab.stop()
        fab.close()


@pytest.mark.parametrize("pack_hot", [True, False])
def test_glm_style_layer_program(pack_hot):
    """The GLM-style layer of the reference's tests/test_fabric_model_glm.py:57-67 as a fabric program:
    sigmoid scoring with a selection bias and a routed scale, FP8-e4m3 experts with per-output-channel
    scales (half of them hot, half read over the link), and a shared expert that every token passes
    through; against the torch oracle on the de-quantised weights, FP8 tolerance rel-L2 <= 3e-2."""
    from monoserve_b200.fabric import Fabric
    from monoserve_b200.lane import MoELane
    from oracle import torch_path as tp
    T, H, I, E, K, Is = 90, 512, 256, 16, 4, 384
    g = torch.Generator().manual_seed(31)
    wr = (torch.randn(E, H, generator=g) * H ** -0.5).to(torch.bfloat16)
    bias = torch.randn(E, generator=g) * 0.2
    q13, s13, d13 = tp.quantize_fp8(torch.randn(E, 2 * I, H, generator=g) * 0.05)
    q2, s2, d2 = tp.quantize_fp8(torch.randn(E, H, I, generator=g) * 0.05)
    sw13 = (torch.randn(2 * Is, H, generator=g) * 0.05).to(torch.bfloat16)
    sw2 = (torch.randn(H, Is, generator=g) * 0.05).to(torch.bfloat16)
    xn, x2 = acts(T, H, 32)
    fab = Fabric(pool_bytes=128 << 20)
    fab.set_max_run(60)
    try:
        lane = MoELane(fab, 0, H, I, E, K, 96, wr, q13, q2, hot=list(range(1, E, 2)), pack_hot=pack_hot,
                       scales=(s13, s2), scoring=1, bias=bias, routed_scale=2.5, shared=(sw13, sw2))
        lane.set_input(xn.cuda(), x2.cuda())
        h = lane.build(T, iterations=2)
        fab.start()
        fab.publish(map=[0] * fab.num_workers, caps=[4], order=[0], programs=[h], forms=[64])
        wait_iterations(fab, 0, 2)
        fab.stop()
        assert fab.progress()["error"] == 0
        ids, w = lane.topk_ids[:T].cpu().long(), lane.topk_w[:T].cpu()
        tw_ref, ti_ref = tp.route(xn.float(), wr, K, scoring="sigmoid", bias=bias, renorm=True, routed_scale=2.5)
        agree = (ids.sort(-1).values == ti_ref.sort(-1).values).all(-1).float().mean().item()
        assert agree > 0.97, agree            # the projection's summation order differs from torch's in the last bit
        ref, _, _ = tp.moe_layer(xn.float(), x2.float(), wr, d13, d2, K, routing=(w, ids),
                                 shared=(sw13.float(), sw2.float()))
        got = lane.x[:T].float().cpu()
        rel = float((got - ref).norm() / ref.norm())
        assert rel < 3e-2, rel
        # the shared expert alone, bf16 weights: tight
        sh = tp.ffn(xn.float(), sw13.float(), sw2.float())
        rel_s = float((lane.shared["y"][:T].cpu() - sh).norm() / sh.norm())
        assert rel_s < 1e-2, rel_s
    finally:
        fab.stop()
        fab.close()
