"""The host loop beside a running fabric: while a prefill program of the tiny Qwen3-style model
repeats, the loop's thread follows the lane's marks, stages host-resident experts of the coming
layer into the lane's staging buffer with the copy engine, switches their table entries and
switches them back when the layer is done (the arrangement of the reference's
monoserve/runtime/host_loop.py with csrc/host/host_loop.cpp).  Whatever the timing of the
copies, every iteration computes the golden logits: an expert is read either from pinned host
memory or from its staged copy, never from a half-written slot."""
import time

import pytest
import torch

from tests.test_gpu_model import check_logits, load_fixture

pytestmark = pytest.mark.gpu


def test_staging_by_the_copy_engine_keeps_the_logits_and_restores_the_tables():
    from monoserve_b200.fabric import Fabric
    from monoserve_b200.host_loop import HostLoop
    from monoserve_b200.model import KVCache, ModelLane, ModelWeights
    cfg, w, tokens, ref = load_fixture()
    hot = [list(range(l % 2, cfg.num_experts, 2)) for l in range(cfg.num_layers)]
    weights = ModelWeights(cfg, w, hot=hot)
    weights.alloc_staging(slots=2 * 4)                     # two halves of four experts
    kv = KVCache(cfg, n_pages=16, page_size=16)
    fab = Fabric(pool_bytes=256 << 20)
    fab.set_max_run(120)
    loop = None
    try:
        lane = ModelLane(fab, 0, cfg, weights, kv, max_tokens=64, max_slots=4, bt_stride=8, staging_index=0)
        lane.set_pages(1, [3, 1, 2])
        iterations = 400
        h = lane.build_prefill([(1, tokens, 0)], iterations=iterations, all_logits=True)
        before = lane.tables.cpu().clone()
        loop = HostLoop(fab, weights)
        loop.add_prefill_lane(lane, 0)
        fab.start()
        loop.start(poll_us=5)
        fab.publish(map=[0] * fab.num_workers, caps=[4], order=[0], programs=[h])
        t0 = time.time()
        while fab.progress()["lanes"][0]["iterations"] < iterations:
            assert time.time() - t0 < 60, (fab.progress()["error"], fab.wait_notes())
            time.sleep(1e-3)
        loop.stop()
        stats = loop.stats()
        fab.stop()
        assert fab.progress()["error"] == 0
        check_logits(lane.logits[:len(tokens)].cpu(), ref)
        assert stats["copies"] > 0 and stats["flips"] > 0, stats
        assert stats["restores"] == stats["flips"], stats
        w13_bytes, w2_bytes = weights.expert_bytes()
        assert stats["bytes"] == stats["copies"] * (w13_bytes + w2_bytes)
        torch.cuda.synchronize()
        assert torch.equal(lane.tables.cpu(), before), "after stop every entry is back where it was"
        # what was staged last is still in the buffer: each slot holds some expert of some layer, byte for byte
        staged = weights.stage_w13[0].cpu()
        pool = [weights.host_w13[l][e] for l in range(cfg.num_layers) for e in range(cfg.num_experts)]
        for slot in range(staged.shape[0]):
            if staged[slot].abs().sum() > 0:
                assert any(torch.equal(staged[slot], t) for t in pool)
    finally:
        if loop is not None:
            loop.stop()
            loop.close()
        fab.stop()
        fab.close()
