"""The serving loop on a GPU: requests arrive while the fabric runs, prompts are prefilled in
batches, finished prompts join the decode batch through a program switch at an iteration
boundary, KV pages grow with the sequences, and every request's tokens must be what the
reference's torch oracle predicts for its own sequence (greedy sampling: at every position the
produced token is the oracle's arg-max, or its logit is within 2 % of the logit range of the
maximum - the rule of the reference's tests/test_fabric_model.py:135-137)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_engine_serves_staggered_requests():
    from oracle import torch_path as tp
    from monoserve_b200.engine import Engine, PagePool, RequestTable
    from monoserve_b200.fabric import Fabric
    from monoserve_b200.model import KVCache, ModelWeights
    from tests.test_gpu_model import load_fixture
    cfg, w, tokens, _ = load_fixture()
    fab = Fabric(num_workers=120, pool_bytes=512 << 20)     # the other SMs run the host's small copies and fills
    fab.set_max_run(120)
    try:
        weights = ModelWeights(cfg, w)
        page, n_pages, slots, bt_stride = 16, 96, 8, 8
        kv = KVCache(cfg, n_pages=n_pages, page_size=page)
        table = RequestTable(fab, slots, bt_stride)
        eng = Engine(fab, cfg, weights, kv, table, PagePool(n_pages), max_decode=4, token_budget=64)
        rng = np.random.default_rng(0)
        requests = []
        for i in range(7):    # more requests than decode rows: some wait for a free row
            n = int(rng.integers(5, 40))
            prompt = rng.integers(0, cfg.vocab, size=n).tolist() if i else tokens[:20]
            requests.append((0.02 * i, i, prompt, int(rng.integers(3, 24))))
        fab.start()
        records = eng.serve(requests, timeout_s=40)
        assert fab.progress()["error"] == 0
    finally:
        fab.stop()
        fab.close()
    assert eng.stats["decode_programs"] >= 3 and eng.stats["prefill_passes"] >= 2
    assert eng.pool.available() == n_pages - 1 and len(eng.free_slots) == slots     # everything was given back
    for t, rid, prompt, max_tokens in requests:
        r = records[rid]
        assert len(r["tokens"]) == max_tokens and r["first_token"] >= t and r["finish"] >= r["first_token"]
        seq = prompt + r["tokens"]
        logits = tp.model_logits(w, cfg, seq[:-1])
        span = float(logits.max() - logits.min())
        for j, tok in enumerate(r["tokens"]):
            row = logits[len(prompt) - 1 + j]
            assert int(row.argmax()) == tok or float(row.max() - row[tok]) < 0.02 * span, (rid, j)
