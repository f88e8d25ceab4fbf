"""The whole decoder as fabric lane programs against the reference's torch oracle: the
scenario of the reference's tests/test_fabric_model.py:86-137 (a tiny Qwen3-style model,
teacher-forced logits of a 41-token prompt; "arg-max equal or within 2 % of the logit
range") on the golden logits that the reference's own `reference_logits` produced
(tests/golden/qwen_tiny_reference_logits.npz), with all experts in HBM and with half of
them read from pinned host memory through link-gated stages; then the same positions
reached by decode steps on top of a shorter prefill."""
import os
import time
import types

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def load_fixture():
    from tests.test_oracle_golden import _load_make_golden
    g = np.load(os.path.join(GOLD, "qwen_tiny_reference_logits.npz"))
    H, I, E, K, L, hq, hkv, V = [int(v) for v in g["cfg"]]
    cfg = types.SimpleNamespace(hidden=H, intermediate=I, num_experts=E, top_k=K, num_layers=L, num_heads=hq,
                                num_kv_heads=hkv, head_dim=128, vocab=V, rope_theta=float(g["rope_theta"]),
                                rms_eps=float(g["rms_eps"]), rotary_dim=128)
    w = _load_make_golden().make_weights(cfg, int(g["weights_seed"]))
    return cfg, w, g["tokens"].tolist(), torch.from_numpy(g["logits"])


def run_once(fab, handle, caps=(4,), timeout=30, forms=None):
    before = fab.progress()["lanes"][0]["iterations"]
    fab.publish(map=[0] * fab.num_workers, caps=list(caps), order=[0], programs=[handle],
                **({"forms": list(forms)} if forms else {}))
    t0 = time.time()
    while fab.progress()["lanes"][0]["iterations"] < before + 1:
        assert time.time() - t0 < timeout, (fab.progress()["error"], fab.wait_notes())
        time.sleep(1e-3)
    assert fab.progress()["error"] == 0


def check_logits(got, ref):
    """tests/test_fabric_model.py:135-137: per position, the arg-max agrees or the logits are
    within 2 % of the logit range; here additionally the mean error is small."""
    rng = float(ref.max() - ref.min())
    err = (got - ref).abs()
    assert float(err.max()) < 0.02 * rng, (float(err.max()), rng)
    assert float(err.mean()) < 0.002 * rng
    agree = (got.argmax(-1) == ref.argmax(-1)).float().mean().item()
    assert agree > 0.9, agree


def check_logits_away_from_ties(got, ref, tie_gap, rows=None, min_gap=5e-3, min_clear=0.7):
    """Rows whose routing is decided clearly must match closely: every logit within 3 % of the logit range
    (three layers of FP8 matrices with a routed scale of 1.5; the BF16 Qwen model is held to 2 %) and the
    median row within 1 %; a row whose K-th and K+1-th selection scores are closer than the bf16 noise of the
    activations (tie_gap < 5e-3 in some layer) may route one expert differently in any implementation that
    is not bit-identical upstream, which changes that row alone: for those the reference's own rule applies
    in its spirit (tests/test_fabric_model_glm.py:118-124 checks sampled tokens, not rows) — the row stays
    finite and within 15 % of the range."""
    rng = float(ref.max() - ref.min())
    rows = range(ref.shape[0]) if rows is None else rows
    clear = 0
    for j, i in enumerate(rows):
        err = float((got[j] - ref[i]).abs().max())
        if float(tie_gap[i]) >= min_gap:
            clear += 1
            assert err < 0.03 * rng, (i, err, float(tie_gap[i]))
        else:
            assert err < 0.15 * rng, (i, err)
    assert clear >= min_clear * len(list(rows))
    row_err = torch.stack([(got[j] - ref[i]).abs().max() for j, i in enumerate(rows)])
    assert float(row_err.median()) < 0.01 * rng, float(row_err.median())


@pytest.fixture
def fab():
    from monoserve_b200.fabric import Fabric
    f = Fabric(pool_bytes=256 << 20)
    f.set_max_run(120)
    yield f
    f.stop()
    f.close()


@pytest.mark.parametrize("placement", ["all_hot", "half_host", "half_host_staged"])
def test_prefill_logits_match_reference(fab, placement):
    """half_host_staged: form 0 with a staging stack and a threshold of 4 rows, so that most host-resident
    experts of both layers go through fetch tiles and the shared staging stack before their GEMM tiles."""
    from monoserve_b200.model import KVCache, ModelLane, ModelWeights
    cfg, w, tokens, ref = load_fixture()
    hot = None if placement == "all_hot" else [list(range(l % 2, cfg.num_experts, 2)) for l in range(cfg.num_layers)]
    weights = ModelWeights(cfg, w, hot=hot)
    kv = KVCache(cfg, n_pages=16, page_size=16)
    staged = placement == "half_host_staged"
    lane = ModelLane(fab, 0, cfg, weights, kv, max_tokens=64, max_slots=4, bt_stride=8, staged=staged,
                     staged_min_rows=4, fetch_chunk=48 * 1024)
    lane.set_pages(1, [3, 1, 2])
    h = lane.build_prefill([(1, tokens, 0)], all_logits=True)
    fab.start()
    run_once(fab, h, forms=[0] if staged else None)
    fab.stop()
    if staged:
        assert int((lane.hist[:, :] > 4).sum()) > 0, "some expert passed the staging threshold"
    check_logits(lane.logits[:len(tokens)].cpu(), ref)
    # the request's next token is the arg-max of its last row
    assert int(lane.last_token[1]) == int(lane.logits[len(tokens) - 1].argmax())
    assert int(lane.host_tokens[1, 0]) == int(lane.last_token[1]) and int(lane.host_steps[1]) == 1


def test_decode_steps_match_reference(fab):
    """Prefill 29 tokens, then 12 teacher-forced decode steps: step i must reproduce the
    reference's logits at position 29 + i (and, through them, the K/V appended by earlier steps)."""
    from monoserve_b200.model import KVCache, ModelLane, ModelWeights
    cfg, w, tokens, ref = load_fixture()
    weights = ModelWeights(cfg, w)
    kv = KVCache(cfg, n_pages=16, page_size=16)
    lane = ModelLane(fab, 0, cfg, weights, kv, max_tokens=64, max_slots=4, bt_stride=8)
    lane.set_pages(2, [5, 4, 7])
    n0 = 29
    h = lane.build_prefill([(2, tokens[:n0], 0)])   # programs are built while the fabric is stopped:
    fab.start()                                     # nothing else can run on the device beside it
    run_once(fab, h)
    fab.stop()
    got = []
    # teacher forcing needs the host between steps, so each step is its own run
    for i in range(n0, len(tokens)):
        lane.set_request(2, seq_len=i, last_token=tokens[i])
        h = lane.build_decode([2])
        fab.start()
        run_once(fab, h)
        fab.stop()
        got.append(lane.logits[0].cpu().clone())
        assert int(lane.seq_len[2]) == i + 1
    check_logits(torch.stack(got), ref[n0:])


@pytest.mark.parametrize("form", [64, 0])
def test_glm_style_model_matches_reference(fab, form):
    """The GLM-4.5-style structure of the reference's tests/test_fabric_model_glm.py:71-124 — FP8 matrices
    with per-row scales everywhere, a dense first layer, a shared expert beside the routed ones, sigmoid
    routing with a selection bias and routed scale, qkv bias, rotary embedding on half of each head, GQA
    12 / 4 — as lane programs, in both kernel forms of the host-resident experts: teacher-forced prefill
    logits of 45 tokens, then decode steps on top of a shorter prefill, against the golden logits the
    reference's own oracle produced on the same quantised weights."""
    from monoserve_b200.model import KVCache, ModelLane, ModelWeights
    from tests.test_oracle_golden import glm_fixture
    from oracle import torch_path as tp
    cfg, w, tokens, ref = glm_fixture()
    gaps = []
    tp.model_logits_glm(w, cfg, tokens, gaps=gaps)           # the oracle, for how close each row's routing is to a tie
    tie_gap = torch.stack(gaps).min(0).values
    hot = [[], list(range(8)), list(range(4, 12))]          # the reference test's placement
    weights = ModelWeights(cfg, w, hot=hot)
    kv = KVCache(cfg, n_pages=16, page_size=16)
    lane = ModelLane(fab, 0, cfg, weights, kv, max_tokens=64, max_slots=4, bt_stride=8)
    lane.set_pages(0, [2, 9, 4])
    h = lane.build_prefill([(0, tokens, 0)], all_logits=True)
    fab.start()
    before = fab.progress()["lanes"][0]["iterations"]
    fab.publish(map=[0] * fab.num_workers, caps=[4], order=[0], programs=[h], forms=[form])
    t0 = time.time()
    while fab.progress()["lanes"][0]["iterations"] < before + 1:
        assert time.time() - t0 < 30, (fab.progress()["error"], fab.wait_notes())
        time.sleep(1e-3)
    fab.stop()
    assert fab.progress()["error"] == 0
    check_logits_away_from_ties(lane.logits[:len(tokens)].cpu(), ref, tie_gap)
    # decode: prefill 40 tokens, then the last 5 positions one step at a time
    kv2 = KVCache(cfg, n_pages=16, page_size=16)
    lane2 = ModelLane(fab, 0, cfg, weights, kv2, max_tokens=64, max_slots=4, bt_stride=8)
    lane2.set_pages(1, [3, 1, 7])
    n0 = 40
    h = lane2.build_prefill([(1, tokens[:n0], 0)])
    fab.start()
    run_once(fab, h)
    fab.stop()
    got = []
    for i in range(n0, len(tokens)):
        lane2.set_request(1, seq_len=i, last_token=tokens[i])
        h = lane2.build_decode([1])
        fab.start()
        run_once(fab, h)
        fab.stop()
        got.append(lane2.logits[0].cpu().clone())
    check_logits_away_from_ties(torch.stack(got), ref, tie_gap, rows=range(n0, len(tokens)))


def test_checkpoint_loader_to_logits(fab, tmp_path):
    """A tiny Qwen3-MoE checkpoint in the Hugging Face layout goes through the checkpoint loader, the
    placement (half of every layer's experts in HBM) and a prefill program; the logits must match the
    reference's torch oracle run on the tensors the loader returned."""
    from monoserve_b200.checkpoint import read_checkpoint
    from monoserve_b200.model import KVCache, ModelLane, ModelWeights
    from oracle import torch_path as tp
    from tests.test_checkpoint import tiny_checkpoint
    tiny_checkpoint(str(tmp_path), glm=False)
    cfg, w = read_checkpoint(str(tmp_path))
    assert w.host_w13[0].is_pinned()
    weights = ModelWeights(cfg, w, hot=[list(range(l % 2, cfg.num_experts, 2)) for l in range(cfg.num_layers)])
    kv = KVCache(cfg, n_pages=16, page_size=16)
    lane = ModelLane(fab, 0, cfg, weights, kv, max_tokens=64, max_slots=4, bt_stride=8)
    lane.set_pages(0, [3, 1, 2])
    tokens = torch.randint(0, cfg.vocab, (33,), generator=torch.Generator().manual_seed(1)).tolist()
    h = lane.build_prefill([(0, tokens, 0)], all_logits=True)
    fab.start()
    run_once(fab, h)
    fab.stop()
    check_logits(lane.logits[:len(tokens)].cpu(), tp.model_logits(w, cfg, tokens))


def test_k_split_projections_match_reference(fab):
    """A model wide enough (hidden 1024, 8 query heads) for the few-row form of the dense projections: qkv and o
    run as K ranges into fp32 slabs that the rope tile and the add-norm tile add in slab order.  Prefill of 20
    tokens, then decode steps (whose attention plans run beside the layers): logits against the torch oracle."""
    from monoserve_b200.model import KVCache, ModelLane, ModelWeights
    from oracle import torch_path as tp
    from tests.test_oracle_golden import _load_make_golden
    cfg = types.SimpleNamespace(hidden=1024, intermediate=128, num_experts=8, top_k=2, num_layers=2, num_heads=8,
                                num_kv_heads=2, head_dim=128, vocab=512, rope_theta=1e6, rms_eps=1e-6, rotary_dim=128)
    w = _load_make_golden().make_weights(cfg, 11)
    weights = ModelWeights(cfg, w)
    kv = KVCache(cfg, n_pages=16, page_size=16)
    lane = ModelLane(fab, 0, cfg, weights, kv, max_tokens=64, max_slots=4, bt_stride=8)
    lane.set_pages(0, [3, 1, 2, 5])
    tokens = torch.randint(0, cfg.vocab, (26,), generator=torch.Generator().manual_seed(3)).tolist()
    ref = tp.model_logits(w, cfg, tokens)
    n0 = 20
    h = lane.build_prefill([(0, tokens[:n0], 0)], all_logits=True)
    fab.start()
    run_once(fab, h)
    fab.stop()
    check_logits(lane.logits[:n0].cpu(), ref[:n0])
    got = []
    for i in range(n0, len(tokens)):   # teacher-forced decode steps, each its own run
        lane.set_request(0, seq_len=i, last_token=tokens[i])
        h = lane.build_decode([0])
        fab.start()
        run_once(fab, h)
        fab.stop()
        got.append(lane.logits[0].cpu().clone())
    check_logits(torch.stack(got), ref[n0:])


def test_full_width_layers_match_reference(fab):
    """The benchmark's layer shapes (hidden 2048, 128 experts of width 768, top-8, 32 / 4 heads) on two layers and
    a small vocabulary: a 48-token prefill (K-split o and qkv projections at their real sizes: 8 and 2 ranges)
    and four decode steps (the small-batch stage forms: norm folded into the projection tiles, permute inside
    expand, every layer's attention plan beside the layers), half of the experts read from pinned host memory:
    logits against the torch oracle."""
    from monoserve_b200.model import KVCache, ModelLane, ModelWeights
    from oracle import torch_path as tp
    from tests.test_oracle_golden import _load_make_golden
    cfg = types.SimpleNamespace(hidden=2048, intermediate=768, num_experts=128, top_k=8, num_layers=2, num_heads=32,
                                num_kv_heads=4, head_dim=128, vocab=4096, rope_theta=1e6, rms_eps=1e-6, rotary_dim=128)
    one = types.SimpleNamespace(**{**vars(cfg), "num_layers": 1})
    w = _load_make_golden().make_weights(one, 5)   # one layer's random weights (2.4 GB of draws), used by both layers
    for name in ("in_norm", "qkv", "q_norm", "k_norm", "o", "post_norm", "router", "host_w13", "host_w2"):
        setattr(w, name, getattr(w, name) * cfg.num_layers)
    weights = ModelWeights(cfg, w, hot=[list(range(l % 2, cfg.num_experts, 2)) for l in range(cfg.num_layers)])
    kv = KVCache(cfg, n_pages=16, page_size=16)
    lane = ModelLane(fab, 0, cfg, weights, kv, max_tokens=64, max_slots=4, bt_stride=8)
    lane.set_pages(1, [6, 2, 9, 4])
    tokens = torch.randint(0, cfg.vocab, (52,), generator=torch.Generator().manual_seed(8)).tolist()
    gaps = []
    ref = tp.model_logits(w, cfg, tokens, gaps=gaps)
    # 128 experts, top-8: the 8th and 9th router logits of a row are often closer than the bf16 noise of the
    # activations (a few 1e-3 in logit units; rows under 0.012 count as near ties); such a row may pick one expert differently and is held to the
    # looser bound, every other row to 3 % of the logit range
    tie_gap = torch.stack(gaps).min(0).values
    n0 = 48
    h = lane.build_prefill([(1, tokens[:n0], 0)], all_logits=True)
    fab.start()
    run_once(fab, h, caps=(8,))
    fab.stop()
    check_logits_away_from_ties(lane.logits[:n0].cpu(), ref, tie_gap, rows=range(n0), min_gap=0.012, min_clear=0.4)
    got = []
    for i in range(n0, len(tokens)):
        lane.set_request(1, seq_len=i, last_token=tokens[i])
        h = lane.build_decode([1])
        fab.start()
        run_once(fab, h, caps=(8,))
        fab.stop()
        got.append(lane.logits[0].cpu().clone())
    check_logits_away_from_ties(torch.stack(got), ref, tie_gap, rows=range(n0, len(tokens)), min_gap=0.012, min_clear=0.25)


def test_glm_style_wide_model_takes_the_few_row_paths(fab):
    """The GLM-4.5 structure on a model wide enough (hidden 1024, 8 / 4 heads) for the few-row forms with FP8
    matrices: K-split qkv (its bias added by the first range) and o projections into fp32 slabs, the norm folded
    into the router projection's tiles with the shared expert waiting for it, the permute inside expand; a dense
    first layer beside them.  20-token prefill and three decode steps against the GLM oracle, tie-aware."""
    from monoserve_b200.model import KVCache, ModelLane, ModelWeights
    from oracle import torch_path as tp
    from tests.test_oracle_golden import _load_make_golden
    cfg = types.SimpleNamespace(hidden=1024, intermediate=128, num_experts=16, top_k=4, num_layers=3, num_heads=8,
                                num_kv_heads=4, head_dim=128, vocab=512, rope_theta=1e6, rms_eps=1e-6, rotary_dim=64,
                                dense_layers=1, dense_intermediate=256, shared_intermediate=128, scoring="sigmoid",
                                routed_scale=1.5, qk_norm=False, qkv_bias=True)
    w = _load_make_golden().make_glm_weights(cfg, 23)
    tokens = torch.randint(0, cfg.vocab, (23,), generator=torch.Generator().manual_seed(4)).tolist()
    gaps = []
    ref = tp.model_logits_glm(w, cfg, tokens, gaps=gaps)
    tie_gap = torch.stack(gaps).min(0).values
    weights = ModelWeights(cfg, w, hot=[[], list(range(8)), list(range(4, 12))])
    kv = KVCache(cfg, n_pages=16, page_size=16)
    lane = ModelLane(fab, 0, cfg, weights, kv, max_tokens=64, max_slots=4, bt_stride=8)
    lane.set_pages(0, [2, 9, 4])
    n0 = 20
    h = lane.build_prefill([(0, tokens[:n0], 0)], all_logits=True)
    fab.start()
    run_once(fab, h)
    fab.stop()
    check_logits_away_from_ties(lane.logits[:n0].cpu(), ref, tie_gap, rows=range(n0), min_clear=0.5)
    got = []
    for i in range(n0, len(tokens)):
        lane.set_request(0, seq_len=i, last_token=tokens[i])
        h = lane.build_decode([0])
        fab.start()
        run_once(fab, h)
        fab.stop()
        got.append(lane.logits[0].cpu().clone())
    check_logits_away_from_ties(torch.stack(got), ref, tie_gap, rows=range(n0, len(tokens)), min_clear=0.0)
