"""The control plane on the CPU: time estimator and plan search against a hand-written
calibration whose curves have the shapes a calibration run measures (rates that rise with the
SM share and saturate, a link rate that grows with the credits up to the link's peak, a
read stretch that grows with exposure).  The scenarios, the calibration numbers and the
expected values are those of the reference's tests/test_control.py:21-252, restated for this
library's Python mirror (monoserve_b200.control)."""
import math
import types

import pytest

import numpy as np

from monoserve_b200.control import (ASYM, Admission, AdmissionConfig, Curve, Estimator, EstimatorOptions, LaneWork,
                                    PlanSearch, Request, Seq, load_calibration, model_shape, profile_view)

SMS = 132
GRID = [8, 16, 24, 32, 48, 64, 96, 132]
LINK_US, PEAK_GBPS = 0.83, 400.0


def solo(tflops, gbps, knee, q):
    return {"sms": GRID, "tflops": [tflops * s / SMS for s in GRID], "gbps": [gbps * min(1.0, s / knee) for s in GRID],
            "q_per_sm": q}


def credit_sweep(efficiency):
    credits = [128, 256, 512, 1024, 2048, 4096, 8192, 10400, 12000]
    return {"credits": credits, "gbps": [min(PEAK_GBPS * efficiency, n * 32 / (LINK_US * 1e-6) / 1e9) for n in credits]}


CAL = {
    "sms": SMS, "R_H_us": 0.34, "R_C_us": LINK_US, "q_max": 96,
    "gamma": {"exposure_entry_us": [2000, 4000, 8000, 12000, 16000], "stretch": [1.0, 1.15, 1.5, 2.0, 2.5]},
    "dense": solo(600, 3600, 70, 64), "attn_prefill": solo(450, 3000, 80, 48), "attn_decode": solo(150, 3200, 64, 80),
    "expert": {"16": solo(160, 3400, 64, 96), "32": solo(300, 3400, 64, 96), "64": solo(480, 3400, 64, 96),
               "128": solo(620, 3400, 64, 96), "asym": solo(320, 3200, 64, 72)},
    "rho": {"16": credit_sweep(1.0), "32": credit_sweep(1.0), "64": credit_sweep(1.0), "128": credit_sweep(1.0),
            "asym": credit_sweep(0.8)},
    "q_form": {"16": 96, "32": 96, "64": 128, "128": 160, "asym": 64},
    "beta_gbps": PEAK_GBPS, "reference_form": 64, "layer_overhead_us": 4.0, "tail_overhead_us": 30.0,
}
QWEN = types.SimpleNamespace(hidden=2048, intermediate=768, num_experts=128, top_k=8, num_layers=48, num_heads=32,
                             num_kv_heads=4, head_dim=128, vocab=151936)


@pytest.fixture(scope="module")
def cal():
    return load_calibration(CAL)


@pytest.fixture(scope="module")
def est(cal):
    return Estimator(model_shape(QWEN), cal)


def blind(cal):
    o = EstimatorOptions()
    o.contention_aware = False
    return Estimator(model_shape(QWEN), cal, o)


def decode_work(batch=8, context=2000, active=27.0, miss=5.0, tpot=0.05):
    w = LaneWork()
    w.decode = True
    w.passes = [[Seq(1, context) for _ in range(batch)]]
    w.active, w.miss, w.deadline = [active] * 48, [miss] * 48, tpot
    return w


def prefill_work(tokens=(4096,), deadline=2.0, staging=0, active=120.0, miss=30.0):
    w = LaneWork()
    w.passes = [[Seq(t, 0) for t in tokens]]
    w.active, w.miss, w.staging, w.deadline = [active] * 48, [miss] * 48, staging, deadline
    return w


def test_curve_ends():
    through_origin = Curve([8.0, 16.0], [80.0, 160.0], True)
    assert through_origin(4) == pytest.approx(40) and through_origin(12) == pytest.approx(120)
    assert through_origin(64) == pytest.approx(160)
    assert Curve([8.0, 16.0], [80.0, 160.0])(4) == pytest.approx(80)
    assert Curve()(3) == 0.0


def test_link_budget_and_exposure_bound(est, cal):
    # Q^link: the fewest credits at which the reference form reaches 99 % of the peak, on the piecewise-linear curve
    sweep = CAL["rho"]["64"]
    i = next(k for k, g in enumerate(sweep["gbps"]) if g >= 0.99 * PEAK_GBPS)
    x0, x1, y0, y1 = sweep["credits"][i - 1], sweep["credits"][i], sweep["gbps"][i - 1], sweep["gbps"][i]
    q_link = x0 + (0.99 * PEAK_GBPS - y0) / (y1 - y0) * (x1 - x0)
    assert est.link_credits == pytest.approx(q_link)
    assert est.exposure_bound == pytest.approx(q_link * 0.83e-6 + 96 * 132 * 0.34e-6)
    assert est.gamma_ratio(0.0) == pytest.approx(cal.gamma(est.exposure_bound))
    assert est.gamma_ratio(est.exposure_bound) == pytest.approx(1.0)
    assert blind(cal).gamma_ratio(0.0) == 1.0


def test_estimate_falls_with_share(est):
    for work in (decode_work(), prefill_work()):
        load = est.load(work)
        t = [est.evaluate(load, s, est.link_credits, 64).total for s in range(1, SMS + 1)]
        assert all(b <= a * (1 + 1e-12) for a, b in zip(t, t[1:]))


def test_link_term(est, cal):
    load = est.load(decode_work(batch=8, active=27.0, miss=5.0))
    s, credits = 40, 2048.0
    e = est.evaluate(load, s, credits, 16)
    # a decode batch bounds an expert's rows by its size: one pass of a 16-row block
    assert e.m_link == pytest.approx(5.0 * model_shape(QWEN).expert_bytes / cal.rho_at(16, min(96 * s, credits)))


def test_staging_guarantee(est, cal):
    s, credits, form = 64, 4096.0, 64
    w = model_shape(QWEN).expert_bytes
    e = est.evaluate(est.load(prefill_work((8192,), staging=16)), s, credits, form)
    assert e.staged == pytest.approx(min(30.0, 16, math.floor(cal.rho_at(form, credits) * e.attn / w)))
    e0 = est.evaluate(est.load(prefill_work((8192,), staging=0)), s, credits, form)
    assert e0.staged == 0 and e.m_link < e0.m_link


def test_one_pass_form_reads_each_expert_once(est, cal):
    # 2048 tokens x top-8 over 128 experts: 128 rows per expert, eight 16-row passes against one
    load = est.load(prefill_work((2048,), active=128.0, miss=40.0))
    s, credits = 64, 8192.0
    blocks, once = est.evaluate(load, s, credits, 16), est.evaluate(load, s, credits, ASYM)
    bytes_blocks = blocks.m_link * cal.rho_at(16, min(96 * s, credits))
    bytes_once = once.m_link * cal.rho_at(ASYM, min(64 * s, credits))
    assert bytes_blocks / bytes_once == pytest.approx(8.0)


def test_one_pass_form_of_this_library_has_no_partial_sum_traffic(cal):
    """With the calibration keys of this library (256-row blocks, partial sums in TMEM) the one-pass
    form's HBM term has no partial-sum bytes: it is below the reference kernel's on the same load."""
    d = dict(CAL, one_pass_rows=256, one_pass_row_bytes=0.0)
    own = Estimator(model_shape(QWEN), load_calibration(d))
    ref = Estimator(model_shape(QWEN), cal)
    work = prefill_work((8192,), active=128.0, miss=100.0)
    a, b = own.evaluate(own.load(work), 64, 8192.0, ASYM), ref.evaluate(ref.load(work), 64, 8192.0, ASYM)
    assert a.m_rd < b.m_rd and a.m_link == pytest.approx(b.m_link)


def test_deadline_floor_is_the_smallest_share(est):
    search = PlanSearch(est)
    for work in (decode_work(tpot=0.03), prefill_work(deadline=0.8)):
        load = est.load(work)
        for form in (16, 64, ASYM):
            brute = next((s for s in range(1, SMS + 1) if est.evaluate(load, s, 4096.0, form).total <= work.deadline),
                         SMS + 1)
            assert search.deadline_floor(load, 4096.0, form) == brute


def test_search_with_two_prefill_lanes(est):
    search = PlanSearch(est)
    works = [decode_work(batch=16, context=1000, tpot=0.05), prefill_work((1000,) * 4, deadline=2.0, staging=32),
             prefill_work((16384,), deadline=10.0, staging=32)]
    lanes = [est.load(w) for w in works]
    plan = search.solve(lanes, decode_key=7)
    assert plan.feasible and plan.min_slack >= 0
    assert sum(p.sms for p in plan.lanes) <= SMS
    assert sum(p.credits for p in plan.lanes) <= est.link_credits * 1.01 + 3 * 160
    assert sum(p.rate for p in plan.lanes) <= PEAK_GBPS * 1e9 * 1.01
    for p, w in zip(plan.lanes, works):
        assert p.est.total <= w.deadline and p.cap >= 1
    again = search.solve(lanes, decode_key=7)   # the decode lane's options are remembered under the key
    assert again.feasible and again.evaluations < plan.evaluations


def test_search_reports_infeasible(est):
    plan = PlanSearch(est).solve([est.load(prefill_work((65536,), deadline=0.01))])
    assert not plan.feasible and len(plan.lanes) == 1 and plan.lanes[0].sms == SMS


def test_contention_blind_estimates_are_smaller(est, cal):
    mca = blind(cal)
    work = decode_work(batch=32, context=4000, tpot=0.03)
    for s in (16, 64, 132):
        assert mca.evaluate(mca.load(work), s, 1e9, 64).total <= est.evaluate(est.load(work), s, est.link_credits, 64).total
    assert PlanSearch(mca).deadline_floor(mca.load(work), mca.link_credits, 64) <= \
        PlanSearch(est).deadline_floor(est.load(work), est.link_credits, 64)


def test_bad_inputs_are_refused(cal):
    bad = load_calibration(CAL)
    bad.sms = 0
    with pytest.raises(RuntimeError, match="SM count"):
        Estimator(model_shape(QWEN), bad)
    est = Estimator(model_shape(QWEN), cal)
    with pytest.raises(RuntimeError, match="credit sweep"):
        est.evaluate(est.load(decode_work()), 8, 100.0, 48)   # no such kernel form
    with pytest.raises(RuntimeError, match="decode lane must be the first"):
        PlanSearch(est).solve([est.load(prefill_work()), est.load(decode_work())])


# ---------------------------------------------------------------- profile view and admission
def test_profile_view_expectations():
    p = np.full((2, 8), 1 / 8)
    view = profile_view(p, p, [[0, 1, 2, 3], []])
    a, m = view.expected(True, 0, 1.0)
    assert a == pytest.approx(1.0) and m == pytest.approx(0.5)
    a, m = view.expected(True, 0, 4096.0)
    assert a == pytest.approx(8, rel=1e-3) and m == pytest.approx(4, rel=1e-3)
    a, m = view.expected(False, 1, 16.0)
    assert m == pytest.approx(a) and a == pytest.approx(8 * (1 - (7 / 8) ** 16), rel=1e-9)


def make_admission(est, **cfg):
    c = AdmissionConfig()
    c.kv_bytes_per_token = model_shape(QWEN).kv_bytes_per_token
    for k, v in cfg.items():
        setattr(c, k, v)
    p = np.full((48, 128), 1 / 128)
    return Admission(est, PlanSearch(est), profile_view(p, p, [list(range(100))] * 48), c)


def test_admission_lanes_join_and_finish(est):
    adm = make_admission(est, token_budget=8192, staging_experts=32)
    d = adm.arrive(Request(1, 2000, 256, 0.0, 2.0, 0.05), 0.0)
    assert d.publish and d.feasible and d.pass_lanes == [1] and d.passes[0].reqs == [1]
    d = adm.arrive(Request(2, 3000, 256, 0.01, 2.0, 0.05), 0.01)
    assert d.pass_lanes == [2] and d.lanes == [1, 2]
    d = adm.arrive(Request(3, 1000, 256, 0.02, 2.0, 0.05), 0.02)
    assert not d.publish and adm.queued == 1        # both prefill lanes are busy
    d = adm.pass_done(1, 0.3)                       # request 1's first token is out
    assert d.joined == [1] and d.pass_lanes == [1] and d.passes[0].reqs == [3]
    assert d.lanes == [0, 2, 1] and d.feasible
    d = adm.finished(1, 0.5)
    assert d.publish and d.decode_changed and d.decode == []
    assert adm.kv_reserved == pytest.approx((3000 + 256 + 1000 + 256) * model_shape(QWEN).kv_bytes_per_token)


def test_admission_chunks_long_prompts(est):
    adm = make_admission(est, token_budget=4096)
    d = adm.arrive(Request(9, 10000, 16, 0.0, 30.0, 0.1), 0.0)
    assert d.pass_lanes == [1]
    p = d.passes[0]
    assert (p.tokens, p.pos0, p.last) == ([3334], [0], [0])
    d = adm.pass_done(1, 1.0)
    assert d.pass_lanes[0] == 1 and d.passes[0].pos0 == [3334]
    d = adm.pass_done(1, 2.0)
    assert d.passes[0].tokens == [3332] and d.passes[0].last == [1]
    d = adm.pass_done(1, 3.0)
    assert d.joined == [9]


def test_admission_rejects_only_hopeless_requests(est):
    kv = model_shape(QWEN).kv_bytes_per_token
    adm = make_admission(est, kv_capacity=kv * 3000)
    d = adm.arrive(Request(1, 65536, 16, 0.0, 1e-4, 0.05), 0.0)
    assert d.rejected == [1] and adm.queued == 0
    d = adm.arrive(Request(2, 2000, 256, 0.0, 5.0, 0.05), 0.0)
    assert d.pass_lanes == [1]
    # memory, not the deadline, holds this one back: it stays queued
    d = adm.arrive(Request(3, 2000, 256, 0.0, 5.0, 0.05), 0.0)
    assert d.pass_lanes == [] and d.rejected == [] and adm.queued == 1


def test_behind_republishes(est):
    adm = make_admission(est)
    adm.arrive(Request(1, 4000, 64, 0.0, 3.0, 0.05), 0.0)
    adm.progress(1, 20)
    d = adm.behind(1, 0.5)
    assert d.publish and d.lanes == [1] and d.searches == 1
    with pytest.raises(RuntimeError, match="already known"):
        adm.arrive(Request(1, 10, 1, 0.0, 1.0, 0.05), 0.6)
    with pytest.raises(RuntimeError, match="not open"):
        adm.pass_done(2, 0.7)


def test_committed_b200_calibration_plans_the_mixed_workload():
    """The calibration shipped with the package loads, and the search over it gives the offload workload
    (128 decoding sequences beside 4 prompts of 2048 tokens, half of the experts host-resident) a feasible
    plan that hands most link credits to the decode lane and the single-pass form to the prefill lane."""
    from monoserve_b200.benchmarks import mixed_lane as ml
    cfg = ml.q_config(48)
    rng = np.random.default_rng(0)
    hot = [sorted(rng.permutation(128)[:64].tolist()) for _ in range(48)]
    ctx = rng.integers(512, 8193, size=128).tolist()
    args = types.SimpleNamespace(tpot=1.0, ttft=3.0, prompt_len=2048, prompts=4)
    plan = ml.search_plan(cfg, args, ctx, hot, False)
    assert plan["feasible"] and sum(plan["sms"]) <= 148 and min(plan["sms"]) >= 1
    assert plan["caps"][0] > plan["caps"][1] >= 1 and sum(plan["caps"]) <= 16
    assert plan["forms"][1] == 0 and plan["forms"][0] in (64, 128, 256)
    assert plan["estimated_s"][0] <= 1.0 and plan["estimated_s"][1] <= 3.0
    args.tpot = 0.3          # below what the link alone allows for the decode lane's host-resident experts
    assert not ml.search_plan(cfg, args, ctx, hot, False)["feasible"]
