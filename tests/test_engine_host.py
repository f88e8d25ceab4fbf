"""Host-side pieces of the serving loop that need no GPU: the arrival process and length draws of
benchmark configuration 5, and the KV page pool."""
import numpy as np
import pytest

from monoserve_b200.engine import PagePool, arrival_times, lognormal_lengths


def test_poisson_arrivals_share_one_pattern_across_rates():
    a, b = arrival_times(2.0, seed=3, num=200), arrival_times(32.0, seed=3, num=200)
    assert a[0] == 0.0 and np.all(np.diff(a) > 0) and len(a) == 200
    assert np.allclose(a * 2.0, b * 32.0)                      # the same unit exponentials, scaled by the rate
    gaps = np.diff(arrival_times(8.0, seed=0, num=20000))
    assert gaps.mean() == pytest.approx(1 / 8.0, rel=0.03)     # exponential gaps: mean 1 / rate, cv 1
    assert gaps.std() == pytest.approx(1 / 8.0, rel=0.05)


def test_lognormal_lengths_are_clipped_and_centred():
    prompts = lognormal_lengths(20000, median=256, sigma=1.0, lo=16, hi=4096, seed=0)
    outputs = lognormal_lengths(20000, median=200, sigma=0.8, lo=8, hi=2048, seed=1)
    assert prompts.min() >= 16 and prompts.max() <= 4096 and outputs.min() >= 8 and outputs.max() <= 2048
    assert np.median(prompts) == pytest.approx(256, rel=0.05) and np.median(outputs) == pytest.approx(200, rel=0.05)


def test_page_pool_never_hands_out_the_sink_or_a_page_twice():
    pool = PagePool(10)
    a = pool.take(4)
    b = pool.take(5)
    assert 0 not in a + b and len(set(a + b)) == 9 and pool.available() == 0
    with pytest.raises(MemoryError):
        pool.take(1)
    pool.give(a)
    assert sorted(pool.take(4)) == sorted(a)


def test_search_planner_splits_the_workers_between_the_lanes():
    """The engine's planner: the control plane's plan search over the committed B200 calibration gives the decode
    lane a share that grows with its batch and shrinks when the prefill pass grows; one lane alone needs no split."""
    from monoserve_b200.benchmarks.mixed_lane import q_config
    from monoserve_b200.engine import SearchPlanner
    cfg = q_config(48)
    planner = SearchPlanner(cfg, [list(range(cfg.num_experts))] * cfg.num_layers, tpot_s=0.05, ttft_s=0.5)
    assert planner.split([], [300], 140) is None and planner.split([100], [], 140) is None
    small = planner.split([1000] * 4, [4000], 140)
    large = planner.split([4000] * 128, [300], 140)
    assert 1 <= small < 140 and 1 <= large < 140 and large >= small
    assert planner.stats["searches"] == 2 and planner.stats["micros"] > 0
