"""One MoE layer as a fabric program that repeats on all SMs, timed by the in-kernel iteration
timer: the protocol of the reference's calibrator for MoE-layer tokens/s
(monoserve/calibrate/calibrator.py:309-319: T / median iteration time of a one-layer program with
iterations = 0, >= 2 warm-up and >= 6 timed iterations).

    python -m monoserve_b200.benchmarks.fabric_layer [--tokens 256] [--caps 8] [--form 64] [--reps 40]

Shapes and data are those of bench.py (benchmark configuration 2: Qwen3-30B-A3B layer, Zipf-skewed routing,
32 hot + 96 host-resident experts); `all_hot` repeats the measurement with every expert in HBM.
One JSON line.
"""
import argparse
import json
import os
import statistics
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def run(wl, hot, tokens, caps, form, reps, idle_cap=0):
    from monoserve_b200.fabric import Fabric
    from monoserve_b200.lane import MoELane
    H, I, E, K = 2048, 768, 128, 8
    fab = Fabric(pool_bytes=512 << 20)
    fab.set_max_run(120)
    if idle_cap:
        fab.set_idle_cap(idle_cap)   # longest back-off of an idle worker's poll, ns
    lane = MoELane(fab, 0, H, I, E, K, 256, wl["wr"], wl["w13"], wl["w2"], hot=hot)
    lane.set_input(wl["xs"][0][:tokens].cuda(), wl["x2s"][0][:tokens].cuda())
    h = lane.build(tokens, iterations=0)
    fab.start()
    fab.publish(map=[0] * fab.num_workers, caps=[caps], order=[0], programs=[h], forms=[form])
    time.sleep(0.05)
    it0 = fab.progress()["lanes"][0]["iterations"]
    ends = fab.iteration_times(0, it0, reps + 3, timeout=60)
    err = fab.progress()["error"]
    fab.stop()
    fab.close()
    d = [(b - a) / 1e3 for a, b in zip(ends[2:], ends[3:])]
    med = statistics.median(d)
    return {"iteration_us_p50": med, "iteration_us_min": min(d), "tokens_per_s": tokens / (med * 1e-6), "error": err}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=256)
    ap.add_argument("--caps", type=int, default=8)
    ap.add_argument("--form", type=int, default=64)
    ap.add_argument("--reps", type=int, default=40)
    ap.add_argument("--idle-cap", type=int, default=0, help="longest back-off of an idle worker's poll in ns (default: the library's)")
    ap.add_argument("--only", choices=["both", "all_hot", "config2"], default="both")
    args = ap.parse_args()
    import bench
    wl = bench.make_workload()
    line = {"workload": "one MoE layer as a repeating fabric program on all SMs (config-2 shapes)", "tokens": args.tokens,
            "caps": args.caps, "form": args.form}
    if args.only in ("both", "config2"):
        line["config2"] = run(wl, wl["hot"], args.tokens, args.caps, args.form, max(6, args.reps // 4), args.idle_cap)
    if args.only in ("both", "all_hot"):
        line["all_hot"] = run(wl, list(range(128)), args.tokens, args.caps, args.form, args.reps, args.idle_cap)
    print(json.dumps(line))


if __name__ == "__main__":
    main()
