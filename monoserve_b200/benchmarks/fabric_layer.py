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


def run(wl, hot, tokens, caps, form, reps, idle_cap=0, trace=False):
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
    tr = None
    if trace:   # the stage timeline (activation / completion of every stage), decoded after the run
        from monoserve_b200.fabric.trace import StageTrace
        tr = StageTrace(capacity=1 << 18)
        tr.start(fab)
    fab.start()
    fab.publish(map=[0] * fab.num_workers, caps=[caps], order=[0], programs=[h], forms=[form])
    time.sleep(0.05)
    it0 = fab.progress()["lanes"][0]["iterations"]
    ends = fab.iteration_times(0, it0, reps + 3, timeout=60)
    err = fab.progress()["error"]
    fab.stop()
    if tr is not None:
        from monoserve_b200.fabric.trace import spans, summary
        rec = tr.stop(fab)
        print(summary(rec, lane.labels, lane=0), file=sys.stderr)
        # one iteration in the middle of the trace: when each kind of stage was activated and completed
        sp = spans(rec, lane.labels, lane=0)
        tags = sorted({s[2] for s in sp})
        if len(tags) > 4:
            one = [s for s in sp if s[2] == tags[len(tags) // 2]]
            t0 = min(s[3] for s in one)
            print("one iteration (us from its start): stage, activated first..last, completed first..last", file=sys.stderr)
            for name in dict.fromkeys(s[0] for s in sorted(one, key=lambda s: s[3])):
                a = [(s[3] - t0) / 1e3 for s in one if s[0] == name]
                c = [(s[4] - t0) / 1e3 for s in one if s[0] == name]
                print(f"  {name:14s} n={len(a):4d}  {min(a):7.1f} .. {max(a):7.1f}   {min(c):7.1f} .. {max(c):7.1f}", file=sys.stderr)
        stamps = lane.expand_stamps.cpu().tolist()
        print("expand tile phases (us):", [round((b - a) / 1e3, 1) for a, b in zip(stamps, stamps[1:]) if a and b], file=sys.stderr)
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
    ap.add_argument("--trace", action="store_true", help="also print the stage timeline of the run (stderr)")
    args = ap.parse_args()
    import bench
    wl = bench.make_workload()
    line = {"workload": "one MoE layer as a repeating fabric program on all SMs (config-2 shapes)", "tokens": args.tokens,
            "caps": args.caps, "form": args.form}
    if args.only in ("both", "config2"):
        line["config2"] = run(wl, wl["hot"], args.tokens, args.caps, args.form, max(6, args.reps // 4), args.idle_cap, args.trace)
    if args.only in ("both", "all_hot"):
        line["all_hot"] = run(wl, list(range(128)), args.tokens, args.caps, args.form, args.reps, args.idle_cap, args.trace)
    print(json.dumps(line))


if __name__ == "__main__":
    main()
