"""Continuous batching under Poisson arrivals on one GPU: the serving loop
(monoserve_b200/engine.py) over a random-init Qwen3-30B-A3B-shaped decoder, the arrival process and
length distributions of benchmark configuration 5 (arrivals at `--rates` requests/s built as the
reference's load generator builds them, eval/loadgen.py:54-70; prompt lengths log-normal with median
256, sigma 1.0, clipped to [16, 4096]; output lengths log-normal with median 200, sigma 0.8, clipped
to [8, 2048]; prompt token ids uniform over the vocabulary, seed 0).

    python -m monoserve_b200.benchmarks.serve [--rates 2,8,32] [--duration 10] [--layers 48] [--distinct 8]
                                              [--max-decode 128] [--token-budget 4096] [--quick]

This is configuration 5 at N = 1: all 128 experts of every layer on the one GPU, in its HBM hot tier
(the configuration partitions the experts over the GPUs; whole-model expert parallelism over several
GPUs is not built).  Per rate: requests served, TTFT and time per output token (mean / p50 / p99),
output tokens/s.  Synthetic, seeded data; `--distinct D` cycles D distinct layers' weights over the
layers to bound set-up time (every layer still streams 1.2 GB of experts per step, far beyond L2).
One JSON line.
"""
import argparse
import json
import time

import numpy as np
import torch

from monoserve_b200.benchmarks.mixed_lane import make_weights, q_config
from monoserve_b200.engine import Engine, PagePool, RequestTable, arrival_times, lognormal_lengths, summarize
from monoserve_b200.fabric import Fabric
from monoserve_b200.model import KVCache, ModelWeights


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rates", default="2,8,32")
    ap.add_argument("--duration", type=float, default=10.0, help="seconds of arrivals per rate")
    ap.add_argument("--layers", type=int, default=48)
    ap.add_argument("--distinct", type=int, default=8)
    ap.add_argument("--max-decode", type=int, default=128)
    ap.add_argument("--token-budget", type=int, default=4096)
    ap.add_argument("--pages", type=int, default=24000)
    ap.add_argument("--spare-sms", type=int, default=8, help="SMs left to the host's copies and fills while the fabric runs")
    ap.add_argument("--plan", choices=["fixed", "search"], default="fixed",
                    help="search: the SM split of the decode and prefill lanes comes from the control plane's plan search "
                         "(deadlines --tpot / --ttft) whenever both lanes run, instead of half / half")
    ap.add_argument("--tpot", type=float, default=0.05, help="decode deadline for --plan search, seconds per step")
    ap.add_argument("--ttft", type=float, default=0.5, help="prefill deadline for --plan search, seconds per pass")
    ap.add_argument("--quick", action="store_true", help="4 layers, short lengths, one rate: a smoke run")
    args = ap.parse_args()
    prompt_clip, output_clip = (16, 4096), (8, 2048)
    if args.quick:
        args.layers, args.distinct, args.rates, args.duration, args.pages = 4, 1, "16", 2.0, 4000
        prompt_clip, output_clip = (16, 512), (8, 64)
    cfg = q_config(args.layers)
    t_setup = time.time()
    w = make_weights(cfg, min(args.distinct, args.layers))
    weights = ModelWeights(cfg, w, hot=[list(range(cfg.num_experts)) for _ in range(cfg.num_layers)])
    page = 16
    max_len = prompt_clip[1] + output_clip[1]
    bt_stride = -(-max_len // page) + 2
    kv = KVCache(cfg, args.pages, page)
    props = torch.cuda.get_device_properties(0)
    fab = Fabric(num_workers=props.multi_processor_count - args.spare_sms, pool_bytes=4 << 30)
    fab.set_max_run(900)
    slots = 2 * args.max_decode
    table = RequestTable(fab, slots, bt_stride)
    results = []
    try:
        planner = None
        if args.plan == "search":
            from monoserve_b200.engine import SearchPlanner
            planner = SearchPlanner(cfg, [list(range(cfg.num_experts)) for _ in range(cfg.num_layers)], tpot_s=args.tpot,
                                    ttft_s=args.ttft)
        eng = Engine(fab, cfg, weights, kv, table, PagePool(args.pages), max_decode=args.max_decode,
                     token_budget=args.token_budget, max_len=max_len, planner=planner)
        torch.cuda.synchronize()
        t_setup = time.time() - t_setup
        fab.start()
        for rate in [float(v) for v in args.rates.split(",")]:
            n = max(2, int(rate * args.duration))
            arrivals = arrival_times(rate, seed=0, num=n)
            prompts = lognormal_lengths(n, 256, 1.0, *prompt_clip, seed=1)
            outputs = lognormal_lengths(n, 200, 0.8, *output_clip, seed=2)
            rng = np.random.default_rng(0)
            reqs = [(float(arrivals[i]), f"r{rate:g}-{i}", rng.integers(0, cfg.vocab, size=int(prompts[i])).tolist(),
                     int(outputs[i])) for i in range(n)]
            eng.reqs.clear()
            before = dict(eng.stats)
            records = eng.serve(reqs, timeout_s=600)
            line = summarize(records)
            line.update(rate_per_s=rate, prompt_tokens=int(prompts.sum()),
                        decode_programs=eng.stats["decode_programs"] - before["decode_programs"],
                        prefill_passes=eng.stats["prefill_passes"] - before["prefill_passes"])
            # host time to build one program (numpy tile arrays + writes through the fabric's staging ring)
            for kind, count in (("prefill", "prefill_passes"), ("decode", "decode_programs")):
                made = line[count]
                line[f"{kind}_build_ms"] = 1e3 * (eng.stats[f"{kind}_build_s"] - before[f"{kind}_build_s"]) / made if made else None
            if planner is not None:
                line["plan_search"] = dict(planner.stats, sm_decode_last=eng.map.count(0))
            results.append(line)
        err = fab.progress()["error"]
    finally:
        fab.stop()
        fab.close()
    print(json.dumps({"workload": "config 5 at N = 1: Qwen3-30B-A3B-shaped decoder, continuous batching under Poisson "
                                  "arrivals, every expert in HBM", "layers": cfg.num_layers,
                      "distinct_weight_layers": min(args.distinct, args.layers), "max_decode": args.max_decode,
                      "token_budget": args.token_budget, "fabric_workers": fab_workers(props, args), "page_size": page,
                      "setup_s": round(t_setup, 1), "error": err, "rates": results}))


def fab_workers(props, args):
    return props.multi_processor_count - args.spare_sms


if __name__ == "__main__":
    main()
