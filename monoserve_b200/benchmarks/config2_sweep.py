"""The sweep that benchmark configuration 2 describes: the Qwen3-30B-A3B MoE layer on one B200 with 32 experts in
the HBM hot tier and 96 in pinned host memory, decode batches 1 / 8 / 32 / 128 / 256 with Zipf(1.1)
+ N(0,1) router logits, link credits 1..16, and both kernel forms for host-resident experts (row
blocks of 64, and the one-pass form that the reference's asymmetric form maps to).

    python -m monoserve_b200.benchmarks.config2_sweep [--reps 20] [--credits 1,2,4,8,16] [--batches 1,8,32,128,256]

Per point: layer time (CUDA events over `reps` steps of the stream path, inputs resident, 8 batches
rotating so that the weights streamed per step exceed L2), tokens/s, activated hot / cold experts, and
the host-link rate = cold experts x 9.44 MB / time.  One JSON line with the table, and a text table on
stderr.  Data and weights are those of bench.py (seeded, synthetic).
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--credits", default="1,2,4,8,16")
    ap.add_argument("--batches", default="1,8,32,128,256")
    ap.add_argument("--forms", default="64,0")
    args = ap.parse_args()
    import bench
    from monoserve_b200.moe import MoELayer
    H, I, E, K = bench.SHAPE["H"], bench.SHAPE["I"], bench.SHAPE["E"], bench.SHAPE["K"]
    wl = bench.make_workload()
    layer = MoELayer(H, I, E, K, bench.BATCH)
    layer.set_router(wl["wr"].cuda())
    layer.set_experts(wl["w13"], wl["w2"], wl["hot"])
    xs = [x.cuda() for x in wl["xs"]]
    x2s = [x.cuda() for x in wl["x2s"]]
    expert_bytes = 3 * H * I * 2
    hot = set(wl["hot"])
    rows = []
    for T in [int(v) for v in args.batches.split(",")]:
        out = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")
        for form in [int(v) for v in args.forms.split(",")]:
            for credits in [int(v) for v in args.credits.split(",")]:
                layer.set_plan(0, credits, form)
                step = lambda i: layer.forward(xs[i % len(xs)][:T].contiguous(), x2s[i % len(xs)][:T].contiguous(), out)  # noqa: E731
                for i in range(3):
                    step(i)
                torch.cuda.synchronize()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                cold_sum = hot_sum = 0
                a.record()
                for i in range(args.reps):
                    step(i)
                b.record()
                b.synchronize()
                layer.status()
                for i in range(min(len(xs), args.reps)):      # activated experts of the batches used
                    step(i)
                    counts = layer.workspace("counts")[:E].cpu()
                    act = [e for e in range(E) if counts[e] > 0]
                    cold_sum += sum(1 for e in act if e not in hot)
                    hot_sum += sum(1 for e in act if e in hot)
                n = min(len(xs), args.reps)
                ms = a.elapsed_time(b) / args.reps
                cold = cold_sum / n
                rows.append(dict(batch=T, form=form, credits=credits, ms=ms, tokens_per_s=T / ms * 1e3,
                                 hot_active=hot_sum / n, cold_active=cold,
                                 host_link_gbs=cold * expert_bytes / (ms * 1e-3) / 1e9))
                r = rows[-1]
                print(f"batch {T:4d} form {form:3d} credits {credits:2d}: {ms:8.3f} ms  {r['tokens_per_s']:9.0f} tok/s  "
                      f"cold {cold:5.1f} hot {r['hot_active']:5.1f}  link {r['host_link_gbs']:5.1f} GB/s", file=sys.stderr)
    print(json.dumps({"workload": "BASELINE config 2 sweep (stream path)", "rows": rows}))
    layer.close()


if __name__ == "__main__":
    main()
