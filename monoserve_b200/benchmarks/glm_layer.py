"""The routed-expert MoE layer at the shape of benchmark configuration 4 (GLM-4.5-Air-shaped: hidden 4096,
128 routed experts of width 1408, top-8, sigmoid scoring with a selection bias and routed scale,
FP8-e4m3 weights drawn from N(0, 0.02) and quantised per output channel with fp32 scales, 25 % of
the experts in the HBM hot tier and all of them in pinned host memory), through the stream path
(`MoELayer`), for the two batch shapes of that config: 64 decode rows, and 2 x 4096 prefill rows.

    python -m monoserve_b200.benchmarks.glm_layer [--reps 10] [--credits 8] [--all-hot] [--only decode|prefill]

The shared expert and the attention of config 4 are not part of this measurement.  Reported per
batch: layer time (CUDA events, inputs resident), tokens/s, activated hot / cold experts, host-link
GB/s = cold expert bytes x passes / time, and the result's rel-L2 against the de-quantised fp32
reference on four sample rows (tolerance 3e-2).  One JSON line.
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--credits", type=int, default=8)
    ap.add_argument("--all-hot", action="store_true", help="every expert in the HBM hot tier (the FP8 kernel against HBM)")
    ap.add_argument("--only", choices=["both", "decode", "prefill"], default="both")
    args = ap.parse_args()
    from monoserve_b200.moe import MoELayer

    def bf(t):
        return t.to(torch.bfloat16).float()

    def ffn(x, w13, w2):   # SwiGLU expert with the bf16-rounded hidden of tests/test_fabric_model_glm.py:29-31
        width = w13.shape[0] // 2
        return bf(torch.nn.functional.silu(x @ w13[:width].t()) * (x @ w13[width:].t())) @ w2.t()
    H, I, E, K = 4096, 1408, 128, 8
    g = torch.Generator(device="cuda").manual_seed(0)
    q13 = torch.empty(E, 2 * I, H, dtype=torch.uint8, pin_memory=True)
    q2 = torch.empty(E, H, I, dtype=torch.uint8, pin_memory=True)
    s13 = torch.empty(E, 2 * I, dtype=torch.float32)
    s2 = torch.empty(E, H, dtype=torch.float32)
    for e in range(E):     # quantise on the GPU, one expert at a time (monoserve/runtime/weights.py:218-229)
        for name, q, s, shape in (("w13", q13, s13, (2 * I, H)), ("w2", q2, s2, (H, I))):
            w = torch.randn(*shape, generator=g, device="cuda") * 0.02
            sc = (w.abs().amax(dim=-1, keepdim=True) / 448.0).clamp_min(1e-12)
            qq = (w / sc).to(torch.float8_e4m3fn)
            q[e].copy_(qq.view(torch.uint8))
            s[e].copy_(sc.squeeze(-1))
    torch.cuda.synchronize()
    wr = (torch.randn(E, H, generator=g, device="cuda") * H ** -0.5).to(torch.bfloat16)
    bias = torch.randn(E, generator=g, device="cuda") * 0.1
    hot = list(range(E)) if args.all_hot else list(range(0, E, 4))   # 25 % hot
    results = {}
    for name, T, form in (("decode_64", 64, 64), ("prefill_2x4096", 8192, 0)):
        if args.only != "both" and not name.startswith(args.only):
            continue
        layer = MoELayer(H, I, E, K, T, scoring="sigmoid", renorm=True, routed_scale=2.5, fp8=True)
        layer.set_router(wr, bias)
        layer.set_experts(q13, q2, hot, scales=(s13, s2))
        layer.set_plan(0, args.credits, form)
        xn = torch.randn(T, H, generator=g, device="cuda").to(torch.bfloat16)
        x2 = torch.randn(T, H, generator=g, device="cuda").to(torch.bfloat16)
        out = torch.empty_like(xn)
        for _ in range(2):
            layer.forward(xn, x2, out)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.reps):
            layer.forward(xn, x2, out)
        b.record()
        b.synchronize()
        layer.status()
        ms = a.elapsed_time(b) / args.reps
        counts = layer.workspace("counts")[:E].cpu()
        # the layer zeroes its counts; recompute activation from the routing it left behind
        ids = layer.workspace("topk_ids")[:T * K].cpu().view(T, K)
        rows_per = torch.bincount(ids.flatten().long(), minlength=E)
        cold = [e for e in range(E) if rows_per[e] > 0 and e not in hot]
        block = form or 256
        passes = sum(-(-int(rows_per[e]) // block) for e in cold)
        link_bytes = passes * 3 * H * I
        # parity on a sample of rows against the de-quantised weights (fp32, on the GPU) of the experts they use
        sample = list(range(0, T, max(1, T // 4)))[:4]
        tw = layer.workspace("topk_w")[:T * K].view(T, K)
        deq = {}

        def weights(e):
            if e not in deq:
                d13 = q13[e].cuda().view(torch.float8_e4m3fn).float() * s13[e].cuda()[:, None]
                d2 = q2[e].cuda().view(torch.float8_e4m3fn).float() * s2[e].cuda()[:, None]
                deq[e] = (d13, d2)
            return deq[e]

        ref = []
        for t in sample:
            x = xn[t:t + 1].float()
            acc = torch.zeros(H, device="cuda")
            for k in range(K):
                d13, d2 = weights(int(ids[t, k]))
                acc += float(tw[t, k]) * ffn(x, d13, d2)[0]
            ref.append(bf(x2[t].float() + acc))
        ref = torch.stack(ref)
        rel = float((out[sample].float() - ref).norm() / ref.norm())
        del deq
        results[name] = {"tokens": T, "form": form, "credits": args.credits, "ms": ms, "tokens_per_s": T / ms * 1e3,
                         "hot_active": int(sum(1 for e in hot if rows_per[e] > 0)), "cold_active": len(cold),
                         "host_link_gbs": link_bytes / (ms * 1e-3) / 1e9, "rel_l2_sample": rel,
                         "sample_rows": len(sample)}
        layer.close()
    print(json.dumps({"workload": "BASELINE config 4 shape: GLM-4.5-Air-shaped routed MoE layer, FP8-e4m3 W8A16, "
                                  "25 % hot, sigmoid routing", "results": results}))


if __name__ == "__main__":
    main()
