"""Paged-KV attention micro-benchmark on the shapes of benchmark configuration 3
(Qwen3-30B-A3B: 32 query heads, 4 KV heads, head_dim 128, page size 16).

    python -m monoserve_b200.benchmarks.attention [--page 16] [--seqs 128] [--reps 20] [--quick]
                                                  [--mode both|decode|prefill] [--part-tiles N]

decode : `seqs` sequences, contexts uniform in [512, 8192], one query token each;
         reported as K+V GB/s = sum(ctx) * hkv * 128 * 2 * 2 bytes / time (HBM-bound).
prefill: 4 prompts of 2048 tokens; reported as TFLOP/s with
         FLOPs = 4 * hq * 128 * sum over prompts of n (n + 1) / 2 (tensor-pipe-bound).
Synthetic, seeded data; the work list is planned once outside the timed region; times are
CUDA-event means of the launches (main kernel + merge of split parts) after warm-up; one JSON line.
"""
import argparse
import json

import torch

from monoserve_b200.attention import AttentionPlan


def make_batch(lens, q_rows, hq, hkv, page, seed):
    g = torch.Generator().manual_seed(seed)
    need = [-(-n // page) for n in lens]
    n_pages = sum(need) + 1
    kc = torch.randn(n_pages, page, hkv, 128, generator=g, dtype=torch.float32).to(torch.bfloat16).cuda()
    vc = torch.randn(n_pages, page, hkv, 128, generator=g, dtype=torch.float32).to(torch.bfloat16).cuda()
    perm = torch.randperm(n_pages - 1, generator=g) + 1
    bt = torch.zeros(len(lens), max(need), dtype=torch.int32)
    at = 0
    for r, n in enumerate(need):
        bt[r, :n] = perm[at:at + n].to(torch.int32)
        at += n
    T = sum(q_rows)
    q = torch.randn(T, hq, 128, generator=g).to(torch.bfloat16).cuda()
    req_info, row = [], 0
    for n, L in zip(q_rows, lens):
        req_info.append((row, L - n, n, L))
        row += n
    return q, kc, vc, bt.cuda(), req_info


def timed(fn, reps):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        fn()
    b.record()
    b.synchronize()
    return a.elapsed_time(b) / reps * 1e-3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--page", type=int, default=16)
    ap.add_argument("--seqs", type=int, default=128)
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--part-tiles", type=int, default=None, help="128-key tiles per split part (default: planned)")
    ap.add_argument("--mode", choices=["both", "decode", "prefill"], default="both")
    ap.add_argument("--quick", action="store_true", help="small case for profiling: 32 sequences / 1 prompt")
    args = ap.parse_args()
    hq, hkv = 32, 4
    line = {}
    if args.mode in ("both", "decode"):
        g = torch.Generator().manual_seed(0)
        seqs = 32 if args.quick else args.seqs
        lens = torch.randint(512, 8193, (seqs,), generator=g).tolist()
        q, kc, vc, bt, info = make_batch(lens, [1] * seqs, hq, hkv, args.page, 1)
        out = torch.empty_like(q)
        plan = AttentionPlan(info, hq, hkv, part_tiles=args.part_tiles)
        sec = timed(lambda: plan.run(q, kc, vc, bt, out=out, check=False), args.reps)
        assert int(plan.status.item()) == 0
        kv_bytes = sum(lens) * hkv * 128 * 2 * 2
        line["decode"] = {"seqs": seqs, "ctx_sum": sum(lens), "page": args.page, "items": int(plan.items.shape[0]),
                          "us": sec * 1e6, "kv_gbs": kv_bytes / sec / 1e9, "kv_bytes": kv_bytes}
    if args.mode in ("both", "prefill"):
        plens = [2048] * (1 if args.quick else 4)
        q, kc, vc, bt, info = make_batch(plens, plens, hq, hkv, args.page, 2)
        out = torch.empty_like(q)
        plan = AttentionPlan(info, hq, hkv, part_tiles=args.part_tiles)
        sec = timed(lambda: plan.run(q, kc, vc, bt, out=out, check=False), max(3, args.reps // 4))
        assert int(plan.status.item()) == 0
        flops = 4 * hq * 128 * sum(n * (n + 1) // 2 for n in plens)
        line["prefill"] = {"prompts": plens, "page": args.page, "items": int(plan.items.shape[0]), "us": sec * 1e6,
                           "tflops": flops / sec / 1e12}
    import os
    peaks = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    # fractions of the peaks measured on this pool (a copy and a cuBLAS bf16 GEMM), else of an earlier measurement
    pk, src = (json.load(open(peaks)), "measured") if os.path.exists(peaks) else \
        ({"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback")
    if "decode" in line:
        line["decode"]["hbm_frac"] = line["decode"]["kv_gbs"] / pk["hbm_gbs"]
    if "prefill" in line:
        line["prefill"]["bf16_frac"] = line["prefill"]["tflops"] / pk["bf16_tflops"]
    line["peaks"] = {"hbm_gbs": pk["hbm_gbs"], "bf16_tflops": pk["bf16_tflops"], "source": src}
    print(json.dumps(line))


if __name__ == "__main__":
    main()
