"""Measure a calibration of the control plane's time estimator on this GPU.

    python -m monoserve_b200.calibrate [--out monoserve_b200/calibration/b200.json] [--quick]

The reference measures its calibration inside its fabric (monoserve/calibrate/calibrator.py: solo
sweeps of every kernel against the SM share, one credit sweep per kernel form, a contention probe).
This module measures the same curves with this library's kernels through their stream entry
points, which take the SM share (`ctas`), the link credits and the kernel form as plan parameters:

  expert[form]   the expert GEMM with every expert in HBM, against the SM share: HBM bytes/s from a
                 decode batch (weight streaming), FLOP/s from a prefill batch (2048 rows)
  rho[form]      the same kernel with every expert in pinned host memory, against the link credits
                 (link slots: workers reading host memory at once).  Measured alone, one slot already pulls
                 57 % of the link and two saturate it; what a plan needs is what a lane gets when several
                 lanes hold slots at once, and then the saturated link is shared in proportion to the slots.
                 The file therefore carries rho as that share model - a straight line from the origin to
                 the form's saturated rate at kShareCredits = 16 credits, so that the lanes' rates add up to
                 the link's - and the raw single-lane sweep under "measured"
  attn_decode / attn_prefill   the paged-KV attention kernel at full size; the curves against the SM
                 share are straight lines through that point (the kernel takes no SM limit)
  dense          the dense projections use the same GEMM tiles as the experts: the 128-row expert curves
  gamma          flat: no read-time stretch under exposure was observed behind PCIe, where the link's
                 51 GB/s is under 1 % of HBM bandwidth
  beta           the saturated rate of the kernel's own reads of host memory (not the copy engine's)

Output: the reference's calibration file format (monoserve/control/calibration.py:1-25) plus the two
keys of this library's one-pass form (256-row blocks, no partial-sum traffic).  Synthetic, seeded data.
"""
import argparse
import json
import os

import torch

SHAPE = dict(H=2048, I=768, E=128, K=8)


def timed(fn, reps, warm=3):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        fn()
    b.record()
    b.synchronize()
    return a.elapsed_time(b) / reps * 1e-3


def expert_kernel_seconds(layer, xn, out, reps):
    """Seconds of the expert GEMM launch alone (CUDA events around it, averaged)."""
    layer.set_profile(1)
    total = 0.0
    for i in range(reps + 2):
        layer.forward(xn, None, out)
        if i >= 2:
            total += layer.last_times()["experts"] * 1e-3
    layer.set_profile(0)
    return total / reps


kShareCredits = 16


def share_model(raw):
    """Per form: credits 1 .. kShareCredits against the form's saturated rate shared in proportion."""
    grid = list(range(1, kShareCredits + 1))   # every whole credit is a grant the plan search may try
    return {name: {"credits": grid, "gbps": [max(v["gbps"]) * c / kShareCredits for c in grid]} for name, v in raw.items()}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=os.path.join(os.path.dirname(os.path.abspath(__file__)), "calibration", "b200.json"))
    ap.add_argument("--quick", action="store_true", help="fewer points and repetitions")
    args = ap.parse_args()
    from monoserve_b200.attention import AttentionPlan
    from monoserve_b200.benchmarks.attention import make_batch
    from monoserve_b200.moe import MoELayer
    H, I, E, K = SHAPE["H"], SHAPE["I"], SHAPE["E"], SHAPE["K"]
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    reps = 5 if args.quick else 12
    g = torch.Generator().manual_seed(0)
    wr = (torch.randn(E, H, generator=g) * H ** -0.5).to(torch.bfloat16).cuda()
    w13 = torch.empty(E, 2 * I, H, dtype=torch.bfloat16, pin_memory=True)
    w2 = torch.empty(E, H, I, dtype=torch.bfloat16, pin_memory=True)
    for e in range(E):
        w13[e] = (torch.randn(2 * I, H, generator=g) * 0.02).to(torch.bfloat16)
        w2[e] = (torch.randn(H, I, generator=g) * 0.02).to(torch.bfloat16)
    expert_bytes = 3 * H * I * 2
    shares = [sms // 8, sms // 4, sms // 2, 3 * sms // 4, sms] if not args.quick else [sms // 4, sms // 2, sms]
    forms = {"16": 16, "32": 32, "64": 64, "128": 128, "asym": 0}

    # ---- experts in HBM: bytes/s from a decode batch, FLOP/s from a prefill batch, against the SM share
    def hbm_sweep(T):
        layer = MoELayer(H, I, E, K, T)
        layer.set_router(wr)
        layer.set_experts(w13, w2, hot=list(range(E)))
        xn = torch.randn(T, H, generator=g).to(torch.bfloat16).cuda()
        out = torch.empty_like(xn)
        rows = []
        for s in shares:
            layer.set_plan(s, 0, 64)
            sec = expert_kernel_seconds(layer, xn, out, reps)
            active = int((layer.workspace("counts")[:E] > 0).sum())
            rows.append((s, active * expert_bytes / sec, 6.0 * T * K * H * I / sec))
        layer.close()
        return rows
    decode_rows, prefill_rows = hbm_sweep(256), hbm_sweep(2048)
    expert = {"sms": shares, "tflops": [r[2] / 1e12 for r in prefill_rows], "gbps": [r[1] / 1e9 for r in decode_rows],
              "q_per_sm": 1}

    # ---- experts in pinned host memory: bytes/s over the link against the credits, per form
    credits = [1, 2, 4, 8, 16] if not args.quick else [1, 2, 8]
    layer = MoELayer(H, I, E, K, 64)
    layer.set_router(wr)
    layer.set_experts(w13, w2, hot=[])
    xn = torch.randn(64, H, generator=g).to(torch.bfloat16).cuda()
    out = torch.empty_like(xn)
    rho = {}
    for name, form in forms.items():
        if args.quick and form not in (64, 0):
            continue
        gbps = []
        for c in credits:
            layer.set_plan(0, c, form)
            sec = expert_kernel_seconds(layer, xn, out, max(3, reps // 3))
            active = int((layer.workspace("counts")[:E] > 0).sum())
            gbps.append(active * expert_bytes / sec / 1e9)     # 64 rows: one pass per expert in every form
        rho[name] = {"credits": credits, "gbps": gbps}
    layer.close()
    if args.quick:
        for name in forms:
            rho.setdefault(name, rho["64"])
    beta = max(max(v["gbps"]) for v in rho.values())
    raw_rho = rho
    rho = share_model(raw_rho)

    # ---- attention at full size
    hq, hkv = 32, 4
    gen = torch.Generator().manual_seed(0)
    lens = torch.randint(512, 8193, (128,), generator=gen).tolist()
    q, kc, vc, bt, info = make_batch(lens, [1] * len(lens), hq, hkv, 16, 1)
    o = torch.empty_like(q)
    plan = AttentionPlan(info, hq, hkv)
    dec_gbps = sum(lens) * hkv * 128 * 4 / timed(lambda: plan.run(q, kc, vc, bt, out=o, check=False), reps) / 1e9
    plens = [2048] * 4
    q, kc, vc, bt, info = make_batch(plens, plens, hq, hkv, 16, 2)
    o = torch.empty_like(q)
    plan = AttentionPlan(info, hq, hkv)
    pre_tflops = 4 * hq * 128 * sum(n * (n + 1) // 2 for n in plens) / timed(lambda: plan.run(q, kc, vc, bt, out=o, check=False), max(3, reps // 2)) / 1e12
    line = lambda full: [full * s / sms for s in shares]  # noqa: E731
    hbm_full = expert["gbps"][-1]
    cal = {
        "sms": sms, "R_H_us": 0.5, "R_C_us": 2.0, "q_max": 1,
        "gamma": {"exposure_entry_us": [1.0, 1e6], "stretch": [1.0, 1.0]},
        "dense": dict(expert),
        "attn_prefill": {"sms": shares, "tflops": line(pre_tflops), "gbps": line(hbm_full), "q_per_sm": 1},
        "attn_decode": {"sms": shares, "tflops": line(pre_tflops), "gbps": line(dec_gbps), "q_per_sm": 1},
        "expert": {name: dict(expert) for name in forms},
        "rho": rho, "q_form": {name: 1 for name in forms}, "beta_gbps": beta, "reference_form": 64,
        "layer_overhead_us": 25.0, "tail_overhead_us": 60.0, "one_pass_rows": 256, "one_pass_row_bytes": 0.0,
        "measured": {"gpu": torch.cuda.get_device_name(0), "rho_single_lane": raw_rho, "attention_decode_gbps": dec_gbps,
                     "attention_prefill_tflops": pre_tflops, "expert_hbm_gbps_all_sms": hbm_full,
                     "expert_tflops_all_sms": expert["tflops"][-1], "command": "python -m monoserve_b200.calibrate"},
    }
    os.makedirs(os.path.dirname(args.out), exist_ok=True)
    with open(args.out, "w") as f:
        json.dump(cal, f, indent=1, sort_keys=True)
    print(json.dumps({"written": args.out, "beta_gbps": beta, "rho_64": rho["64"], "expert": expert,
                      "attn_decode_gbps": dec_gbps, "attn_prefill_tflops": pre_tflops}))


if __name__ == "__main__":
    main()
