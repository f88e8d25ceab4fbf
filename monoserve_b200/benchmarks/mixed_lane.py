"""Mixed-lane benchmark on the shapes of benchmark configuration 3: a random-init Qwen3-30B-A3B-shaped
decoder (48 layers, hidden 2048, 32 / 4 heads of 128, 128 experts top-8 of width 768, vocabulary
151936, BF16) with a prefill lane (4 prompts of 2048 tokens) and a decode lane (128 sequences,
paged KV with page size 16, contexts uniform in [512, 8192]) running concurrently inside one
persistent fabric kernel, half of every layer's experts in the HBM hot tier and all of them in
pinned host memory.

    python -m monoserve_b200.benchmarks.mixed_lane [--layers 48] [--distinct 48] [--decode 128]
        [--prompts 4] [--prompt-len 2048] [--hot 64] [--sm-decode 74] [--caps 8,2] [--forms 64,0] [--no-staged]
        [--steps 8] [--decode-only] [--quick]

Reported (one JSON line): decode TPOT p50 = median of the decode lane's iteration end-time deltas
(the in-kernel timer, as monoserve/calibrate/calibrator.py:309-319 and Fabric.iteration_times),
taken while the prefill lane's program repeats on its share of the SMs; the prefill lane's tokens/s;
the SM split, link credits and kernel forms that were published.

`--model glm` runs benchmark configuration 4 instead: a GLM-4.5-Air-shaped decoder (46 layers, the first one dense
with an FFN width of 10944 — the configuration does not give it, this is the value chosen —, hidden 4096,
96 / 8 heads of 128 with rotary on 64 dims and qkv bias, 128 routed experts of width 1408 top-8 with sigmoid
routing plus a shared expert of width 1408), every matrix FP8-e4m3 with per-output-channel scales, 25 % of
the experts hot, a prefill lane of 2 x 4096 tokens beside 64 decode sequences with contexts uniform in
[1024, 16384].  Its expert stacks are 2.2 GB per layer, so `--distinct` defaults to 8 there.

Synthetic, seeded data stand in for everything.  The default holds 48 distinct layers' weights: 58 GB
of pinned host memory, 29 GB of hot tier and 57 GB of KV cache in HBM.  `--distinct D` makes only D
distinct layers' weights and cycles them over the layers, for hosts with less memory (every layer still
streams its own experts' bytes per step: one layer's hot tier, 604 MB, is far larger than the 126 MB
L2); the output states it.  The default plan (74 + 74 SMs, 8 + 2 link credits, row-block form 64 for the
decode lane and form 0 for the prefill lane, where a host-resident expert with more than 256 rows is
copied once into the lane's HBM staging stack and computed from there; `--no-staged` reads every
256-row block over the link instead) is one point of the plan space the reference's control plane
searches; other points are a flag away.
"""
import argparse
import sys
import json
import time
import types

import numpy as np
import torch

from monoserve_b200.fabric import Fabric
from monoserve_b200.model import KVCache, ModelLane, ModelWeights


def q_config(layers):
    return types.SimpleNamespace(hidden=2048, intermediate=768, num_experts=128, top_k=8, num_layers=layers,
                                 num_heads=32, num_kv_heads=4, head_dim=128, vocab=151936, rope_theta=1e6,
                                 rms_eps=1e-6, rotary_dim=128)


def make_weights(cfg, distinct, seed=0):
    """Random bf16 weights, N(0, 0.02); the expert stacks go to pinned host memory."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    H, I, E, V = cfg.hidden, cfg.intermediate, cfg.num_experts, cfg.vocab
    qkv_dim = (cfg.num_heads + 2 * cfg.num_kv_heads) * 128

    def rnd(*shape, scale=0.02):
        return (torch.randn(*shape, generator=g, device="cuda") * scale).to(torch.bfloat16)

    def pinned(*shape):
        out = torch.empty(*shape, dtype=torch.bfloat16, pin_memory=True)
        for e in range(shape[0]):
            out[e].copy_(rnd(*shape[1:]))
        return out

    ones = lambda n: torch.ones(n, dtype=torch.bfloat16, device="cuda")  # noqa: E731
    layers = []
    for _ in range(distinct):
        layers.append(dict(in_norm=ones(H), qkv=rnd(qkv_dim, H), q_norm=ones(128), k_norm=ones(128),
                           o=rnd(H, cfg.num_heads * 128), post_norm=ones(H), router=rnd(E, H, scale=H ** -0.5),
                           host_w13=pinned(E, 2 * I, H), host_w2=pinned(E, H, I)))
    torch.cuda.synchronize()
    w = types.SimpleNamespace(embed=rnd(V, H, scale=1.0), lm_head=rnd(V, H), final_norm=ones(H))
    for name in layers[0]:
        setattr(w, name, [layers[l % distinct][name] for l in range(cfg.num_layers)])
    return w


def glm_config(layers):
    return types.SimpleNamespace(hidden=4096, intermediate=1408, num_experts=128, top_k=8, num_layers=layers,
                                 num_heads=96, num_kv_heads=8, head_dim=128, vocab=151552, rope_theta=1e6,
                                 rms_eps=1e-5, rotary_dim=64, qk_norm=False, qkv_bias=True, scoring="sigmoid",
                                 routed_scale=1.0, dense_layers=1, dense_intermediate=10944, shared_intermediate=1408)


def make_glm_weights(cfg, distinct, seed=0):
    """Random weights N(0, 0.02), every matrix quantised to e4m3 per output channel
    (monoserve/runtime/weights.py:218-229); expert stacks in pinned host memory."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    H, I, E, V, L = cfg.hidden, cfg.intermediate, cfg.num_experts, cfg.vocab, cfg.num_layers
    qkv_dim = (cfg.num_heads + 2 * cfg.num_kv_heads) * 128

    def quant(rows, cols, scale=0.02):
        w = torch.randn(rows, cols, generator=g, device="cuda") * scale
        sc = (w.abs().amax(dim=-1, keepdim=True) / 448.0).clamp_min(1e-12)
        return (w / sc).to(torch.float8_e4m3fn).view(torch.uint8), sc.squeeze(-1)

    def stack(n, rows, cols):
        q = torch.empty(n, rows, cols, dtype=torch.uint8, pin_memory=True)
        s = torch.empty(n, rows, dtype=torch.float32, device="cuda")
        for e in range(n):
            b, sc = quant(rows, cols)
            q[e].copy_(b)
            s[e] = sc
        return q, s

    ones = lambda n: torch.ones(n, dtype=torch.bfloat16, device="cuda")  # noqa: E731
    shared_layers = []
    for _ in range(distinct):
        w13, s13 = stack(E, 2 * I, H)
        w2, s2 = stack(E, H, I)
        shared_layers.append(dict(
            in_norm=ones(H), post_norm=ones(H), qkv=quant(qkv_dim, H), qkv_bias=torch.zeros(qkv_dim, dtype=torch.bfloat16,
                                                                                          device="cuda"),
            o=quant(H, cfg.num_heads * 128), router=(torch.randn(E, H, generator=g, device="cuda") * H ** -0.5).to(torch.bfloat16),
            router_bias=torch.zeros(E, device="cuda"), shared_w13=quant(2 * cfg.shared_intermediate, H),
            shared_w2=quant(H, cfg.shared_intermediate), host_w13=w13, host_w2=w2, w13_scale=s13, w2_scale=s2))
    torch.cuda.synchronize()
    w = types.SimpleNamespace(embed=(torch.randn(V, H, generator=g, device="cuda")).to(torch.bfloat16),
                              lm_head=(torch.randn(V, H, generator=g, device="cuda") * 0.02).to(torch.bfloat16),
                              final_norm=ones(H))
    nd = cfg.dense_layers
    for name in shared_layers[0]:
        setattr(w, name, [shared_layers[l % distinct][name] for l in range(L)])
    for name in ("router", "router_bias", "shared_w13", "shared_w2", "host_w13", "host_w2", "w13_scale", "w2_scale"):
        for l in range(nd):
            getattr(w, name)[l] = None
    mlp13, mlp2 = quant(2 * cfg.dense_intermediate, H), quant(H, cfg.dense_intermediate)
    w.mlp_w13 = [mlp13 if l < nd else None for l in range(L)]
    w.mlp_w2 = [mlp2 if l < nd else None for l in range(L)]
    return w


def measure_link_peak(mib=256, reps=6):
    """GB/s of a pinned host -> device copy of `mib` MiB by the copy engine (best of `reps`)."""
    src = torch.empty(mib << 20, dtype=torch.uint8).pin_memory()
    dst = torch.empty(mib << 20, dtype=torch.uint8, device="cuda")
    best = 0.0
    for _ in range(reps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        dst.copy_(src, non_blocking=True)
        b.record()
        b.synchronize()
        best = max(best, (mib << 20) / (a.elapsed_time(b) * 1e-3) / 1e9)
    del src, dst
    return best


def search_plan(cfg, args, ctx, hot, glm):
    """The control plane's plan for this workload: one decode lane (its sequences' contexts, deadline --tpot) and
    one prefill lane (its prompts, deadline --ttft), expected activations from uniform routing shares and the
    hot sets, the B200 calibration measured by `python -m monoserve_b200.calibrate`."""
    import os
    from monoserve_b200 import control
    cal_path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "calibration", "b200.json")
    shape = types.SimpleNamespace(**vars(cfg), fp8=glm)
    est = control.Estimator(control.model_shape(shape), control.load_calibration(cal_path))
    E, L = cfg.num_experts, cfg.num_layers
    p = np.full((L, E), 1.0 / E)
    view = control.profile_view(p, p, hot)
    dense = getattr(cfg, "dense_layers", 0)

    def work(decode, seqs, deadline, rows):
        w = control.LaneWork()
        w.decode, w.deadline = decode, deadline
        w.passes = [[control.Seq(t, c) for t, c in seqs]]
        on = [view.expected(decode, l, rows * cfg.top_k) if l >= dense else (0.0, 0.0) for l in range(L)]
        w.active, w.miss = [a for a, _ in on], [m for _, m in on]
        return w
    lanes = [est.load(work(True, [(1, c) for c in ctx], args.tpot, len(ctx))),
             est.load(work(False, [(args.prompt_len, 0)] * args.prompts, args.ttft, args.prompts * args.prompt_len))]
    plan = control.PlanSearch(est).solve(lanes)
    return {"feasible": plan.feasible, "sms": [l.sms for l in plan.lanes], "caps": [l.cap for l in plan.lanes],
            "forms": [l.form for l in plan.lanes], "estimated_s": [l.est.total for l in plan.lanes],
            "slack": [l.slack for l in plan.lanes], "evaluations": plan.evaluations, "search_us": plan.micros,
            "deadlines_s": [args.tpot, args.ttft]}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", choices=["qwen", "glm"], default="qwen")
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--distinct", type=int, default=None)
    ap.add_argument("--decode", type=int, default=None)
    ap.add_argument("--prompts", type=int, default=None)
    ap.add_argument("--prompt-len", type=int, default=None)
    ap.add_argument("--ctx-lo", type=int, default=None)
    ap.add_argument("--ctx-hi", type=int, default=None)
    ap.add_argument("--hot", type=int, default=None)
    ap.add_argument("--sm-decode", type=int, default=74)
    ap.add_argument("--caps", default="8,2")
    ap.add_argument("--forms", default="64,0")
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--page", type=int, default=16)
    ap.add_argument("--decode-only", action="store_true", help="no prefill lane: every SM decodes")
    ap.add_argument("--no-staged", dest="staged", action="store_false",
                    help="prefill lane: read every 256-row block of a host-resident expert over the link instead of "
                         "copying experts with more than 256 rows once into the HBM staging stack (form 0)")
    ap.add_argument("--host-loop", type=int, default=0, metavar="SLOTS",
                    help="run the host loop beside the fabric: the copy engine stages up to SLOTS host-resident "
                         "experts of the prefill lane's coming layer into an HBM staging buffer (two halves)")
    ap.add_argument("--plan", choices=["given", "search"], default="given",
                    help="search: take the SM split, link credits and kernel forms from the control plane's plan search "
                         "(monoserve_b200.control) over the B200 calibration, with --tpot / --ttft as the lanes' deadlines")
    ap.add_argument("--tpot", type=float, default=1.0, help="decode deadline for --plan search, seconds per step")
    ap.add_argument("--ttft", type=float, default=3.0, help="prefill deadline for --plan search, seconds per pass")
    ap.add_argument("--trace", action="store_true",
                    help="also print the decode lane's stage timeline summary (per stage name: count, mean / p50 / max span) on stderr")
    ap.add_argument("--quick", action="store_true", help="2 layers, 16 sequences, 1 prompt of 256: a smoke run")
    args = ap.parse_args()
    glm = args.model == "glm"
    defaults = dict(layers=46, distinct=8, decode=64, prompts=2, prompt_len=4096, ctx_lo=1024, ctx_hi=16384, hot=32) if glm \
        else dict(layers=48, distinct=48, decode=128, prompts=4, prompt_len=2048, ctx_lo=512, ctx_hi=8192, hot=64)
    for k, v in defaults.items():
        if getattr(args, k) is None:
            setattr(args, k, v)
    if args.quick:
        args.layers, args.distinct, args.decode, args.prompts, args.prompt_len = (3 if glm else 2), 1, 16, 1, 256
        args.ctx_lo, args.ctx_hi, args.steps = 128, 1024, 4
    cfg = glm_config(args.layers) if glm else q_config(args.layers)
    caps = [int(v) for v in args.caps.split(",")]
    forms = [int(v) for v in args.forms.split(",")]
    searched = None
    # before the weights are pinned: a buffer pinned after tens of GB of weights has been seen to land where
    # the copy engine reaches only 46 GB/s, below what the kernel's own reads of the weights sustain
    link_peak = max(measure_link_peak() for _ in range(2))
    t_setup = time.time()
    w = (make_glm_weights if glm else make_weights)(cfg, min(args.distinct, args.layers))
    rng = np.random.default_rng(0)
    hot = [sorted(rng.permutation(cfg.num_experts)[:args.hot].tolist()) for _ in range(cfg.num_layers)]
    weights = ModelWeights(cfg, w, hot=hot)
    if args.host_loop and not args.decode_only:
        weights.alloc_staging(2 * args.host_loop)
    page = args.page
    ctx = rng.integers(args.ctx_lo, args.ctx_hi + 1, size=args.decode).tolist()
    grow = args.steps + 16
    pages_dec = [-(-(c + grow) // page) for c in ctx]
    pages_pre = -(-args.prompt_len // page)
    n_pages = 1 + sum(pages_dec) + args.prompts * pages_pre
    kv = KVCache(cfg, n_pages, page)
    for l in range(cfg.num_layers):
        kv.k[l].normal_(0, 1)
        kv.v[l].normal_(0, 1)
    bt_stride = max(max(pages_dec), pages_pre)
    fab = Fabric(pool_bytes=2 << 30)
    fab.set_max_run(600)
    min_form = min([f for f in forms if f] + [64])
    dec = ModelLane(fab, 0, cfg, weights, kv, max_tokens=args.decode, max_slots=args.decode, bt_stride=bt_stride,
                    logit_rows=args.decode, min_form=min_form)
    at = 1
    perm = rng.permutation(n_pages - 1) + 1          # shuffled pages, page 0 stays the sink
    for s, n in enumerate(pages_dec):
        dec.set_pages(s, perm[at - 1:at - 1 + n].tolist())
        at += n
        dec.set_request(s, seq_len=ctx[s], last_token=int(rng.integers(0, cfg.vocab)))
    h_dec = dec.build_decode(list(range(args.decode)), iterations=0)
    programs, lanes_map = [h_dec], [0] * fab.num_workers
    pre = None
    if not args.decode_only:
        T = args.prompts * args.prompt_len
        pre = ModelLane(fab, 1, cfg, weights, kv, max_tokens=T, max_slots=args.prompts, bt_stride=bt_stride,
                        logit_rows=args.prompts, min_form=min_form, staged=args.staged,
                        staging_index=0 if args.host_loop else None)
        batch = []
        for s in range(args.prompts):
            pre.set_pages(s, perm[at - 1:at - 1 + pages_pre].tolist())
            at += pages_pre
            batch.append((s, rng.integers(0, cfg.vocab, size=args.prompt_len).tolist(), 0))
        programs.append(pre.build_prefill(batch, iterations=0))
        lanes_map = [0] * args.sm_decode + [1] * (fab.num_workers - args.sm_decode)
    if args.plan == "search" and pre is not None:
        searched = search_plan(cfg, args, ctx, hot, glm)
        if searched["feasible"]:
            caps, forms = searched["caps"], searched["forms"]
            args.sm_decode = min(fab.num_workers - 1, max(1, searched["sms"][0] * fab.num_workers // sum(searched["sms"])))
            lanes_map = [0] * args.sm_decode + [1] * (fab.num_workers - args.sm_decode)
    loop = None
    if args.host_loop and pre is not None:
        from monoserve_b200.host_loop import HostLoop
        loop = HostLoop(fab, weights)
        loop.add_prefill_lane(pre, 0)
    torch.cuda.synchronize()
    t_setup = time.time() - t_setup
    tr = None
    if args.trace:
        from monoserve_b200.fabric.trace import StageTrace
        tr = StageTrace(capacity=1 << 21)
        tr.start(fab)
    fab.start()
    if loop is not None:
        loop.start(poll_us=5)
    fab.publish(map=lanes_map, caps=caps[:len(programs)], order=list(range(len(programs))), programs=programs,
                forms=forms[:len(programs)])
    warm = 2
    ends = fab.iteration_times(0, 0, warm + args.steps, timeout=600)
    pre_ends = fab.iteration_times(1, fab.progress()["lanes"][1]["iterations"], 2, timeout=600) if pre else []
    prog = fab.progress()
    err = prog["error"]
    notes = fab.wait_notes() if err else {}
    loop_stats = None
    if loop is not None:
        loop.stop()
        loop_stats = loop.stats()
    fab.stop()
    torch.cuda.synchronize()
    if tr is not None:
        from monoserve_b200.fabric.trace import summary
        print(summary(tr.stop(fab), dec.labels, lane=0), file=sys.stderr)
    deltas = np.diff(np.array(ends[warm - 1:], dtype=np.float64)) * 1e-6    # ms per decode step
    hist = dec.hist.cpu().numpy()
    iters = warm + args.steps
    line = {"workload": ("config 4: GLM-4.5-Air-shaped FP8 decoder" if glm else "config 3: Qwen3-30B-A3B-shaped decoder") +
                        ", prefill + decode lanes in one fabric kernel",
            "layers": cfg.num_layers, "distinct_weight_layers": min(args.distinct, args.layers),
            "decode_seqs": args.decode, "ctx_sum": int(sum(ctx)), "prefill": f"{args.prompts}x{args.prompt_len}",
            "hot_experts_per_layer": args.hot, "page_size": page,
            "sm_split": {"decode": args.sm_decode if pre else fab.num_workers,
                         "prefill": fab.num_workers - args.sm_decode if pre else 0},
            "caps": caps[:len(programs)], "forms": forms[:len(programs)],
            "decode_tpot_ms_p50": float(np.median(deltas)), "decode_tpot_ms_min": float(deltas.min()),
            "decode_tpot_ms_max": float(deltas.max()), "decode_tokens_per_s": args.decode / float(np.median(deltas)) * 1e3,
            "decode_steps_timed": int(len(deltas)),
            "activated_experts_per_layer_step": float((hist > 0).sum() / max(1, cfg.num_layers)),
            "routed_rows_per_layer_step": float(hist.sum() / max(1, cfg.num_layers) / iters),
            "setup_s": round(t_setup, 1), "error": err}
    # Host-link traffic: every activated cold expert's 3 H I weights cross the link once per pass over
    # its rows (row blocks of `form` rows; form 0 = 256-row blocks), per layer.  Computed from the mean rows
    # per expert and iteration, which is exact when every cold expert is activated in every iteration (the
    # full configurations: 1024 or 512 routed decode rows over 128 experts) and an over-estimate for the
    # `--quick` case, whose 16 sequences leave a third of the experts idle in a step.
    expert_bytes = 3 * cfg.hidden * cfg.intermediate * (1 if glm else 2)

    def link_bytes(lane, form, iterations, staged=False):
        h = lane.hist.cpu().numpy().astype(np.float64) / max(1, iterations)     # rows per expert, layer, iteration
        total = 0.0
        for l in range(getattr(cfg, "dense_layers", 0), cfg.num_layers):
            cold = np.ones(cfg.num_experts, dtype=bool)
            cold[hot[l]] = False
            passes = np.ceil(h[l][cold] / (form or 256))
            if staged and form == 0:   # a staged expert crosses the link once
                passes = np.minimum(passes, 1.0)
            total += float(passes.sum()) * expert_bytes
        return total

    dec_iters = prog["lanes"][0]["iterations"]
    dec_link = link_bytes(dec, forms[0], dec_iters)
    line["decode_link_bytes_per_step"] = dec_link
    link_rate = dec_link / (float(np.median(deltas)) * 1e-3)
    if pre is not None and len(pre_ends) >= 2:
        pre_ms = (pre_ends[-1] - pre_ends[-2]) * 1e-6
        line["prefill_iteration_ms"] = pre_ms
        line["prefill_tokens_per_s"] = args.prompts * args.prompt_len / pre_ms * 1e3
        pre_link = link_bytes(pre, forms[1], prog["lanes"][1]["iterations"], staged=args.staged)
        line["prefill_staged"] = bool(args.staged)
        line["prefill_link_bytes_per_iteration"] = pre_link
        link_rate += pre_link / (pre_ms * 1e-3)
    line["host_link_gbs"] = link_rate / 1e9
    # Roofline of the run: both lanes are bound by the host link, so the fraction to read is the expert bytes
    # that crossed it per second against the copy peak measured in this process; the decode step's own lower
    # bound is its link bytes at that peak, i.e. with no prefill lane beside it and every other term hidden.
    line["host_link_peak_gbs"] = link_peak
    line["host_link_frac"] = link_rate / 1e9 / link_peak if link_peak else None
    line["decode_tpot_link_bound_ms"] = dec_link / (link_peak * 1e9) * 1e3 if link_peak else None
    if searched is not None:
        line["searched_plan"] = searched
    if loop_stats is not None:
        # experts the copy engine staged are read from HBM by the prefill lane: the figure above counts them
        # as link reads of the kernel, so with the host loop it is an upper bound of the kernel's own reads
        line["host_loop"] = dict(loop_stats, slots_per_half=args.host_loop)
    if notes:
        line["wait_notes"] = {str(k): v for k, v in list(notes.items())[:4]}
    print(json.dumps(line))
    fab.close()


if __name__ == "__main__":
    main()
