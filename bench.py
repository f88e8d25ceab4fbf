#!/usr/bin/env python
"""Benchmark of the MoE-layer hot path (metric: MoE layer tokens/s).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N = 1): benchmark configuration 2 — one Qwen3-30B-A3B-shaped MoE layer in BF16
(128 experts, top-8, hidden 2048, expert intermediate 768, SwiGLU, softmax routing
with renormalisation), 32 experts in the HBM hot tier and 96 read in place from
pinned host memory, a decode batch of 256 tokens per step, router logits
N(0,1) + a Zipf(s=1.1) log-prior over a seeded expert permutation.  All data is
synthetic and seeded; weights N(0, 0.02).

One step = one pass of the whole layer (router projection, top-k, plan, pack, w13,
w2, combine) over one batch.  `value` is measured with the inputs resident in HBM;
`e2e` goes through the host-buffer entry point of the C ABI with the host->device
and device->host copies inside the timed region.  `--impl reference` times the
reference's PyTorch MoE path (restated in oracle/torch_path.py) on the host CPU
cores on the same workload.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SHAPE = dict(H=2048, I=768, E=128, K=8)
BATCH = 256
N_HOT = 32
N_BATCHES = 8          # distinct input batches rotated through the steps
CREDITS = 8
FORM = 64


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"], source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")


def zipf_prior(E, seed):
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(E, generator=g)
    rank = torch.empty(E, dtype=torch.float32)
    rank[perm] = torch.arange(1, E + 1, dtype=torch.float32)
    return -1.1 * torch.log(rank)      # log(rank^-1.1)


def make_workload(seed=0, experts=None):
    """Weights and input batches of config 2.  The router weight carries the Zipf
    log-prior in column 0, which every activation row holds at 1.0, so that
    logits = N(0,1) + prior."""
    H, I, E, K = SHAPE["H"], SHAPE["I"], SHAPE["E"], SHAPE["K"]
    g = torch.Generator().manual_seed(seed)
    prior = zipf_prior(E, seed + 1)
    wr = torch.randn(E, H, generator=g) * (H - 1) ** -0.5
    wr[:, 0] = prior
    wr = wr.to(torch.bfloat16)
    w13 = torch.empty(E, 2 * I, H, dtype=torch.bfloat16)
    w2 = torch.empty(E, H, I, dtype=torch.bfloat16)
    for e in range(E):   # chunked to keep the fp32 temporaries small
        w13[e] = (torch.randn(2 * I, H, generator=g) * 0.02).to(torch.bfloat16)
        w2[e] = (torch.randn(H, I, generator=g) * 0.02).to(torch.bfloat16)
    g1 = torch.Generator().manual_seed(seed + 2)
    xs, x2s = [], []
    for _ in range(N_BATCHES):
        x = torch.randn(BATCH, H, generator=g1)
        x[:, 0] = 1.0
        xs.append(x.to(torch.bfloat16))
        x2s.append(torch.randn(BATCH, H, generator=g1).to(torch.bfloat16))
    hot = torch.argsort(prior, descending=True)[:N_HOT].tolist()
    return dict(wr=wr, w13=w13, w2=w2, xs=xs, x2s=x2s, hot=sorted(hot), prior=prior)


class ClockSampler:
    """nvidia-smi samples of SM clock and throttle reasons during the timed region."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.path = index, None, None

    def start(self):
        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=f,
                                         stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        out = dict(sm_mhz=None, sm_max_mhz=None, reasons=[], samples=0)
        if not self.proc:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for line in open(self.path):
            c = [v.strip() for v in line.split(",")]
            if len(c) < 9:
                continue
            try:
                sm.append(float(c[1]))
                mx.append(float(c[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), c[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        return out


def measure_h2d_gbs(nbytes=256 << 20, reps=5):
    """Copy-engine host->device bandwidth from pinned memory: the host-link peak."""
    src = torch.empty(nbytes, dtype=torch.uint8, pin_memory=True)
    dst = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    best = 0.0
    for _ in range(reps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        dst.copy_(src, non_blocking=True)
        b.record()
        b.synchronize()
        best = max(best, nbytes / (a.elapsed_time(b) * 1e-3) / 1e9)
    return best


def cpu_layer_time(wl, threads, reps, warm):
    """Seconds per batch of the reference's PyTorch MoE path on the host CPU."""
    from oracle import torch_path as tp
    torch.set_num_threads(threads)
    K = SHAPE["K"]
    times = []
    with torch.no_grad():
        for i in range(warm + reps):
            x, x2 = wl["xs"][i % N_BATCHES].float(), wl["x2s"][i % N_BATCHES].float()
            t0 = time.perf_counter()
            tp.moe_layer(x, x2, wl["wr"], wl["w13"], wl["w2"], K)
            dt = time.perf_counter() - t0
            if i >= warm:
                times.append(dt)
    return times


def config_dict(n_gpus):
    return {"workload": "BASELINE config 2: Qwen3-30B-A3B MoE layer BF16, 32 experts HBM hot tier + 96 in pinned "
                        "host memory read in place, decode batch 256, Zipf(1.1)+N(0,1) router logits",
            "hidden": SHAPE["H"], "expert_intermediate": SHAPE["I"], "experts": SHAPE["E"], "top_k": SHAPE["K"],
            "tokens_per_step_per_gpu": BATCH, "hot_experts": N_HOT, "credits": CREDITS, "form": FORM,
            "parallelism": "1 GPU" if n_gpus == 1 else
            f"ep{n_gpus}: {SHAPE['E'] // n_gpus} experts per GPU (up to {N_HOT} of them in HBM, the rest in pinned host "
            f"memory), {BATCH} tokens per GPU per step, NCCL all-to-all dispatch/return",
            "l2": "weights streamed per step (302 MB HBM hot tier + host reads) exceed the 126 MB L2; "
                  f"{N_BATCHES} input batches rotate"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    wl = make_workload()
    threads = os.cpu_count() or 1
    times = cpu_layer_time(wl, threads, reps=max(1, args.steps), warm=max(1, min(args.warmup, 3)))
    sec = sum(times) / len(times)
    value = BATCH / sec
    line = {"impl": "reference", "metric": "moe_layer_tokens_per_s", "value": value, "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": len(times), "warmup": args.warmup, "ms_per_step": sec * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": config_dict(1),
            "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port",
                             "sample": f"{len(times)} batches of {BATCH} tokens, whole layer, "
                                       "oracle/torch_path.py (reference's PyTorch MoE loop) on the host CPU"},
            "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def run_profile_target(args):
    """A short, quiet run of the layer for `ncu` (one GPU).  --ep: the expert-parallel layer as a single
    rank, so that its exchange kernels (counts, dispatch, return) run with this GPU as their own peer."""
    from monoserve_b200.moe import MoELayer
    H, I, E, K = SHAPE["H"], SHAPE["I"], SHAPE["E"], SHAPE["K"]
    wl = make_workload()
    if args.ep:
        from monoserve_b200.ep import ExpertParallelMoE
        ep = ExpertParallelMoE(H, I, E, K, BATCH, rank=0, world=1)
        ep.connect([ep.export()])
        wr = wl["wr"].cuda()
        ep.set_router(wr)
        ep.set_local_experts(wl["w13"], wl["w2"], list(range(E)) if args.all_hot else wl["hot"])
        ep.set_plan(0, CREDITS, FORM)
        out = torch.empty(BATCH, H, dtype=torch.bfloat16, device="cuda")
        xs, x2s = [x.cuda() for x in wl["xs"]], [x.cuda() for x in wl["x2s"]]
        for i in range(args.warmup + args.steps):
            ep.forward(xs[i % N_BATCHES], x2s[i % N_BATCHES], out)
        torch.cuda.synchronize()
        ep.local.status()
        ep.close()
        return
    layer = MoELayer(H, I, E, K, BATCH)
    layer.set_router(wl["wr"].cuda())
    layer.set_experts(wl["w13"], wl["w2"], list(range(E)) if args.all_hot else wl["hot"])
    layer.set_plan(0, CREDITS, FORM)
    out = torch.empty(BATCH, H, dtype=torch.bfloat16, device="cuda")
    xs, x2s = [x.cuda() for x in wl["xs"]], [x.cuda() for x in wl["x2s"]]
    for i in range(args.warmup + args.steps):
        layer.forward(xs[i % N_BATCHES], x2s[i % N_BATCHES], out)
    torch.cuda.synchronize()
    layer.status()
    layer.close()


def ep_check(layer, xn, x2, out, wl, rank, world):
    """One pass of this rank checked against the oracle: routing bit for bit against the C
    oracle, the layer output against the reference's PyTorch MoE path (rel-L2 <= 1e-2)."""
    import numpy as np
    import oracle
    from oracle import torch_path as tp
    K = SHAPE["K"]
    T = xn.shape[0]
    ids_d, w_d = layer.ids[:T].cpu(), layer.w[:T].cpu()
    logits = oracle.router_logits(oracle.bf16_bits(xn.cpu()), oracle.bf16_bits(wl["wr"]))
    ids, w, _ = oracle.router_topk(logits, K)
    exact = bool(np.array_equal(ids_d.numpy(), ids) and np.array_equal(w_d.numpy().view(np.int32), w.view(np.int32)))
    ref, _, _ = tp.moe_layer(xn.cpu().float(), x2.cpu().float(), wl["wr"], wl["w13"], wl["w2"], K,
                             routing=(w_d, ids_d.long()))
    rel = float((out.cpu().float() - ref).norm() / ref.norm())
    return rel, exact


def run_ours_ep(args, wl, world, rank, local):
    """N > 1: experts partitioned over the ranks; every rank brings its own batch of
    BATCH tokens per step (weak scaling).  The headline is the peer exchange (this
    library's own dispatch / return kernels over NVLink); the NCCL all-to-all exchange
    is timed beside it as the library baseline.  Before anything is timed, one pass of
    every rank is checked against the oracle."""
    import torch.distributed as dist
    from monoserve_b200.ep import ExpertParallelMoE
    H, I, E, K = SHAPE["H"], SHAPE["I"], SHAPE["E"], SHAPE["K"]
    El = E // world
    lo = rank * El
    # the HBM hot tier keeps its per-GPU capacity: the N_HOT most probable local experts
    prior_local = wl["prior"][lo:lo + El]
    hot = sorted(torch.argsort(prior_local, descending=True)[:min(N_HOT, El)].tolist())
    w13_l, w2_l = wl["w13"][lo:lo + El].contiguous(), wl["w2"][lo:lo + El].contiguous()
    wr_d = wl["wr"].cuda()
    g = torch.Generator().manual_seed(50 + rank)
    xs, x2s = [], []
    for _ in range(N_BATCHES):
        x = torch.randn(BATCH, H, generator=g)
        x[:, 0] = 1.0
        xs.append(x.to(torch.bfloat16).cuda())
        x2s.append(torch.randn(BATCH, H, generator=g).to(torch.bfloat16).cuda())
    xs_h = [x.cpu().pin_memory() for x in xs]
    x2s_h = [x.cpu().pin_memory() for x in x2s]
    xin, x2in = torch.empty_like(xs[0]), torch.empty_like(xs[0])
    out = torch.empty(BATCH, H, dtype=torch.bfloat16, device="cuda")
    out_h = torch.empty(BATCH, H, dtype=torch.bfloat16, pin_memory=True)

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    def all_max(v):
        t = torch.tensor([v], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def measure(exchange):
        layer = ExpertParallelMoE(H, I, E, K, BATCH, exchange=exchange)
        layer.set_router(wr_d)
        layer.set_local_experts(w13_l, w2_l, hot)
        layer.set_plan(0, CREDITS, FORM)

        def step(i):
            layer.forward(xs[i % N_BATCHES], x2s[i % N_BATCHES], out)

        def step_e2e(i):
            xin.copy_(xs_h[i % N_BATCHES], non_blocking=True)
            x2in.copy_(x2s_h[i % N_BATCHES], non_blocking=True)
            layer.forward(xin, x2in, out)
            out_h.copy_(out, non_blocking=True)
            torch.cuda.current_stream().synchronize()

        # parity first: every rank checks one pass against the oracle
        step(1)
        torch.cuda.synchronize()
        layer.local.status()
        rel, exact = ep_check(layer, xs[1], x2s[1], out, wl, rank, world)
        rel = all_max(rel)
        exact = all_max(0.0 if exact else 1.0) == 0.0
        res = {"parity_checked": True, "rel_l2_max_over_ranks": rel, "routing_bit_exact": exact}
        # The timed steps take a few milliseconds, less than one nvidia-smi sample: the sampler runs over them
        # and over `hold` untimed steps of the same kind before and after, so that its samples show the clocks
        # under this load.
        hold = max(0, 1500 - args.steps)
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        for i in range(args.warmup + hold):
            step(i)
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(args.steps):
            step(args.warmup + i)
        b.record()
        barrier()
        res["ms_dev"] = all_max(a.elapsed_time(b))
        for i in range(hold):
            step(i)
        torch.cuda.synchronize()
        res["clocks"] = sampler.stop() if rank == 0 else {}
        if rank == 0:
            res["clocks"]["window"] = f"the {args.steps} timed steps and {hold} untimed steps of the same kind on either side"
        layer.local.status()
        for i in range(3):
            step_e2e(i)
        barrier()
        t0 = time.perf_counter()
        for i in range(args.steps):
            step_e2e(i)
        barrier()
        res["sec_e2e"] = all_max(time.perf_counter() - t0)
        layer.local.status()
        if exchange == "peer":
            # per-phase device times (CUDA events on the launching stream), a separate pass
            layer.set_profile(1)
            acc, active = {}, []
            n_prof = min(args.steps, 20)
            for i in range(n_prof):
                step(i)
                for k, v in layer.last_times().items():
                    acc.setdefault(k, []).append(v)
                active.append(int((layer.local.workspace("counts")[:El] > 0).sum()))
            layer.set_profile(0)
            res["phase_ms"] = {k: sum(v) / len(v) for k, v in acc.items()}
            res["active_local_experts"] = sum(active) / len(active)
            barrier()
        res["n_hot_local"] = len(hot)
        layer.close()
        return res

    peer = measure("peer")
    nccl = measure("nccl")
    anchor = None
    if rank == 0:
        # like-for-like anchor: the one-GPU layer with every expert in HBM, same batch size, on this GPU
        from monoserve_b200.moe import MoELayer
        solo = MoELayer(H, I, E, K, BATCH)
        solo.set_router(wr_d)
        solo.set_region(1, solo.pack_w13(wl["w13"].cuda()), wl["w2"].cuda(), packed=True)
        tbl = torch.ones(E, 2, dtype=torch.int32)
        tbl[:, 1] = torch.arange(E)
        solo.set_table(tbl)
        for i in range(5):
            solo.forward(xs[i % N_BATCHES], x2s[i % N_BATCHES], out)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(args.steps):
            solo.forward(xs[i % N_BATCHES], x2s[i % N_BATCHES], out)
        b.record()
        torch.cuda.synchronize()
        solo.status()
        anchor = BATCH * args.steps / (a.elapsed_time(b) * 1e-3)
        solo.close()
    dist.barrier()
    if rank == 0:
        tokens = BATCH * world
        pk = peaks()
        expert_bytes = 3 * I * H * 2
        n_cold = El - peer["n_hot_local"]
        line = {"metric": "moe_layer_tokens_per_s", "value": tokens * args.steps / (peer["ms_dev"] * 1e-3),
                "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": peer["ms_dev"] / args.steps, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config_dict(world),
                "clocks": peer["clocks"],
                "e2e": {"value": tokens * args.steps / peer["sec_e2e"], "unit": "tokens/s",
                        "h2d_bytes_per_step": 2 * BATCH * H * 2, "d2h_bytes_per_step": BATCH * H * 2},
                "gpu_launches": 8 * args.steps,
                "exchange": "peer stores over NVLink (libmonofab dispatch / return kernels)",
                "ep_check": {k: peer[k] for k in ("parity_checked", "rel_l2_max_over_ranks", "routing_bit_exact")},
                "phase_ms_rank0": peer["phase_ms"],
                "nccl_exchange": {"value": tokens * args.steps / (nccl["ms_dev"] * 1e-3), "unit": "tokens/s",
                                  "ms_per_step": nccl["ms_dev"] / args.steps,
                                  "e2e": tokens * args.steps / nccl["sec_e2e"],
                                  "ep_check": {k: nccl[k] for k in ("parity_checked", "rel_l2_max_over_ranks",
                                                                     "routing_bit_exact")},
                                  "note": "the same layer with torch.distributed all-to-all(-v) over NCCL: two host "
                                          "round trips per layer for the split sizes"},
                "anchor_all_hot_n1_tokens_per_s_per_gpu": anchor,
                "per_gpu_vs_anchor": tokens * args.steps / (peer["ms_dev"] * 1e-3) / world / anchor,
                "cpu_baseline": None}
        if n_cold == 0:
            # every local expert is in HBM: the expert kernel against the HBM roofline on rank 0
            ach = peer["active_local_experts"] * expert_bytes / (peer["phase_ms"]["experts"] * 1e-3) / 1e9
            line["roofline"] = {"kernel": "expert_gemm_kernel (rank 0)", "bound": "hbm", "achieved": ach,
                                "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": ach / pk["hbm_gbs"],
                                "peak_source": pk["source"], "traffic": None,
                                "algorithmic_bytes": peer["active_local_experts"] * expert_bytes}
        else:
            line["roofline"] = {"kernel": "expert_gemm_kernel (rank 0)", "bound": "host_link", "achieved": None,
                                "peak": None, "unit": "GB/s", "frac": None, "traffic": None,
                                "note": f"{n_cold} of {El} local experts are read over the host link; the N=1 line "
                                        "carries the host-link roofline of this kernel"}
        line["note"] = ("weak scaling changes the placement: per-GPU hot tier of %d experts holds %d of %d local "
                        "experts; compare per-GPU tokens/s with the N=1 line's roofline_all_hot.layer_tokens_per_s "
                        "(every expert in HBM)" % (N_HOT, peer["n_hot_local"], El))
        print(json.dumps(line), flush=True)
    dist.destroy_process_group()


def config1_workload():
    """Benchmark configuration 1: weights N(0, 0.02) from seed 0 in the order router [E, H], w13 [E, 2I, H],
    w2 [E, H, I]; activations N(0, 1) from seed 1 for a ragged batch of 64 decode tokens plus one 512-token
    prefill (576 rows for the MoE layer)."""
    H, I, E = SHAPE["H"], SHAPE["I"], SHAPE["E"]
    g = torch.Generator().manual_seed(0)
    wr = (torch.randn(E, H, generator=g) * 0.02).to(torch.bfloat16)
    w13 = (torch.randn(E, 2 * I, H, generator=g) * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(E, H, I, generator=g) * 0.02).to(torch.bfloat16)
    xn = torch.randn(576, H, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16)
    return wr, w13, w2, xn


def run_config1(steps):
    """Config 1 on the GPU (every expert in HBM, stream path, CUDA events over `steps` passes) and the
    reference's PyTorch MoE loop on the host cores on the same batch."""
    from monoserve_b200.moe import MoELayer
    from oracle import torch_path as tp
    H, I, E, K = SHAPE["H"], SHAPE["I"], SHAPE["E"], SHAPE["K"]
    wr, w13, w2, xn = config1_workload()
    T = xn.shape[0]
    layer = MoELayer(H, I, E, K, T)
    layer.set_router(wr.cuda())
    layer.set_region(1, layer.pack_w13(w13.cuda()), w2.cuda(), packed=True)
    tbl = torch.ones(E, 2, dtype=torch.int32)
    tbl[:, 1] = torch.arange(E)
    layer.set_table(tbl)
    xd, out = xn.cuda(), torch.empty(T, H, dtype=torch.bfloat16, device="cuda")
    for _ in range(3):
        layer.forward(xd, None, out)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        layer.forward(xd, None, out)
    b.record()
    b.synchronize()
    layer.status()
    ms = a.elapsed_time(b) / steps
    layer.set_profile(1)
    layer.forward(xd, None, out)
    kt = layer.last_times()
    layer.set_profile(0)
    active = int((layer.workspace("counts")[:E] > 0).sum())
    ids = layer.workspace("topk_ids")[:T * K].view(T, K).cpu().long()
    tw = layer.workspace("topk_w")[:T * K].view(T, K).cpu()
    got = out.float().cpu()
    layer.close()
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    times = []
    with torch.no_grad():
        for i in range(4):
            t0 = time.perf_counter()
            ref, _, _ = tp.moe_layer(xn.float(), None, wr, w13, w2, K, routing=(tw, ids))
            times.append(time.perf_counter() - t0)
    sec = sum(times[1:]) / len(times[1:])
    pk = peaks()
    bytes_alg = active * 3 * H * I * 2
    return {"workload": "BASELINE config 1: 576 rows (64 decode + one 512-token prefill), every expert in HBM",
            "tokens": T, "ms": ms, "tokens_per_s": T / ms * 1e3, "kernel_ms": kt, "active_experts": active,
            "experts_kernel_hbm_gbs": bytes_alg / (kt["experts"] * 1e-3) / 1e9,
            "experts_kernel_hbm_frac": bytes_alg / (kt["experts"] * 1e-3) / 1e9 / pk["hbm_gbs"],
            "layer_hbm_frac": bytes_alg / (ms * 1e-3) / 1e9 / pk["hbm_gbs"],
            "rel_l2_vs_cpu_reference": float((got - ref).norm() / ref.norm()),
            "cpu_baseline": {"value": T / sec, "unit": "tokens/s", "cores": threads, "kind": "port",
                             "sample": "3 passes of the same 576-row batch, oracle/torch_path.py on the host CPU"}}


def run_sweep(args):
    """The sweep benchmark configuration 2 describes: decode batches 1 / 8 / 32 / 128 / 256, link credits 1..16
    and both kernel forms for host-resident experts (row blocks of 64, and the one-pass form the reference's
    asymmetric form maps to).  Per point: layer time (CUDA events over `--steps` passes of the stream path,
    inputs resident, the input batches rotating), tokens/s, activated hot / cold experts and the host-link rate
    = cold experts x 9.44 MB / time.  A text table on stderr, one JSON line on stdout."""
    from monoserve_b200.moe import MoELayer
    H, I, E, K = SHAPE["H"], SHAPE["I"], SHAPE["E"], SHAPE["K"]
    torch.cuda.set_device(0)
    wl = make_workload()
    layer = MoELayer(H, I, E, K, BATCH)
    layer.set_router(wl["wr"].cuda())
    layer.set_experts(wl["w13"], wl["w2"], wl["hot"])
    xs, x2s = [x.cuda() for x in wl["xs"]], [x.cuda() for x in wl["x2s"]]
    expert_bytes, hot, rows = 3 * H * I * 2, set(wl["hot"]), []
    for T in (1, 8, 32, 128, 256):
        out = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")
        for form in (64, 0):
            for credits in (1, 2, 4, 8, 16):
                layer.set_plan(0, credits, form)

                def step(i):
                    layer.forward(xs[i % N_BATCHES][:T].contiguous(), x2s[i % N_BATCHES][:T].contiguous(), out)
                for i in range(3):
                    step(i)
                torch.cuda.synchronize()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                for i in range(args.steps):
                    step(i)
                b.record()
                b.synchronize()
                layer.status()
                cold_sum = hot_sum = 0
                n = min(N_BATCHES, args.steps)
                for i in range(n):      # activated experts of the batches used
                    step(i)
                    counts = layer.workspace("counts")[:E].cpu()
                    act = [e for e in range(E) if counts[e] > 0]
                    cold_sum += sum(1 for e in act if e not in hot)
                    hot_sum += sum(1 for e in act if e in hot)
                ms = a.elapsed_time(b) / args.steps
                rows.append(dict(batch=T, form=form, credits=credits, ms=ms, tokens_per_s=T / ms * 1e3,
                                 hot_active=hot_sum / n, cold_active=cold_sum / n,
                                 host_link_gbs=cold_sum / n * expert_bytes / (ms * 1e-3) / 1e9))
                r = rows[-1]
                print(f"batch {T:4d} form {form:3d} credits {credits:2d}: {ms:8.3f} ms  {r['tokens_per_s']:9.0f} tok/s  "
                      f"cold {r['cold_active']:5.1f} hot {r['hot_active']:5.1f}  link {r['host_link_gbs']:5.1f} GB/s",
                      file=sys.stderr)
    print(json.dumps({"workload": "BASELINE config 2 sweep (stream path)", "rows": rows}))
    layer.close()


def run_ours(args):
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from monoserve_b200.moe import MoELayer
    H, I, E, K = SHAPE["H"], SHAPE["I"], SHAPE["E"], SHAPE["K"]
    wl = make_workload()
    if world > 1:
        return run_ours_ep(args, wl, world, rank, local)
    layer = MoELayer(H, I, E, K, BATCH)
    layer.set_router(wl["wr"].cuda())
    layer.set_experts(wl["w13"], wl["w2"], wl["hot"])
    layer.set_plan(0, CREDITS, FORM)
    xs = [x.cuda() for x in wl["xs"]]
    x2s = [x.cuda() for x in wl["x2s"]]
    xs_h = [x.pin_memory() for x in wl["xs"]]
    x2s_h = [x.pin_memory() for x in wl["x2s"]]
    out = torch.empty(BATCH, H, dtype=torch.bfloat16, device="cuda")
    out_h = torch.empty(BATCH, H, dtype=torch.bfloat16, pin_memory=True)
    link_peak = measure_h2d_gbs() if rank == 0 else 0.0

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warm):
        for i in range(warm):
            fn(i)
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(steps):
            fn(warm + i)
        b.record()
        barrier()
        ms = torch.tensor([a.elapsed_time(b)], device="cuda")
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    # device-resident pass
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms_dev = timed(lambda i: layer.forward(xs[i % N_BATCHES], x2s[i % N_BATCHES], out), args.steps, args.warmup)
    clocks = sampler.stop() if rank == 0 else {}
    layer.status()

    # end to end through the host-buffer entry point (copies inside the timed region)
    t_e2e = []

    def e2e_step(i):
        layer.forward_host(xs_h[i % N_BATCHES], x2s_h[i % N_BATCHES], out_h)
    for i in range(min(args.warmup, 3)):
        e2e_step(i)
    barrier()
    t0 = time.perf_counter()
    for i in range(args.steps):
        e2e_step(i)
    barrier()
    sec_e2e = torch.tensor([time.perf_counter() - t0], device="cuda")
    if world > 1:
        dist.all_reduce(sec_e2e, op=dist.ReduceOp.MAX)
    sec_e2e = float(sec_e2e.item())
    layer.status()

    # per-kernel times with CUDA events on the launching stream (separate pass)
    layer.set_profile(1)
    kt = {}
    prof_steps = min(args.steps, 20)
    step_counts = []   # per profiled step: the routed rows of every expert (the batches differ)
    for i in range(prof_steps):
        layer.forward(xs[i % N_BATCHES], x2s[i % N_BATCHES], out)
        for k, v in layer.last_times().items():
            kt.setdefault(k, []).append(v)
        step_counts.append(layer.workspace("counts")[:E].cpu())
    layer.set_profile(0)
    kt = {k: sum(v) / len(v) for k, v in kt.items()}

    # the same layer with every expert in the HBM hot tier: the kernel against the HBM roofline
    hot_kt = None
    if rank == 0:
        layer_hot = MoELayer(H, I, E, K, BATCH)
        layer_hot.set_router(wl["wr"].cuda())
        layer_hot.set_region(1, layer_hot.pack_w13(wl["w13"].cuda()), wl["w2"].cuda(), packed=True)
        tbl = torch.ones(E, 2, dtype=torch.int32)
        tbl[:, 1] = torch.arange(E)
        layer_hot.set_table(tbl)
        layer_hot.set_profile(1)
        hot_kt = {}
        hot_active_steps = []
        for i in range(3 + prof_steps):
            layer_hot.forward(xs[i % N_BATCHES], x2s[i % N_BATCHES], out)
            if i >= 3:
                for k, v in layer_hot.last_times().items():
                    hot_kt.setdefault(k, []).append(v)
                hot_active_steps.append(int((layer_hot.workspace("counts")[:E] > 0).sum()))
        hot_kt = {k: sum(v) / len(v) for k, v in hot_kt.items()}
        layer_hot.set_profile(0)
        hot_ms_step = timed(lambda i: layer_hot.forward(xs[i % N_BATCHES], x2s[i % N_BATCHES], out),
                            args.steps, 3) / args.steps if world == 1 else float("nan")
        hot_active = sum(hot_active_steps) / len(hot_active_steps)   # mean over the steps whose times are averaged
        layer_hot.status()
        layer_hot.close()

    if rank == 0:
        # algorithmic bytes of the dominant kernel (w13): every activated expert's w13 once
        # mean over the profiled steps (the kernel time below is the mean over the same steps)
        table = layer.table
        is_cold = torch.tensor([int(table[e, 0]) == 0 for e in range(E)])
        cold = sum(float(((c > 0) & is_cold).sum()) for c in step_counts) / len(step_counts)
        hot = sum(float(((c > 0) & ~is_cold).sum()) for c in step_counts) / len(step_counts)
        w13_bytes = 3 * I * H * 2      # one expert: w13 + w2, read by the single fused GEMM launch
        pk = peaks()
        dom = "experts"
        link_bytes, hbm_bytes = cold * w13_bytes, hot * w13_bytes
        achieved = link_bytes / (kt[dom] * 1e-3) / 1e9 if kt[dom] > 0 else 0.0
        tokens = BATCH * world
        cpu_threads = os.cpu_count() or 1
        cpu_times = cpu_layer_time(wl, cpu_threads, reps=5, warm=1) if world == 1 else None
        line = {
            "metric": "moe_layer_tokens_per_s", "value": tokens * args.steps / (ms_dev * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_dev / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": config_dict(world), "clocks": clocks,
            "e2e": {"value": tokens * args.steps / sec_e2e, "unit": "tokens/s",
                    "h2d_bytes_per_step": 2 * BATCH * H * 2, "d2h_bytes_per_step": BATCH * H * 2},
            "gpu_launches": 6 * args.steps,
            "kernel_ms": kt,
            "roofline": {"kernel": "expert_gemm_kernel (w13 + w2 tiles, one launch)", "bound": "host_link", "achieved": achieved,
                         "peak": link_peak, "unit": "GB/s", "frac": achieved / link_peak if link_peak else None,
                         "peak_source": "cudaMemcpyAsync H2D of 256 MiB pinned, measured in this run",
                         "algorithmic_bytes": {"host_link": link_bytes, "hbm": hbm_bytes,
                                               "cold_experts_active": cold, "hot_experts_active": hot},
                         "hbm_peak": pk["hbm_gbs"], "hbm_peak_source": pk["source"], "traffic": None},
        }
        hbm_ach = hot_active * w13_bytes / (hot_kt["experts"] * 1e-3) / 1e9
        line["roofline_all_hot"] = {"kernel": "expert_gemm_kernel (w13 + w2 tiles, one launch)", "bound": "hbm", "achieved": hbm_ach,
                                    "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": hbm_ach / pk["hbm_gbs"],
                                    "peak_source": pk["source"], "active_experts": hot_active,
                                    "note": "same batch with all 128 experts in HBM", "kernel_ms": hot_kt,
                                    "algorithmic_bytes": hot_active * w13_bytes, "traffic": None,
                                    "layer_tokens_per_s": BATCH / (hot_ms_step * 1e-3)}
        if cpu_times:
            sec = sum(cpu_times) / len(cpu_times)
            line["cpu_baseline"] = {"value": BATCH / sec, "unit": "tokens/s", "cores": cpu_threads, "kind": "port",
                                    "sample": f"{len(cpu_times)} batches of {BATCH} tokens, whole layer, "
                                              "oracle/torch_path.py on the host CPU"}
        if world == 1:
            line["config1"] = run_config1(min(args.steps, 20))
        if world == 1 and not args.no_mixed_lane:
            line["fabric_layer"] = side_run(["monoserve_b200.benchmarks.fabric_layer"], 300)
            line["attention"] = side_run(["monoserve_b200.benchmarks.attention"], 300)
            line["mixed_lane"] = side_run(["monoserve_b200.benchmarks.mixed_lane", "--steps", "20"], 900)
            line["config4"] = side_run(["monoserve_b200.benchmarks.mixed_lane", "--model", "glm", "--steps", "8"], 900)
            line["serve"] = side_run(["monoserve_b200.benchmarks.serve", "--rates", "2,8"], 600)
        print(json.dumps(line), flush=True)
    layer.close()
    if world > 1:
        dist.destroy_process_group()


def side_run(module_args, timeout_s):
    """More measurements ride on the N = 1 line, each made by a module of
    monoserve_b200/benchmarks in a process of its own: `fabric_layer`, the same MoE layer as a
    repeating fabric program timed by the in-kernel iteration timer (the reference's protocol for
    MoE-layer tokens/s); `attention`, the paged-KV attention kernel on config-3 shapes (decode
    K+V GB/s, prefill TFLOP/s); `mixed_lane`, the second headline metric: decode TPOT p50
    on config 3 (the full 48-layer Qwen3-30B-A3B-shaped decoder, a 4 x 2048 prefill lane beside a
    128-sequence decode lane in one persistent kernel; it pins 58 GB of host memory); `config4`,
    the same for the GLM-4.5-Air-shaped FP8 decoder of config 4; and `serve`, config 5 at N = 1:
    continuous batching under Poisson arrivals at 2 and 8 requests/s (TTFT, time per output token,
    output tokens/s, host time per program build)."""
    cmd = [sys.executable, "-m"] + module_args
    try:
        out = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout_s,
                             cwd=os.path.dirname(os.path.abspath(__file__)))
        last = [ln for ln in out.stdout.splitlines() if ln.startswith("{")]
        if out.returncode != 0 or not last:
            return {"error": (out.stderr or out.stdout)[-300:]}
        return json.loads(last[-1])
    except Exception as exc:   # the headline line is printed regardless
        return {"error": repr(exc)[:300]}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--ncu", action="store_true",
                    help="profiling target: only W warm-up + K device-resident steps, no JSON line")
    ap.add_argument("--all-hot", action="store_true", help="with --ncu: place all 128 experts in HBM")
    ap.add_argument("--ep", action="store_true", help="with --ncu: run the expert-parallel layer as one rank")
    ap.add_argument("--no-mixed-lane", action="store_true",
                    help="skip the side runs that the N=1 line carries (`fabric_layer`, `attention`, `mixed_lane`, "
                         "`config4`, `serve`)")
    ap.add_argument("--sweep", action="store_true",
                    help="the batch x credits x form sweep of benchmark configuration 2 instead of the bench line")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.sweep:
        run_sweep(args)
    elif args.ncu:
        run_profile_target(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
