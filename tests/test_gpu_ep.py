"""Expert parallelism on GPUs: the one-rank path against the plain layer; four
ranks standing on ONE GPU, their phases run in lockstep, against the plain layer and
the oracle (the peer exchange's layout, flags and buffer reuse need no second GPU to
be checked); and, when the box has two or more GPUs, two ranks as processes, each
exchange against the oracle."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _weights(H, I, E, seed):
    g = torch.Generator().manual_seed(seed)
    wr = (torch.randn(E, H, generator=g) * H ** -0.5).to(torch.bfloat16)
    w13 = (torch.randn(E, 2 * I, H, generator=g) * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(E, H, I, generator=g) * 0.02).to(torch.bfloat16)
    return wr, w13, w2


def _tokens(rank, T, H):
    g = torch.Generator().manual_seed(1000 + rank)
    return torch.randn(T, H, generator=g).to(torch.bfloat16), torch.randn(T, H, generator=g).to(torch.bfloat16)


@pytest.mark.parametrize("exchange", ["peer", "nccl"])
def test_single_rank_path_equals_plain_layer(exchange):
    from monoserve_b200.ep import ExpertParallelMoE
    from monoserve_b200.moe import MoELayer
    T, H, I, E, K = 70, 512, 256, 16, 4
    wr, w13, w2 = _weights(H, I, E, 1)
    xn, x2 = _tokens(0, T, H)
    plain = MoELayer(H, I, E, K, T)
    plain.set_router(wr.cuda())
    plain.set_experts(w13, w2, hot=list(range(8)))
    want = plain.forward(xn.cuda(), x2.cuda()).clone()
    ep = ExpertParallelMoE(H, I, E, K, T, exchange=exchange)
    wr_d = wr.cuda()
    ep.set_router(wr_d)
    ep.set_local_experts(w13, w2, hot=list(range(8)))
    for _ in range(2):
        got = ep.forward(xn.cuda(), x2.cuda())
        torch.cuda.synchronize()
        assert ep.local.status() == 0
        assert torch.equal(got, want)
    plain.close()
    ep.close()


@pytest.mark.parametrize("world,tokens", [(4, [70, 33, 0, 64]), (2, [5, 90])])
def test_ranks_on_one_gpu_in_lockstep(world, tokens):
    """`world` expert-parallel ranks as objects of this process on one GPU.  Phase p of every rank
    is launched before phase p + 1 of any, on one stream, so every flag a kernel waits for was
    raised by a kernel launched before it.  Three passes in a row (buffer and flag reuse, counts
    table parity), token counts that differ per rank and a rank with none.  Each rank's output
    must equal, bit for bit, what the one-GPU layer holding all experts gives for its tokens."""
    import oracle
    from monoserve_b200.ep import ExpertParallelMoE
    from monoserve_b200.moe import MoELayer
    H, I, E, K = 512, 256, 16, 4
    Tmax = max(tokens)
    El = E // world
    wr, w13, w2 = _weights(H, I, E, 3)
    wr_d = wr.cuda()
    plain = MoELayer(H, I, E, K, Tmax)
    plain.set_router(wr_d)
    plain.set_experts(w13, w2, hot=list(range(0, E, 2)))
    ranks = [ExpertParallelMoE(H, I, E, K, Tmax, rank=r, world=world) for r in range(world)]
    handles = [r.export() for r in ranks]
    for r, layer in enumerate(ranks):
        layer.connect(handles)
        layer.set_router(wr_d)
        layer.set_local_experts(w13[r * El:(r + 1) * El].contiguous(), w2[r * El:(r + 1) * El].contiguous(),
                                hot=list(range(0, El, 2)))
    for step in range(3):
        xs = [_tokens(10 * step + r, tokens[(r + step) % world], H) for r in range(world)]
        xs = [(a.cuda(), b.cuda()) for a, b in xs]
        outs = [torch.empty_like(a) for a, _ in xs]
        for p in range(4):
            for r, layer in enumerate(ranks):
                layer.phase(p, xs[r][0], xs[r][1], outs[r])
        torch.cuda.synchronize()
        for r, layer in enumerate(ranks):
            assert layer.local.status() == 0
            T = xs[r][0].shape[0]
            if T == 0:
                continue
            want = plain.forward(xs[r][0], xs[r][1]).clone()
            assert torch.equal(layer.ids[:T], plain.workspace("topk_ids")[:T * K].view(T, K))
            assert torch.equal(outs[r], want), (step, r, float((outs[r].float() - want.float()).abs().max()))
            logits = oracle.router_logits(oracle.bf16_bits(xs[r][0].cpu()), oracle.bf16_bits(wr))
            ids, w, _ = oracle.router_topk(logits, K)
            assert np.array_equal(layer.ids[:T].cpu().numpy(), ids)
            assert np.array_equal(layer.w[:T].cpu().numpy().view(np.int32), w.view(np.int32))
    for layer in ranks:
        layer.disconnect()
    for layer in ranks:
        layer.close()
    plain.close()


def test_receive_capacity_overflow_is_reported():
    """A receive buffer smaller than the rows routed to a rank: the rows beyond it are not sent and
    the pass reports MONOFAB_STATUS_PLAN_OVERFLOW instead of writing out of bounds."""
    from monoserve_b200.ep import ExpertParallelMoE
    H, I, E, K, T, world = 512, 256, 16, 4, 64, 2
    El = E // world
    wr, w13, w2 = _weights(H, I, E, 3)
    wr_d = wr.cuda()
    ranks = [ExpertParallelMoE(H, I, E, K, T, rank=r, world=world, capacity_factor=0.25) for r in range(world)]
    handles = [r.export() for r in ranks]
    for r, layer in enumerate(ranks):
        layer.connect(handles)
        layer.set_router(wr_d)
        layer.set_local_experts(w13[r * El:(r + 1) * El].contiguous(), w2[r * El:(r + 1) * El].contiguous(),
                                hot=list(range(El)))
    xs = [tuple(t.cuda() for t in _tokens(r, T, H)) for r in range(world)]
    outs = [torch.empty_like(a) for a, _ in xs]
    for p in range(4):
        for r, layer in enumerate(ranks):
            layer.phase(p, xs[r][0], xs[r][1], outs[r])
    torch.cuda.synchronize()
    for layer in ranks:
        with pytest.raises(RuntimeError, match="overflow"):
            layer.local.status()
    for layer in ranks:
        layer.disconnect()
    for layer in ranks:
        layer.close()


def _ep_worker(rank, world, port, T, H, I, E, K, result_dir, exchange):
    import torch.distributed as dist
    from monoserve_b200.ep import ExpertParallelMoE
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        wr, w13, w2 = _weights(H, I, E, 1)
        El = E // world
        layer = ExpertParallelMoE(H, I, E, K, T, exchange=exchange)
        wr_d = wr.cuda()
        layer.set_router(wr_d)
        layer.set_local_experts(w13[rank * El:(rank + 1) * El].contiguous(), w2[rank * El:(rank + 1) * El].contiguous(),
                                hot=list(range(0, El, 2)))
        xn, x2 = _tokens(rank, T, H)
        for _ in range(3):   # passes in a row: flags and buffers are reused without a barrier
            out = layer.forward(xn.cuda(), x2.cuda())
        torch.cuda.synchronize()
        assert layer.local.status() == 0
        torch.save(dict(out=out.cpu(), ids=layer.ids[:T].cpu(), w=layer.w[:T].cpu()), os.path.join(result_dir, f"r{rank}.pt"))
        layer.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("exchange", ["peer", "nccl"])
def test_two_ranks_match_the_reference_path(tmp_path, exchange):
    import torch.multiprocessing as mp
    from oracle import torch_path as tp
    T, H, I, E, K = 90, 512, 256, 16, 4
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    mp.spawn(_ep_worker, args=(2, port, T, H, I, E, K, str(tmp_path), exchange), nprocs=2, join=True)
    wr, w13, w2 = _weights(H, I, E, 1)
    for rank in range(2):
        r = torch.load(os.path.join(tmp_path, f"r{rank}.pt"))
        xn, x2 = _tokens(rank, T, H)
        ref, _, _ = tp.moe_layer(xn.float(), x2.float(), wr, w13, w2, K, routing=(r["w"], r["ids"].long()))
        rel = float((r["out"].float() - ref).norm() / ref.norm())
        assert rel < 1e-2, rel
        # routing is local and exact
        import oracle
        logits = oracle.router_logits(oracle.bf16_bits(xn), oracle.bf16_bits(wr))
        ids, w, _ = oracle.router_topk(logits, K)
        assert np.array_equal(r["ids"].numpy(), ids)
        assert np.array_equal(r["w"].numpy().view(np.int32), w.view(np.int32))
