"""Expert parallelism on GPUs: the one-rank path against the plain layer, and
(when the box has two or more GPUs) two NCCL ranks against the oracle."""
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


def test_single_rank_path_equals_plain_layer():
    from monoserve_b200.ep import ExpertParallelMoE
    from monoserve_b200.moe import MoELayer
    T, H, I, E, K = 70, 512, 256, 16, 4
    wr, w13, w2 = _weights(H, I, E, 1)
    xn, x2 = _tokens(0, T, H)
    plain = MoELayer(H, I, E, K, T)
    plain.set_router(wr.cuda())
    plain.set_experts(w13, w2, hot=list(range(8)))
    want = plain.forward(xn.cuda(), x2.cuda()).clone()
    ep = ExpertParallelMoE(H, I, E, K, T)
    ep.set_router(wr.cuda())
    ep.set_local_experts(w13, w2, hot=list(range(8)))
    got = ep.forward(xn.cuda(), x2.cuda())
    torch.cuda.synchronize()
    assert ep.local.status() == 0
    assert torch.equal(got, want)
    plain.close()
    ep.close()


def _ep_worker(rank, world, port, T, H, I, E, K, result_dir):
    import torch.distributed as dist
    from monoserve_b200.ep import ExpertParallelMoE
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        wr, w13, w2 = _weights(H, I, E, 1)
        El = E // world
        layer = ExpertParallelMoE(H, I, E, K, T)
        layer.set_router(wr.cuda())
        layer.set_local_experts(w13[rank * El:(rank + 1) * El].contiguous(), w2[rank * El:(rank + 1) * El].contiguous(),
                                hot=list(range(0, El, 2)))
        xn, x2 = _tokens(rank, T, H)
        out = layer.forward(xn.cuda(), x2.cuda())
        torch.cuda.synchronize()
        assert layer.local.status() == 0
        torch.save(dict(out=out.cpu(), ids=layer.ids[:T].cpu(), w=layer.w[:T].cpu()), os.path.join(result_dir, f"r{rank}.pt"))
        layer.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_match_the_reference_path(tmp_path):
    import torch.multiprocessing as mp
    from oracle import torch_path as tp
    T, H, I, E, K = 90, 512, 256, 16, 4
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    mp.spawn(_ep_worker, args=(2, port, T, H, I, E, K, str(tmp_path)), nprocs=2, join=True)
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
