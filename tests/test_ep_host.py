"""Expert-parallel exchange plumbing on the CPU: two gloo ranks run the same
host-side functions the GPU path uses (counts exchange, dispatch, return) on
rows packed by the oracle, and every rank checks what it received and what came
back against the definition."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _routing(rank, T, E, K):
    g = torch.Generator().manual_seed(100 + rank)
    ids = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).to(torch.int32)
    w = torch.rand(T, K, generator=g)
    return ids, w


def _rows(rank, T, H):
    # row content identifies (rank, token)
    return (torch.arange(T)[:, None] * 1000 + rank * 100000 + torch.arange(H)[None, :]).float()


def _worker(rank, world, port, T, E, K, H):
    import oracle
    from monoserve_b200 import ep
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        El = E // world
        ids, w = _routing(rank, T, E, K)
        counts = np.bincount(ids.numpy().ravel(), minlength=E).astype(np.int32)
        starts = oracle.scan(counts)
        pt, pw, pp = oracle.pack(ids.numpy(), w.numpy(), starts)
        x = _rows(rank, T, H)
        send = x[torch.from_numpy(pt).long()]
        counts_t = torch.from_numpy(counts)
        recv_counts = ep.exchange_counts(counts_t)
        send_splits = ep.split_plan(counts_t, world)
        recv_splits = recv_counts.sum(1).tolist()
        assert send_splits == [int(counts[d * El:(d + 1) * El].sum()) for d in range(world)]
        recv_buf = torch.zeros(T * K * world, H)
        got = ep.dispatch_rows(send, send_splits, recv_buf, recv_splits)
        # expected: for every source rank, its packed rows of MY experts, in its packed order
        exp_rows, exp_expert = [], []
        for s in range(world):
            ids_s, _ = _routing(s, T, E, K)
            c_s = np.bincount(ids_s.numpy().ravel(), minlength=E).astype(np.int32)
            st_s = oracle.scan(c_s)
            pt_s, _, _ = oracle.pack(ids_s.numpy(), np.zeros((T, K), np.float32), st_s)
            lo, hi = st_s[rank * El], st_s[(rank + 1) * El]
            exp_rows.append(_rows(s, T, H)[torch.from_numpy(pt_s[lo:hi]).long()])
            assert np.array_equal(recv_counts[s].numpy(), c_s[rank * El:(rank + 1) * El])
            for e in range(El):
                exp_expert += [e] * int(c_s[rank * El + e])
        assert torch.equal(got, torch.cat(exp_rows))
        # "expert FFN": y = row * (global expert id + 1); segments are (source, local expert)
        seg_expert = torch.tensor(exp_expert) + rank * El
        y_local = got * (seg_expert[:, None].float() + 1)
        y_back = ep.return_rows(y_local, recv_splits, torch.zeros(T * K, H), send_splits)
        e_of_pos = np.repeat(np.arange(E), counts)
        want = send * (torch.from_numpy(e_of_pos)[:, None].float() + 1)
        assert torch.equal(y_back, want)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,T,E,K", [(2, 37, 8, 2), (2, 5, 16, 4)])
def test_dispatch_and_return_over_gloo(world, T, E, K):
    mp.spawn(_worker, args=(world, _free_port(), T, E, K, 8), nprocs=world, join=True)


def test_split_plan_requires_even_partition():
    from monoserve_b200 import ep
    with pytest.raises(AssertionError):
        ep.split_plan(torch.ones(10, dtype=torch.int32), 4)
    assert ep.split_plan(torch.tensor([1, 2, 3, 4], dtype=torch.int32), 2) == [3, 7]


def test_peer_exchange_layout():
    """dest_base (and its C twin, the arithmetic the dispatch kernel does) against a receive buffer
    built by concatenation: the owner's experts in order, inside an expert the source ranks in order."""
    from monoserve_b200 import _C, ep
    rng = np.random.default_rng(5)
    for world, E in [(2, 8), (4, 16), (8, 128), (1, 4)]:
        El = E // world
        counts = rng.integers(0, 7, (world, E)).astype(np.int32)
        counts[rng.integers(0, world), :] = 0          # a rank without tokens
        for owner in range(world):
            want, row = {}, 0
            for e in range(owner * El, (owner + 1) * El):
                for src in range(world):
                    want[(src, e)] = row
                    row += int(counts[src, e])
            for (src, e), base in want.items():
                assert ep.dest_base(counts, src, e) == base
                assert _C.lib.monofab_ep_dest_base(counts.ctypes.data, E, world, E, src, e) == base
