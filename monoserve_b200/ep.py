"""Expert parallelism for one MoE layer: experts partitioned over the ranks of
one node, token dispatch and return as all-to-all exchanges over NVLink (NCCL
through torch.distributed), everything else local.

The reference has no collective of its own; its only multi-GPU mode is stock
vLLM expert parallelism (monoserve/baselines/serve_ep.py:24-28).  Here rank r
owns experts [r * E/N, (r + 1) * E/N); routing, packing and combining are
data-parallel over each rank's own tokens.

Per layer and rank:
  1. router logits + top-k on the local tokens (all E experts);
  2. stable pack by GLOBAL expert id: the packed rows of a destination rank are
     one contiguous range of the send buffer, in (expert, token, pick) order;
  3. counts exchange: all-to-all of int32 [E/N] per peer;
  4. dispatch: all-to-all-v of bf16 rows, received straight into the local
     layer's packed-row workspace, ordered (source rank, local expert, row);
  5. expert FFN over N * E/N segments (monofab_moe_experts);
  6. return: all-to-all-v of the fp32 expert-output rows, back in packed order;
  7. weighted combine in pick order (deterministic).
With N = 1 nothing is exchanged.

`split_plan`, `exchange_counts`, `dispatch_rows` and `return_rows` hold the
host-side logic and work on any backend (the CPU tests run them over gloo).
"""
import ctypes

import torch
import torch.distributed as dist


def split_plan(counts, world):
    """Rows this rank sends to every peer, from its per-expert pair counts
    (int64/32 CPU tensor [E]); experts are partitioned contiguously."""
    E = counts.numel()
    assert E % world == 0, "experts must divide evenly over the ranks"
    return counts.view(world, E // world).sum(1).tolist()


def exchange_counts(counts, group=None):
    """counts: int32 [E] on the exchange device.  Returns recv_counts int32
    [world, E/world]: rows coming from every source rank for each local expert."""
    world = dist.get_world_size(group)
    recv = torch.empty_like(counts)
    dist.all_to_all_single(recv, counts.contiguous(), group=group)
    return recv.view(world, counts.numel() // world)


def dispatch_rows(send, send_splits, recv_buf, recv_splits, group=None):
    """All-to-all-v of packed rows.  send: [P, H]; recv_buf: [>= sum(recv_splits), H]."""
    n = sum(recv_splits)
    assert recv_buf.shape[0] >= n, f"receive buffer of {recv_buf.shape[0]} rows cannot take {n}"
    out = recv_buf[:n]
    dist.all_to_all_single(out, send.contiguous(), output_split_sizes=recv_splits, input_split_sizes=send_splits,
                           group=group)
    return out


def return_rows(y_local, recv_splits, y_back, send_splits, group=None):
    """The reverse exchange: every rank sends back the outputs of the rows it
    received; y_back ends up in the sender's packed order."""
    dist.all_to_all_single(y_back, y_local.contiguous(), output_split_sizes=send_splits,
                           input_split_sizes=recv_splits, group=group)
    return y_back


class ExpertParallelMoE:
    """One MoE layer over the ranks of `group` (None = the default group).

    layer = ExpertParallelMoE(H, I, E, K, max_tokens)
    layer.set_router(wr)                          # bf16 [E, H] on this GPU (replicated)
    layer.set_local_experts(w13, w2, hot=[...])   # THIS rank's experts [E/N, 2I, H], [E/N, H, I]
    out = layer.forward(xn, x2)                   # local tokens in, local tokens out
    """

    def __init__(self, hidden, intermediate, experts, top_k, max_tokens, group=None, capacity_factor=None):
        from monoserve_b200 import _C
        from monoserve_b200.moe import MoELayer
        self._C = _C
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        assert experts % self.world == 0
        self.H, self.I, self.E, self.K, self.T = hidden, intermediate, experts, top_k, max_tokens
        self.El = experts // self.world
        # worst case every pair of every rank lands here; capacity_factor trims the workspace
        rows_cap = max_tokens * top_k * self.world
        if capacity_factor is not None:
            rows_cap = int(max_tokens * top_k * capacity_factor)
        self.rows_cap = rows_cap
        self.local = MoELayer(hidden, intermediate, self.El, 1, rows_cap)
        P = max_tokens * top_k
        dev = "cuda"
        self.logits = torch.empty(max_tokens, experts, device=dev)
        self.ids = torch.empty(max_tokens, top_k, dtype=torch.int32, device=dev)
        self.w = torch.empty(max_tokens, top_k, device=dev)
        self.counts = torch.empty(experts, dtype=torch.int32, device=dev)
        self.starts = torch.empty(experts + 1, dtype=torch.int32, device=dev)
        self.pair_token = torch.empty(P, dtype=torch.int32, device=dev)
        self.pair_weight = torch.empty(P, device=dev)
        self.pair_pos = torch.empty(P, dtype=torch.int32, device=dev)
        self.send = torch.empty(P, hidden, dtype=torch.bfloat16, device=dev)
        self.y_back = torch.empty(P, hidden, device=dev)
        self.scratch = torch.empty(max(_C.lib.monofab_pack_scratch_bytes(max_tokens, experts, top_k), 16),
                                   dtype=torch.uint8, device=dev)
        self.seg_expert = torch.arange(self.El, dtype=torch.int32, device=dev).repeat(self.world).contiguous()
        self.wr = None

    def set_router(self, wr):
        assert wr.is_cuda and wr.dtype == torch.bfloat16 and wr.shape == (self.E, self.H) and wr.is_contiguous()
        self.wr = wr

    def set_local_experts(self, w13, w2, hot, pack_hot=True):
        assert w13.shape[0] == self.El and w2.shape[0] == self.El
        self.local.set_experts(w13, w2, hot, pack_hot=pack_hot)

    def set_plan(self, ctas=0, credits=8, form=64):
        self.local.set_plan(ctas, credits, form)

    def forward(self, xn, x2=None, out=None):
        C, lib = self._C, self._C.lib
        T = xn.shape[0]
        assert T <= self.T and xn.is_cuda and xn.dtype == torch.bfloat16 and xn.is_contiguous()
        if out is None:
            out = torch.empty_like(xn)
        st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        P = T * self.K
        C.check(lib.monofab_router_logits(xn.data_ptr(), self.wr.data_ptr(), self.logits.data_ptr(), T, self.H, self.E, st))
        C.check(lib.monofab_router_topk(self.logits.data_ptr(), None, self.ids.data_ptr(), self.w.data_ptr(), None, None,
                                        None, T, self.E, self.K, 0, 1, 1.0, 0, st))
        C.check(lib.monofab_pack_pairs(self.ids.data_ptr(), self.w.data_ptr(), T, self.E, self.K, self.H, xn.data_ptr(),
                                       self.send.data_ptr(), self.counts.data_ptr(), self.starts.data_ptr(),
                                       self.pair_token.data_ptr(), self.pair_weight.data_ptr(), self.pair_pos.data_ptr(),
                                       self.scratch.data_ptr(), self.scratch.numel(), st))
        xp = self.local.workspace("xp").view(-1, self.H)
        y = self.local.workspace("y").view(-1, self.H)
        if self.world == 1:
            xp[:P].copy_(self.send[:P])
            self.local.experts(self.counts)
            y_back = y[:P]
        else:
            recv_counts = exchange_counts(self.counts, self.group)          # [world, El] on the GPU
            send_splits = split_plan(self.counts.cpu(), self.world)         # host sync: NCCL needs host split sizes
            recv_splits = recv_counts.sum(1).cpu().tolist()
            if sum(recv_splits) > self.rows_cap:
                raise RuntimeError(f"monofab: {sum(recv_splits)} rows routed to rank {self.rank} exceed the "
                                   f"workspace of {self.rows_cap} rows")
            dispatch_rows(self.send[:P], send_splits, xp, recv_splits, self.group)
            self.local.experts(recv_counts.reshape(-1).contiguous(), self.seg_expert)
            y_back = return_rows(y[:sum(recv_splits)], recv_splits, self.y_back[:P], send_splits, self.group)
        C.check(lib.monofab_combine(y_back.data_ptr(), self.pair_pos.data_ptr(), self.w.data_ptr(),
                                    x2.data_ptr() if x2 is not None else None, out.data_ptr(), None, None, T, self.K,
                                    self.H, 0.0, st))
        return out

    def close(self):
        self.local.close()
