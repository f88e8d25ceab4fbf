"""Expert parallelism for one MoE layer: experts partitioned over the ranks of
one node (one process per GPU), everything else local.

The reference has no collective of its own; its only multi-GPU mode is stock
vLLM expert parallelism (monoserve/baselines/serve_ep.py:24-28).  Here rank r
owns experts [r * E/N, (r + 1) * E/N); routing, packing and combining are
data-parallel over each rank's own tokens.

Two exchanges are built:

  exchange="peer" (the product): libmonofab's own kernels store every routed
      row straight into the owning GPU's packed-row buffer over NVLink, signal
      with flags in peer memory, and push the fp32 expert outputs back the same
      way (csrc/ep_exchange.cu).  No collective call and no host round trip per
      layer; torch.distributed is used once, to hand the buffer handles round.
  exchange="nccl" (the library baseline it is measured against): all-to-all of
      counts, all-to-all-v of rows and of outputs through torch.distributed,
      which needs the split sizes on the host and so blocks twice per layer.

Per layer and rank, either way:
  1. router logits + top-k on the local tokens (all E experts);
  2. stable order by GLOBAL expert id: the rows of a destination rank are
     ordered (expert, token, pick) at the source;
  3. counts exchange;
  4. dispatch of bf16 rows into the owning rank's packed-row workspace, ordered
     (local expert, source rank, row) by the peer exchange - one segment per
     expert - and (source rank, local expert, row) by NCCL's all-to-all-v;
  5. expert FFN over those segments (monofab_moe_experts);
  6. return of the fp32 expert-output rows to the sender's packed order;
  7. weighted combine in pick order (deterministic).

`split_plan`, `exchange_counts`, `dispatch_rows`, `return_rows` and `dest_base`
hold the host-side logic and work on any backend (the CPU tests run them over gloo).
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


def dest_base(counts_all, src, e):
    """First row, in the packed-row buffer of the rank that owns expert e, of the
    rows rank `src` sends for e: every rank's rows of the owner's lower experts,
    then the lower ranks' rows of e - so an expert's rows from all sources are one
    segment.  counts_all: int [world, E].  This is the layout the dispatch kernel
    writes (monofab_ep_dest_base is its C twin)."""
    world, E = counts_all.shape
    El = E // world
    lo = (e // El) * El
    return int(counts_all[:, lo:e].sum() + counts_all[:src, e].sum())


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


_PHASES = ("router_logits", "router_topk", "counts_post", "dispatch", "plan", "experts", "return", "combine")


class ExpertParallelMoE:
    """One MoE layer over the ranks of `group` (None = the default group).

    layer = ExpertParallelMoE(H, I, E, K, max_tokens)        # collective: every rank
    layer.set_router(wr)                          # bf16 [E, H] on this GPU (replicated)
    layer.set_local_experts(w13, w2, hot=[...])   # THIS rank's experts [E/N, 2I, H], [E/N, H, I]
    out = layer.forward(xn, x2)                   # local tokens in, local tokens out (collective)
    layer.close()                                 # collective

    rank / world / handles: for ranks that are objects of one process (tests on one GPU) pass
    rank and world explicitly and call `connect([h.export() for h in ranks])` on each.
    """

    def __init__(self, hidden, intermediate, experts, top_k, max_tokens, group=None, capacity_factor=None,
                 exchange="peer", rank=None, world=None):
        from monoserve_b200 import _C
        from monoserve_b200.moe import MoELayer
        assert exchange in ("peer", "nccl")
        self._C = _C
        self.group = group
        self.exchange = exchange
        self._standalone = rank is not None
        if rank is None:
            world = dist.get_world_size(group) if dist.is_initialized() else 1
            rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world, self.rank = world, rank
        assert experts % self.world == 0
        self.H, self.I, self.E, self.K, self.T = hidden, intermediate, experts, top_k, max_tokens
        self.El = experts // self.world
        # worst case every pair of every rank lands here; capacity_factor trims the workspace
        rows_cap = max_tokens * top_k * self.world
        if capacity_factor is not None:
            rows_cap = min(rows_cap, int(max_tokens * top_k * capacity_factor))
        self.rows_cap = rows_cap
        self.wr = None
        self._ep = None
        dev = "cuda"
        if exchange == "peer":
            cfg = _C.MoEConfigC(hidden=hidden, intermediate=intermediate, experts=experts, top_k=top_k,
                                max_tokens=max_tokens, scoring=0, renorm=1, routed_scale=1.0, fp8=0)
            self._ep = ctypes.c_void_p()
            _C.check(_C.lib.monofab_ep_create(ctypes.byref(cfg), self.rank, self.world, rows_cap, ctypes.byref(self._ep)))
            self.local = MoELayer.borrowed(_C.lib.monofab_ep_local(self._ep), hidden, intermediate, self.El, 1, rows_cap)
            self.ids = self._workspace("topk_ids", torch.int32).view(max_tokens, top_k)
            self.w = self._workspace("topk_w", torch.float32).view(max_tokens, top_k)
            if not self._standalone:
                self.connect(self._gather_handles())
            return
        self.local = MoELayer(hidden, intermediate, self.El, 1, rows_cap)
        P = max_tokens * top_k
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

    # ---- peer exchange set-up ---------------------------------------------------
    def _workspace(self, name, dt):
        from monoserve_b200.moe import _from_device_address
        ptr, nbytes = ctypes.c_void_p(), ctypes.c_size_t()
        self._C.check(self._C.lib.monofab_ep_workspace(self._ep, name.encode(), ctypes.byref(ptr), ctypes.byref(nbytes)))
        return _from_device_address(ptr.value, nbytes.value // 4, dt)

    def export(self):
        """This rank's buffer handle: plain bytes to hand to every other rank."""
        buf = (ctypes.c_ubyte * self._C.EP_HANDLE_BYTES)()
        self._C.check(self._C.lib.monofab_ep_export(self._ep, buf))
        return bytes(buf)

    def _gather_handles(self):
        mine = torch.frombuffer(bytearray(self.export()), dtype=torch.uint8)
        if self.world == 1:
            return [bytes(mine.numpy())]
        backend = dist.get_backend(self.group)
        mine = mine.cuda() if backend == "nccl" else mine
        every = [torch.empty_like(mine) for _ in range(self.world)]
        dist.all_gather(every, mine, group=self.group)
        return [bytes(t.cpu().numpy()) for t in every]

    def connect(self, handles):
        assert len(handles) == self.world
        blob = b"".join(handles)
        self._C.check(self._C.lib.monofab_ep_connect(self._ep, blob))

    # ---- weights ----------------------------------------------------------------
    def set_router(self, wr):
        assert wr.is_cuda and wr.dtype == torch.bfloat16 and wr.shape == (self.E, self.H) and wr.is_contiguous()
        self.wr = wr
        if self._ep:
            self._C.check(self._C.lib.monofab_ep_set_router(self._ep, wr.data_ptr(), None))

    def set_local_experts(self, w13, w2, hot, pack_hot=True):
        assert w13.shape[0] == self.El and w2.shape[0] == self.El
        self.local.set_experts(w13, w2, hot, pack_hot=pack_hot)

    def set_plan(self, ctas=0, credits=8, form=64):
        self.local.set_plan(ctas, credits, form)

    # ---- compute ----------------------------------------------------------------
    def _check(self, xn, x2, out):
        T = xn.shape[0]
        assert T <= self.T and xn.is_cuda and xn.dtype == torch.bfloat16 and xn.is_contiguous()
        if out is None:
            out = torch.empty_like(xn)
        st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        return T, out, st

    def phase(self, p, xn, x2=None, out=None):
        """One phase of a pass (peer exchange only; see monofab_ep_phase)."""
        T, out, st = self._check(xn, x2, out)
        self._C.check(self._C.lib.monofab_ep_phase(self._ep, p, xn.data_ptr(), x2.data_ptr() if x2 is not None else None,
                                                   out.data_ptr(), T, st))
        return out

    def forward(self, xn, x2=None, out=None):
        C, lib = self._C, self._C.lib
        T, out, st = self._check(xn, x2, out)
        if self._ep:
            C.check(lib.monofab_ep_forward(self._ep, xn.data_ptr(), x2.data_ptr() if x2 is not None else None,
                                           out.data_ptr(), T, st))
            return out
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

    def set_profile(self, on):
        self._C.check(self._C.lib.monofab_ep_set_profile(self._ep, int(on)))

    def last_times(self):
        """Milliseconds of the last profiled pass by phase (peer exchange only); the
        waits for peers are inside dispatch (counts), plan (rows) and combine (outputs)."""
        ms = (ctypes.c_float * 8)()
        self._C.check(self._C.lib.monofab_ep_last_times(self._ep, ctypes.byref(ms)))
        return dict(zip(_PHASES, list(ms)))

    def disconnect(self):
        if self._ep:
            self._C.lib.monofab_ep_disconnect(self._ep)

    def close(self):
        """Collective when the ranks are processes: peers unmap each other's buffers,
        meet at a barrier, and only then free their own."""
        if self._ep:
            self.disconnect()
            if not self._standalone and self.world > 1 and dist.is_initialized():
                dist.barrier(group=self.group)
            self.local.close()
            self._C.lib.monofab_ep_destroy(self._ep)
            self._ep = None
        elif self.local is not None:
            self.local.close()
        self.local = None
