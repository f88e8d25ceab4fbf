"""Lane programs for the MoE layer: the layer's stage chain as a fabric program.

The reference builds, per layer, router_gemm -> router -> expand -> permute ->
per expert (w13 -> red -> w2) -> add_norm (monoserve/runtime/lane.py:340-380), with
the expert stages filled at run time by the expand tile and flagged as link stages
when the layer's (region, slot) table places the expert in pinned host memory.
`MoELane` builds the same chain on this library's tiles:

  router_logits (48) -> router (38, with stable ranks) -> expand (39) -> permute (40)
  -> per expert: w13[e] (GEMM tiles, SiLU-mul) -> w2[e] (GEMM tiles, fp32 rows; no reduce
  stage between them: nothing is K-split) -> combine (47: un-permute + weighted sum in pick
  order + residual)

All device memory is allocated here, before the fabric starts
(monoserve/runtime/lane.py:101-122 lists the same workspaces).
"""
import torch

from monoserve_b200 import _C
from monoserve_b200.fabric import Program, Tile, tile_array
from monoserve_b200.fabric.args import pack

K_GEMM, K_ROUTER, K_EXPAND, K_PERMUTE, K_COMBINE, K_LOGITS = 32, 38, 39, 40, 47, 48
REGION_HOST, REGION_HOT = 0, 1
CHUNK = 16    # rows of one rank chunk of the stable pack (kFabChunk)
SUB = 4       # rows per router / permute tile: one per exec warp; divides CHUNK, so a tile stays inside a chunk
LOGIT_ROWS, LOGIT_EXPERTS = 16, 16   # a router-projection tile: rows x experts (256 tokens x 128 experts: one wave of 128 tiles)
EPI_SILU_MUL, EPI_ROWS_F32 = 1, 5


def _block(name, **fields):
    return torch.frombuffer(bytearray(pack(name, **fields)), dtype=torch.uint8).cuda()


def _u64(values):
    return torch.tensor([int(v) for v in values], dtype=torch.int64).cuda()


def logits_tiles(args_ptr, T, E, rows=LOGIT_ROWS):
    """Router-projection tiles (kind 48): blocks of `rows` rows x LOGIT_EXPERTS experts."""
    import numpy as np
    r0, e0 = np.meshgrid(np.arange(0, T, rows), np.arange(0, E, LOGIT_EXPERTS), indexing="ij")
    return tile_array(K_LOGITS, i0=r0, i1=np.minimum(rows, T - r0), i2=e0, i3=np.minimum(LOGIT_EXPERTS, E - e0),
                      a0=args_ptr)


def _row_tiles(kind, args, rows, per):
    return [Tile(kind, i=(r0, min(per, rows - r0)), a=(args.data_ptr(),)) for r0 in range(0, rows, per)]


class MoELane:
    """lane = MoELane(fab, lane_id, H, I, E, K, max_tokens, wr, w13, w2, hot)
    lane.set_input(xn, x2); h = lane.build(T, iterations=1); fab.publish(..., programs=[h]) ..."""

    def __init__(self, fab, lane_id, hidden, intermediate, experts, top_k, max_tokens, wr, w13, w2, hot,
                 pack_hot=True, scales=None, scoring=0, bias=None, routed_scale=1.0, shared=None, staged=False,
                 staged_min_rows=256, fetch_chunk=256 * 1024):
        """w13 / w2: bf16, or e4m3 bytes (uint8) with scales = (fp32 [E][2I], fp32 [E][H]) per output
        channel.  scoring 1 = sigmoid with the optional fp32 [E] selection bias; routed_scale multiplies
        the renormalised weights.  shared = (w13 bf16 [2 Is][H], w2 bf16 [H][Is]): a shared expert every
        token passes through, added to the routed sum (tests/test_fabric_model_glm.py:29-31,57-67).
        staged: under form 0 a host-resident expert with more than staged_min_rows rows is first copied
        into an HBM staging stack by fetch tiles (chunks of fetch_chunk bytes) and its GEMM tiles read the
        copy, so its weights cross the host link once whatever its row count."""
        self.fab, self.lane_id = fab, lane_id
        self.H, self.I, self.E, self.K, self.T = hidden, intermediate, experts, top_k, max_tokens
        H, I, E, K, T = hidden, intermediate, experts, top_k, max_tokens
        P = T * K
        dev = "cuda"
        self.wr = wr.to(torch.bfloat16).contiguous().cuda()
        # placement (monoserve/runtime/weights.py:100-143): the full set pinned, the hot experts copied to HBM
        self.host_w13 = w13 if w13.is_pinned() else w13.contiguous().pin_memory()
        self.host_w2 = w2 if w2.is_pinned() else w2.contiguous().pin_memory()
        self.hot = list(hot)
        idx = torch.tensor(self.hot if self.hot else [0])
        self.fp8 = self.host_w13.dtype == torch.uint8
        assert self.fp8 == (scales is not None), "e4m3 weights come with per-output-channel scales"
        hot13 = self.host_w13[idx].cuda()
        if pack_hot:
            packed = torch.empty_like(hot13)
            _C.check(_C.lib.monofab_pack_w13(hot13.data_ptr(), packed.data_ptr(), hot13.shape[0], I, H,
                                             hot13.element_size(), None))
            torch.cuda.synchronize()
            hot13 = packed
        self.hot_w13, self.hot_w2 = hot13, self.host_w2[idx].cuda()
        table = torch.zeros(E, 2, dtype=torch.int32)
        table[:, 1] = torch.arange(E)
        if self.hot:
            table[idx, 0] = REGION_HOT
            table[idx, 1] = torch.arange(len(self.hot), dtype=torch.int32)
        self.table = table.cuda()

        def wmap(t, base, packed=False):
            z, rows, k = t.shape
            if t.dtype == torch.uint8:   # e4m3 bytes: byte strides, no swizzle (monoserve/runtime/weights.py:38-40)
                return fab.tensor_map(base, [k, rows, z], [k, rows * k], [128, 64, 1], dtype=2, swizzle=0, packed=packed)
            return fab.tensor_map(base, [k, rows, z], [k * 2, rows * k * 2], [64, 64, 1], packed=packed)

        m13 = [wmap(self.host_w13, _C.host_device_pointer(self.host_w13.data_ptr())),
               wmap(self.hot_w13, self.hot_w13.data_ptr(), packed=pack_hot), 0, 0]
        m2 = [wmap(self.host_w2, _C.host_device_pointer(self.host_w2.data_ptr())),
              wmap(self.hot_w2, self.hot_w2.data_ptr()), 0, 0]
        self.staging = None
        if staged:   # region 3: the lane's staging stack, one slot per expert, the reference's row order
            self.stage_w13 = torch.empty(self.host_w13.shape, dtype=self.host_w13.dtype, device=dev)
            self.stage_w2 = torch.empty(self.host_w2.shape, dtype=self.host_w2.dtype, device=dev)
            m13[3], m2[3] = wmap(self.stage_w13, self.stage_w13.data_ptr()), wmap(self.stage_w2, self.stage_w2.data_ptr())
            b13 = self.host_w13[0].numel() * self.host_w13.element_size()
            b2 = self.host_w2[0].numel() * self.host_w2.element_size()
            self.fetch_tiles = -(-b13 // fetch_chunk) + -(-b2 // fetch_chunk)
            self.staging = _block("StagingArgs", w13_src=_C.host_device_pointer(self.host_w13.data_ptr()),
                                  w13_dst=self.stage_w13.data_ptr(), w13_bytes=b13,
                                  w2_src=_C.host_device_pointer(self.host_w2.data_ptr()),
                                  w2_dst=self.stage_w2.data_ptr(), w2_bytes=b2, chunk_bytes=fetch_chunk,
                                  min_rows=staged_min_rows)
        self.w13_maps, self.w2_maps = _u64(m13), _u64(m2)
        # workspaces
        z = lambda *shape, dt=torch.int32: torch.zeros(*shape, dtype=dt, device=dev)  # noqa: E731
        self.xn, self.x2, self.x = (z(T, H, dt=torch.bfloat16) for _ in range(3))
        self.logits = z(T, E, dt=torch.float32)
        self.topk_ids, self.topk_w = z(T, K), z(T, K, dt=torch.float32)
        self.counts, self.fill, self.starts = z(E), z(E), z(E + 1)
        self.chunks = -(-T // CHUNK)
        self.chunk_counts, self.chunk_prefix = z(self.chunks, E), z(self.chunks, E)
        self.pair_token, self.pair_weight, self.pair_pos = z(P), z(P, dt=torch.float32), z(T, K)
        self.xp, self.h = z(P + 256, H, dt=torch.bfloat16), z(P + 256, I, dt=torch.bfloat16)
        self.y = z(P + 256, H, dt=torch.float32)
        self.hist = z(E)
        self.expand_stamps = torch.zeros(8, dtype=torch.int64, device=dev)   # phase time stamps of the expand tile
        # operand blocks
        self.logits_args = None
        self.bias = bias.float().cuda() if bias is not None else None
        self.router_args = _block("RouterArgs", logits=self.logits, topk_ids=self.topk_ids, topk_w=self.topk_w,
                                  counts=self.counts, bias=self.bias if self.bias is not None else 0, E=E, K=K,
                                  scoring=scoring, renorm=1, scale=routed_scale, chunk_counts=self.chunk_counts)
        self.scales = (scales[0].float().contiguous().cuda(), scales[1].float().contiguous().cuda()) if scales else None
        # shared expert: two dense GEMMs over all tokens, fp32 rows that the combine tile adds
        self.shared = None
        if shared is not None:
            sw13, sw2 = shared[0].to(torch.bfloat16).contiguous().cuda(), shared[1].to(torch.bfloat16).contiguous().cuda()
            Is = sw2.shape[1]
            self.shared = dict(w13=sw13, w2=sw2, Is=Is, h=z(T + 256, Is, dt=torch.bfloat16),
                               y=z(T, H, dt=torch.float32),
                               m13=fab.tensor_map(sw13.data_ptr(), [H, 2 * Is, 1], [H * 2, 2 * Is * H * 2], [64, 64, 1]),
                               m2=fab.tensor_map(sw2.data_ptr(), [Is, H, 1], [Is * 2, H * Is * 2], [64, 64, 1]))
        self.permute_args = _block("PermuteArgs", topk_ids=self.topk_ids, topk_w=self.topk_w, starts=self.starts,
                                   fill=self.fill, pair_token=self.pair_token, pair_weight=self.pair_weight,
                                   src=self.xn, dst=self.xp, K=K, H=H, chunk_prefix=self.chunk_prefix,
                                   pair_pos=self.pair_pos, E=E)
        self.combine_args = _block("CombineArgs", y=self.y, pair_pos=self.pair_pos, topk_w=self.topk_w, x2=self.x2,
                                   x=self.x, K=K, H=H, eps=0.0, shared=self.shared["y"] if self.shared else 0)
        heights = [16, 32, 64, 128, 256]
        self.xp_maps = _u64([fab.tensor_map(self.xp.data_ptr(), [H, P + 256], [H * 2], [64, bm]) for bm in heights])
        self.h_maps = _u64([fab.tensor_map(self.h.data_ptr(), [I, P + 256], [I * 2], [64, bm]) for bm in heights])
        self._gemm_blocks = []
        a13, a2 = [], []
        for bm in heights:
            b13 = torch.frombuffer(bytearray(_C.gemm_args(out=self.h.data_ptr(), ld_out=I, k_tiles=H // 64,
                                                          epi=EPI_SILU_MUL, bm=bm, n_limit=I, up_offset=I,
                                                          w_fp8=int(self.fp8))), dtype=torch.uint8).cuda()
            b2 = torch.frombuffer(bytearray(_C.gemm_args(out=self.y.data_ptr(), ld_out=H, k_tiles=I // 64,
                                                         epi=EPI_ROWS_F32, bm=bm, n_limit=H, w_fp8=int(self.fp8))),
                                  dtype=torch.uint8).cuda()
            self._gemm_blocks += [b13, b2]
            a13.append(b13.data_ptr())
            a2.append(b2.data_ptr())
        self.w13_args, self.w2_args = _u64(a13), _u64(a2)
        self._keep = []

    def set_input(self, xn, x2=None):
        """Copy the batch into the lane's input buffers (before the program runs)."""
        T = xn.shape[0]
        self.xn[:T].copy_(xn)
        if x2 is not None:
            self.x2[:T].copy_(x2)
        else:
            self.x2[:T].zero_()

    def dynamic_tiles(self, T):
        """Most GEMM tiles the expander can write for T tokens (form 16, ragged tails)."""
        n = (T * self.K // 16 + self.E) * (self.I // 64 + self.H // 128)
        return n + (self.E * self.fetch_tiles if self.staging is not None else 0)

    def build(self, T, iterations=1, mark_layer=0):
        """Upload the one-layer program for a batch of T tokens; returns its handle."""
        assert 0 < T <= self.T
        H, E = self.H, self.E
        nw = self.fab.num_workers
        p = Program()
        logits_args = _block("LogitsArgs", x=self.xn, wr=self.wr, logits=self.logits, T=T, H=H, E=E)
        s_lg = p.stage(logits_tiles(logits_args.data_ptr(), T, E), label=("router_logits", mark_layer))
        s_rt = p.stage(_row_tiles(K_ROUTER, self.router_args, T, SUB), label=("router", mark_layer))
        p.after(s_lg, s_rt)
        ex = torch.zeros(_C.struct_layouts()["ExpandArgs"][0], dtype=torch.uint8, device="cuda")
        s_ex = p.stage(tile_array(K_EXPAND, a0=ex.data_ptr()), label=("expand", mark_layer))
        p.after(s_rt, s_ex)
        s_pm = p.stage(_row_tiles(K_PERMUTE, self.permute_args, T, SUB), label=("permute", mark_layer))
        p.after(s_ex, s_pm)
        w13 = [p.stage(label=("w13", mark_layer)) for _ in range(E)]
        w2 = [p.stage(label=("w2", mark_layer)) for _ in range(E)]
        per_cb = max(2, -(-T // (2 * nw)))
        s_cb = p.stage(_row_tiles(K_COMBINE, self.combine_args, T, per_cb), mark=(mark_layer << 8) | 3,
                       label=("combine", mark_layer))
        if self.shared:   # runs beside the routed chain, joins at the combine stage
            sh = self.shared
            bm = next(h for h in (16, 32, 64, 128, 256) if T <= h or h == 256)
            xm = self.fab.tensor_map(self.xn.data_ptr(), [H, self.T], [H * 2], [64, bm])
            hm = self.fab.tensor_map(sh["h"].data_ptr(), [sh["Is"], self.T + 256], [sh["Is"] * 2], [64, bm])
            g13 = torch.frombuffer(bytearray(_C.gemm_args(out=sh["h"].data_ptr(), ld_out=sh["Is"], k_tiles=H // 64,
                                                          epi=EPI_SILU_MUL, bm=bm, n_limit=sh["Is"], up_offset=sh["Is"])),
                                   dtype=torch.uint8).cuda()
            g2 = torch.frombuffer(bytearray(_C.gemm_args(out=sh["y"].data_ptr(), ld_out=H, k_tiles=sh["Is"] // 64, epi=3,
                                                         bm=bm, n_limit=H)), dtype=torch.uint8).cuda()
            self._keep += [g13, g2]
            t13 = [Tile(K_GEMM, i=(f0, m0, min(bm, T - m0), 0), a=(g13.data_ptr(), sh["m13"], xm))
                   for m0 in range(0, T, bm) for f0 in range(0, sh["Is"], 64)]
            t2 = [Tile(K_GEMM, i=(n0, m0, min(bm, T - m0), 0), a=(g2.data_ptr(), sh["m2"], hm))
                  for m0 in range(0, T, bm) for n0 in range(0, H, 128)]
            s_s13 = p.stage(t13, label=("shared_w13", mark_layer))
            s_s2 = p.stage(t2, label=("shared_w2", mark_layer))
            p.after(s_lg, s_s13)
            p.after(s_s13, s_s2)
            p.after(s_s2, s_cb)
        fetch = [p.stage(label=("fetch", mark_layer)) for _ in range(E)] if self.staging is not None else None
        for e in range(E):
            p.after(s_pm, w13[e])
            if fetch:   # the copy into the staging stack starts as soon as the expert's row count is known
                p.after(s_ex, fetch[e])
                p.after(fetch[e], w13[e])
            p.after(w13[e], w2[e])
            p.after(w2[e], s_cb)
        dyn = self.dynamic_tiles(T)
        p.reserve(dyn)
        blob = pack("ExpandArgs", counts=self.counts, starts=self.starts, fill=self.fill, table=self.table,
                    w13_maps=self.w13_maps, w2_maps=self.w2_maps, xp_maps=self.xp_maps, h_maps=self.h_maps,
                    w13_args=self.w13_args, w2_args=self.w2_args, hist=self.hist, E=E, H=H, I=self.I,
                    host_region=REGION_HOST, w13_stage0=w13[0], w2_stage0=w2[0], red_stage0=0xffffffff,
                    dyn_first=p.dynamic_first, dyn_cap=dyn, lane=self.lane_id, join_stage=s_cb,
                    staging=self.staging if self.staging is not None else 0, fetch_stage0=fetch[0] if fetch else 0,
                    chunks=-(-T // CHUNK), chunk_counts=self.chunk_counts, chunk_prefix=self.chunk_prefix,
                    red_args=self.expand_stamps, w13_scale=self.scales[0] if self.scales else 0,
                    w2_scale=self.scales[1] if self.scales else 0)
        ex.copy_(torch.frombuffer(bytearray(blob), dtype=torch.uint8))
        torch.cuda.synchronize()
        self._keep += [logits_args, ex]
        self.labels = p.labels()   # stage names, for monoserve_b200.fabric.trace.summary
        return p.upload(self.fab, first=s_lg, iterations=iterations)
