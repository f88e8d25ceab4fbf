"""A Qwen3-MoE-style decoder as fabric lane programs.

The reference builds one program per lane whose per-layer chain is
qkv GEMM -> rope -> attention -> o GEMM -> norm -> router -> expand -> permute ->
per expert (w13 -> red -> w2) -> add_norm, then lm_head and sample
(monoserve/runtime/lane.py:309-420), over the workspaces of lane.py:101-122 and the
weight placement of monoserve/runtime/weights.py:100-158.  `ModelLane` builds the same
chain on this library's tiles:

  embed (42) -> per layer [ qkv GEMM (32) -> qk_rope (37) -> attention items (33/34, planned
  on the host for prefill and by the plan tile 44 for decode) -> merge (35) -> o GEMM (32,
  + residual) -> RMSNorm (36) -> router_logits (48) -> router (38) -> expand (39) ->
  permute (40) -> experts (32, SiLU-mul / fp32 rows) -> combine (47, + next norm) ]
  -> final norm with gather (36) -> lm_head GEMM (32, fp32) -> sample (43)

All device memory is allocated when the lane is built, before the fabric starts.
"""
import numpy as np
import torch

from monoserve_b200 import _C
from monoserve_b200.attention import SCALE_LOG2, fabric_maps, fabric_tiles, plan_items
from monoserve_b200.fabric import Program, Tile, tile_array
from monoserve_b200.fabric.args import pack
from monoserve_b200.lane import SUB, logits_tiles

K_GEMM, K_ATTN_PREFILL, K_ATTN_DECODE, K_ATTN_MERGE, K_RMSNORM, K_QKROPE = 32, 33, 34, 35, 36, 37
K_ADDNORM, K_NORM_LOGITS = 41, 50
FUSE_ROWS, FUSE_PERMUTE_ROWS = 32, 16   # batches this small fold the norm into the projection's tiles, and the permute into expand
SPLIT_ROWS, SPLIT_PARTS, QKV_PARTS = 64, 8, 2   # a dense GEMM of at most SPLIT_ROWS rows may run as up to SPLIT_PARTS K ranges
O_SPLIT_ROWS, O_WIDE_PARTS = 512, 4   # the o projection (a residual epilogue of 2-byte loads and stores) keeps the form up to here
K_ROUTER, K_EXPAND, K_PERMUTE, K_EMBED, K_SAMPLE, K_ATTN_PLAN, K_COMBINE, K_LOGITS = 38, 39, 40, 42, 43, 44, 47, 48
EPI_STORE, EPI_SILU_MUL, EPI_F32, EPI_ROWS_F32 = 0, 1, 3, 5
REGION_HOST, REGION_HOT = 0, 1
CHUNK = 16            # rows per router / permute tile = rank chunk of the stable pack
ROPE_ITEMS = 48       # (row, head) items per qk_rope tile (monoserve/runtime/lane.py:27)
HEIGHTS = [16, 32, 64, 128, 256]


def _block(name, **fields):
    return torch.frombuffer(bytearray(pack(name, **fields)), dtype=torch.uint8).cuda()


def _u64(values):
    return torch.tensor([int(v) for v in values], dtype=torch.int64).cuda()


class _Blob:
    """A piece of device memory by address (what `pack` and the tile builders need of a tensor)."""

    def __init__(self, addr, nbytes):
        self.addr, self.nbytes = addr, nbytes

    def data_ptr(self):
        return self.addr


class _Arena:
    """Device memory for the operand blocks of one program build, carved from one buffer that is
    allocated with the lane and filled through Fabric.write: a build then neither allocates device
    memory nor launches a kernel, both of which would wait for a resident fabric kernel."""

    def __init__(self, fab, nbytes):
        self.fab, self.buf, self.at = fab, torch.zeros(nbytes, dtype=torch.uint8, device="cuda"), 0
        self.host, self.flushed = bytearray(nbytes), 0   # the blocks of the current build; [flushed, at) not yet written

    def reset(self):
        self.at = self.flushed = 0

    def put(self, data):
        """Room for `data` in the arena; the bytes reach the device with the next flush()."""
        size = (len(data) + 255) & ~255
        if self.at + size > self.buf.numel():
            raise RuntimeError("monofab: the lane's operand arena is full")
        blob = _Blob(self.buf.data_ptr() + self.at, len(data))
        self.host[self.at:self.at + len(data)] = data
        self.at += size
        return blob

    def patch(self, blob, data):
        """Replace the contents of a block put earlier in this build."""
        at = blob.addr - self.buf.data_ptr()
        assert self.flushed <= at and at + len(data) <= self.at, "the block is not of the current build"
        self.host[at:at + len(data)] = data

    def flush(self):
        """One write of everything put since the last flush (a build has hundreds of blocks of 64 to 256 bytes)."""
        if self.at > self.flushed:
            self.fab.write(self.buf.data_ptr() + self.flushed, bytes(self.host[self.flushed:self.at]))
            self.flushed = self.at


def _bm(rows):
    """Row-block height of a dense GEMM over `rows` activation rows."""
    for h in HEIGHTS:
        if rows <= h:
            return h
    return HEIGHTS[-1]


def _retarget(template, a0=None, a1=None, a2=None, a4=None):
    """A copy of a tile array with other operand addresses.  The tiles of a stage depend on the layer only
    through the addresses they name, so a lane keeps one array per shape and re-addresses a copy per layer."""
    t = template.copy()
    for col, v in ((3, a0), (4, a1), (5, a2), (7, a4)):
        if v is not None:
            t[:, col] = v
    return t


def rope_table(theta, rot_dim, max_pos):
    """cos/sin fp32 [max_pos][rot_dim / 2][2], computed as the reference's oracle does
    (tests/test_fabric_model.py:35-42; the lane's host table: monoserve/runtime/lane.py:36-48)."""
    half = rot_dim // 2
    j = torch.arange(half, dtype=torch.float32)
    inv = 1.0 / torch.pow(torch.tensor(theta, dtype=torch.float32), 2 * j / rot_dim)
    ang = torch.arange(max_pos, dtype=torch.float32)[:, None] * inv[None]
    return torch.stack([ang.cos(), ang.sin()], -1).contiguous()


class Mat:
    """A weight matrix on the device: bf16, or e4m3 bytes with an fp32 scale per output row."""

    def __init__(self, data, scale=None):
        self.data, self.scale = data, scale
        self.fp8 = data.dtype == torch.uint8


class ModelWeights:
    """Weights of the decoder on the device, expert stacks placed as the reference places them
    (monoserve/runtime/weights.py:100-158): the full expert set of every layer in pinned host
    memory (region 0, slot = expert id), the layer's hot experts copied to HBM (region 1,
    w13 in the packed SwiGLU row order), and a per-layer (region, slot) table.

    w: an object with CPU (or CUDA) tensors embed [V,H], lm_head [V,H], final_norm [H] and per-layer lists
    in_norm, qkv, o, post_norm, and for MoE layers router, host_w13 [E,2I,H], host_w2 [E,H,I].  A matrix is
    a bf16 tensor, or a pair (e4m3 bytes as uint8, fp32 scale per output row); expert stacks in e4m3 come
    with lists w13_scale [E,2I] / w2_scale [E,H].  Optional members, by model family: q_norm / k_norm
    (per-head norms), qkv_bias, router_bias (fp32 [E], selection only), shared_w13 / shared_w2 (a shared
    expert), mlp_w13 / mlp_w2 (the dense FFN of the first cfg.dense_layers layers).
    hot: per layer, the expert ids kept in HBM (default: all)."""

    def __init__(self, cfg, w, hot=None):
        self.cfg = cfg
        L, E, I, H = cfg.num_layers, cfg.num_experts, cfg.intermediate, cfg.hidden
        self.dense_layers = getattr(cfg, "dense_layers", 0)
        # A tensor object that appears for several layers (a benchmark that cycles a few distinct
        # layers' weights) is placed once.
        dev_cache, pin_cache, hot_cache = {}, {}, {}

        def d(t):
            if id(t) not in dev_cache:
                dev_cache[id(t)] = t.contiguous().cuda() if t.dtype in (torch.uint8, torch.float32) else \
                    t.to(torch.bfloat16).contiguous().cuda()
            return dev_cache[id(t)]

        def mat(v):
            return Mat(d(v[0]), d(v[1].float())) if isinstance(v, (tuple, list)) else Mat(d(v))

        def pin(t):
            if id(t) not in pin_cache:
                pin_cache[id(t)] = t if t.is_pinned() else t.contiguous().pin_memory()
            return pin_cache[id(t)]

        def per_layer(name, f, layers=range(L)):
            src = getattr(w, name, None)
            return [f(src[l]) if src is not None and l in layers and src[l] is not None else None for l in range(L)]

        moe_layers = range(self.dense_layers, L)
        self.embed, self.lm_head, self.final_norm = d(w.embed), d(w.lm_head), d(w.final_norm)
        for name in ("in_norm", "post_norm", "q_norm", "k_norm", "qkv_bias"):
            setattr(self, name, per_layer(name, d))
        for name in ("qkv", "o"):
            setattr(self, name, per_layer(name, mat))
        for name in ("mlp_w13", "mlp_w2"):
            setattr(self, name, per_layer(name, mat, range(self.dense_layers)))
        for name in ("shared_w13", "shared_w2"):
            setattr(self, name, per_layer(name, mat, moe_layers))
        self.router = per_layer("router", d, moe_layers)
        self.router_bias = per_layer("router_bias", lambda t: d(t.float()), moe_layers)
        self.w13_scale = per_layer("w13_scale", lambda t: d(t.float()), moe_layers)
        self.w2_scale = per_layer("w2_scale", lambda t: d(t.float()), moe_layers)
        self.host_w13 = per_layer("host_w13", pin, moe_layers)
        self.host_w2 = per_layer("host_w2", pin, moe_layers)
        self.fp8_experts = any(t is not None and t.dtype == torch.uint8 for t in self.host_w13)
        self.hot = [list(h) for h in hot] if hot is not None else [list(range(E)) for _ in range(L)]
        self.hot_w13, self.hot_w2, self.table = [None] * L, [None] * L, [None] * L
        for l in moe_layers:
            idx = torch.tensor(self.hot[l] if self.hot[l] else [0])
            key = (id(w.host_w13[l]), id(w.host_w2[l]), tuple(self.hot[l]))
            if key not in hot_cache:
                h13 = self.host_w13[l][idx].cuda()
                packed = torch.empty_like(h13)
                _C.check(_C.lib.monofab_pack_w13(h13.data_ptr(), packed.data_ptr(), h13.shape[0], I, H,
                                                 h13.element_size(), None))
                torch.cuda.synchronize()
                hot_cache[key] = (packed, self.host_w2[l][idx].cuda())
            self.hot_w13[l], self.hot_w2[l] = hot_cache[key]
            table = torch.zeros(E, 2, dtype=torch.int32)
            table[:, 1] = torch.arange(E)
            if self.hot[l]:
                table[idx, 0] = REGION_HOT
                table[idx, 1] = torch.arange(len(self.hot[l]), dtype=torch.int32)
            self.table[l] = table.cuda()
        self.stage_w13, self.stage_w2, self.staging_slots = [], [], 0

    def expert_bytes(self):
        """(bytes of one expert's w13 block, of its w2 block) (monoserve/runtime/weights.py)."""
        l = next(i for i, t in enumerate(self.host_w13) if t is not None)
        return (self.host_w13[l][0].numel() * self.host_w13[l].element_size(),
                self.host_w2[l][0].numel() * self.host_w2[l].element_size())

    def alloc_staging(self, slots, buffers=1):
        """Staging buffers in HBM for the host loop (regions 2, 3 ...): each holds `slots` experts in
        the reference's row order, in two halves of slots // 2 (one layer's worth each)
        (monoserve/runtime/weights.py: stage_w13 / stage_w2 / staging_slots)."""
        l = next(i for i, t in enumerate(self.host_w13) if t is not None)
        h13, h2 = self.host_w13[l], self.host_w2[l]
        self.staging_slots = slots
        for _ in range(buffers):
            self.stage_w13.append(torch.zeros((slots,) + tuple(h13.shape[1:]), dtype=h13.dtype, device="cuda"))
            self.stage_w2.append(torch.zeros((slots,) + tuple(h2.shape[1:]), dtype=h2.dtype, device="cuda"))


class KVCache:
    """Paged K and V per layer, bf16 [pages][page_size][hkv][128] (monoserve/runtime/kv.py:8-11 with
    the page size a parameter).  Page 0 is a write sink (monoserve/engine.py:113)."""

    def __init__(self, cfg, n_pages, page_size=16):
        self.n_pages, self.page = n_pages, page_size
        shape = (n_pages, page_size, cfg.num_kv_heads, 128)
        self.k = [torch.zeros(shape, dtype=torch.bfloat16, device="cuda") for _ in range(cfg.num_layers)]
        self.v = [torch.zeros(shape, dtype=torch.bfloat16, device="cuda") for _ in range(cfg.num_layers)]


class ModelLane:
    """One lane of the fabric running the decoder: buffers, operand blocks and tensor maps are
    made once; `build_prefill` / `build_decode` upload programs over them.

    Request state lives in slot-indexed arrays (block table row, sequence length, last token),
    as in the reference's lane (StepArgs, csrc/fabric/model_types.h:116-128)."""

    def __init__(self, fab, lane_id, cfg, weights, kv, max_tokens, max_slots, bt_stride, max_chunks=8, max_pos=None,
                 logit_rows=None, min_form=16, staged=False, staged_min_rows=256, fetch_chunk=256 * 1024,
                 staging_index=None, requests=None):
        """staging_index: the weights' staging buffer (ModelWeights.alloc_staging) a host loop fills for
        this lane; its experts are region 2 of the lane's own (region, slot) tables.
        staged: under form 0 a host-resident expert with more than staged_min_rows rows is copied once
        into this lane's HBM staging stack (one slot per expert, shared by all layers) by fetch tiles of
        fetch_chunk bytes, and its GEMM tiles read the copy.
        requests: a RequestTable (monoserve_b200/engine.py) whose slot-indexed request state (block table,
        lengths, last tokens, token rings) this lane uses instead of arrays of its own, so that several
        lanes (a prefill lane, two decode buffers) see the same requests (monoserve/runtime/requests.py)."""
        self.fab, self.lane_id, self.cfg, self.w, self.kv = fab, lane_id, cfg, weights, kv
        self.staged, self.staged_min_rows, self.fetch_chunk = staged, staged_min_rows, fetch_chunk
        self.staging_index = staging_index
        # the lane's own (region, slot) tables int32 [layers][experts][2]: a host loop moves entries of
        # one lane between the host region and that lane's staging buffer without touching other lanes
        E_, L_ = cfg.num_experts, cfg.num_layers
        self.tables = torch.zeros(L_, E_, 2, dtype=torch.int32, device="cuda")
        for l_ in range(L_):
            if weights.table[l_] is not None:
                self.tables[l_].copy_(weights.table[l_])
        self.T, self.S, self.bt_stride, self.max_chunks = max_tokens, max_slots, bt_stride, max_chunks
        # rows of the lm_head (requests that continue; every row when a caller wants all logits), and the
        # smallest row-block height the published plans will use for host-resident experts
        self.logit_rows = logit_rows or max(max_tokens, max_slots)
        self.min_form = min_form
        H, I, E, K, L, V = cfg.hidden, cfg.intermediate, cfg.num_experts, cfg.top_k, cfg.num_layers, cfg.vocab
        hq, hkv = cfg.num_heads, cfg.num_kv_heads
        self.qkv_dim = (hq + 2 * hkv) * 128
        T, S, P = max_tokens, max_slots, max_tokens * K
        dev = "cuda"
        z = lambda *shape, dt=torch.int32: torch.zeros(*shape, dtype=dt, device=dev)  # noqa: E731
        bf = torch.bfloat16
        # residual stream and projections (monoserve/runtime/lane.py:101-122)
        self.x, self.x2, self.xn = z(T, H, dt=bf), z(T, H, dt=bf), z(T, H, dt=bf)
        self.qkv = z(T, self.qkv_dim, dt=bf)
        self.q, self.ao = z(T, hq, 128, dt=bf), z(T, hq, 128, dt=bf)
        self.xlast, self.logits = z(self.logit_rows, H, dt=bf), z(self.logit_rows, V, dt=torch.float32)
        # routing and expert workspaces
        self.rl = z(T, E, dt=torch.float32)
        self.topk_ids, self.topk_w = z(T, K), z(T, K, dt=torch.float32)
        self.counts, self.fill, self.starts, self.hist = z(E), z(E), z(E + 1), z(L, E)
        self.chunk_counts, self.chunk_prefix = z(-(-T // CHUNK), E), z(-(-T // CHUNK), E)
        self.pair_token, self.pair_weight, self.pair_pos = z(P), z(P, dt=torch.float32), z(T, K)
        self.xp, self.h = z(P + 256, H, dt=bf), z(P + 256, I, dt=bf)
        self.y = z(P + 256, H, dt=torch.float32)
        self.o_rows = min(O_SPLIT_ROWS, (T + 63) // 64 * 64)
        self.o_slabs = z(SPLIT_PARTS * self.o_rows, H, dt=torch.float32)   # K-split partial sums of the o projection
        self.qkv_slabs = z(QKV_PARTS * SPLIT_ROWS, self.qkv_dim, dt=torch.float32)   # and of the qkv projection
        # dense FFN of the first layers / shared expert: hidden rows and fp32 output rows
        self.Id, self.Is = getattr(cfg, "dense_intermediate", 0), getattr(cfg, "shared_intermediate", 0)
        wide = max(self.Id, self.Is)
        self.hd = z(T + 256, wide, dt=bf) if wide else None
        self.y_shared = z(T, H, dt=torch.float32) if self.Is else None
        # token and request state
        self.tokens, self.tok_pos, self.tok_slot, self.gather = z(T), z(T), z(T), z(T)
        self.req_info = z(max(T, S), 4)
        self.row_req = z(max(T, S))
        if requests is not None:
            assert requests.slots >= S and requests.bt_stride == bt_stride
            self.bt, self.seq_len, self.last_token, self.steps = requests.bt, requests.seq_len, requests.last_token, requests.steps
            self.temperature, self.ring = requests.temperature, requests.ring
            self.host_tokens, self.host_steps = requests.host_tokens, requests.host_steps
        else:
            self.bt = z(S, bt_stride)
            self.seq_len, self.last_token, self.steps = z(S), z(S), z(S)
            self.temperature = z(S, dt=torch.float32)
            self.ring = 64
            self.host_tokens = torch.zeros(S, self.ring, dtype=torch.int32).pin_memory()
            self.host_steps = torch.zeros(S, dtype=torch.int64).pin_memory()
        # attention split workspace: (max, sum) pairs after the fp32 rows
        self.ws_rows = max(max_chunks * S * hq, 4 * T * hq // 8 + 1024)
        self.ws = z(self.ws_rows * 130, dt=torch.float32)
        max_pos = max_pos or bt_stride * kv.page
        self.max_pos = max_pos
        self.cos_sin = rope_table(cfg.rope_theta, cfg.rotary_dim, max_pos).cuda()
        self._keep = []
        self.arena = _Arena(fab, (64 << 10) * (L + 2))
        self._templates = {}   # tile arrays by shape, re-addressed per layer (_retarget)
        self._maps()

    # ------------------------------------------------------------------ maps and operand blocks
    def _wmap(self, t, base=None, packed=False):
        if isinstance(t, Mat):
            t = t.data
        if t.dim() == 2:
            rows, k, zdim = t.shape[0], t.shape[1], 1
        else:
            zdim, rows, k = t.shape
        base = base if base is not None else t.data_ptr()
        if t.dtype == torch.uint8:   # e4m3 bytes: byte strides, no swizzle (monoserve/runtime/weights.py:38-40)
            return self.fab.tensor_map(base, [k, rows, zdim], [k, rows * k], [128, 64, 1], dtype=2, swizzle=0, packed=packed)
        return self.fab.tensor_map(base, [k, rows, zdim], [k * 2, rows * k * 2], [64, 64, 1], packed=packed)

    def _amaps(self, t, rows, k):
        """Activation maps of a [rows][k] bf16 buffer for every row-block height."""
        return [self.fab.tensor_map(t.data_ptr(), [k, rows], [k * 2], [64, bm]) for bm in HEIGHTS]

    def _maps(self):
        cfg, w, fab = self.cfg, self.w, self.fab
        H, I, E, K, L = cfg.hidden, cfg.intermediate, cfg.num_experts, cfg.top_k, cfg.num_layers
        hq, hkv = cfg.num_heads, cfg.num_kv_heads
        T, P = self.T, self.T * K
        self.m_xn = self._amaps(self.xn, T, H)
        self.m_ao = self._amaps(self.ao, T, hq * 128)
        self.m_xlast = self._amaps(self.xlast, self.xlast.shape[0], H)
        self.m_qkv = [self._wmap(w.qkv[l]) for l in range(L)]
        self.m_o = [self._wmap(w.o[l]) for l in range(L)]
        self.m_lm = self._wmap(w.lm_head)
        opt = lambda lst, l: self._wmap(lst[l]) if lst[l] is not None else 0  # noqa: E731
        self.m_mlp13, self.m_mlp2 = [opt(w.mlp_w13, l) for l in range(L)], [opt(w.mlp_w2, l) for l in range(L)]
        self.m_sh13, self.m_sh2 = [opt(w.shared_w13, l) for l in range(L)], [opt(w.shared_w2, l) for l in range(L)]
        if self.hd is not None:
            self.m_hd = self._amaps(self.hd, T + 256, self.hd.shape[1])
        moe = [l for l in range(L) if w.host_w13[l] is not None]
        self.w13_maps, self.w2_maps = [None] * L, [None] * L
        self.staging, self.fetch_tiles = [None] * L, 0
        st13 = st2 = hl13 = hl2 = 0
        if self.staging_index is not None:   # region 2: the staging buffer a host loop fills
            hl13, hl2 = self._wmap(w.stage_w13[self.staging_index]), self._wmap(w.stage_w2[self.staging_index])
        if self.staged and moe:   # region 3: the lane's own staging stack, one slot per expert, filled by fetch tiles
            h13, h2 = w.host_w13[moe[0]], w.host_w2[moe[0]]
            self.stage_w13 = torch.empty(h13.shape, dtype=h13.dtype, device="cuda")
            self.stage_w2 = torch.empty(h2.shape, dtype=h2.dtype, device="cuda")
            st13, st2 = self._wmap(self.stage_w13), self._wmap(self.stage_w2)
            b13, b2 = h13[0].numel() * h13.element_size(), h2[0].numel() * h2.element_size()
            self.fetch_tiles = -(-b13 // self.fetch_chunk) + -(-b2 // self.fetch_chunk)
        for l in moe:
            self.w13_maps[l] = _u64([self._wmap(w.host_w13[l], _C.host_device_pointer(w.host_w13[l].data_ptr())),
                                     self._wmap(w.hot_w13[l], packed=True), hl13, st13])
            self.w2_maps[l] = _u64([self._wmap(w.host_w2[l], _C.host_device_pointer(w.host_w2[l].data_ptr())),
                                    self._wmap(w.hot_w2[l]), hl2, st2])
            if st13:
                self.staging[l] = _block(
                    "StagingArgs", w13_src=_C.host_device_pointer(w.host_w13[l].data_ptr()),
                    w13_dst=self.stage_w13.data_ptr(), w13_bytes=b13,
                    w2_src=_C.host_device_pointer(w.host_w2[l].data_ptr()), w2_dst=self.stage_w2.data_ptr(),
                    w2_bytes=b2, chunk_bytes=self.fetch_chunk, min_rows=self.staged_min_rows)
        self.xp_maps = _u64(self._amaps(self.xp, P + 256, H))
        self.h_maps = _u64(self._amaps(self.h, P + 256, I))
        a13, a2 = [], []
        for bm in HEIGHTS:
            b13 = torch.frombuffer(bytearray(_C.gemm_args(out=self.h.data_ptr(), ld_out=I, k_tiles=H // 64,
                                                          epi=EPI_SILU_MUL, bm=bm, n_limit=I, up_offset=I,
                                                          w_fp8=int(w.fp8_experts))), dtype=torch.uint8).cuda()
            b2 = torch.frombuffer(bytearray(_C.gemm_args(out=self.y.data_ptr(), ld_out=H, k_tiles=I // 64,
                                                         epi=EPI_ROWS_F32, bm=bm, n_limit=H, w_fp8=int(w.fp8_experts))),
                                  dtype=torch.uint8).cuda()
            self._keep += [b13, b2]
            a13.append(b13.data_ptr())
            a2.append(b2.data_ptr())
        self.w13_args, self.w2_args = _u64(a13), _u64(a2)
        # attention: one AttnArgs block per layer (the layer's cache maps)
        self.attn_args = []
        group = hq // hkv
        for l in range(L):
            q_map, q_small, k_map, v_map = fabric_maps(fab, self.q, self.kv.k[l], self.kv.v[l])
            self.attn_args.append(_block(
                "AttnArgs", q_map=q_map, k_map=k_map, v_map=v_map, out=self.ao, ws_o=self.ws,
                ws_m=self.ws.data_ptr() + self.ws_rows * 512, block_table=self.bt, req_info=self.req_info,
                scale_log2=SCALE_LOG2, bt_stride=self.bt_stride, hq=hq, hkv=hkv, group=group,
                max_chunks=self.max_chunks, page_size=self.kv.page, q_map_small=q_small))
        scoring = {"softmax": 0, "sigmoid": 1}[getattr(cfg, "scoring", "softmax")]
        self.router_args = [_block("RouterArgs", logits=self.rl, topk_ids=self.topk_ids, topk_w=self.topk_w,
                                   counts=self.counts, bias=w.router_bias[l] if w.router_bias[l] is not None else 0,
                                   E=E, K=K, scoring=scoring, renorm=1, scale=getattr(cfg, "routed_scale", 1.0),
                                   chunk_counts=self.chunk_counts) for l in range(L)]
        self.permute_args = _block("PermuteArgs", topk_ids=self.topk_ids, topk_w=self.topk_w, starts=self.starts,
                                   fill=self.fill, pair_token=self.pair_token, pair_weight=self.pair_weight,
                                   src=self.xn, dst=self.xp, K=K, H=H, chunk_prefix=self.chunk_prefix,
                                   pair_pos=self.pair_pos, E=E)
        self.step_args = _block("StepArgs", row_req=self.row_req, last_token=self.last_token, seq_len=self.seq_len,
                                block_table=self.bt, tok_pos=self.tok_pos, tok_slot=self.tok_slot,
                                req_info=self.req_info, bt_stride=self.bt_stride, page_size=self.kv.page)
        self.sample_args = _block("SampleArgs", logits=self.logits, temperature=self.temperature,
                                  last_token=self.last_token, steps=self.steps,
                                  host_tokens=_C.host_device_pointer(self.host_tokens.data_ptr()),
                                  host_steps=_C.host_device_pointer(self.host_steps.data_ptr()), seed=0x5eed,
                                  V=cfg.vocab, ring=self.ring)

    # ------------------------------------------------------------------ device memory of a build
    def _dev(self, name, **fields):
        """An operand block in the lane's arena."""
        return self.arena.put(pack(name, **fields))

    def _put(self, tensor, values, dtype=np.int32):
        """Write the first len(values) elements of a device tensor without launching a kernel."""
        data = np.ascontiguousarray(values, dtype=dtype)
        if data.size:
            self.fab.write(tensor.data_ptr(), data.tobytes())

    # ------------------------------------------------------------------ stage builders
    def _gemm_split(self, p, wmap, amaps, rows, n_out, k, slabs, parts, label, mark=None, mat=None, bias=None,
                    slab_rows=SPLIT_ROWS):
        """The same product for few rows as `parts` K ranges, every range storing its fp32 partial sums in its own
        slab of `slabs` ([parts][slab_rows][n_out]); the add-norm tile behind it adds the slabs in order.  A 128-row
        weight slice over all of K is a megabyte that one worker streams alone; the ranges spread it over
        parts x n_out / 128 workers, and the sum keeps a defined order (no atomics)."""
        bm = _bm(rows)
        fp8 = mat is not None and mat.fp8
        xm = amaps[HEIGHTS.index(bm)]
        kt = k // 64
        per = -(-kt // parts)
        ptrs, ranges = [], []
        for q in range(parts):
            k0, kn = q * per, min(per, kt - q * per)
            args = self.arena.put(_C.gemm_args(out=slabs.data_ptr() + 4 * q * slab_rows * n_out, ld_out=n_out, k_tiles=kt,
                                               epi=EPI_F32, bm=bm, n_limit=n_out, w_fp8=int(fp8),
                                               bias=bias.data_ptr() if bias is not None else 0))   # added by the first range
            ptrs.append(args.data_ptr())
            ranges.append(k0 | (kn << 16))
        key = ("split", rows, bm, n_out, parts, kt)
        tmpl = self._templates.get(key)
        if tmpl is None:
            m0, n0 = np.meshgrid(np.arange(0, rows, bm), np.arange(0, n_out, 128), indexing="ij")
            by_range = np.asarray(ranges, dtype=np.int64)[:, None, None]   # (range, row block, slice)
            tmpl = self._templates[key] = tile_array(K_GEMM, i0=n0[None], i1=m0[None], i2=np.minimum(bm, rows - m0)[None],
                                                     a3=by_range)
        per_range = len(tmpl) // parts
        tiles = _retarget(tmpl, a0=np.repeat(np.asarray(ptrs, dtype=np.uint64), per_range), a1=wmap, a2=xm,
                          a4=mat.scale.data_ptr() if fp8 else 0)
        return p.stage(tiles, mark=mark, label=label)

    def _gemm(self, p, wmap, amaps, rows, n_out, k, out, ld_out, epi, label, residual=None, ld_res=0, mark=None,
              mat=None, bias=None, up_offset=0):
        """A dense GEMM stage: out[rows][n_out] = act[rows][k] x weight[n_out (x2 for SiLU-mul)][k]^T.
        mat: the weight's Mat (e4m3 weights carry their scales into the tiles)."""
        bm = _bm(rows)
        fp8 = mat is not None and mat.fp8
        args = self.arena.put(_C.gemm_args(
            out=out.data_ptr(), ld_out=ld_out, k_tiles=k // 64, epi=epi, bm=bm, n_limit=n_out,
            residual=residual.data_ptr() if residual is not None else 0, ld_res=ld_res,
            bias=bias.data_ptr() if bias is not None else 0, up_offset=up_offset, w_fp8=int(fp8)))
        xm = amaps[HEIGHTS.index(bm)]
        step = 64 if epi == EPI_SILU_MUL else 128
        key = ("gemm", rows, bm, n_out, step)
        tmpl = self._templates.get(key)
        if tmpl is None:
            m0, n0 = np.meshgrid(np.arange(0, rows, bm), np.arange(0, n_out, step), indexing="ij")
            tmpl = self._templates[key] = tile_array(K_GEMM, i0=n0, i1=m0, i2=np.minimum(bm, rows - m0))
        tiles = _retarget(tmpl, a0=args.data_ptr(), a1=wmap, a2=xm, a4=mat.scale.data_ptr() if fp8 else 0)
        return p.stage(tiles, mark=mark, label=label)

    def _rows(self, kind, args, rows, per):
        key = ("rows", kind, rows, per)
        tmpl = self._templates.get(key)
        if tmpl is None:
            r0 = np.arange(0, rows, per)
            tmpl = self._templates[key] = tile_array(kind, i0=r0, i1=np.minimum(per, rows - r0))
        return _retarget(tmpl, a0=args.data_ptr())

    def _per(self, T):
        """Rows per tile of a stage whose tiles give each exec warp one row at a time: up to four rows per tile
        while that keeps the stage to one round of tiles over the workers (150 tiles on 148 workers are two
        rounds), a multiple of four beyond."""
        nw = self.fab.num_workers
        if T <= 4 * nw:
            return max(1, -(-T // nw))
        return -(-(-(-T // (2 * nw))) // 4) * 4

    def _logit_rows(self, T, E):
        """Rows per router-projection tile (of 16 experts): the height in 8 .. 32 that costs the fewest rounds x
        (rows + 4), the 4 standing for what a tile costs before its first row."""
        nw, groups = self.fab.num_workers, -(-E // 16)
        best = None
        for rows in range(8, 33, 2):
            cost = -(-(-(-T // rows) * groups) // nw) * (rows + 4)
            if best is None or cost < best[0]:
                best = (cost, rows)
        return best[1]

    def _one(self, kind, args):
        """The single tile of an expand or plan stage."""
        key = ("one", kind)
        tmpl = self._templates.get(key)
        if tmpl is None:
            tmpl = self._templates[key] = tile_array(kind)
        return _retarget(tmpl, a0=args.data_ptr())

    def _logits(self, args, T, E):
        key = ("logits", T, E)
        tmpl = self._templates.get(key)
        if tmpl is None:
            tmpl = self._templates[key] = logits_tiles(0, T, E, rows=self._logit_rows(T, E))
        return _retarget(tmpl, a0=args.data_ptr())

    def _moe(self, p, l, T, prev, norm_w, expands, fuse_norm=None):
        """Stages of layer l's MoE block after `prev` (xn, x2 ready); returns the combine stage.
        fuse_norm = (norm tile kind, its NormArgs): `prev` is the stage BEFORE the post-attention norm, and that norm
        is folded into the router projection's tiles (a small batch: a stage hop costs more than repeating the
        norm of a few rows in each expert-range tile)."""
        cfg = self.cfg
        H, E = cfg.hidden, cfg.num_experts
        nw = self.fab.num_workers
        lg = self._dev("LogitsArgs", x=self.xn, wr=self.w.router[l], logits=self.rl, T=T, H=H, E=E)
        shared = self.w.shared_w13[l] is not None
        cb = self._dev("CombineArgs", y=self.y, pair_pos=self.pair_pos, topk_w=self.topk_w, x2=self.x2, x=self.x,
                       w=norm_w if norm_w is not None else 0, out=self.xn, K=cfg.top_k, H=H, eps=cfg.rms_eps,
                       shared=self.y_shared if shared else 0)
        ex = self.arena.put(bytes(_C.struct_layouts()["ExpandArgs"][0]))   # filled once the dynamic region is laid out
        per = self._per(T)
        if fuse_norm is not None:
            kind, nrm = fuse_norm
            key = ("norm_logits", T, E)
            tmpl = self._templates.get(key)
            if tmpl is None:
                # four rows per tile: one row's norm per exec warp, then their projection
                tmpl = self._templates[key] = logits_tiles(0, T, E, rows=4)
                tmpl[:, 0] = (tmpl[:, 0] & np.uint64(0xFFFFFFFFFFFF0000)) | np.uint64(K_NORM_LOGITS)
            tiles = _retarget(tmpl, a0=nrm.data_ptr(), a1=lg.data_ptr())
            tiles[:, 6] = kind   # a[3]: which norm
            s_lg = p.stage(tiles, label=("norm_logits", l))
        else:
            s_lg = p.stage(self._logits(lg, T, E), label=("router_logits", l))
        s_rt = p.stage(self._rows(K_ROUTER, self.router_args[l], T, SUB), label=("router", l))
        p.after(prev, s_lg)
        p.after(s_lg, s_rt)
        xn_ready = s_lg if fuse_norm is not None else prev
        s_ex = p.stage(self._one(K_EXPAND, ex), label=("expand", l))
        p.after(s_rt, s_ex)
        permute_in_expand = T <= FUSE_PERMUTE_ROWS
        if permute_in_expand:
            s_pm = s_ex
        else:
            s_pm = p.stage(self._rows(K_PERMUTE, self.permute_args, T, SUB), label=("permute", l))
            p.after(s_ex, s_pm)
        w13_0 = p.stages(E, label=("w13", l))
        w2_0 = p.stages(E, label=("w2", l))
        s_cb = p.stage(self._rows(K_COMBINE, cb, T, per), mark=(l << 8) | 3, label=("combine", l))
        fetch_0 = p.stages(E, label=("fetch", l)) if self.staging[l] is not None else None
        p.fan_out(s_pm, w13_0, E)
        if fetch_0 is not None:   # the copy into the staging stack starts as soon as the expert's row count is known
            p.fan_out(s_ex, fetch_0, E)
            p.pairwise(fetch_0, w13_0, E)
        p.pairwise(w13_0, w2_0, E)
        p.fan_in(w2_0, E, s_cb)
        if shared:   # the shared expert runs beside the routed chain and joins at the combine stage
            s_s13 = self._gemm(p, self.m_sh13[l], self.m_xn, T, self.Is, H, self.hd, self.hd.shape[1], EPI_SILU_MUL,
                               ("shared_w13", l), mat=self.w.shared_w13[l], up_offset=self.Is)
            s_s2 = self._gemm(p, self.m_sh2[l], self.m_hd, T, H, self.Is, self.y_shared, H, EPI_F32, ("shared_w2", l),
                              mat=self.w.shared_w2[l])
            p.after(xn_ready, s_s13)
            p.after(s_s13, s_s2)
            p.after(s_s2, s_cb)
        dyn = (T * cfg.top_k // self.min_form + E) * (cfg.intermediate // 64 + H // 128)
        if fetch_0 is not None:
            dyn += E * self.fetch_tiles
        expands.append((ex, l, T, w13_0, 0xffffffff, w2_0, s_cb, dyn, fetch_0 if fetch_0 is not None else 0,
                        permute_in_expand))
        return s_cb

    def _finish_dynamic(self, p, expands, plans):
        """Hand each expand / plan tile its part of the dynamic region, now that every static tile is counted."""
        at = p.dynamic_first
        for ex, l, T, w13_0, red_0, w2_0, s_cb, dyn, fetch_0, pm_in in expands:
            p.reserve(dyn)
        for blob, fields, dyn in plans:
            p.reserve(dyn)
        cfg = self.cfg
        at = p.dynamic_first
        for ex, l, T, w13_0, red_0, w2_0, s_cb, dyn, fetch_0, pm_in in expands:
            blob = pack("ExpandArgs", permute_args=self.permute_args if pm_in else 0, permute_rows=T if pm_in else 0, counts=self.counts, starts=self.starts, fill=self.fill, table=self.tables[l],
                        w13_maps=self.w13_maps[l], w2_maps=self.w2_maps[l], xp_maps=self.xp_maps, h_maps=self.h_maps,
                        w13_args=self.w13_args, w2_args=self.w2_args, hist=self.hist[l], E=cfg.num_experts, H=cfg.hidden,
                        I=cfg.intermediate, host_region=REGION_HOST, w13_stage0=w13_0, w2_stage0=w2_0, red_stage0=red_0,
                        dyn_first=at, dyn_cap=dyn, lane=self.lane_id, join_stage=s_cb, chunks=-(-T // CHUNK),
                        chunk_counts=self.chunk_counts, chunk_prefix=self.chunk_prefix,
                        staging=self.staging[l] if self.staging[l] is not None else 0, fetch_stage0=fetch_0,
                        w13_scale=self.w.w13_scale[l] if self.w.w13_scale[l] is not None else 0,
                        w2_scale=self.w.w2_scale[l] if self.w.w2_scale[l] is not None else 0)
            self.arena.patch(ex, blob)
            at += dyn
        for blob, fields, dyn in plans:
            self.arena.patch(blob, pack("AttnPlanArgs", dyn_first=at, dyn_cap=dyn, **fields))
            at += dyn

    def _layers(self, p, T, first_stage, attention, sample_rows, n_rows):
        """The decoder after the embedding stage; `attention(p, l, prev)` adds layer l's attention
        stages after `prev` and returns the stage that completes `ao`.  Returns the last stage."""
        cfg, w = self.cfg, self.w
        H, L = cfg.hidden, cfg.num_layers
        hq, hkv = cfg.num_heads, cfg.num_kv_heads
        heads = hq + 2 * hkv
        prev = first_stage
        expands = []
        for l in range(L):
            qkv_parts = min(QKV_PARTS, (H // 64) // 8) if T <= SPLIT_ROWS else 1
            if qkv_parts > 1:
                s_qkv = self._gemm_split(p, self.m_qkv[l], self.m_xn, T, self.qkv_dim, H, self.qkv_slabs, qkv_parts,
                                         ("qkv", l), mat=w.qkv[l], bias=w.qkv_bias[l])
            else:
                s_qkv = self._gemm(p, self.m_qkv[l], self.m_xn, T, self.qkv_dim, H, self.qkv, self.qkv_dim, EPI_STORE,
                                   ("qkv", l), mat=w.qkv[l], bias=w.qkv_bias[l])
            p.after(prev, s_qkv)
            qk = self._dev("QkArgs", qkv=self.qkv_slabs if qkv_parts > 1 else self.qkv, qkv_parts=qkv_parts,
                        qkv_rows=SPLIT_ROWS, q_out=self.q, k_cache=self.kv.k[l], v_cache=self.kv.v[l],
                        q_norm=w.q_norm[l] if w.q_norm[l] is not None else 0,
                        k_norm=w.k_norm[l] if w.k_norm[l] is not None else 0, tok_pos=self.tok_pos, tok_slot=self.tok_slot,
                        cos_sin=self.cos_sin, ld_qkv=self.qkv_dim, hq=hq, hkv=hkv, rot_dim=cfg.rotary_dim,
                        theta=cfg.rope_theta, eps=cfg.rms_eps, max_pos=self.max_pos)
            # a small batch: few items per tile, so that every worker has one (an item is a chain of exposed loads)
            rope_items = min(ROPE_ITEMS, max(4, -(-(T * heads) // (4 * self.fab.num_workers)) * 4))
            s_rope = p.stage(self._rows(K_QKROPE, qk, T * heads, rope_items), mark=(l << 8) | 1, label=("rope", l))
            p.after(s_qkv, s_rope)
            s_attn = attention(p, l, s_rope)
            o_parts = min(SPLIT_PARTS if T <= SPLIT_ROWS else O_WIDE_PARTS, (hq * 128 // 64) // 8) if T <= self.o_rows else 1
            if o_parts > 1:
                # few rows: K ranges into fp32 slabs, then x2 = bf16(x + sum of the slabs) and its norm in one tile
                s_o = self._gemm_split(p, self.m_o[l], self.m_ao, T, H, hq * 128, self.o_slabs, o_parts, ("o", l),
                                       mark=(l << 8) | 2, mat=w.o[l], slab_rows=self.o_rows)
                nrm = self._dev("NormArgs", x=self.x2, x2=self.x, acc=self.o_slabs, w=w.post_norm[l], out=self.xn, H=H, ld=H,
                                eps=cfg.rms_eps, acc_parts=o_parts, acc_rows=self.o_rows)
                norm_kind = K_ADDNORM
            else:
                s_o = self._gemm(p, self.m_o[l], self.m_ao, T, H, hq * 128, self.x2, H, EPI_STORE, ("o", l),
                                 residual=self.x, ld_res=H, mark=(l << 8) | 2, mat=w.o[l])
                nrm = self._dev("NormArgs", x=self.x2, w=w.post_norm[l], out=self.xn, H=H, ld=H, eps=cfg.rms_eps)
                norm_kind = K_RMSNORM
            p.after(s_attn, s_o)
            next_norm = w.in_norm[l + 1] if l + 1 < L else None
            if w.mlp_w13[l] is None and T <= FUSE_ROWS:
                prev = self._moe(p, l, T, s_o, next_norm, expands, fuse_norm=(norm_kind, nrm))
                continue
            s_norm = p.stage(self._rows(norm_kind, nrm, T, self._per(T)),
                             label=("norm", l))
            p.after(s_o, s_norm)
            next_norm = w.in_norm[l + 1] if l + 1 < L else None
            if w.mlp_w13[l] is not None:
                # a dense layer: x = bf16(x2 + ffn(xn)), then the next layer's input norm
                s_d13 = self._gemm(p, self.m_mlp13[l], self.m_xn, T, self.Id, H, self.hd, self.hd.shape[1], EPI_SILU_MUL,
                                   ("mlp_w13", l), mat=w.mlp_w13[l], up_offset=self.Id)
                s_d2 = self._gemm(p, self.m_mlp2[l], self.m_hd, T, H, self.Id, self.x, H, EPI_STORE, ("mlp_w2", l),
                                  residual=self.x2, ld_res=H, mark=(l << 8) | 3, mat=w.mlp_w2[l])
                p.after(s_norm, s_d13)
                p.after(s_d13, s_d2)
                prev = s_d2
                if next_norm is not None:
                    nn = self._dev("NormArgs", x=self.x, w=next_norm, out=self.xn, H=H, ld=H, eps=cfg.rms_eps)
                    prev = p.stage(self._rows(K_RMSNORM, nn, T, self._per(T)),
                                   label=("in_norm", l + 1))
                    p.after(s_d2, prev)
                continue
            prev = self._moe(p, l, T, s_norm, next_norm, expands)
        # final norm of the rows that continue (gather), lm_head over those rows, next tokens
        R = n_rows
        fin = self._dev("NormArgs", x=self.x, w=w.final_norm, out=self.xn, gather=self.gather, out2=self.xlast, H=H, ld=H,
                     eps=cfg.rms_eps)
        s_fin = p.stage(self._rows(K_RMSNORM, fin, T, self._per(T)), label=("final_norm", L))
        p.after(prev, s_fin)
        s_lm = self._gemm(p, self.m_lm, self.m_xlast, R, cfg.vocab, H, self.logits, cfg.vocab, EPI_F32, ("lm_head", L))
        p.after(s_fin, s_lm)
        s_sample = p.stage([Tile(K_SAMPLE, i=(row, slot), a=(self.sample_args.data_ptr(),)) for row, slot in sample_rows],
                           label=("sample", L))
        p.after(s_lm, s_sample)
        return s_sample, expands

    # ------------------------------------------------------------------ programs
    def build_prefill(self, batch, iterations=1, all_logits=False):
        """batch: list of (slot, tokens, pos0): the request in `slot` appends `tokens` at positions
        pos0 .. (its pages must already be in the lane's block table row `slot`).  The program
        computes the batch, appends K/V to the caches, and samples one next token per request.
        all_logits: keep the logits of every row (row r of `logits`), not only each request's last."""
        page = self.kv.page
        self.arena.reset()   # the operand blocks of this lane's previous program: it must have ended
        if len(self._templates) > 256:   # shapes of many different batches: start over rather than grow
            self._templates.clear()
        tokens, pos, slots, req_info, sample_rows = [], [], [], [], []
        gather = []
        stride = self.bt.shape[1]
        row = 0
        for r, (slot, toks, pos0) in enumerate(batch):
            n = len(toks)
            req_info.append((row, pos0, n, pos0 + n))
            # the request's row of the block table (read through the fabric: nothing may be launched beside it)
            pages = np.frombuffer(self.fab.read(self.bt.data_ptr() + 4 * slot * stride, 4 * stride), dtype=np.int32)
            ppos = pos0 + np.arange(n)
            tokens.append(np.asarray(toks, dtype=np.int32))
            pos.append(ppos.astype(np.int32))
            slots.append((pages[ppos // page].astype(np.int64) * page + ppos % page).astype(np.int32))
            if all_logits:
                gather.append(np.arange(row, row + n, dtype=np.int32))
            else:
                g = np.full(n, -1, dtype=np.int32)
                g[n - 1] = r
                gather.append(g)
            sample_rows.append((row + n - 1 if all_logits else r, slot))
            row += n
        T = row
        assert 0 < T <= self.T and (T if all_logits else len(batch)) <= self.logit_rows
        self._put(self.tokens, np.concatenate(tokens))
        self._put(self.tok_pos, np.concatenate(pos))
        self._put(self.tok_slot, np.concatenate(slots))
        self._put(self.gather, np.concatenate(gather))
        self._put(self.req_info, req_info)
        cfg = self.cfg
        hq, hkv = cfg.num_heads, cfg.num_kv_heads
        items, merge, ws_rows = plan_items(req_info, hq, hkv, sms=self.fab.num_workers)
        assert ws_rows <= self.ws_rows, "attention split workspace too small"
        slot_of = torch.tensor([b[0] for b in batch], dtype=torch.int32)
        items[:, 0] = slot_of[items[:, 0].long()]
        p = Program()
        emb = self._dev("NormArgs", x=self.x, w=self.w.in_norm[0], out=self.xn, embed=self.w.embed, tokens=self.tokens,
                     H=cfg.hidden, ld=cfg.hidden, eps=cfg.rms_eps)
        s_embed = p.stage(self._rows(K_EMBED, emb, T, CHUNK), label=("embed", 0))

        item_tiles, merge_tiles = fabric_tiles(items, merge, 0, K_ATTN_PREFILL)   # the same work list in every layer

        def attention(p, l, prev):
            at = self.attn_args[l].data_ptr()
            s_a = p.stage(_retarget(item_tiles, a0=at), label=("attn", l))
            s_m = p.stage(_retarget(merge_tiles, a0=at), label=("attn_merge", l))
            p.after(prev, s_a)
            p.after(s_a, s_m)
            return s_m

        n_rows = T if all_logits else len(batch)
        last, expands = self._layers(p, T, s_embed, attention, sample_rows, n_rows)
        self._finish_dynamic(p, expands, [])
        self.rows_out = n_rows
        self.labels = p.labels()   # stage names, for monoserve_b200.fabric.trace.summary
        self.arena.flush()
        return p.upload(self.fab, first=s_embed, iterations=iterations)

    def build_decode(self, slots, iterations=1, chunk_keys=0):
        """One decode step per iteration for the requests in `slots` (row r = slots[r]): the
        embedding tiles take each request's last token and advance its length, the plan tile
        writes the step's attention items, and the sample tiles publish the next tokens."""
        cfg = self.cfg
        R = len(slots)
        assert 0 < R <= min(self.T, 256, self.logit_rows)
        self.arena.reset()   # the operand blocks of this lane's previous program: it must have ended
        if len(self._templates) > 256:   # shapes of many different batches: start over rather than grow
            self._templates.clear()
        self._put(self.row_req, slots)
        self._put(self.gather, np.arange(R))
        hq, hkv = cfg.num_heads, cfg.num_kv_heads
        p = Program()
        emb = self._dev("NormArgs", x=self.x, w=self.w.in_norm[0], out=self.xn, embed=self.w.embed, step=self.step_args,
                     H=cfg.hidden, ld=cfg.hidden, eps=cfg.rms_eps)
        s_embed = p.stage(self._rows(K_EMBED, emb, R, CHUNK), label=("embed", 0))
        plans = []

        def attention(p, l, prev):
            blob = self.arena.put(bytes(_C.struct_layouts()["AttnPlanArgs"][0]))   # filled with the dynamic region
            s_plan = p.stage(self._one(K_ATTN_PLAN, blob), label=("attn_plan", l))
            s_a = p.stage(label=("attn", l))
            s_m = p.stage(label=("attn_merge", l))
            # The plan needs the step's sequence lengths only (the embed tiles' bookkeeping), so every layer's
            # plan tile runs right after the embed stage, beside the layers before it, instead of between the
            # layer's rope and attention stages.
            p.after(s_embed, s_plan)
            p.after(s_plan, s_a)
            p.after(prev, s_a)
            p.after(s_a, s_m)
            fields = dict(attn=self.attn_args[l].data_ptr(), req_info=self.req_info.data_ptr(), rows=R, hkv=hkv,
                          chunk_keys=chunk_keys, stage_attn=s_a, stage_comb=s_m, workers=self.fab.num_workers,
                          row_req=self.row_req.data_ptr())
            plans.append((blob, fields, R * hkv * (self.max_chunks + 1)))
            return s_m

        last, expands = self._layers(p, R, s_embed, attention, [(r, s) for r, s in enumerate(slots)], R)
        self._finish_dynamic(p, expands, plans)
        self.rows_out = R
        self.labels = p.labels()
        self.arena.flush()
        return p.upload(self.fab, first=s_embed, iterations=iterations)

    # ------------------------------------------------------------------ request state
    def set_pages(self, slot, pages):
        row = np.zeros(self.bt_stride, dtype=np.int32)
        row[:len(pages)] = pages
        self.fab.write(self.bt.data_ptr() + 4 * slot * self.bt_stride, row.tobytes())

    def set_request(self, slot, seq_len, last_token, temperature=0.0):
        import struct
        self.fab.write(self.seq_len.data_ptr() + 4 * slot, struct.pack("<i", seq_len))
        self.fab.write(self.last_token.data_ptr() + 4 * slot, struct.pack("<i", last_token))
        self.fab.write(self.steps.data_ptr() + 4 * slot, struct.pack("<i", 0))
        self.fab.write(self.temperature.data_ptr() + 4 * slot, struct.pack("<f", temperature))
