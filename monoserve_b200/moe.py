"""One MoE layer on the B200 hot path: routing, stable pack, grouped SwiGLU
expert GEMMs from the HBM hot tier or in place from pinned host memory, and the
fused un-permute + weighted combine.

This is the host-side mirror of what the reference spreads over
monoserve/runtime/weights.py (expert stacks in pinned host memory, hot tier in
HBM, the per-layer (region, slot) table and `set_location`), the per-layer stage
chain of monoserve/runtime/lane.py:340-380, and the parts of a published plan a
layer consumes (SM count, link credits, kernel form: csrc/bindings.cpp:211-232).
All compute happens in libmonofab.so through its C ABI; torch only owns memory
and streams.  There is no CPU fallback.
"""
import ctypes

import torch

from monoserve_b200 import _C

REGION_HOST, REGION_HOT = 0, 1   # monoserve/runtime/kinds.py:16-18
_WORKSPACES = {"logits": torch.float32, "topk_ids": torch.int32, "topk_w": torch.float32,
               "counts": torch.int32, "starts": torch.int32, "pair_token": torch.int32,
               "pair_weight": torch.float32, "pair_pos": torch.int32, "xp": torch.bfloat16,
               "h": torch.bfloat16, "y": torch.float32, "queues": torch.int32, "hist": torch.int32,
               "table": torch.int32, "trace": torch.int32}


def _stream_ptr(stream=None):
    s = stream if stream is not None else torch.cuda.current_stream()
    return ctypes.c_void_p(s.cuda_stream)


def pin(t):
    """Pinned, device-mapped host copy of `t` (monoserve/runtime/weights.py:57-58)."""
    p = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
    p.copy_(t)
    return p


class MoELayer:
    """moe = MoELayer(hidden, intermediate, experts, top_k, max_tokens)
    moe.set_router(wr)                     # bf16 [E, H] on the GPU
    moe.set_experts(w13, w2, hot=[...])    # full stacks -> pinned host + HBM hot tier
    moe.set_plan(ctas=0, credits=8, form=64)
    out = moe.forward(xn, x2)              # bf16 [T, H] = bf16(x2 + moe(xn))
    """

    def __init__(self, hidden, intermediate, experts, top_k, max_tokens, scoring="softmax", renorm=True,
                 routed_scale=1.0, fp8=False):
        if not torch.cuda.is_available():
            raise RuntimeError("monofab: a CUDA device is required (there is no CPU fallback)")
        self.H, self.I, self.E, self.K, self.max_tokens = hidden, intermediate, experts, top_k, max_tokens
        cfg = _C.MoEConfigC(hidden=hidden, intermediate=intermediate, experts=experts, top_k=top_k,
                            max_tokens=max_tokens, scoring={"softmax": 0, "sigmoid": 1}[scoring],
                            renorm=int(bool(renorm)), routed_scale=float(routed_scale), fp8=int(bool(fp8)))
        self.fp8 = bool(fp8)
        self._h = ctypes.c_void_p()
        _C.check(_C.lib.monofab_moe_create(ctypes.byref(cfg), ctypes.byref(self._h)))
        self._keep = {}
        self.hot = []
        self.table = None
        self._owned = True

    @classmethod
    def borrowed(cls, handle, hidden, intermediate, experts, top_k, max_tokens, fp8=False):
        """A view of a layer that another native object owns (the local expert layer of an
        expert-parallel layer); close() does not destroy it."""
        self = cls.__new__(cls)
        self.H, self.I, self.E, self.K, self.max_tokens = hidden, intermediate, experts, top_k, max_tokens
        self.fp8 = bool(fp8)
        self._h = ctypes.c_void_p(handle)
        self._keep = {}
        self.hot = []
        self.table = None
        self._owned = False
        return self

    def close(self):
        if getattr(self, "_h", None) and self._h.value and _C is not None and _C.lib is not None:
            if self._owned:
                _C.lib.monofab_moe_destroy(self._h)
            self._h = ctypes.c_void_p()

    __del__ = close

    # ---- weights and placement -------------------------------------------------
    def set_router(self, wr, bias=None):
        assert wr.is_cuda and wr.dtype == torch.bfloat16 and wr.shape == (self.E, self.H) and wr.is_contiguous()
        if bias is not None:
            assert bias.is_cuda and bias.dtype == torch.float32 and bias.shape == (self.E,)
        self._keep["router"] = (wr, bias)
        _C.check(_C.lib.monofab_moe_set_router(self._h, wr.data_ptr(), bias.data_ptr() if bias is not None else None))

    def set_region(self, region, w13, w2, packed=False):
        """Register the weight stacks of one region: pinned host tensors for
        REGION_HOST, CUDA tensors for REGION_HOT.  packed: w13 is already in the
        packed SwiGLU row order (see pack_w13)."""
        assert w13.shape[1:] == (2 * self.I, self.H) and w2.shape[1:] == (self.H, self.I)
        assert w13.shape[0] == w2.shape[0] and w13.is_contiguous() and w2.is_contiguous()
        want = torch.uint8 if self.fp8 else torch.bfloat16
        assert w13.dtype == want and w2.dtype == want, f"expert weights must be {want}"
        if region == REGION_HOST:
            assert w13.is_pinned() and w2.is_pinned(), "host-resident experts must be in pinned memory"
        else:
            assert w13.is_cuda and w2.is_cuda
        self._keep[("region", region)] = (w13, w2)
        _C.check(_C.lib.monofab_moe_set_region(self._h, region, w13.data_ptr(), w2.data_ptr(), w13.shape[0]))
        _C.check(_C.lib.monofab_moe_set_w13_packed(self._h, region, int(packed)))

    def pack_w13(self, w13):
        """HBM copy of w13 stacks [n, 2I, H] (pinned host or CUDA) in the packed
        SwiGLU row order: 16 gate rows, then their 16 up rows, per group of 16 features."""
        n = w13.shape[0]
        dst = torch.empty(w13.shape, dtype=w13.dtype, device="cuda")
        src = w13.data_ptr() if w13.is_cuda else _C.host_device_pointer(w13.data_ptr())
        _C.check(_C.lib.monofab_pack_w13(src, dst.data_ptr(), n, self.I, self.H, w13.element_size(), _stream_ptr()))
        torch.cuda.current_stream().synchronize()
        return dst

    def set_scales(self, s13, s2):
        """FP8: fp32 per-output-channel scales [E, 2I] and [E, H] on the GPU, indexed by expert id."""
        assert s13.is_cuda and s2.is_cuda and s13.dtype == torch.float32 and s2.dtype == torch.float32
        assert s13.shape == (self.E, 2 * self.I) and s2.shape == (self.E, self.H)
        assert s13.is_contiguous() and s2.is_contiguous()
        self._keep["scales"] = (s13, s2)
        _C.check(_C.lib.monofab_moe_set_scales(self._h, s13.data_ptr(), s2.data_ptr()))

    def set_table(self, table):
        """table: int32 [E, 2] = (region, slot) per expert (monoserve/runtime/weights.py:127-158)."""
        t = torch.as_tensor(table, dtype=torch.int32).contiguous().cpu()
        assert t.shape == (self.E, 2)
        _C.check(_C.lib.monofab_moe_set_table(self._h, t.data_ptr(), _stream_ptr()))
        self.table = t

    def set_experts(self, w13, w2, hot, pack_hot=True, scales=None):
        """The reference's placement: the FULL expert set in pinned host memory,
        and a copy of the `hot` experts in HBM (monoserve/runtime/weights.py:100-115).
        pack_hot: store the hot tier's w13 in the packed SwiGLU row order."""
        hot = list(hot)
        if scales is not None:
            self.set_scales(scales[0].cuda().contiguous(), scales[1].cuda().contiguous())
        host13, host2 = (w13 if w13.is_pinned() else pin(w13.cpu())), (w2 if w2.is_pinned() else pin(w2.cpu()))
        self.set_region(REGION_HOST, host13, host2)
        table = torch.zeros(self.E, 2, dtype=torch.int32)
        table[:, 1] = torch.arange(self.E)
        if hot:
            idx = torch.tensor(hot)
            hot13 = host13[idx].cuda()
            if pack_hot:
                hot13 = self.pack_w13(hot13)
            self.set_region(REGION_HOT, hot13, host2[idx].cuda(), packed=pack_hot)
            table[idx, 0] = REGION_HOT
            table[idx, 1] = torch.arange(len(hot), dtype=torch.int32)
        self.hot = hot
        self.set_table(table)

    def set_plan(self, ctas=0, credits=8, form=64):
        _C.check(_C.lib.monofab_moe_set_plan(self._h, ctas, credits, form))

    # ---- compute -------------------------------------------------------------------
    def forward(self, xn, x2=None, out=None):
        T = xn.shape[0]
        assert xn.is_cuda and xn.dtype == torch.bfloat16 and xn.shape == (T, self.H) and xn.is_contiguous()
        if x2 is not None:
            assert x2.is_cuda and x2.dtype == torch.bfloat16 and x2.shape == xn.shape and x2.is_contiguous()
        if out is None:
            out = torch.empty_like(xn)
        _C.check(_C.lib.monofab_moe_forward(self._h, xn.data_ptr(), x2.data_ptr() if x2 is not None else None,
                                            out.data_ptr(), T, _stream_ptr()))
        return out

    def experts(self, seg_counts, seg_expert=None):
        """Expert FFN over the rows already in workspace("xp"): segment s = seg_counts[s]
        consecutive rows of expert seg_expert[s] (int32 CUDA tensors).  Results in
        workspace("y") (fp32 rows) and workspace("h")."""
        assert seg_counts.is_cuda and seg_counts.dtype == torch.int32 and seg_counts.is_contiguous()
        if seg_expert is not None:
            assert seg_expert.is_cuda and seg_expert.dtype == torch.int32 and seg_expert.numel() == seg_counts.numel()
        _C.check(_C.lib.monofab_moe_experts(self._h, seg_counts.data_ptr(),
                                            seg_expert.data_ptr() if seg_expert is not None else None,
                                            seg_counts.numel(), _stream_ptr()))

    def forward_host(self, xn_host, x2_host, out_host):
        """Host buffers in, host buffer out (synchronous)."""
        T = xn_host.shape[0]
        for t in (xn_host, x2_host, out_host):
            assert t is None or (not t.is_cuda and t.dtype == torch.bfloat16 and t.is_contiguous())
        _C.check(_C.lib.monofab_moe_forward_host(self._h, xn_host.data_ptr(),
                                                 x2_host.data_ptr() if x2_host is not None else None,
                                                 out_host.data_ptr(), T, _stream_ptr()))
        return out_host

    def status(self):
        """Device status word; raises RuntimeError if a kernel reported an error."""
        st = ctypes.c_int32()
        _C.check(_C.lib.monofab_moe_status(self._h, ctypes.byref(st), _stream_ptr()))
        return st.value

    def workspace(self, name):
        """A torch view (no copy) of a named device workspace."""
        ptr, nbytes = ctypes.c_void_p(), ctypes.c_size_t()
        _C.check(_C.lib.monofab_moe_workspace(self._h, name.encode(), ctypes.byref(ptr), ctypes.byref(nbytes)))
        dt = _WORKSPACES[name]
        n = nbytes.value // torch.empty((), dtype=dt).element_size()
        return _from_device_address(ptr.value, n, dt)

    def set_profile(self, on):
        _C.check(_C.lib.monofab_moe_set_profile(self._h, int(on)))

    def last_times(self):
        """Milliseconds of the last profiled forward, by kernel."""
        ms = (ctypes.c_float * 6)()
        _C.check(_C.lib.monofab_moe_last_times(self._h, ctypes.byref(ms)))
        names = ["router_logits", "router_topk", "plan", "pack", "experts", "combine"]
        return dict(zip(names, list(ms)))


class _CudaArray:
    def __init__(self, ptr, n, dt):
        item = torch.empty((), dtype=dt).element_size()
        typestr = {torch.float32: "<f4", torch.int32: "<i4", torch.bfloat16: "<u2"}[dt]
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": typestr, "data": (ptr, False), "version": 3,
                                         "strides": (item,)}


def _from_device_address(ptr, n, dt):
    t = torch.as_tensor(_CudaArray(ptr, n, dt), device="cuda")
    return t.view(torch.bfloat16) if dt == torch.bfloat16 else t
