"""CPU oracle of the MonoFab MoE hot path — TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs import
this package, and only as the checker; nothing under monoserve_b200/ does.

`oracle.c_lib()` loads oracle/liboracle.so (built by `make -C oracle` or
`oracle.build()`), the plain-C restatement in monofab_oracle.c; the functions
below wrap it over numpy arrays.  bf16 tensors travel as uint16 bit patterns.
`oracle.torch_path` is the restatement of the reference's PyTorch MoE path
used for large shapes and as the timed CPU baseline.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def build():
    subprocess.run(["make", "-C", _HERE, "-s"], check=True)
    return os.path.join(_HERE, "liboracle.so")


def c_lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "liboracle.so")
        src = os.path.join(_HERE, "monofab_oracle.c")
        if not os.path.exists(path) or os.path.getmtime(path) < os.path.getmtime(src):
            build()
        _LIB = ctypes.CDLL(path)
        _LIB.orc_expf.restype = ctypes.c_float
        _LIB.orc_expf.argtypes = [ctypes.c_float]
        _LIB.orc_sigmoidf.restype = ctypes.c_float
        _LIB.orc_sigmoidf.argtypes = [ctypes.c_float]
    return _LIB


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _c(a, dtype):
    return None if a is None else np.ascontiguousarray(a, dtype=dtype)


def bf16_bits(t):
    """torch bf16 tensor (or float array to be rounded) -> uint16 numpy bits."""
    import torch
    if isinstance(t, torch.Tensor):
        return t.detach().cpu().to(torch.bfloat16).contiguous().view(torch.int16).numpy().view(np.uint16)
    return bf16_bits(torch.from_numpy(np.asarray(t, dtype=np.float32)))


def bits_to_f32(bits):
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def expf(x):
    lib = c_lib()
    return np.array([lib.orc_expf(float(v)) for v in np.asarray(x, dtype=np.float32).ravel()],
                    dtype=np.float32).reshape(np.shape(x))


def router_logits(x_bits, wr_bits):
    x_bits, wr_bits = _c(x_bits, np.uint16), _c(wr_bits, np.uint16)
    T, H = x_bits.shape
    E = wr_bits.shape[0]
    out = np.zeros((T, E), dtype=np.float32)
    c_lib().orc_router_logits(_p(x_bits), _p(wr_bits), _p(out), T, H, E)
    return out


def router_topk(logits, K, bias=None, scoring=0, renorm=1, scale=1.0):
    logits = _c(logits, np.float32)
    bias = _c(bias, np.float32)
    T, E = logits.shape
    ids = np.zeros((T, K), dtype=np.int32)
    w = np.zeros((T, K), dtype=np.float32)
    counts = np.zeros(E, dtype=np.int32)
    r = c_lib().orc_router_topk(_p(logits), _p(bias), _p(ids), _p(w), _p(counts), T, E, K, int(scoring),
                                int(renorm), ctypes.c_float(scale))
    if r:
        raise ValueError("router_topk: E or K outside the supported range")
    return ids, w, counts


def scan(counts):
    counts = _c(counts, np.int32)
    starts = np.zeros(len(counts) + 1, dtype=np.int32)
    c_lib().orc_scan(_p(counts), _p(starts), len(counts))
    return starts


def pack(ids, w, starts):
    ids, w, starts = _c(ids, np.int32), _c(w, np.float32), _c(starts, np.int32)
    T, K = ids.shape
    E = len(starts) - 1
    pt = np.zeros(T * K, dtype=np.int32)
    pw = np.zeros(T * K, dtype=np.float32)
    pp = np.zeros((T, K), dtype=np.int32)
    c_lib().orc_pack(_p(ids), _p(w), _p(starts), T, K, E, _p(pt), _p(pw), _p(pp))
    return pt, pw, pp


def permute_rows(x_bits, pair_token):
    x_bits, pair_token = _c(x_bits, np.uint16), _c(pair_token, np.int32)
    P, H = len(pair_token), x_bits.shape[1]
    xp = np.zeros((P, H), dtype=np.uint16)
    c_lib().orc_permute_rows(_p(x_bits), _p(pair_token), P, H, _p(xp))
    return xp


def expert_ffn(xp_bits, starts, w13_bits, w2_bits, scale13=None, scale2=None):
    xp_bits, starts = _c(xp_bits, np.uint16), _c(starts, np.int32)
    w13_bits, w2_bits = _c(w13_bits, np.uint16), _c(w2_bits, np.uint16)
    scale13, scale2 = _c(scale13, np.float32), _c(scale2, np.float32)
    E, twoI, H = w13_bits.shape
    I = twoI // 2
    P = xp_bits.shape[0]
    h = np.zeros((P, I), dtype=np.uint16)
    y = np.zeros((P, H), dtype=np.float32)
    c_lib().orc_expert_ffn(_p(xp_bits), _p(starts), _p(w13_bits), _p(w2_bits), _p(scale13), _p(scale2), E, H, I,
                           _p(h), _p(y))
    return h, y


def combine(y, pair_pos, topk_w, x2_bits=None, norm_w_bits=None, eps=0.0):
    y, pair_pos, topk_w = _c(y, np.float32), _c(pair_pos, np.int32), _c(topk_w, np.float32)
    x2_bits, norm_w_bits = _c(x2_bits, np.uint16), _c(norm_w_bits, np.uint16)
    T, K = pair_pos.shape
    H = y.shape[1]
    x = np.zeros((T, H), dtype=np.uint16)
    normed = np.zeros((T, H), dtype=np.uint16) if norm_w_bits is not None else None
    c_lib().orc_combine(_p(y), _p(pair_pos), _p(topk_w), _p(x2_bits), _p(x), _p(norm_w_bits), _p(normed), T, K, H,
                        ctypes.c_float(eps))
    return (x, normed) if normed is not None else x


def moe_layer(xn_bits, x2_bits, wr_bits, w13_bits, w2_bits, K, bias=None, scoring=0, renorm=1, scale=1.0):
    """The whole layer in C (small shapes).  Returns a dict of every intermediate."""
    logits = router_logits(xn_bits, wr_bits)
    ids, w, counts = router_topk(logits, K, bias, scoring, renorm, scale)
    starts = scan(counts)
    pt, pw, pp = pack(ids, w, starts)
    xp = permute_rows(xn_bits, pt)
    h, y = expert_ffn(xp, starts, w13_bits, w2_bits)
    out = combine(y, pp, w, x2_bits)
    return dict(logits=logits, topk_ids=ids, topk_w=w, counts=counts, starts=starts, pair_token=pt,
                pair_weight=pw, pair_pos=pp, xp=xp, h=h, y=y, out=out)
