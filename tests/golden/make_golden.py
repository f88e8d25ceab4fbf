"""Generates tests/golden/*.npz by running the REFERENCE's own torch oracle.

Run where the reference checkout is available, with $MONOSERVE_REFERENCE naming it:

    MONOSERVE_REFERENCE=<path of the reference checkout> python tests/golden/make_golden.py

It imports the reference's test modules tests/test_fabric_model.py and
tests/test_fabric_model_glm.py and calls their `reference_logits` unchanged.
Those functions hard-code device="cuda" and expect the reference's native
module; so, for the duration of the call only, a stub `monoserve._C` is put in
sys.modules and the torch factory functions they use are wrapped to place
tensors on the CPU (Tensor.cuda becomes the identity).  No reference source is
copied: the functions run from where they lie.

Weights are drawn from a seeded generator in a fixed order (see `make_weights`)
so the tests can regenerate them; the fixture stores their CRC-32 values.
"""
import importlib
import os
import sys
import types
import zlib
from contextlib import contextmanager

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.environ.get("MONOSERVE_REFERENCE")   # checkout of the reference project; required to (re)generate


@contextmanager
def reference_on_cpu():
    """Make the reference's test oracles importable and runnable without a GPU."""
    stub = types.ModuleType("monoserve._C")
    saved_mod = sys.modules.get("monoserve._C")
    sys.modules["monoserve._C"] = stub
    sys.path[:0] = [REF, os.path.join(REF, "tests")]
    names = ["tensor", "arange", "zeros", "ones"]
    saved = {n: getattr(torch, n) for n in names}
    saved_cuda = torch.Tensor.cuda

    def on_cpu(fn):
        def wrapped(*a, **k):
            if k.get("device") == "cuda":
                k["device"] = "cpu"
            return fn(*a, **k)
        return wrapped

    for n in names:
        setattr(torch, n, on_cpu(saved[n]))
    torch.Tensor.cuda = lambda self, *a, **k: self
    try:
        yield
    finally:
        for n in names:
            setattr(torch, n, saved[n])
        torch.Tensor.cuda = saved_cuda
        del sys.path[:2]
        if saved_mod is None:
            sys.modules.pop("monoserve._C", None)
        else:
            sys.modules["monoserve._C"] = saved_mod


def bf16_bits(t):
    return t.to(torch.bfloat16).contiguous().view(torch.int16).numpy().view(np.uint16)


def make_weights(cfg, seed):
    """Random bf16 weights of a tiny Qwen3-style model, drawn in this order."""
    g = torch.Generator().manual_seed(seed)
    H, I, E, L, V = cfg.hidden, cfg.intermediate, cfg.num_experts, cfg.num_layers, cfg.vocab
    hq, hkv, D = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim

    def rnd(*shape, scale=1.0):
        return (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16)

    w = types.SimpleNamespace()
    w.embed = rnd(V, H)
    w.lm_head = rnd(V, H, scale=H ** -0.5)
    w.final_norm = (1 + 0.1 * torch.randn(H, generator=g)).to(torch.bfloat16)
    for name in ("in_norm", "qkv", "q_norm", "k_norm", "o", "post_norm", "router", "host_w13", "host_w2"):
        setattr(w, name, [])
    for _ in range(L):
        w.in_norm.append((1 + 0.1 * torch.randn(H, generator=g)).to(torch.bfloat16))
        w.qkv.append(rnd((hq + 2 * hkv) * D, H, scale=H ** -0.5))
        w.q_norm.append((1 + 0.1 * torch.randn(D, generator=g)).to(torch.bfloat16))
        w.k_norm.append((1 + 0.1 * torch.randn(D, generator=g)).to(torch.bfloat16))
        w.o.append(rnd(H, hq * D, scale=(hq * D) ** -0.5))
        w.post_norm.append((1 + 0.1 * torch.randn(H, generator=g)).to(torch.bfloat16))
        w.router.append(rnd(E, H, scale=H ** -0.5))
        w.host_w13.append(rnd(E, 2 * I, H, scale=H ** -0.5))
        w.host_w2.append(rnd(E, H, I, scale=I ** -0.5))
    return w


def quantize_fp8(w):
    """Per-output-channel e4m3 quantisation as the reference's weights do it
    (monoserve/runtime/weights.py:218-229): scale = amax / 448, clamped at 1e-12."""
    s = (w.float().abs().amax(dim=-1, keepdim=True) / 448.0).clamp_min(1e-12)
    q = (w.float() / s).to(torch.float8_e4m3fn)
    return q.view(torch.uint8).contiguous(), s.squeeze(-1).contiguous(), q.float() * s


def make_glm_weights(cfg, seed):
    """Random weights of a tiny GLM-4.5-style model, drawn in this order; every matrix quantised to e4m3 with
    per-row scales.  Returns an object that offers both what the reference's oracle reads (`dequantized`,
    `expert_weights`, the norm / bias / router tensors) and what this library's ModelWeights reads (pairs of
    bytes and scales)."""
    g = torch.Generator().manual_seed(seed)
    H, I, E, L, V = cfg.hidden, cfg.intermediate, cfg.num_experts, cfg.num_layers, cfg.vocab
    hq, hkv, D = cfg.num_heads, cfg.num_kv_heads, 128
    Id, Is, nd = cfg.dense_intermediate, cfg.shared_intermediate, cfg.dense_layers

    def rnd(*shape, scale=1.0):
        return torch.randn(*shape, generator=g) * scale

    w = types.SimpleNamespace()
    w.embed = rnd(V, H).to(torch.bfloat16)
    w.lm_head = rnd(V, H, scale=H ** -0.5).to(torch.bfloat16)
    w.final_norm = (1 + 0.1 * rnd(H)).to(torch.bfloat16)
    deq = {}
    for name in ("in_norm", "post_norm", "qkv", "qkv_bias", "o", "mlp_w13", "mlp_w2", "router", "router_bias",
                 "shared_w13", "shared_w2", "host_w13", "host_w2", "w13_scale", "w2_scale"):
        setattr(w, name, [None] * L)

    def q(name, l, t):
        b, s, d = quantize_fp8(t)
        deq[(name, l)] = d
        return (b, s)

    for l in range(L):
        w.in_norm[l] = (1 + 0.1 * rnd(H)).to(torch.bfloat16)
        w.post_norm[l] = (1 + 0.1 * rnd(H)).to(torch.bfloat16)
        w.qkv[l] = q("qkv", l, rnd((hq + 2 * hkv) * D, H, scale=H ** -0.5))
        w.qkv_bias[l] = (0.1 * rnd((hq + 2 * hkv) * D)).to(torch.bfloat16)
        w.o[l] = q("o", l, rnd(H, hq * D, scale=(hq * D) ** -0.5))
        if l < nd:
            w.mlp_w13[l] = q("mlp_w13", l, rnd(2 * Id, H, scale=H ** -0.5))
            w.mlp_w2[l] = q("mlp_w2", l, rnd(H, Id, scale=Id ** -0.5))
        else:
            w.router[l] = rnd(E, H, scale=H ** -0.5).to(torch.bfloat16)
            w.router_bias[l] = 0.1 * rnd(E)
            w.shared_w13[l] = q("shared_w13", l, rnd(2 * Is, H, scale=H ** -0.5))
            w.shared_w2[l] = q("shared_w2", l, rnd(H, Is, scale=Is ** -0.5))
            b13, s13, d13 = quantize_fp8(rnd(E, 2 * I, H, scale=H ** -0.5))
            b2, s2, d2 = quantize_fp8(rnd(E, H, I, scale=I ** -0.5))
            w.host_w13[l], w.w13_scale[l], w.host_w2[l], w.w2_scale[l] = b13, s13, b2, s2
            deq[("experts", l)] = (d13, d2)
    w.dequantized = lambda name, l: deq[(name, l)]
    w.expert_weights = lambda l: deq[("experts", l)]
    return w


def glm_fixture():
    with reference_on_cpu():
        ref = importlib.import_module("test_fabric_model_glm")
        cfg = ref.CFG   # 3 layers (first dense), 12 / 4 heads, rotary 64, sigmoid routing x 1.5, shared expert, FP8
        w = make_glm_weights(cfg, seed=17)
        g = torch.Generator().manual_seed(5)
        tokens = torch.randint(0, cfg.vocab, (45,), generator=g).tolist()
        logits = ref.reference_logits(w, cfg, tokens)
    out = {"tokens": np.array(tokens, dtype=np.int32), "logits": logits.numpy().astype(np.float32),
           "cfg": np.array([cfg.hidden, cfg.intermediate, cfg.num_experts, cfg.top_k, cfg.num_layers, cfg.num_heads,
                            cfg.num_kv_heads, cfg.vocab, cfg.rotary_dim, cfg.dense_layers, cfg.dense_intermediate,
                            cfg.shared_intermediate], dtype=np.int64),
           "rope_theta": np.float64(cfg.rope_theta), "rms_eps": np.float64(cfg.rms_eps),
           "routed_scale": np.float64(cfg.routed_scale), "weights_seed": np.int64(17),
           "crc_embed": np.uint32(zlib.crc32(bf16_bits(w.embed).tobytes())),
           "crc_experts": np.uint32(zlib.crc32(w.host_w13[cfg.num_layers - 1].numpy().tobytes()))}
    np.savez_compressed(os.path.join(HERE, "glm_tiny_reference_logits.npz"), **out)
    print("glm fixture: logits", logits.shape, "max |logit|", float(logits.abs().max()))



def qwen_fixture():
    with reference_on_cpu():
        ref = importlib.import_module("test_fabric_model")
        cfg = ref.CFG   # hidden 512, intermediate 256, 16 experts top-4, 2 layers, 4/2 heads, vocab 1024
        w = make_weights(cfg, seed=11)
        g = torch.Generator().manual_seed(3)
        tokens = torch.randint(0, cfg.vocab, (41,), generator=g).tolist()
        logits = ref.reference_logits(w, cfg, tokens)
    out = {"tokens": np.array(tokens, dtype=np.int32), "logits": logits.numpy().astype(np.float32),
           "cfg": np.array([cfg.hidden, cfg.intermediate, cfg.num_experts, cfg.top_k, cfg.num_layers,
                            cfg.num_heads, cfg.num_kv_heads, cfg.vocab], dtype=np.int64),
           "rope_theta": np.float64(cfg.rope_theta), "rms_eps": np.float64(cfg.rms_eps)}
    # The weights are NOT stored (24 MB); tests rebuild them with make_weights(cfg, 11)
    # and compare these CRC-32 values first, so a drift of torch's RNG stream is
    # reported as such instead of as a parity failure.
    crc = {}
    for name in ("embed", "lm_head", "final_norm"):
        crc[name] = zlib.crc32(bf16_bits(getattr(w, name)).tobytes())
    for name in ("in_norm", "qkv", "q_norm", "k_norm", "o", "post_norm", "router", "host_w13", "host_w2"):
        crc[name] = zlib.crc32(np.stack([bf16_bits(t) for t in getattr(w, name)]).tobytes())
    out["crc_names"] = np.array(sorted(crc))
    out["crc_values"] = np.array([crc[k] for k in sorted(crc)], dtype=np.uint32)
    out["weights_seed"] = np.int64(11)
    np.savez_compressed(os.path.join(HERE, "qwen_tiny_reference_logits.npz"), **out)
    print("qwen fixture: logits", logits.shape, "max |logit|", float(logits.abs().max()))


def helper_fixture():
    """bf / rms / rope of the reference on seeded inputs (tests/test_fabric_model.py:26-42)."""
    with reference_on_cpu():
        ref = importlib.import_module("test_fabric_model")
        g = torch.Generator().manual_seed(5)
        x = torch.randn(7, 512, generator=g).to(torch.bfloat16).float()
        wn = (1 + 0.1 * torch.randn(512, generator=g)).to(torch.bfloat16)
        q = torch.randn(7, 4, 128, generator=g)
        pos = torch.tensor([0, 1, 2, 3, 100, 1000, 4095])
        out = {"x": x.numpy(), "norm_w": bf16_bits(wn), "rms": ref.rms(x, wn, 1e-6).numpy(),
               "q": q.numpy(), "pos": pos.numpy(), "rope_full": ref.rope(q, pos, 1e6, 128).numpy(),
               "rope_half": ref.rope(q, pos, 1e4, 64).numpy()}
    np.savez_compressed(os.path.join(HERE, "helpers_reference.npz"), **out)
    print("helper fixture written")


def program_spec(mod):
    """The same two programs built through any Program/Tile implementation."""
    out = {}
    p = mod.Program()
    a = p.stage([mod.Tile(mod.KIND["spin"], i=(i, 0), a=(1000 + i, 77)) for i in range(5)])
    b = p.stage([mod.Tile(33, i=(1, 2, 3, 4), a=(5, 6, 7, 8, 9), flags=3)], link=True, mark=0x201)
    c = p.stage(mod.tile_array(32, i0=np.arange(7) * 128, i1=3, i2=9, i3=1, a0=111, a1=222, a2=333))
    d = p.stage()
    p.after(a, b)
    p.after(a, c)
    p.after(b, d)
    p.after(c, d)
    p.reserve(11)
    out["dag"] = p.pack(a, iterations=3, reset_tiles=4)
    q = mod.Program()
    q.stage([mod.Tile(mod.KIND["nop"])] * 40)
    out["flat"] = q.pack(0, iterations=0)
    return out


def program_fixture():
    """Wire format of packed programs from the reference's own monoserve/fabric/program.py."""
    sys.path.insert(0, REF)
    try:
        ref = importlib.import_module("monoserve.fabric.program")
    finally:
        sys.path.pop(0)
    out = {}
    for name, (tiles, stages, succ, first, reset, it) in program_spec(ref).items():
        out[name + "_tiles"] = tiles.numpy()
        out[name + "_stages"] = stages.numpy()
        out[name + "_succ"] = succ.numpy()
        out[name + "_meta"] = np.array([first, reset, it], dtype=np.int64)
    np.savez_compressed(os.path.join(HERE, "program_pack_reference.npz"), **out)
    print("program fixture written")


if __name__ == "__main__":
    if not REF or not os.path.isdir(REF):
        sys.exit("set MONOSERVE_REFERENCE to a checkout of the reference project to regenerate the fixtures")
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    qwen_fixture()
    glm_fixture()
    helper_fixture()
    program_fixture()
