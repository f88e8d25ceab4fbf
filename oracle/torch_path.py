"""The reference's PyTorch MoE path, restated for the host CPU — TEST
INFRASTRUCTURE ONLY (checker for large shapes, and the timed CPU baseline).

The reference's own torch oracle is `reference_logits` in
tests/test_fabric_model.py:46-82 (Qwen3-style: softmax routing, q/k norm) and
tests/test_fabric_model_glm.py:34-68 (GLM-style: sigmoid routing with a
selection bias, routed scale, shared expert, dense first layers, partial
rotary, qkv bias, FP8 weights de-quantised to fp32).  Both hard-code
device="cuda" and take the reference's ModelWeights; here the same arithmetic is
split into per-operator functions over plain tensors on any device, with the
same rounding points (`bf` after every operator that stores bf16).

tests/golden/make_golden.py runs the reference's functions themselves on the
CPU and stores their outputs; tests/test_oracle_golden.py checks this file
against those fixtures.
"""
import torch
import torch.nn.functional as F


def bf(t):
    """Round to bf16, keep fp32 (tests/test_fabric_model.py:26-27)."""
    return t.to(torch.bfloat16).float()


def rms(x, w, eps):
    """RMSNorm with the reference's two roundings (tests/test_fabric_model.py:30-32)."""
    inv = torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    return bf(bf(x * inv) * w.float())


def rope(x, pos, theta, rot):
    """Neox rotary embedding on the first `rot` dims (tests/test_fabric_model.py:35-42)."""
    half = rot // 2
    j = torch.arange(half, device=x.device, dtype=torch.float32)
    inv = 1.0 / torch.pow(torch.tensor(theta, dtype=torch.float32, device=x.device), 2 * j / rot)
    ang = pos[:, None].float() * inv[None]
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    x1, x2 = x[..., :half], x[..., half:rot]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s, x[..., rot:]], -1)


def ffn(x, w13, w2):
    """SwiGLU expert: bf16-rounded hidden, fp32 output (tests/test_fabric_model_glm.py:29-31)."""
    width = w13.shape[0] // 2
    return bf(F.silu(x @ w13[:width].t()) * (x @ w13[width:].t())) @ w2.t()


def route(xn, router_w, top_k, scoring="softmax", bias=None, renorm=True, routed_scale=1.0):
    """Routing weights and ids (tests/test_fabric_model.py:67-69,
    tests/test_fabric_model_glm.py:57-60)."""
    logits = xn @ router_w.float().t()
    if scoring == "softmax":
        p = logits.softmax(-1)
        tw, ti = p.topk(top_k, -1)
    else:
        p = torch.sigmoid(logits)
        sel = p + bias.float() if bias is not None else p
        _, ti = sel.topk(top_k, -1)
        tw = p.gather(1, ti)
    if renorm:
        tw = tw / tw.sum(-1, keepdim=True)
    return tw * routed_scale, ti


def moe_layer(xn, x2, router_w, w13, w2, top_k, scoring="softmax", bias=None, renorm=True,
              routed_scale=1.0, shared=None, routing=None):
    """x = bf16(x2 + moe(xn)): the per-expert loop of tests/test_fabric_model.py:70-80.

    xn, x2: fp32 [T, H] holding bf16 values; w13 [E, 2I, H], w2 [E, H, I] in bf16
    (or fp32 de-quantised FP8), upcast per expert as the reference does.
    routing = (tw, ti) overrides the router (to check the expert path on given
    routing).  shared = (w13, w2) adds a shared expert as in the GLM variant."""
    T, H = xn.shape
    E = w13.shape[0]
    tw, ti = routing if routing is not None else route(xn, router_w, top_k, scoring, bias, renorm, routed_scale)
    moe = ffn(xn, shared[0].float(), shared[1].float()) if shared is not None else torch.zeros(T, H, device=xn.device)
    for e in range(E):
        rows, slot = (ti == e).nonzero(as_tuple=True)
        if len(rows) == 0:
            continue
        moe.index_add_(0, rows, tw[rows, slot][:, None] * ffn(xn[rows], w13[e].float(), w2[e].float()))
    base = x2 if x2 is not None else torch.zeros_like(moe)
    return bf(base + moe), tw, ti


def attention_dense(q, k, v, hq, hkv, D):
    """Causal GQA attention over one sequence, dense softmax
    (tests/test_fabric_model.py:60-64). q [n, hq, D], k/v [n, hkv, D] fp32."""
    n = q.shape[0]
    kk, vv = k.repeat_interleave(hq // hkv, 1), v.repeat_interleave(hq // hkv, 1)
    s = torch.einsum("qhd,khd->hqk", q, kk) / D ** 0.5
    s = s.masked_fill(torch.triu(torch.ones(n, n, device=q.device, dtype=torch.bool), 1)[None], float("-inf"))
    return bf(torch.einsum("hqk,khd->qhd", s.softmax(-1), vv)).reshape(n, hq * D)


@torch.no_grad()
def model_logits(w, cfg, tokens, device="cpu", gaps=None):
    """Whole-model logits with teacher forcing: the Qwen3-style reference oracle
    (tests/test_fabric_model.py:46-82).  `w` is any object with the attributes
    that function reads (embed, in_norm, qkv, q_norm, k_norm, o, post_norm, router,
    host_w13, host_w2, final_norm, lm_head).
    gaps (a list, optional) receives per layer the difference between the K-th and the K+1-th
    router logit of every row: how close each routing decision is to a tie."""
    L, Kt = cfg.num_layers, cfg.top_k
    hq, hkv, D = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
    n = len(tokens)
    tok = torch.tensor(tokens, device=device)
    pos = torch.arange(n, device=device)
    x = w.embed[tok].float()
    for l in range(L):
        xn = rms(x, w.in_norm[l], cfg.rms_eps)
        qkv = bf(xn @ w.qkv[l].float().t())
        q = qkv[:, :hq * D].view(n, hq, D)
        k = qkv[:, hq * D:(hq + hkv) * D].view(n, hkv, D)
        v = qkv[:, (hq + hkv) * D:].view(n, hkv, D)
        qn = bf(q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True) + cfg.rms_eps)) * w.q_norm[l].float()
        kn = bf(k * torch.rsqrt(k.pow(2).mean(-1, keepdim=True) + cfg.rms_eps)) * w.k_norm[l].float()
        q = bf(rope(qn, pos, cfg.rope_theta, cfg.rotary_dim))
        k = bf(rope(kn, pos, cfg.rope_theta, cfg.rotary_dim))
        ao = attention_dense(q, k, v, hq, hkv, D)
        x2 = bf(x + ao @ w.o[l].float().t())
        xn2 = rms(x2, w.post_norm[l], cfg.rms_eps)
        if gaps is not None:
            top = (xn2 @ w.router[l].float().t()).sort(-1, descending=True).values
            gaps.append(top[:, Kt - 1] - top[:, Kt])
        x, _, _ = moe_layer(xn2, x2, w.router[l], w.host_w13[l], w.host_w2[l], Kt)
    xn = rms(x, w.final_norm, cfg.rms_eps)
    return xn @ w.lm_head.float().t()


@torch.no_grad()
def model_logits_glm(w, cfg, tokens, device="cpu", gaps=None):
    """Whole-model logits of the GLM-4.5-style reference oracle (tests/test_fabric_model_glm.py:34-68):
    FP8 matrices de-quantised to fp32 (`w.dequantized(name, l)`, `w.expert_weights(l)`), qkv bias, rotary
    embedding on cfg.rotary_dim of each head and no head norm, dense FFN in the first cfg.dense_layers
    layers, then sigmoid routing with a selection bias, renormalised and scaled, plus a shared expert.
    gaps (a list, optional) receives per MoE layer the difference between the K-th and the K+1-th
    selection score of every row: how close each routing decision is to a tie."""
    L, Kt = cfg.num_layers, cfg.top_k
    hq, hkv, D = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
    n = len(tokens)
    pos = torch.arange(n, device=device)
    x = w.embed[torch.tensor(tokens, device=device)].float()
    for l in range(L):
        xn = rms(x, w.in_norm[l], cfg.rms_eps)
        qkv = bf(xn @ w.dequantized("qkv", l).t() + w.qkv_bias[l].float())
        q = bf(rope(qkv[:, :hq * D].view(n, hq, D), pos, cfg.rope_theta, cfg.rotary_dim))
        k = bf(rope(qkv[:, hq * D:(hq + hkv) * D].view(n, hkv, D), pos, cfg.rope_theta, cfg.rotary_dim))
        v = qkv[:, (hq + hkv) * D:].view(n, hkv, D)
        ao = attention_dense(q, k, v, hq, hkv, D)
        x2 = bf(x + ao @ w.dequantized("o", l).t())
        xn2 = rms(x2, w.post_norm[l], cfg.rms_eps)
        if l < cfg.dense_layers:
            x = bf(x2 + ffn(xn2, w.dequantized("mlp_w13", l), w.dequantized("mlp_w2", l)))
            continue
        w13, w2 = w.expert_weights(l)
        if gaps is not None:
            sel = torch.sigmoid(xn2 @ w.router[l].float().t()) + w.router_bias[l].float()
            top = sel.sort(-1, descending=True).values
            gaps.append(top[:, Kt - 1] - top[:, Kt])
        x, _, _ = moe_layer(xn2, x2, w.router[l], w13, w2, Kt, scoring="sigmoid", bias=w.router_bias[l], renorm=True,
                            routed_scale=cfg.routed_scale,
                            shared=(w.dequantized("shared_w13", l), w.dequantized("shared_w2", l)))
    return rms(x, w.final_norm, cfg.rms_eps) @ w.lm_head.float().t()


def quantize_fp8(w):
    """Per-output-channel e4m3 quantisation (monoserve/runtime/weights.py:218-229,
    tests/test_fabric_gemm.py:246-251): returns (raw bytes, fp32 scale per row,
    de-quantised fp32 weight)."""
    s = (w.float().abs().amax(dim=-1, keepdim=True) / 448.0).clamp_min(1e-12)
    q = (w.float() / s).to(torch.float8_e4m3fn)
    return q.view(torch.uint8).contiguous(), s.squeeze(-1).contiguous(), q.float() * s
