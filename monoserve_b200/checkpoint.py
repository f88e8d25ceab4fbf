"""Load a Hugging Face MoE checkpoint into this library's weight layout: the role of the reference's
monoserve/runtime/checkpoint.py:99-196.  Every layer's routed experts are stacked, as their tensors
stream by, into one pinned host tensor per projection (w13 = [gate; up] as [E, 2I, H], w2 as
[E, H, I]); everything else is kept by name and handed to `ModelWeights`, which places the dense
tensors and the hot tier in HBM.  Supported: Qwen3-MoE (bf16) and GLM-4.5 MoE (bf16, or e4m3 with one
fp32 scale per output channel, the compressed-tensors layout).

The reference streams through vLLM's weight iterator; here the safetensors files are read directly
(the format is an 8-byte little-endian header length, a JSON header {name: {dtype, shape,
data_offsets}}, then the raw tensors), so nothing but torch and numpy is needed, and the model's
shape comes from the checkpoint's config.json.

    cfg, w = read_checkpoint(folder)                 # cfg: the model shape; w: tensors by role
    weights = ModelWeights(cfg, w, hot=hot)          # monoserve_b200/model.py
"""
import glob
import json
import mmap
import os
import re
import struct
import types
import warnings

import numpy as np
import torch

_DTYPES = {"BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2), "F32": (torch.float32, 4), "F64": (torch.float64, 8),
           "F8_E4M3": (torch.float8_e4m3fn, 1), "I64": (torch.int64, 8), "I32": (torch.int32, 4), "I16": (torch.int16, 2),
           "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1)}
_EXPERT = re.compile(r"model\.layers\.(\d+)\.mlp\.experts\.(\d+)\.(gate|up|down)_proj\.(weight|weight_scale)$")


def safetensors_tensors(path):
    """Yield (name, tensor) for every tensor of one .safetensors file, in file order.  The tensors
    are views of a read-only mapping of the file: copy what must outlive the iteration."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
    base = 8 + n
    raw = np.frombuffer(mm, dtype=np.uint8)
    entries = [(k, v) for k, v in header.items() if k != "__metadata__"]
    for name, meta in sorted(entries, key=lambda kv: kv[1]["data_offsets"][0]):
        if meta["dtype"] not in _DTYPES:
            raise ValueError(f"{path}: tensor {name} has unsupported dtype {meta['dtype']}")
        dt, size = _DTYPES[meta["dtype"]]
        lo, hi = meta["data_offsets"]
        count = int(np.prod(meta["shape"])) if meta["shape"] else 1
        if hi - lo != count * size:
            raise ValueError(f"{path}: tensor {name} spans {hi - lo} bytes, its shape needs {count * size}")
        with warnings.catch_warnings():   # the mapping is read-only on purpose; nothing here writes through the view
            warnings.simplefilter("ignore", UserWarning)
            t = torch.from_numpy(raw[base + lo:base + hi])
        yield name, t.view(dt).reshape(meta["shape"])


def checkpoint_files(folder):
    """The .safetensors files of a checkpoint directory: those its index names, else all of them."""
    index = os.path.join(folder, "model.safetensors.index.json")
    if os.path.exists(index):
        with open(index) as f:
            names = sorted(set(json.load(f)["weight_map"].values()))
        return [os.path.join(folder, n) for n in names]
    files = sorted(glob.glob(os.path.join(folder, "*.safetensors")))
    if not files:
        raise FileNotFoundError(f"no .safetensors files in {folder}")
    return files


def model_config(folder):
    """The model shape from config.json, with the attribute names the rest of this library uses
    (monoserve/runtime/config.py:46-66 makes the same translation from the Hugging Face config)."""
    with open(os.path.join(folder, "config.json")) as f:
        c = json.load(f)
    kind = c.get("model_type")
    if kind not in ("qwen3_moe", "glm4_moe"):
        raise NotImplementedError(f"model type {kind}")
    head_dim = c.get("head_dim") or c["hidden_size"] // c["num_attention_heads"]
    cfg = types.SimpleNamespace(
        model_type=kind, hidden=c["hidden_size"], intermediate=c["moe_intermediate_size"],
        num_experts=c.get("num_experts") or c.get("n_routed_experts"), top_k=c["num_experts_per_tok"],
        num_layers=c["num_hidden_layers"], num_heads=c["num_attention_heads"], num_kv_heads=c["num_key_value_heads"],
        head_dim=head_dim, vocab=c["vocab_size"], rope_theta=float(c.get("rope_theta", 1e6)),
        rms_eps=float(c.get("rms_norm_eps", 1e-6)), rotary_dim=int(head_dim * c.get("partial_rotary_factor", 1.0)),
        scoring="softmax", routed_scale=1.0, dense_layers=0, dense_intermediate=0, shared_intermediate=0,
        qk_norm=True, qkv_bias=False, fp8=False)
    if kind == "glm4_moe":
        cfg.scoring, cfg.routed_scale = "sigmoid", float(c.get("routed_scaling_factor", 1.0))
        cfg.dense_layers, cfg.dense_intermediate = c.get("first_k_dense_replace", 0), c.get("intermediate_size", 0)
        cfg.shared_intermediate = c.get("n_shared_experts", 0) * c["moe_intermediate_size"]
        cfg.qk_norm, cfg.qkv_bias = bool(c.get("use_qk_norm", False)), bool(c.get("attention_bias", False))
        q = c.get("quantization_config") or {}
        cfg.fp8 = "float8" in json.dumps(q) or q.get("quant_method") == "fp8"
    if cfg.head_dim != 128:
        raise NotImplementedError("the attention kernels of this library are built for head_dim 128")
    return cfg


class _ExpertStacks:
    """Pinned per-layer stacks that the routed experts are copied into as they stream by."""

    def __init__(self, cfg, layers, fp8, pin):
        E, I, H = cfg.num_experts, cfg.intermediate, cfg.hidden
        dt = torch.uint8 if fp8 else torch.bfloat16
        self.I, self.layers = I, set(layers)
        self.w13 = {l: torch.empty(E, 2 * I, H, dtype=dt, pin_memory=pin) for l in self.layers}
        self.w2 = {l: torch.empty(E, H, I, dtype=dt, pin_memory=pin) for l in self.layers}
        self.s13 = {l: torch.empty(E, 2 * I) for l in self.layers} if fp8 else None
        self.s2 = {l: torch.empty(E, H) for l in self.layers} if fp8 else None
        self.expected = len(self.layers) * E * 3 * (2 if fp8 else 1)
        self.seen = 0

    def take(self, layer, expert, proj, kind, t):
        if layer not in self.layers:   # dense leading layers have none; a next-token-prediction layer is skipped
            return
        I = self.I
        if kind == "weight":
            dst = {"gate": self.w13[layer][expert, :I], "up": self.w13[layer][expert, I:], "down": self.w2[layer][expert]}[proj]
            dst.copy_(t.view(torch.uint8) if dst.dtype == torch.uint8 else t)
        elif self.s13 is not None:
            dst = {"gate": self.s13[layer][expert, :I], "up": self.s13[layer][expert, I:], "down": self.s2[layer][expert]}[proj]
            dst.copy_(t.float().reshape(-1))
        else:
            return
        self.seen += 1


def read_checkpoint(folder, pin=True, log=None):
    """(cfg, w): the model shape and an object with the tensors by role, as `ModelWeights` takes them.
    pin=False keeps the expert stacks in pageable memory (for machines without a CUDA driver)."""
    cfg = model_config(folder)
    L, glm = cfg.num_layers, cfg.model_type == "glm4_moe"
    stacks = _ExpertStacks(cfg, range(cfg.dense_layers, L), cfg.fp8, pin)
    named = {}
    for path in checkpoint_files(folder):
        for name, t in safetensors_tensors(path):
            m = _EXPERT.match(name)
            if m:
                stacks.take(int(m[1]), int(m[2]), m[3], m[4], t)
            else:
                named[name] = t.clone()
        if log:
            log(f"read {os.path.basename(path)}: {stacks.seen} of {stacks.expected} expert tensors")
    if stacks.seen != stacks.expected:
        raise ValueError(f"the checkpoint holds {stacks.seen} of {stacks.expected} expert tensors")

    def linear(name):
        """A linear layer: its bf16 weight, or (e4m3 bytes, fp32 scale per output row)."""
        wt = named[name + ".weight"]
        if name + ".weight_scale" in named:
            return wt.view(torch.uint8), named[name + ".weight_scale"].float().reshape(-1)
        return wt

    def stacked(names):
        parts = [linear(n) for n in names]
        if isinstance(parts[0], tuple):
            return torch.cat([p[0] for p in parts]), torch.cat([p[1] for p in parts])
        return torch.cat(parts)

    w = types.SimpleNamespace(embed=named["model.embed_tokens.weight"], final_norm=named["model.norm.weight"])
    w.lm_head = named.get("lm_head.weight", w.embed)
    per_layer = ("in_norm", "post_norm", "qkv", "qkv_bias", "q_norm", "k_norm", "o", "router", "router_bias", "shared_w13",
                 "shared_w2", "mlp_w13", "mlp_w2", "host_w13", "host_w2", "w13_scale", "w2_scale")
    for name in per_layer:
        setattr(w, name, [None] * L)
    for l in range(L):
        p = f"model.layers.{l}."
        w.in_norm[l], w.post_norm[l] = named[p + "input_layernorm.weight"], named[p + "post_attention_layernorm.weight"]
        w.qkv[l] = stacked([p + f"self_attn.{n}_proj" for n in "qkv"])
        if cfg.qkv_bias:
            w.qkv_bias[l] = torch.cat([named[p + f"self_attn.{n}_proj.bias"] for n in "qkv"])
        if p + "self_attn.q_norm.weight" in named:
            w.q_norm[l], w.k_norm[l] = named[p + "self_attn.q_norm.weight"], named[p + "self_attn.k_norm.weight"]
        w.o[l] = linear(p + "self_attn.o_proj")
        if l < cfg.dense_layers:
            w.mlp_w13[l] = stacked([p + "mlp.gate_proj", p + "mlp.up_proj"])
            w.mlp_w2[l] = linear(p + "mlp.down_proj")
            continue
        w.router[l] = named[p + "mlp.gate.weight"]
        if glm:
            w.router_bias[l] = named[p + "mlp.gate.e_score_correction_bias"].float()
            if cfg.shared_intermediate:
                w.shared_w13[l] = stacked([p + "mlp.shared_experts.gate_proj", p + "mlp.shared_experts.up_proj"])
                w.shared_w2[l] = linear(p + "mlp.shared_experts.down_proj")
        w.host_w13[l], w.host_w2[l] = stacks.w13[l], stacks.w2[l]
        if stacks.s13 is not None:
            w.w13_scale[l], w.w2_scale[l] = stacks.s13[l], stacks.s2[l]
    return cfg, w


def write_safetensors(path, tensors):
    """Write {name: tensor} as one .safetensors file (for tests and for exporting synthetic weights)."""
    names = {v[0]: k for k, v in _DTYPES.items()}
    header, blobs, at = {}, [], 0
    for name, t in tensors.items():
        t = t.contiguous()
        data = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": names[t.dtype], "shape": list(t.shape), "data_offsets": [at, at + len(data)]}
        blobs.append(data)
        at += len(data)
    head = json.dumps(header, separators=(",", ":")).encode()
    head += b" " * (-len(head) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(head)))
        f.write(head)
        for b in blobs:
            f.write(b)
