"""The checkpoint loader on the CPU: tiny Qwen3-MoE and GLM-4.5-MoE (e4m3 with per-channel scales)
checkpoints are written in the Hugging Face layout (config.json, sharded .safetensors with an index),
read back through this library's own safetensors reader, and every expert must sit in its layer's
stack and every dense tensor under its role, bit for bit (the scenario of the reference's
tests/test_checkpoint.py:13-40, which needs vLLM and a GPU; this one needs neither)."""
import json
import os

import pytest
import torch

from monoserve_b200.checkpoint import checkpoint_files, read_checkpoint, safetensors_tensors, write_safetensors


def tiny_checkpoint(folder, glm):
    os.makedirs(folder, exist_ok=True)
    H, I, E, L, hq, hkv, V = 256, 128, 8, 3, 4, 2, 512
    dense = 1 if glm else 0
    cfg = {"model_type": "glm4_moe" if glm else "qwen3_moe", "hidden_size": H, "moe_intermediate_size": I,
           "num_experts_per_tok": 2, "num_hidden_layers": L, "num_attention_heads": hq, "num_key_value_heads": hkv,
           "head_dim": 128, "vocab_size": V, "rope_theta": 1e6, "rms_norm_eps": 1e-5}
    if glm:
        cfg.update(n_routed_experts=E, n_shared_experts=1, first_k_dense_replace=dense, intermediate_size=384,
                   partial_rotary_factor=0.5, attention_bias=True, routed_scaling_factor=1.5,
                   quantization_config={"quant_method": "compressed-tensors", "format": "float8"})
    else:
        cfg["num_experts"] = E
    json.dump(cfg, open(os.path.join(folder, "config.json"), "w"))
    g = torch.Generator().manual_seed(5)
    t = {}

    def lin(name, rows, cols):
        wt = torch.randn(rows, cols, generator=g) * 0.05
        if glm:
            s = (wt.abs().amax(-1, keepdim=True) / 448).clamp_min(1e-12)
            t[name + ".weight"] = (wt / s).to(torch.float8_e4m3fn)
            t[name + ".weight_scale"] = s.to(torch.bfloat16)
        else:
            t[name + ".weight"] = wt.to(torch.bfloat16)

    bf = lambda *shape: torch.randn(*shape, generator=g).to(torch.bfloat16)  # noqa: E731
    t["model.embed_tokens.weight"], t["lm_head.weight"], t["model.norm.weight"] = bf(V, H), bf(V, H), bf(H)
    for l in range(L):
        p = f"model.layers.{l}."
        t[p + "input_layernorm.weight"], t[p + "post_attention_layernorm.weight"] = bf(H), bf(H)
        for n, rows in (("q", hq * 128), ("k", hkv * 128), ("v", hkv * 128)):
            lin(p + f"self_attn.{n}_proj", rows, H)
            if glm:
                t[p + f"self_attn.{n}_proj.bias"] = bf(rows)
        if not glm:
            t[p + "self_attn.q_norm.weight"], t[p + "self_attn.k_norm.weight"] = bf(128), bf(128)
        lin(p + "self_attn.o_proj", H, hq * 128)
        if l < dense:
            lin(p + "mlp.gate_proj", 384, H), lin(p + "mlp.up_proj", 384, H), lin(p + "mlp.down_proj", H, 384)
            continue
        t[p + "mlp.gate.weight"] = bf(E, H)
        if glm:
            t[p + "mlp.gate.e_score_correction_bias"] = torch.randn(E, generator=g)
            lin(p + "mlp.shared_experts.gate_proj", I, H), lin(p + "mlp.shared_experts.up_proj", I, H)
            lin(p + "mlp.shared_experts.down_proj", H, I)
        for e in range(E):
            q = p + f"mlp.experts.{e}."
            lin(q + "gate_proj", I, H), lin(q + "up_proj", I, H), lin(q + "down_proj", H, I)
    names = sorted(t)
    shards = [names[0::2], names[1::2]]     # two shards, interleaved, so a layer's experts span both files
    weight_map = {}
    for i, part in enumerate(shards):
        fn = f"model-{i + 1:05d}-of-00002.safetensors"
        write_safetensors(os.path.join(folder, fn), {n: t[n] for n in part})
        weight_map.update({n: fn for n in part})
    json.dump({"weight_map": weight_map}, open(os.path.join(folder, "model.safetensors.index.json"), "w"))
    return t, cfg


@pytest.mark.parametrize("glm", [False, True])
def test_checkpoint_lands_in_the_stacks_bit_for_bit(tmp_path, glm):
    t, hf = tiny_checkpoint(str(tmp_path), glm)
    cfg, w = read_checkpoint(str(tmp_path), pin=False)
    assert (cfg.hidden, cfg.intermediate, cfg.num_experts, cfg.top_k, cfg.num_layers) == (256, 128, 8, 2, 3)
    assert cfg.fp8 == glm and cfg.dense_layers == (1 if glm else 0) and cfg.rotary_dim == (64 if glm else 128)
    I = cfg.intermediate
    raw = lambda x: x.view(torch.uint8) if x.dtype == torch.float8_e4m3fn else x  # noqa: E731
    for l in range(cfg.dense_layers, cfg.num_layers):
        p = f"model.layers.{l}."
        for e in range(cfg.num_experts):
            q = p + f"mlp.experts.{e}."
            assert torch.equal(w.host_w13[l][e, :I], raw(t[q + "gate_proj.weight"]))
            assert torch.equal(w.host_w13[l][e, I:], raw(t[q + "up_proj.weight"]))
            assert torch.equal(w.host_w2[l][e], raw(t[q + "down_proj.weight"]))
            if glm:
                assert torch.equal(w.w13_scale[l][e, :I], t[q + "gate_proj.weight_scale"].float().reshape(-1))
                assert torch.equal(w.w2_scale[l][e], t[q + "down_proj.weight_scale"].float().reshape(-1))
        assert torch.equal(w.router[l], t[p + "mlp.gate.weight"])
    for l in range(cfg.num_layers):
        p = f"model.layers.{l}."
        qkv = torch.cat([raw(t[p + f"self_attn.{n}_proj.weight"]) for n in "qkv"])
        got = w.qkv[l][0] if glm else w.qkv[l]
        assert torch.equal(got, qkv)
        if glm:
            assert torch.equal(w.qkv[l][1], torch.cat([t[p + f"self_attn.{n}_proj.weight_scale"].float().reshape(-1) for n in "qkv"]))
            assert torch.equal(w.qkv_bias[l], torch.cat([t[p + f"self_attn.{n}_proj.bias"] for n in "qkv"]))
    if glm:
        assert w.mlp_w13[0] is not None and w.host_w13[0] is None and w.shared_w13[1] is not None
        assert torch.equal(w.router_bias[1], t["model.layers.1.mlp.gate.e_score_correction_bias"])
    assert torch.equal(w.embed, t["model.embed_tokens.weight"]) and torch.equal(w.lm_head, t["lm_head.weight"])


def test_reader_rejects_truncated_and_unknown_tensors(tmp_path):
    path = str(tmp_path / "a.safetensors")
    write_safetensors(path, {"x": torch.arange(6, dtype=torch.int32).reshape(2, 3), "y": torch.ones(4, dtype=torch.bfloat16)})
    got = dict(safetensors_tensors(path))
    assert torch.equal(got["x"], torch.arange(6, dtype=torch.int32).reshape(2, 3)) and got["y"].dtype == torch.bfloat16
    assert checkpoint_files(str(tmp_path)) == [path]
    raw = bytearray(open(path, "rb").read())
    raw = raw.replace(b'"I32"', b'"Q99"')
    open(path, "wb").write(raw)
    with pytest.raises(ValueError, match="unsupported dtype"):
        list(safetensors_tensors(path))
    json.dump({"model_type": "llama"}, open(tmp_path / "config.json", "w"))
    with pytest.raises(NotImplementedError):
        read_checkpoint(str(tmp_path), pin=False)
    with pytest.raises(FileNotFoundError):
        checkpoint_files(str(tmp_path / "nowhere"))
