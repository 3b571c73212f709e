"""Shared by the tests: tiny configurations, random weights made by the tests themselves
(not by the library's random mode), model folders in temporary directories, and error norms."""
from __future__ import annotations

import json
import os

import torch

# Two tiny configurations that differ in every size and option, and a third with a window.
TINY_A = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, hidden_size=64,
              num_attention_heads=4, num_key_value_heads=2, head_dim=16, intermediate_size=128, vocab_size=256,
              rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=4096,
              hidden_act="silu", eos_token_id=7)
TINY_B = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=3, hidden_size=96,
              num_attention_heads=6, num_key_value_heads=3, head_dim=32, intermediate_size=224, vocab_size=509,
              rope_theta=1000000.0, rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=2048,
              hidden_act="silu")
TINY_C = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=4, hidden_size=80,
              num_attention_heads=5, num_key_value_heads=1, head_dim=48, intermediate_size=176, vocab_size=1000,
              rope_theta=500000.0, rms_norm_eps=3e-6, tie_word_embeddings=False, max_position_embeddings=1024,
              hidden_act="silu", sliding_window=20,
              layer_types=["sliding_attention", "full_attention", "sliding_attention", "sliding_attention"])
TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C}


def weight_names(cfg):
    """(name, shape, is_norm) of every tensor of a Qwen3 dense checkpoint."""
    H, F, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    hd = cfg.get("head_dim") or H // cfg["num_attention_heads"]
    Q, KV = cfg["num_attention_heads"] * hd, cfg["num_key_value_heads"] * hd
    out = [("model.embed_tokens.weight", (V, H), False)]
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        out += [(p + "input_layernorm.weight", (H,), True),
                (p + "self_attn.q_proj.weight", (Q, H), False), (p + "self_attn.k_proj.weight", (KV, H), False),
                (p + "self_attn.v_proj.weight", (KV, H), False), (p + "self_attn.o_proj.weight", (H, Q), False),
                (p + "self_attn.q_norm.weight", (hd,), True), (p + "self_attn.k_norm.weight", (hd,), True),
                (p + "post_attention_layernorm.weight", (H,), True),
                (p + "mlp.gate_proj.weight", (F, H), False), (p + "mlp.up_proj.weight", (F, H), False),
                (p + "mlp.down_proj.weight", (H, F), False)]
    out.append(("model.norm.weight", (H,), True))
    if not cfg.get("tie_word_embeddings"):
        out.append(("lm_head.weight", (V, H), False))
    return out


def random_weights(cfg, seed, dtype=torch.bfloat16, std=0.02, norm_std=0.1):
    """Matrices ~ N(0, std), norm weights 1 + N(0, norm_std), rounded to ``dtype`` (as a file holds them)."""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, shape, is_norm in weight_names(cfg):
        t = torch.randn(shape, generator=g) * (norm_std if is_norm else std) + (1.0 if is_norm else 0.0)
        w[name] = t.to(dtype)
    return w


def write_folder(folder, cfg, weights):
    from titan_b200.weights import write_safetensors
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    names = list(weights)
    write_safetensors(os.path.join(folder, "model.safetensors"),
                      [(n, tuple(weights[n].shape), weights[n].dtype) for n in names], lambda n: weights[n])
    return folder


def random_tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def rel_l2(a, b):
    a, b = a.double().flatten(), b.double().flatten()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


# Bounds, fixed before the first run on a GPU.  float32: the engine differs from the plain
# implementation by summation order only.  bfloat16: activations are rounded to 8 bits of mantissa
# (2^-9 relative) at every part's output.
TOL = {"float32": 5e-5, "bfloat16": 3e-2}


def rows_close(got, want, dtype, what="", row_factor=4.0):
    """The whole tensor within the bound, and every row within ``row_factor`` times the bound: one wrong row
    among a thousand right ones does not hide in the tensor's norm."""
    got, want = got.float().cpu(), want.float().cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} instead of {tuple(want.shape)}"
    err = rel_l2(got, want)
    assert err < TOL[dtype], f"{what}: relative error {err:.3e} over the bound {TOL[dtype]:.0e}"
    g, w = got.double().reshape(-1, got.shape[-1]), want.double().reshape(-1, want.shape[-1])
    per_row = (g - w).norm(dim=1) / w.norm(dim=1).clamp_min(1e-30)
    worst = int(per_row.argmax())
    assert float(per_row[worst]) < row_factor * TOL[dtype], \
        f"{what}: row {worst} of {g.shape[0]} is off by {float(per_row[worst]):.3e} (bound {row_factor * TOL[dtype]:.0e})"


# Mid-size models whose head sizes take the tensor-core attention kernels (the kernels that serving runs).
MID = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, hidden_size=1024,
           num_attention_heads=8, num_key_value_heads=2, head_dim=128, intermediate_size=2816, vocab_size=5000,
           rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=4096)
MID64 = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, hidden_size=512,
             num_attention_heads=16, num_key_value_heads=8, head_dim=64, intermediate_size=1408, vocab_size=3000,
             rope_theta=10000.0, rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=2048)
