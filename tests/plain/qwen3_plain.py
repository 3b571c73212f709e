"""Plain, slow, whole-sequence Qwen3-dense forward pass on the CPU.

This is the oracle of the test-suite.  It shares no code with ``titan_b200``:
it reads ``config.json`` as a plain dict, takes weights as a dict of tensors by
their safetensors names, has no cache and no batching, and has one function per
part.  Every function restates a formula of berniehans/titan's CPU reference
bank (``engine/engine-core/src/forward_cpu.rs``); the cited lines are paths
inside that project.

berniehans/titan's model code is Rust and cannot be compiled here (no cargo),
so this file rests on the formulas.  The one piece of the reference that does
run here, its numpy forward in ``tools/build_synthetic_gguf.py``, is compared
with this file once in ``tests/golden/make_golden.py``.

All arithmetic is float32 with float64 reductions where the reference bank
uses them (norm sum of squares, attention scores, softmax and PV).
"""
from __future__ import annotations

import math

import torch

F32 = torch.float32
F64 = torch.float64


# --------------------------------------------------------------------------- #
# configuration (read straight from the config.json dict)
# --------------------------------------------------------------------------- #
def layer_windows(cfg: dict) -> list:
    """Per-layer attention window (None = all keys).

    berniehans/titan has full attention in every layer
    (forward_cpu.rs:445-507); the window is this architecture's own
    config.json option: ``layer_types[i] == "sliding_attention"`` or, without
    ``layer_types``, ``use_sliding_window`` with layers ``>= max_window_layers``
    windowed.
    """
    n = cfg["num_hidden_layers"]
    win = cfg.get("sliding_window")
    types = cfg.get("layer_types")
    if types is not None:
        return [win if t == "sliding_attention" else None for t in types]
    if cfg.get("use_sliding_window") and win is not None:
        first = cfg.get("max_window_layers", n)
        return [win if i >= first else None for i in range(n)]
    return [None] * n


def head_dim_of(cfg: dict) -> int:
    # engine-io/src/config.rs:119-120: key_length defaults to hidden / heads
    return cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]


# --------------------------------------------------------------------------- #
# parts
# --------------------------------------------------------------------------- #
def embed_lookup(table: torch.Tensor, tokens: torch.Tensor) -> torch.Tensor:
    """Row gather, no scale (forward_cpu.rs:144-159)."""
    assert int(tokens.max()) < table.shape[0] and int(tokens.min()) >= 0
    return table.to(F32)[tokens.long()]


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * 1/sqrt(mean(x^2) + eps) * w; eps inside the sqrt, float32
    squares summed in float64, weight used as stored (forward_cpu.rs:189-200)."""
    x = x.to(F32)
    sq = (x * x).to(F64).sum(dim=-1, keepdim=True)
    mean = (sq / x.shape[-1]).to(F32)
    scale = 1.0 / torch.sqrt(mean + torch.tensor(eps, dtype=F32))
    return x * scale * w.to(F32)


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """y = x . W^T with W [out, in], no bias (forward_cpu.rs:165-184).  The
    sum runs in float64 and is rounded once, so that the oracle is not itself a
    source of float32 reduction-order noise."""
    return (x.to(F64) @ w.to(F64).t()).to(F32)


def rope_neox(x: torch.Tensor, pos: torch.Tensor, theta_base: float) -> torch.Tensor:
    """Half-split rotary over the whole head (forward_cpu.rs:226-241; n_rot =
    head_dim, forward_driver.rs:608).  x: [T, heads, hd], pos: [T].
    theta_k = pos * base^(-2k/hd); pairs (k, k + hd/2)."""
    hd = x.shape[-1]
    half = hd // 2
    k = torch.arange(half, dtype=F64)
    inv_freq = torch.tensor(theta_base, dtype=F64) ** (-2.0 * k / hd)
    ang = pos.to(F64)[:, None] * inv_freq[None, :]          # [T, half]
    c = torch.cos(ang).to(F32)[:, None, :]
    s = torch.sin(ang).to(F32)[:, None, :]
    x = x.to(F32)
    x0, x1 = x[..., :half], x[..., half:]
    return torch.cat([x0 * c - x1 * s, x0 * s + x1 * c], dim=-1)


def causal_attention(q, k, v, window=None) -> torch.Tensor:
    """q [T, nh, hd], k/v [T, nkv, hd] of ONE sequence, positions 0..T-1.
    Query head qh uses kv head qh // (nh/nkv); score = q.k / sqrt(hd); keys
    t <= query position; softmax with max subtraction; float64 throughout
    (forward_cpu.rs:440-507).  ``window``: keys with p - window < t <= p."""
    T, nh, hd = q.shape
    nkv = k.shape[1]
    assert nh % nkv == 0
    group = nh // nkv
    out = torch.zeros(T, nh, hd, dtype=F32)
    scale = 1.0 / math.sqrt(hd)
    idx = torch.arange(T)
    allowed = idx[None, :] <= idx[:, None]
    if window is not None:
        allowed &= idx[None, :] > (idx[:, None] - window)
    for h in range(nh):
        kh = h // group
        s = (q[:, h].to(F64) @ k[:, kh].to(F64).t()) * scale     # [T, T]
        s = s.masked_fill(~allowed, float("-inf"))
        s = s - s.max(dim=-1, keepdim=True).values
        p = torch.exp(s)
        p = p / p.sum(dim=-1, keepdim=True)
        out[:, h] = (p @ v[:, kh].to(F64)).to(F32)
    return out


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """silu(g) * u with silu(g) = g / (1 + exp(-g)) (forward_cpu.rs:210-219)."""
    g = gate.to(F32)
    return g / (1.0 + torch.exp(-g)) * up.to(F32)


# --------------------------------------------------------------------------- #
# arrangement
# --------------------------------------------------------------------------- #
def attention_part(cfg, w, prefix, xn, pos, window):
    """QKV -> per-head RMSNorm on Q and K (same eps, before the rotation) ->
    rotary on Q and K -> causal GQA attention -> output projection
    (forward_cpu.rs:300-366)."""
    nh, nkv = cfg["num_attention_heads"], cfg.get("num_key_value_heads") or cfg["num_attention_heads"]
    hd = head_dim_of(cfg)
    eps = cfg.get("rms_norm_eps", 1e-5)          # engine-io/src/config.rs:31
    theta = cfg.get("rope_theta", 10000.0)       # engine-io/src/config.rs:29
    T = xn.shape[0]
    q = linear(xn, w[prefix + "self_attn.q_proj.weight"]).view(T, nh, hd)
    k = linear(xn, w[prefix + "self_attn.k_proj.weight"]).view(T, nkv, hd)
    v = linear(xn, w[prefix + "self_attn.v_proj.weight"]).view(T, nkv, hd)
    q = rms_norm(q, w[prefix + "self_attn.q_norm.weight"], eps)
    k = rms_norm(k, w[prefix + "self_attn.k_norm.weight"], eps)
    q = rope_neox(q, pos, theta)
    k = rope_neox(k, pos, theta)
    a = causal_attention(q, k, v, window).reshape(T, nh * hd)
    return linear(a, w[prefix + "self_attn.o_proj.weight"])


def mlp_part(w, prefix, xn):
    """down(silu(gate(x)) * up(x)) (forward_cpu.rs:369-386)."""
    g = linear(xn, w[prefix + "mlp.gate_proj.weight"])
    u = linear(xn, w[prefix + "mlp.up_proj.weight"])
    return linear(swiglu(g, u), w[prefix + "mlp.down_proj.weight"])


def block(cfg, w, i, x, pos, window):
    """x -> norm -> attention -> +x -> norm -> MLP -> + (forward_cpu.rs:281-386)."""
    eps = cfg.get("rms_norm_eps", 1e-5)
    p = f"model.layers.{i}."
    h1 = x + attention_part(cfg, w, p, rms_norm(x, w[p + "input_layernorm.weight"], eps), pos, window)
    return h1 + mlp_part(w, p, rms_norm(h1, w[p + "post_attention_layernorm.weight"], eps))


def forward_logits(cfg: dict, w: dict, tokens) -> torch.Tensor:
    """Logits [T, vocab] at every position of ONE whole sequence.  Final
    RMSNorm, then the LM head, which is the embedding when tied
    (forward_cpu.rs:390-395, forward_driver.rs:621-625)."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    pos = torch.arange(tokens.shape[0])
    x = embed_lookup(w["model.embed_tokens.weight"], tokens)
    wins = layer_windows(cfg)
    for i in range(cfg["num_hidden_layers"]):
        x = block(cfg, w, i, x, pos, wins[i])
    xn = rms_norm(x, w["model.norm.weight"], cfg.get("rms_norm_eps", 1e-5))
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings") else w["lm_head.weight"]
    return linear(xn, head)


# --------------------------------------------------------------------------- #
# sampling
# --------------------------------------------------------------------------- #
MASK64 = (1 << 64) - 1


def uniform_draw(seed: int, sequence: int, step: int) -> float:
    """Counter-based uniform in [0, 1) with 24 bits, one value per
    (seed, sequence, step).  berniehans/titan draws ``(x >> 40) / 2^24`` from a
    xorshift stream per request (sampler.rs:62-82); a stream cannot be
    independent of batching, so the stream is replaced by a hash (splitmix64
    finaliser) of the three counters; the 24-bit mapping is kept."""
    z = (seed * 0x9E3779B97F4A7C15 + sequence * 0xBF58476D1CE4E5B9 + step * 0x94D049BB133111EB + 0x2545F4914F6CDD1D) & MASK64
    for _ in range(2):
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK64
        z = z ^ (z >> 31)
    return (z >> 40) / float(1 << 24)


def sample(logits, context, temperature=0.0, top_k=0, top_p=1.0, repetition_penalty=1.0, u=0.0) -> int:
    """One token from one row of logits, after sampler.rs:109-240:
    repetition penalty over the distinct context tokens (positive logit / pen,
    else * pen, 132-145); temperature <= 1e-4 -> argmax, lowest index on ties
    (148-158, 351-361); else logits / T (161-164), keep the top_k largest
    (167-177), softmax with max subtraction (184-200), keep the shortest
    descending prefix whose mass reaches top_p and renormalise (203-226), draw
    the first index whose running sum reaches ``u`` (229-239).

    Two stated differences: top_k = 0 keeps the whole vocabulary (the
    reference silently keeps 1024), and the running sum of the draw runs in
    vocabulary order, not in descending-probability order (same distribution;
    no sort on the device).  Ties at the top_k / top_p boundary keep the lower
    index."""
    x = torch.as_tensor(logits, dtype=F32).clone()
    V = x.shape[0]
    if repetition_penalty > 1.0 and len(context):
        for t in set(int(c) for c in context):
            if t < V:
                x[t] = x[t] / repetition_penalty if x[t] > 0 else x[t] * repetition_penalty
    if temperature <= 1e-4:
        return int(torch.argmax(x))          # torch.argmax returns the first maximum
    x = x * torch.tensor(1.0 / temperature, dtype=F32)
    keep = torch.ones(V, dtype=torch.bool)
    order = sorted(range(V), key=lambda i: (-float(x[i]), i))
    if 0 < top_k < V:
        keep[:] = False
        keep[order[:top_k]] = True
    p = torch.where(keep, torch.exp(x - x[keep].max()), torch.zeros(()))
    p = p / p.sum()
    if top_p < 1.0:
        run, kept = 0.0, []
        for i in order:
            if not keep[i]:
                continue
            kept.append(i)
            run += float(p[i])
            if run >= top_p:
                break
        keep[:] = False
        keep[kept] = True
        p = torch.where(keep, p, torch.zeros(()))
        p = p / p.sum()
    target = u * float(p.sum())
    run = 0.0
    last = 0
    for i in range(V):
        if keep[i]:
            run += float(p[i])
            last = i
            if run > target:
                return i
    return last
