#!/usr/bin/env python3
"""Compares the plain implementation (tests/plain/qwen3_plain.py) with the one piece of
berniehans/titan's model code that runs here on the CPU: the numpy forward of
``tools/build_synthetic_gguf.py`` (its Rust crates cannot be built: no cargo in this image).

    python tests/golden/make_golden.py /path/to/berniehans-titan  ->  tests/golden/reference_numpy.json

What is written: (1) outputs of the reference's ``rms_norm`` (:318-331), ``matmul_q``
(:334-342) and ``softmax_1`` (:345-350) on seeded random inputs, which the test-suite
recomputes with the plain functions; (2) the reference's whole forward (:353-409) of its
synthetic model (hidden 256, 2 query heads, 1 kv head, head_dim 128, ffn 256, vocab 16, eps
1e-5, theta 1e6, tied head; one token at position 0) next to the plain implementation's
logits for the same dequantised weights.  That model is one token at position 0 with a zero
down projection, so rotation at later positions, softmax over several keys, head grouping and
the MLP's contribution rest on the formulas alone.
"""
import importlib.util
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, ".."))
from plain import qwen3_plain as P  # noqa: E402


def load_reference(root):
    spec = importlib.util.spec_from_file_location("titan_synth", os.path.join(root, "tools", "build_synthetic_gguf.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def op_inputs():
    rng = np.random.default_rng(20240601)
    return {"x": rng.standard_normal(96).astype(np.float32), "w": (1 + 0.1 * rng.standard_normal(96)).astype(np.float32),
            "m": (0.05 * rng.standard_normal((24, 96))).astype(np.float32), "s": (3 * rng.standard_normal(17)).astype(np.float32)}


def plain_whole_forward(R):
    tensors = R.parse_tensor_section(R.build_gguf(R.TENSOR_DEFS), R.TENSOR_DEFS)
    deq = lambda n: torch.from_numpy(np.array(R.dequant_tensor(*tensors[n]), dtype=np.float32))
    vec = lambda n: torch.from_numpy(np.frombuffer(tensors[n][2], dtype="<f4").astype(np.float32))
    names = {"attn_q": "self_attn.q_proj", "attn_k": "self_attn.k_proj", "attn_v": "self_attn.v_proj",
             "attn_output": "self_attn.o_proj", "ffn_gate": "mlp.gate_proj", "ffn_up": "mlp.up_proj", "ffn_down": "mlp.down_proj"}
    w = {"model.embed_tokens.weight": deq("token_embd.weight"), "model.norm.weight": vec("output_norm.weight")}
    for g, h in names.items():
        w[f"model.layers.0.{h}.weight"] = deq(f"blk.0.{g}.weight")
    for g, h in {"attn_norm": "input_layernorm", "ffn_norm": "post_attention_layernorm",
                 "attn_q_norm": "self_attn.q_norm", "attn_k_norm": "self_attn.k_norm"}.items():
        w[f"model.layers.0.{h}.weight"] = vec(f"blk.0.{g}.weight")
    cfg = dict(num_hidden_layers=1, hidden_size=R.H, num_attention_heads=R.N_HEAD, num_key_value_heads=R.N_KV,
               head_dim=R.HEAD_DIM, intermediate_size=R.FFN, vocab_size=R.VOCAB, rms_norm_eps=R.EPS,
               rope_theta=R.FREQ_BASE, tie_word_embeddings=True)
    ref = R.reference_forward(tensors)
    mine = P.forward_logits(cfg, w, [R.TOKEN_ID])[0]
    return ref, mine


def main(root):
    R = load_reference(root)
    i = op_inputs()
    ref, mine = plain_whole_forward(R)
    out = {
        "source": "berniehans/titan tools/build_synthetic_gguf.py: rms_norm :318-331, matmul_q :334-342, softmax_1 :345-350, reference_forward :353-409",
        "inputs": "numpy default_rng(20240601): x, w [96], m [24,96], s [17] (see op_inputs in make_golden.py)",
        "rms_norm_eps": 1e-5,
        "rms_norm": [float(v) for v in R.rms_norm(i["x"], i["w"], 1e-5)],
        "matmul_q": [float(v) for v in R.matmul_q(i["m"], i["x"])],
        "softmax_1": [float(v) for v in R.softmax_1(i["s"])],
        "whole_forward_reference_logits": ref["logits"],
        "whole_forward_plain_logits": [float(v) for v in mine],
    }
    with open(os.path.join(HERE, "reference_numpy.json"), "w") as f:
        json.dump(out, f, indent=1)
    d = np.abs(np.array(ref["logits"]) - mine.numpy()).max()
    print(f"whole forward: max |reference - plain| = {d:.3e} over logits of magnitude {np.abs(ref['logits']).max():.3f}")


def reference_dir():
    """Where the reference's checkout is looked for: ``TITAN_REFERENCE_DIR``, else a folder ``reference``
    beside this repository."""
    return os.environ.get("TITAN_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(HERE))), "reference")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else reference_dir())
