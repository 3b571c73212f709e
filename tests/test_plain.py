"""The plain implementation itself: hand-computed cases in the manner of berniehans/titan's
engine/engine-core/tests/forward_cpu_tests.rs:22-150, and the committed outputs of the
reference's numpy functions (tests/golden/reference_numpy.json).  No GPU."""
import json
import math
import os

import numpy as np
import pytest
import torch

from golden.make_golden import op_inputs, reference_dir
from helpers import TINY_A, TINY_C, random_tokens, random_weights
from plain import qwen3_plain as P

GOLD = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_numpy.json")))


def test_rms_norm_eps_inside_the_sqrt():
    x, w = torch.tensor([3.0, 4.0]), torch.tensor([1.0, 2.0])
    s = 1 / math.sqrt(12.5 + 0.5)
    assert torch.allclose(P.rms_norm(x, w, 0.5), torch.tensor([3 * s, 8 * s]), atol=1e-7)


def test_rope_identity_at_zero_and_pairs_across_halves():
    x = torch.arange(1.0, 9.0).view(1, 1, 8)
    assert torch.equal(P.rope_neox(x, torch.tensor([0]), 10000.0), x)
    y = P.rope_neox(x, torch.tensor([1]), 10000.0)[0, 0]
    c, s = math.cos(1.0), math.sin(1.0)                  # k = 0: angle = pos * base^0
    assert abs(float(y[0]) - (1 * c - 5 * s)) < 1e-6 and abs(float(y[4]) - (1 * s + 5 * c)) < 1e-6
    a = 10000.0 ** (-2 * 3 / 8)
    assert abs(float(y[3]) - (4 * math.cos(a) - 8 * math.sin(a))) < 1e-6


def test_silu_and_swiglu():
    g, u = torch.tensor([0.0, 1.0, -2.0]), torch.tensor([5.0, 2.0, 3.0])
    want = [0.0, 1 / (1 + math.exp(-1)) * 2, -2 / (1 + math.exp(2)) * 3]
    assert torch.allclose(P.swiglu(g, u), torch.tensor(want), atol=1e-7)


def test_attention_is_causal_grouped_and_windowed():
    torch.manual_seed(0)
    q, k, v = torch.randn(5, 4, 8), torch.randn(5, 2, 8), torch.randn(5, 2, 8)
    out = P.causal_attention(q, k, v)
    assert torch.allclose(out[0, :2], v[0, 0].expand(2, 8)) and torch.allclose(out[0, 2:], v[0, 1].expand(2, 8))
    s = (q[3, 3] @ k[:4, 1].t()) / math.sqrt(8)
    assert torch.allclose(out[3, 3], torch.softmax(s, 0) @ v[:4, 1], atol=1e-6)
    k2, v2 = k.clone(), v.clone()
    k2[4], v2[4] = 100.0, 100.0                          # the future does not leak
    assert torch.equal(P.causal_attention(q, k2, v2)[:4], out[:4])
    w = P.causal_attention(q, k, v, window=2)
    s = (q[4, 0] @ k[3:5, 0].t()) / math.sqrt(8)
    assert torch.allclose(w[4, 0], torch.softmax(s, 0) @ v[3:5, 0], atol=1e-6)
    assert torch.allclose(P.causal_attention(q, k, v, window=5), out)


def test_against_the_references_numpy_functions():
    i = {k: torch.from_numpy(v) for k, v in op_inputs().items()}
    assert np.allclose(P.rms_norm(i["x"], i["w"], GOLD["rms_norm_eps"]).numpy(), GOLD["rms_norm"], rtol=2e-7, atol=0)
    assert np.allclose(P.linear(i["x"][None], i["m"])[0].numpy(), GOLD["matmul_q"], rtol=0, atol=2e-6)
    # softmax: the plain implementation's own max-subtract / exp / normalise code, inside its attention.  One query
    # over 17 keys whose scores are the golden inputs (q = 5 e_0, k_t = s_t e_0, head_dim 25 so that the scale is
    # 1/5), values one-hot: the output row is the softmax itself.
    T, hd = 17, 25
    q, k, v = torch.zeros(T, 1, hd), torch.zeros(T, 1, hd), torch.zeros(T, 1, hd)
    q[:, 0, 0] = 5.0
    k[:, 0, 0] = i["s"]
    v[torch.arange(T), 0, torch.arange(T)] = 1.0
    assert np.allclose(P.causal_attention(q, k, v)[T - 1, 0, :T].numpy(), GOLD["softmax_1"], rtol=2e-6, atol=1e-9)
    ref, mine = np.array(GOLD["whole_forward_reference_logits"]), np.array(GOLD["whole_forward_plain_logits"])
    assert np.abs(ref - mine).max() < 1e-6 * np.abs(ref).max()


@pytest.mark.skipif(not os.path.isfile(os.path.join(reference_dir(), "tools", "build_synthetic_gguf.py")), reason="reference not mounted")
def test_whole_forward_against_the_reference_when_it_is_mounted():
    from golden.make_golden import load_reference, plain_whole_forward
    with np.errstate(over="ignore"):
        ref, mine = plain_whole_forward(load_reference(reference_dir()))
    assert np.abs(np.array(ref["logits"]) - mine.numpy()).max() < 1e-6 * np.abs(ref["logits"]).max()


def test_prefix_property_of_the_whole_model():
    """Logits at position t depend on tokens 0..t only; a window changes them once it is exceeded."""
    for cfg in (TINY_A, TINY_C):
        w = random_weights(cfg, 3, torch.float32, std=0.2)
        toks = random_tokens(30, cfg["vocab_size"], 1)
        full = P.forward_logits(cfg, w, toks)
        assert torch.allclose(P.forward_logits(cfg, w, toks[:13]), full[:13], atol=1e-5)
    nowin = {k: v for k, v in TINY_C.items() if k not in ("sliding_window", "layer_types")}
    other = P.forward_logits(nowin, w, toks)
    assert torch.allclose(other[:20], full[:20], atol=1e-5) and not torch.allclose(other[25:], full[25:], atol=1e-3)


def test_plain_sampler():
    logits = [0.0, 2.0, 2.0, -1.0, 1.0]
    assert P.sample(logits, []) == 1                                  # lowest index on a tie
    assert P.sample(logits, [1], repetition_penalty=2.0) == 2         # 2.0 / 2 = 1.0
    assert P.sample([-1.0, -3.0], [0], repetition_penalty=4.0) == 1   # negative logits are multiplied
    assert P.sample(logits, [], temperature=1.0, top_k=1, u=0.99) == 1
    assert {P.sample(logits, [], temperature=1.0, top_k=2, u=u) for u in (0.0, 0.49, 0.51, 0.99)} == {1, 2}
    p = torch.softmax(torch.tensor(logits), 0)
    assert float(p[1] + p[2]) > 0.7 and P.sample(logits, [], temperature=1.0, top_p=0.7, u=0.99) == 2
    assert P.sample(logits, [], temperature=1.0, top_p=0.8, u=0.999) == 4   # the third token is needed for 0.8
    counts = [0] * 5
    for step in range(4000):
        counts[P.sample(logits, [], temperature=1.0, u=P.uniform_draw(7, 3, step))] += 1
    assert all(abs(c / 4000 - float(q)) < 0.03 for c, q in zip(counts, p))
    assert P.uniform_draw(7, 3, 5) == P.uniform_draw(7, 3, 5) != P.uniform_draw(7, 4, 5)
