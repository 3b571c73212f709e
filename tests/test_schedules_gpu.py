"""Schedules of the step function and ways into the library that the other files do not run: a step that
mixes a fresh prompt, a continuation chunk and single tokens on a model whose head size takes the
tensor-core kernels; the command line as a subprocess; positions at the end of a 32,768-token context; a
step that fails between a product and its consumer; the model's position limit."""
import json
import math
import os
import subprocess
import sys

import pytest
import torch

from helpers import MID, TINY, random_tokens, random_weights, rel_l2, rows_close, write_folder
from plain import qwen3_plain as P

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_one_step_with_a_fresh_prompt_a_continuation_chunk_and_single_tokens(dtype):
    """Four sequences in ONE step: one brings its whole prompt, one a chunk of 70 tokens onto 200 cached ones,
    two a single token each (onto 130 and onto 64 cached ones, a page border).  berniehans/titan's chunked
    prompt path is the same situation for one sequence (engine/engine-core/src/forward_driver.rs:939-1242)."""
    from titan_b200 import Engine, StepEntry
    from titan_b200.config import config_from_dict
    w = random_weights(MID, 31, torch.bfloat16, std=0.03)
    w32 = {k: v.float() for k, v in w.items()}
    e = Engine.from_tensors(config_from_dict(MID), w, dtype=dtype, max_tokens=2048, max_context=512, mark_freed_pages=True)
    reqs = [random_tokens(n, MID["vocab_size"], 40 + n) for n in (150, 290, 135, 68)]
    held = [0, 200, 130, 64]                                           # tokens in the cache before the mixed step
    brings = [150, 70, 1, 1]
    want = [P.forward_logits(MID, w32, r) for r in reqs]
    for round_ in range(2):                                            # twice: the second round finds used pages
        slots = [e.alloc_slot() for _ in reqs]
        e.step([StepEntry(slots[i], reqs[i][:held[i]], []) for i in (1, 2, 3)])
        out = e.step([StepEntry(slots[i], reqs[i][held[i]:held[i] + brings[i]], list(range(brings[i]))) for i in range(4)])
        at = 0
        for i in range(4):
            rows_close(out[at:at + brings[i]], want[i][held[i]:held[i] + brings[i]], dtype, f"round {round_}, sequence {i}")
            at += brings[i]
        # and the cache it left is right: the next tokens one by one
        fed = [h + b for h, b in zip(held, brings)]
        for _ in range(3):
            live = [i for i in range(4) if fed[i] < len(reqs[i])]
            out = e.step([StepEntry(slots[i], [reqs[i][fed[i]]], [0]) for i in live])
            for k, i in enumerate(live):
                rows_close(out[k:k + 1], want[i][fed[i]:fed[i] + 1], dtype, f"round {round_}, sequence {i}, token {fed[i]}")
                fed[i] += 1
        for s in slots:
            e.free_slot(s)
    e.check_kernels()
    e.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_command_line_generates(tmp_path, dtype):
    cfg = TINY["B"]
    w = random_weights(cfg, 8, torch.bfloat16, std=0.08)
    folder = write_folder(str(tmp_path / "model"), cfg, w)
    w32 = {k: v.float() for k, v in w.items()}
    prompts = [random_tokens(n, cfg["vocab_size"], 60 + n) for n in (9, 30)]
    cmd = [sys.executable, os.path.join(ROOT, "bin", "titan_b200"), "run", "-m", folder, "-t", "0", "--repetition-penalty", "1.0",
           "--max-tokens", "6", "--stop-ids", "", "--dtype", dtype, "--max-context", "128", "--max-batch", "1", "-c", "256"]
    for p in prompts:
        cmd += ["--prompt-ids", ",".join(str(t) for t in p)]
    run = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stderr[-2000:]
    lines = [json.loads(l) for l in run.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 2 and [l["prompt_tokens"] for l in lines] == [9, 30] and all(l["finish_reason"] == "length" for l in lines)
    for p, l in zip(prompts, lines):
        assert len(l["tokens"]) == 6
        logits = P.forward_logits(cfg, w32, list(p) + l["tokens"])
        for j, tok in enumerate(l["tokens"]):
            row = logits[len(p) - 1 + j]
            best = int(torch.argmax(row))
            if tok != best:
                assert dtype == "bfloat16" and float(row[best] - row[tok]) < 0.05 * float(row.abs().max()), (j, tok, best)
    # a folder without a model: one line on stderr, status 1, no traceback
    bad = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "titan_b200"), "run", "-m", str(tmp_path / "nowhere"), "--prompt-ids", "1"],
                         capture_output=True, text=True, timeout=600)
    assert bad.returncode == 1 and "ConfigError" in bad.stderr and "Traceback" not in bad.stderr
    # a prompt beyond --max-context is refused the same way
    long = subprocess.run(cmd[:cmd.index("--prompt-ids")] + ["--prompt-ids", ",".join(["1"] * 200)], capture_output=True, text=True, timeout=600)
    assert long.returncode != 0 and "200 tokens" in long.stderr


def test_rotation_at_the_end_of_a_long_context():
    """Head norm and rotation at positions 32,000 to 32,767 against float64: angles of tens of thousands of
    radians, where a float32 product position * frequency has lost five digits (the reference computes the
    same float32 product, engine/engine-core/src/forward_cpu.rs:233-234)."""
    from titan_b200 import kernels as K
    from titan_b200.engine.batch import StepEntry, StepLayout
    nh, nkv, hd, theta, eps = 4, 2, 128, 1e6, 1e-6
    T = 768
    g = torch.Generator().manual_seed(3)
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, generator=g)
    qw, kw = 1 + 0.1 * torch.randn(hd, generator=g), 1 + 0.1 * torch.randn(hd, generator=g)
    lay = StepLayout([StepEntry(0, [0] * T, [])], [32000], "cuda")
    k = torch.arange(hd // 2, dtype=torch.float64)
    inv64 = torch.tensor(theta, dtype=torch.float64) ** (-2 * k / hd)
    inv = inv64.float().cuda()
    pos = torch.arange(32000, 32000 + T)

    def ref(x, w):                                          # float64 throughout, with the float32 table the kernel is given
        x = x.double()
        y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w.double()
        ang = pos.double()[:, None, None] * inv.cpu().double()[None, None, :]
        a, b = y[..., :hd // 2], y[..., hd // 2:]
        return torch.cat([a * ang.cos() - b * ang.sin(), a * ang.sin() + b * ang.cos()], -1)
    Q, KV = nh * hd, nkv * hd
    want_q, want_k = ref(qkv[:, :Q].view(T, nh, hd), qw), ref(qkv[:, Q:Q + KV].view(T, nkv, hd), kw)
    for dtype, bound in ((torch.float32, 3e-3), (torch.bfloat16, 8e-3)):
        buf = qkv.to(dtype).cuda()
        keep = (qw.cuda(), kw.cuda())
        a = K.QkArgs()
        a.inp, a.in_stride, a.q_out, a.q_stride = buf.data_ptr(), buf.shape[1], buf.data_ptr(), buf.shape[1]
        a.k_out, a.k_stride = buf.data_ptr() + Q * buf.element_size(), buf.shape[1]
        a.q_w, a.k_w, a.rope = keep[0].data_ptr(), keep[1].data_ptr(), K.RotaryArgs(inv.data_ptr(), hd, 0.0, 1.0)
        a.eps, a.nh, a.nkv, a.hd = eps, nh, nkv, hd
        a.pos_of, a.seq_of, a.slot_of_seq = lay.pos_of.data_ptr(), lay.seq_of.data_ptr(), lay.slot_of_seq.data_ptr()
        a.append, a.T = 0, T
        K.qk_norm_rope(a, dtype, dtype, K.current_stream())
        got = buf.float().cpu()
        # float32: position * frequency is rounded to 24 bits (an angle of 32,767 radians is off by up to 2e-3); nothing more
        assert rel_l2(got[:, :Q], want_q.reshape(T, Q)) < bound, dtype
        assert rel_l2(got[:, Q:Q + KV], want_k.reshape(T, KV)) < bound, dtype
        # the slow dims (small angles) are exact to rounding
        slow = torch.cat([torch.arange(48, 64), torch.arange(112, 128)])
        assert rel_l2(got[:, :Q].view(T, nh, hd)[..., slow], want_q[..., slow]) < (2e-6 if dtype == torch.float32 else 6e-3)


def plain_last_rows(cfg, w, toks, first):
    """Logits of rows ``first ..`` of a ONE-layer model by the plain implementation's parts, with the attention of
    those rows alone in float64 (the whole-sequence function would hold a 32,768 x 32,768 score matrix)."""
    T, hd = len(toks), cfg["head_dim"]
    nh, nkv, eps, p = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["rms_norm_eps"], "model.layers.0."
    pos = torch.arange(T)
    x = P.embed_lookup(w["model.embed_tokens.weight"], torch.tensor(toks))
    h = P.rms_norm(x, w[p + "input_layernorm.weight"], eps)
    q = P.rope_neox(P.rms_norm(P.linear(h[first:], w[p + "self_attn.q_proj.weight"]).view(-1, nh, hd), w[p + "self_attn.q_norm.weight"], eps), pos[first:], cfg["rope_theta"])
    k = P.rope_neox(P.rms_norm(P.linear(h, w[p + "self_attn.k_proj.weight"]).view(T, nkv, hd), w[p + "self_attn.k_norm.weight"], eps), pos, cfg["rope_theta"])
    v = P.linear(h, w[p + "self_attn.v_proj.weight"]).view(T, nkv, hd)
    rows = []
    for i in range(T - first):
        n = first + i + 1                                              # keys 0 .. first + i
        heads = []
        for hq in range(nh):
            kh = hq // (nh // nkv)
            sc = (k[:n, kh].double() @ q[i, hq].double()) / math.sqrt(hd)
            heads.append((torch.softmax(sc, 0) @ v[:n, kh].double()).float())
        rows.append(torch.cat(heads))
    x = x[first:] + P.linear(torch.stack(rows), w[p + "self_attn.o_proj.weight"])
    x = x + P.mlp_part(w, p, P.rms_norm(x, w[p + "post_attention_layernorm.weight"], eps))
    return P.linear(P.rms_norm(x, w["model.norm.weight"], eps), w["lm_head.weight"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decoding_at_the_end_of_a_32768_token_context(dtype):
    """One layer with heads of 128, a sequence of 32,700 tokens fed in chunks, then single tokens up to the
    context's last place, against the plain implementation: split-KV decode over 511 pages and a block table of
    512 entries.  One key far back is made to stand out, so that a lost early page would show."""
    from titan_b200 import Engine, StepEntry, StepError
    from titan_b200.config import config_from_dict
    cfg = dict(MID, num_hidden_layers=1, hidden_size=256, num_attention_heads=2, num_key_value_heads=1, intermediate_size=512,
               vocab_size=300, max_position_embeddings=32768)
    w = random_weights(cfg, 17, torch.bfloat16, std=0.05)
    n, tail = 32700, 68
    toks = random_tokens(n + tail, 300, 9)
    toks[5] = 299                                                      # a rare token early on ...
    e16 = w["model.embed_tokens.weight"]
    e16[299] = (e16[299].float() * 6).to(torch.bfloat16)               # ... whose key and value are large
    w32 = {k: v.float() for k, v in w.items()}
    want = plain_last_rows(cfg, w32, toks, n - 1)
    e = Engine.from_tensors(config_from_dict(cfg), w, dtype=dtype, max_tokens=32768, max_slots=1)
    assert e.max_context == 32768
    s = e.alloc_slot()
    rows = []
    for at in range(0, n, 8192):
        m = min(8192, n - at)
        out = e.step([StepEntry(s, toks[at:at + m], [m - 1] if at + m == n else [])])
        if out is not None:
            rows.append(out)
    for t in toks[n:]:
        e.advance([s], [t])                                             # captured steps from the third on
        rows.append(e.last_logits.clone())
    assert e.cache.length[s] == 32768
    with pytest.raises(StepError):
        e.step([StepEntry(s, [1], [0])])                                # the context is full
    e.free_slot(s)
    e.check_kernels()
    rows_close(torch.cat(rows), want, dtype, "positions 32,699 to 32,767")


def test_a_step_that_fails_between_a_product_and_its_consumer_spoils_no_later_step(monkeypatch):
    """Decode products add their K slices into a float32 buffer that the next kernel consumes and leaves zeroed.
    A step that ends between the two (here: the consumer's launcher refuses once) must not leave its sums
    there for the next step of the same shape, eager or captured; with the consumer as a kernel of its own too."""
    from titan_b200 import Engine, StepEntry, kernels as K
    from titan_b200.config import config_from_dict
    w = random_weights(MID, 33, torch.bfloat16, std=0.03)
    w32 = {k: v.float() for k, v in w.items()}
    e = Engine.from_tensors(config_from_dict(MID), w, dtype="bfloat16", max_tokens=512, decode_graphs=False)
    toks = random_tokens(40, MID["vocab_size"], 2)
    want = P.forward_logits(MID, w32, toks)
    s = e.alloc_slot()
    e.step([StepEntry(s, toks[:30], [])])
    rows_close(e.step([StepEntry(s, [toks[30]], [0])]), want[30:31], "bfloat16", "before the failure")
    assert any(k.startswith("acc_") for k in e.scratch)
    real, calls = K.attn_decode_mma, {"n": 0}       # the consumer of the sums: the attention kernel (head norm inside it)

    def refuse_once(*a, **k):
        calls["n"] += 1
        if calls["n"] == 2:                                             # the second layer's: the first layer's sums were consumed, these are not
            raise K.KernelError("refused for the test")
        return real(*a, **k)
    monkeypatch.setattr(K, "attn_decode_mma", refuse_once)
    with pytest.raises(K.KernelError):
        e.step([StepEntry(s, [toks[31]], [0])])
    monkeypatch.setattr(K, "attn_decode_mma", real)
    assert e.cache.length[s] == 31                                      # nothing was committed
    # the failed step wrote the first layer's key and value of position 31, which the same token now writes again
    rows_close(e.step([StepEntry(s, [toks[31]], [0])]), want[31:32], "bfloat16", "the step after the failure")
    rows_close(e.step([StepEntry(s, [toks[32]], [0])]), want[32:33], "bfloat16", "and the one after")
    e.free_slot(s)


def test_the_models_position_limit_bounds_the_context():
    from titan_b200 import Engine, SamplerParams, StepError
    from titan_b200.config import config_from_dict
    cfg = dict(TINY["A"], max_position_embeddings=96)
    w = random_weights(cfg, 1, torch.bfloat16, std=0.08)
    e = Engine.from_tensors(config_from_dict(cfg), w, dtype="float32", max_tokens=1024)
    assert e.max_context == 96                                          # not the cache's 1,024
    with pytest.raises(ValueError, match="does not fit"):
        e.generate([list(range(97))], max_tokens=4)
    out = e.generate([list(range(90))], max_tokens=50, params=SamplerParams.greedy(), stop_tokens=[])
    assert out[0].finish_reason == "length" and len(out[0].tokens) == 7  # positions 90 .. 95 are fed back; the seventh token has no place
    with pytest.raises(StepError, match="beyond the model"):
        Engine.from_tensors(config_from_dict(cfg), w, dtype="float32", max_tokens=1024, max_context=200)
    assert Engine.from_tensors(config_from_dict(cfg), w, dtype="float32", max_tokens=1024, max_context=64).max_context == 64


def test_a_prompt_in_chunks_takes_the_tensor_core_kernels(monkeypatch):
    """A prompt fed as four chunks of 512 runs its continuation chunks on the tensor-core prompt attention (keys from
    the cache's pages), not on the any-size kernel, and gives the logits of the prompt fed whole."""
    from titan_b200 import Engine, StepEntry, kernels as K
    from titan_b200.config import config_from_dict
    w = random_weights(MID, 35, torch.bfloat16, std=0.03)
    e = Engine.from_tensors(config_from_dict(MID), w, dtype="bfloat16", max_tokens=4096, max_context=2048)
    toks = random_tokens(2048, MID["vocab_size"], 4)
    used = {"tc": 0, "plain": 0}
    tc, plain = K.attn_prefill_tc, K.attn_prefill
    monkeypatch.setattr(K, "attn_prefill_tc", lambda *a, **k: (used.__setitem__("tc", used["tc"] + 1), tc(*a, **k))[1])
    monkeypatch.setattr(K, "attn_prefill", lambda *a, **k: (used.__setitem__("plain", used["plain"] + 1), plain(*a, **k))[1])
    want_rows = sorted(set(range(0, 2048, 61)) | {511, 512, 1535, 2047})
    s = e.alloc_slot()
    whole = e.step([StepEntry(s, toks, want_rows)])
    e.free_slot(s)
    s = e.alloc_slot()
    parts = []
    for at in range(0, 2048, 512):
        parts.append(e.step([StepEntry(s, toks[at:at + 512], [r - at for r in want_rows if at <= r < at + 512])]))
    e.free_slot(s)
    e.check_kernels()
    assert used["plain"] == 0 and used["tc"] == 2 * 5                   # two layers: one whole prompt and four chunks
    rows_close(torch.cat(parts), whole.float().cpu(), "bfloat16", "chunks against the whole prompt")
