"""Sizes beyond the tiny models: a mid-size model against the plain implementation (several tiles of the
tensor-core kernels per matrix, head_dim 128, prompts over several pages), and one layer of the
benchmark's sizes in bfloat16 against the same engine in true float32."""
import pytest
import torch

from helpers import MID, TOL, random_tokens, random_weights, rel_l2, rows_close
from plain import qwen3_plain as P

pytestmark = pytest.mark.gpu

BIG = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=1, hidden_size=4096,
           num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288, vocab_size=151936,
           rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=40960)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mid_size_model_against_the_plain_implementation(dtype):
    from titan_b200 import Engine, StepEntry
    from titan_b200.config import config_from_dict
    w = random_weights(MID, 11, torch.bfloat16, std=0.03)
    w32 = {k: v.float() for k, v in w.items()}
    e = Engine.from_tensors(config_from_dict(MID), w, dtype=dtype, max_tokens=2048)
    reqs = [random_tokens(n, MID["vocab_size"], 50 + n) for n in (300, 130, 70)]
    want = [P.forward_logits(MID, w32, r) for r in reqs]
    slots = [e.alloc_slot() for _ in reqs]
    cut = [260, 100, 69]
    out = e.step([StepEntry(s, r[:c], list(range(c))) for s, r, c in zip(slots, reqs, cut)])
    got, at = [], 0
    for c in cut:
        got.append([out[at:at + c]])
        at += c
    fed = list(cut)
    while any(f < len(r) for f, r in zip(fed, reqs)):
        live = [i for i in range(3) if fed[i] < len(reqs[i])]
        out = e.step([StepEntry(slots[i], [reqs[i][fed[i]]], [0]) for i in live])
        for k, i in enumerate(live):
            got[i].append(out[k:k + 1])
            fed[i] += 1
    for i in range(3):
        assert rel_l2(torch.cat(got[i]).float().cpu(), want[i]) < TOL[dtype], i
        e.free_slot(slots[i])


def test_benchmark_layer_sizes_against_the_plain_implementation_and_bfloat16_against_float32():
    """One layer of the benchmark's sizes, weights from the library's own generator (made on the device, the
    same bits as on the CPU): a short prompt and a few decoded tokens against the plain implementation in both
    dtypes; longer unequal prompts in bfloat16 against the true 32-bit engine; and 24 greedy tokens (captured
    steps from the third on), each of which must be the 32-bit engine's choice for the same sequence or lose
    a near-tie to rounding."""
    from titan_b200 import Engine, SamplerParams, StepEntry, kernels as K
    from titan_b200.config import config_from_dict
    from titan_b200.parts import declare_weights
    from titan_b200.weights.random_init import make_tensor
    cfg = config_from_dict(BIG)
    w = {d.name: make_tensor(d, 3, torch.bfloat16, "cuda").cpu() for d in declare_weights(cfg.to_model_spec())}
    short = random_tokens(44, 151936, 5)
    want_short = P.forward_logits(BIG, {k: v.float() for k, v in w.items()}, short)
    logits, tokens = {}, {}
    prompts = [random_tokens(n, 151936, n) for n in (333, 64, 129)]
    engines = {}
    for dtype in ("bfloat16", "float32"):
        e = engines[dtype] = Engine.from_tensors(cfg, w, dtype=dtype, max_tokens=4096, max_context=1024)
        s = e.alloc_slot()
        got = [e.step([StepEntry(s, short[:40], list(range(40)))])] + [e.step([StepEntry(s, [t], [0])]) for t in short[40:]]
        e.free_slot(s)
        rows_close(torch.cat(got), want_short, dtype, f"{dtype} against the plain implementation")
        slots = [e.alloc_slot() for _ in prompts]
        first = e.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
        rows = [first]
        feed = [7, 8, 9]
        for _ in range(3):
            rows.append(e.step([StepEntry(s, [t], [0]) for s, t in zip(slots, feed)]))
        for s in slots:
            e.free_slot(s)
        logits[dtype] = torch.cat(rows).float().cpu()
        e.check_kernels()
    rows_close(logits["bfloat16"], logits["float32"], "bfloat16", "bfloat16 against float32")
    out = engines["bfloat16"].generate(prompts, max_tokens=24, params=SamplerParams.greedy(), stop_tokens=[])     # graphs after the first steps
    engines["bfloat16"].check_kernels()
    assert engines["bfloat16"].graph_launches > 0
    e32 = engines["float32"]
    for p, r in zip(prompts, out):
        s = e32.alloc_slot()
        seq = list(p) + r.tokens[:-1]
        ref = e32.step([StepEntry(s, seq, list(range(len(p) - 1, len(seq))))]).float().cpu()
        e32.free_slot(s)
        for j, tok in enumerate(r.tokens):
            best = int(torch.argmax(ref[j]))
            if tok != best:
                assert float(ref[j][best] - ref[j][tok]) < 0.05 * float(ref[j].abs().max()), (j, tok, best)


def test_long_prompts_and_decoding_fast_kernels_against_plain_kernels():
    """The same mid-size model in bfloat16 with the tensor-core kernels and with the any-size CUDA-core
    kernels: prompts of thousands of tokens (dozens of key tiles, several chunks of decode attention,
    cluster merges), then 48 single-token steps, one batch after another so that slots are used again.
    Both must agree within the bfloat16 tolerance, and no kernel may have given up on a wait."""
    from titan_b200 import Engine, StepEntry, kernels as K
    from titan_b200.config import config_from_dict
    w = random_weights(MID, 12, torch.bfloat16, std=0.03)
    kw = dict(dtype="bfloat16", max_tokens=3 * 3072, max_context=3072, mark_freed_pages=True)    # a stale row of the round before would show
    engines = {"fast": Engine.from_tensors(config_from_dict(MID), w, **kw),
               "plain kernels": Engine.from_tensors(config_from_dict(MID), w, gemm="plain", attention="plain", **kw)}
    got = {}
    for name, e in engines.items():
        rows = []
        for round_ in range(2):
            reqs = [random_tokens(n, MID["vocab_size"], 70 + n + round_) for n in (2300, 900, 1500)]
            slots = [e.alloc_slot() for _ in reqs]
            rows.append(e.step([StepEntry(s, r, sorted({len(r) - 1, 0, len(r) // 2} | set(range(5, len(r), 97)))) for s, r in zip(slots, reqs)]))      # dozens of rows spread over every prompt
            for step in range(48):
                live = slots if step < 30 else slots[:2]               # the third sequence ends earlier
                rows.append(e.step([StepEntry(s, [(11 * step + 3 * i) % MID["vocab_size"]], [0]) for i, s in enumerate(live)]))
            for s in slots:
                e.free_slot(s)
        e.check_kernels()
        got[name] = torch.cat(rows).float().cpu()
    assert K.wait_errors() == {}
    rows_close(got["fast"], got["plain kernels"], "bfloat16", "tensor-core kernels against the any-size ones")


def _random_configuration(seed):
    """A Qwen3 configuration drawn at random: head sizes in steps of 16 up to 256, any number of heads and
    groups (group sizes beyond what the tensor-core kernels take included), widths and vocabularies that are
    no power of two, windows on some layers."""
    import random
    r = random.Random(seed)
    hd = r.choice([64, 128]) if r.random() < 0.4 else 16 * r.randint(1, 16)
    nkv = r.choice([1, 1, 2, 3, 4, 5, 8])
    group = r.choice([1, 2, 3, 4, 4, 5, 7, 8, 16, 20])
    while nkv * group * hd > 4096:
        group = max(1, group // 2)
    layers = r.randint(1, 3)
    cfg = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=layers,
               hidden_size=r.choice([512, 1024, 2048]) if r.random() < 0.3 else 8 * r.randint(8, 200),
               num_attention_heads=nkv * group, num_key_value_heads=nkv, head_dim=hd,
               intermediate_size=8 * r.randint(8, 400), vocab_size=r.randint(100, 7000),
               rope_theta=r.choice([1e4, 5e5, 1e6]), rms_norm_eps=r.choice([1e-6, 1e-5, 3e-6]),
               tie_word_embeddings=r.random() < 0.3, max_position_embeddings=4096)
    if r.random() < 0.35:
        cfg["sliding_window"] = r.randint(5, 300)
        cfg["layer_types"] = [r.choice(["sliding_attention", "full_attention"]) for _ in range(layers)]
    return cfg, [r.randint(1, 900), r.randint(1, 300), r.randint(1, 64)]


@pytest.mark.parametrize("seed", range(2000, 2010))
def test_random_configurations_against_the_plain_implementation(seed):
    """Unequal prompts in one step, then single tokens (the shortest request ends earlier), in both dtypes."""
    from titan_b200 import Engine, StepEntry
    from titan_b200.config import config_from_dict
    cfg, lens = _random_configuration(seed)
    steps = 5
    w = random_weights(cfg, seed, torch.bfloat16, std=0.03)
    w32 = {k: v.float() for k, v in w.items()}
    reqs = [random_tokens(n + steps, cfg["vocab_size"], 7 * n + seed) for n in lens]
    want = [P.forward_logits(cfg, w32, q) for q in reqs]
    for dtype in ("bfloat16", "float32"):
        e = Engine.from_tensors(config_from_dict(cfg), w, dtype=dtype, max_tokens=2048, max_context=1024)
        slots = [e.alloc_slot() for _ in reqs]
        out = e.step([StepEntry(s, q[:n], list(range(n))) for s, q, n in zip(slots, reqs, lens)])
        got, at = [], 0
        for n in lens:
            got.append([out[at:at + n]])
            at += n
        for d in range(steps):
            live = [0, 1, 2] if d < 3 else [0, 1]
            out = e.step([StepEntry(slots[i], [reqs[i][lens[i] + d]], [0]) for i in live])
            for k, i in enumerate(live):
                got[i].append(out[k:k + 1])
        e.check_kernels()
        for i in range(3):
            g = torch.cat(got[i]).float().cpu()
            assert rel_l2(g, want[i][:g.shape[0]]) < TOL[dtype], (cfg, lens, dtype, i)
        del e
