"""The path that serving and the benchmark run, against the plain implementation: bfloat16, decode steps
replayed as CUDA graphs, decode attention on tensor cores (head sizes 128 and 64) with its splits merged
inside a thread-block cluster, lengths read from the committed per-slot state before the step's earlier
kernels have ended, K slices of the decode products summed in float32.

Teacher-forced: the tokens fed are the request's own, so every step's logits have a plain counterpart,
and they are compared row by row.  berniehans/titan checks its captured decode pass the same way, graph
against stream and token by token (engine/engine-cuda/tests/cuda_graphs_test.rs:143-148,
engine/engine-core/tests/driver_graph_parity.rs:54-78)."""
import pytest
import torch

from helpers import MID, MID64, TOL, random_tokens, random_weights, rel_l2, rows_close
from plain import qwen3_plain as P

pytestmark = pytest.mark.gpu

STEPS = 100
PROMPTS = {1: [100], 3: [1, 63, 250], 8: [30, 60, 64, 65, 120, 127, 200, 600]}     # lengths that cross pages (64) and splits (128) on the way
MODELS = {"hd128": (MID, 21), "hd64": (MID64, 22)}


@pytest.fixture(scope="module")
def models():
    out = {}
    for name, (cfg, seed) in MODELS.items():
        w = random_weights(cfg, seed, torch.bfloat16, std=0.03)
        out[name] = (cfg, w, {k: v.float() for k, v in w.items()})
    return out


def teacher_forced(engine, reqs, prompt_lens, steps):
    """Prompts in one step, then ``steps`` single-token steps through Engine.advance (captured from the third
    step of a batch size on); the logits of every step, per request."""
    from titan_b200 import SamplerParams
    B = len(reqs)
    slots, _ = engine.start([r[:n] for r, n in zip(reqs, prompt_lens)], [SamplerParams.greedy()] * B, list(range(B)))
    rows = [[engine.last_logits[i:i + 1].clone()] for i in range(B)]
    for d in range(steps):
        engine.advance(slots, [r[n + d] for r, n in zip(reqs, prompt_lens)])
        for i in range(B):
            rows[i].append(engine.last_logits[i:i + 1].clone())
    for s in slots:
        engine.finish(s)
    engine.check_kernels()
    return [torch.cat(r).float().cpu() for r in rows]


@pytest.mark.parametrize("variant", ["default", "lengths after the wait", "merge through scratch", "next kernel let in at once"])
@pytest.mark.parametrize("B", [1, 3, 8])
@pytest.mark.parametrize("model", ["hd128", "hd64"])
def test_captured_decode_steps_against_the_plain_implementation(models, model, B, variant):
    from titan_b200 import Engine, kernels as K
    from titan_b200.config import config_from_dict
    cfg, w, w32 = models[model]
    lens = PROMPTS[B]
    reqs = [random_tokens(n + STEPS, cfg["vocab_size"], 300 + 7 * n + B) for n in lens]
    want = [P.forward_logits(cfg, w32, r)[n - 1:] for r, n in zip(reqs, lens)]
    kw = dict(dtype="bfloat16", max_tokens=B * 768, max_context=768, mark_freed_pages=True)
    if variant == "lengths after the wait":
        kw["early_pages"] = False
    K.set_attn_decode_cluster(variant != "merge through scratch")
    K.set_attn_decode_late_trigger(variant != "next kernel let in at once")
    try:
        graph = Engine.from_tensors(config_from_dict(cfg), w, decode_graphs=True, **kw)
        got = teacher_forced(graph, reqs, lens, STEPS)
        assert graph.graph_launches > 0
        for i in range(B):
            rows_close(got[i], want[i], "bfloat16", f"{model}, batch {B}, {variant}, request {i} (captured)")
        if variant == "default":
            eager = Engine.from_tensors(config_from_dict(cfg), w, decode_graphs=False, **kw)
            plain_steps = teacher_forced(eager, reqs, lens, STEPS)
            assert eager.graph_launches == 0
            for i in range(B):
                rows_close(plain_steps[i], want[i], "bfloat16", f"{model}, batch {B}, request {i} (eager)")
                rows_close(got[i], plain_steps[i], "bfloat16", f"{model}, batch {B}, request {i} (captured against eager)")
    finally:
        K.set_attn_decode_cluster(True)
        K.set_attn_decode_late_trigger(True)


@pytest.mark.parametrize("model", ["hd128", "hd64"])
def test_decoding_on_the_device_against_the_plain_implementation(models, model):
    """64 steps with the host out of the loop (every step feeds the token the step before sampled, from the
    slot's state), one replay at a time so that every token can be read: each must be the plain
    implementation's greedy choice for the sequence so far, or lose a near-tie to rounding."""
    from titan_b200 import Engine, SamplerParams
    from titan_b200.config import config_from_dict
    cfg, w, w32 = models[model]
    prompts = [random_tokens(n, cfg["vocab_size"], 900 + n) for n in (70, 3, 129)]
    e = Engine.from_tensors(config_from_dict(cfg), w, dtype="bfloat16", max_tokens=3 * 256, max_context=256)
    slots, first = e.start(prompts, [SamplerParams.greedy()] * 3, [0, 1, 2])
    second = e.advance(slots, first)
    made = [[a, b] for a, b in zip(first, second)]
    for _ in range(64):
        for i, t in enumerate(e.decode_on_device(slots, 1).cpu().tolist()):
            made[i].append(t)
    for s in slots:
        e.finish(s)
    e.check_kernels()
    e.cache.check()
    for p, toks in zip(prompts, made):
        logits = P.forward_logits(cfg, w32, list(p) + toks)
        for j, tok in enumerate(toks):
            row = logits[len(p) - 1 + j]
            best = int(torch.argmax(row))
            if tok != best:
                assert float(row[best] - row[tok]) < 0.05 * float(row.abs().max()), (model, j, tok, best)
    # and 64 steps in one call, nothing read in between: every token again the plain choice for its own sequence so far
    # (the two runs may part at a near-tie: the float32 sums of K slices add in any order)
    slots, first = e.start(prompts, [SamplerParams.greedy()] * 3, [0, 1, 2])
    second = e.advance(slots, first)
    rest = e.decode_on_device(slots, 64, keep_all=True).cpu().tolist()
    for s in slots:
        e.finish(s)
    e.check_kernels()
    for i, p in enumerate(prompts):
        toks = [first[i], second[i]] + [row[i] for row in rest]
        logits = P.forward_logits(cfg, w32, list(p) + toks)
        for j, tok in enumerate(toks):
            row = logits[len(p) - 1 + j]
            best = int(torch.argmax(row))
            if tok != best:
                assert float(row[best] - row[tok]) < 0.05 * float(row.abs().max()), (model, j, tok, best)


@pytest.mark.parametrize("B", [1, 8, 20])
def test_folded_norms_change_results_by_rounding_only(models, B):
    """Decode steps with the norms folded into the products that consume them (the default) and with the norms as
    kernels of their own: both against the plain implementation, and the option really switches (launch counts)."""
    from titan_b200 import Engine, kernels as K
    from titan_b200.config import config_from_dict
    cfg, w, w32 = models["hd128"]
    lens = [40 + 13 * i for i in range(B)]
    reqs = [random_tokens(n + 12, cfg["vocab_size"], 500 + n) for n in lens]
    want = [P.forward_logits(cfg, w32, r)[n - 1:] for r, n in zip(reqs, lens)]
    launches = {}
    for fold in (True, False):
        e = Engine.from_tensors(config_from_dict(cfg), w, dtype="bfloat16", max_tokens=B * 384, max_context=384, max_batch=B, fold_norms=fold,
                                fold_norms_rows=32)       # 20 rows too: the default folds up to 16
        before = K.launch_count
        got = teacher_forced(e, reqs, lens, 12)
        launches[fold] = K.launch_count - before + e.graph_launches
        for i in range(B):
            rows_close(got[i], want[i], "bfloat16", f"batch {B}, fold_norms={fold}, request {i}")
    assert launches[True] < launches[False]
    # what one eager decode step of this model launches, by launcher: with every kernel on its own, and by default
    from titan_b200 import SamplerParams
    layers = cfg["num_hidden_layers"]
    logs = {}
    for name, kw in (("apart", dict(fold_norms=False, fold_head_norm=False)), ("default", {})):
        e = Engine.from_tensors(config_from_dict(cfg), w, dtype="bfloat16", max_tokens=512, decode_graphs=False, **kw)
        slots, first = e.start([r[:5] for r in reqs[:1]], [SamplerParams.greedy()], [0])
        K.launch_log_start()
        e.advance(slots, first)
        logs[name] = K.launch_log_stop()
        e.finish(slots[0])
    log = logs["apart"]
    assert log["rmsnorm"] == 2 * layers + 1 and log["qk_norm_rope"] == layers and log["attn_decode_mma"] == layers
    assert log["gemm_tc"] == 4 * layers + 1 and log["embed"] == 1 and "gemm_tc_normed" not in log
    log = logs["default"]
    assert log["rmsnorm"] == 1 and "qk_norm_rope" not in log and log["attn_decode_mma"] == layers
    assert log["gemm_tc_normed"] == 2 * layers and log["gemm_tc"] == 2 * layers + 1


@pytest.mark.parametrize("model", ["hd128", "hd64"])
def test_head_norm_inside_the_attention_kernel_changes_results_by_rounding_only(models, model):
    """Decode steps with head norm, rotation and cache append inside the attention kernel (the default) and as a
    kernel of their own, on sequences that cross pages while they grow (the new key's row moves through a page and
    into the next; the split that holds it changes): both against the plain implementation, and the caches they
    leave are the same to rounding (a later prompt step reads them)."""
    from titan_b200 import Engine, StepEntry
    from titan_b200.config import config_from_dict
    cfg, w, w32 = models[model]
    lens = [62, 1, 127, 190]
    reqs = [random_tokens(n + 70, cfg["vocab_size"], 700 + n) for n in lens]
    want = [P.forward_logits(cfg, w32, r) for r in reqs]
    for fold in (True, False):
        e = Engine.from_tensors(config_from_dict(cfg), w, dtype="bfloat16", max_tokens=4 * 320, max_context=320, fold_head_norm=fold,
                                decode_graphs=False, mark_freed_pages=True)
        for round_ in range(2):
            got = teacher_forced(e, reqs, lens, 66) if round_ == 0 else None
            if got is not None:
                for i in range(4):
                    rows_close(got[i], want[i][lens[i] - 1:lens[i] + 66], "bfloat16", f"{model}, fold_head_norm={fold}, request {i}")
        # the cache that decoding left: decode 66 tokens, then read all of it with a chunk of 4 more tokens
        slots = [e.alloc_slot() for _ in reqs]
        e.step([StepEntry(s, r[:n], []) for s, r, n in zip(slots, reqs, lens)])
        for d in range(66):
            e.step([StepEntry(s, [r[n + d]], []) for s, r, n in zip(slots, reqs, lens)])
        out = e.step([StepEntry(s, r[n + 66:n + 70], [0, 1, 2, 3]) for s, r, n in zip(slots, reqs, lens)])
        for i in range(4):
            rows_close(out[4 * i:4 * i + 4], want[i][lens[i] + 66:lens[i] + 70], "bfloat16", f"{model}, fold_head_norm={fold}, cache of request {i}")
        for s in slots:
            e.free_slot(s)
        e.check_kernels()


@pytest.mark.parametrize("hd", [64, 128])
def test_captured_decode_over_a_ring_cache(hd):
    """Layers with a window keep a ring of rows: the attention kernel that appends the new key itself writes
    position p into row p % ring, and the page it patches in shared memory is the ring's.  Sequences that
    start inside the window and decode far past it (the ring wraps several times), captured steps."""
    from titan_b200 import Engine
    from titan_b200.config import config_from_dict
    cfg = dict(MID64 if hd == 64 else MID, sliding_window=100, layer_types=["sliding_attention", "full_attention"], max_position_embeddings=1024)
    w = random_weights(cfg, 40 + hd, torch.bfloat16, std=0.03)
    w32 = {k: v.float() for k, v in w.items()}
    lens = [60, 130, 1]
    steps = 300
    reqs = [random_tokens(n + steps, cfg["vocab_size"], 800 + n) for n in lens]
    want = [P.forward_logits(cfg, w32, r)[n - 1:] for r, n in zip(reqs, lens)]
    e = Engine.from_tensors(config_from_dict(cfg), w, dtype="bfloat16", max_tokens=3 * 512, max_context=512, mark_freed_pages=True)
    assert sorted(g.ring_rows for g in e.cache.groups) == [0, 128]
    got = teacher_forced(e, reqs, lens, steps)
    assert e.graph_launches > 0
    for i in range(3):
        rows_close(got[i], want[i], "bfloat16", f"head size {hd}, request {i}")
        rows_close(got[i][-40:], want[i][-40:], "bfloat16", f"head size {hd}, request {i}, the last steps")


@pytest.mark.parametrize("heads,kv_heads,hd", [(12, 1, 64), (16, 1, 128), (10, 2, 128)])
def test_captured_decode_with_large_and_odd_groups(heads, kv_heads, hd):
    """More than eight query heads per kv head (both halves of the tensor-core tile's rows are live), and a group of
    five: the attention kernel norms and rotates a group's queries with its four warps taking heads in turn."""
    from titan_b200 import Engine
    from titan_b200.config import config_from_dict
    cfg = dict(MID, num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=hd, hidden_size=640, intermediate_size=1280,
               vocab_size=1500, rms_norm_eps=1e-5)
    w = random_weights(cfg, heads + hd, torch.bfloat16, std=0.03)
    w32 = {k: v.float() for k, v in w.items()}
    lens = [5, 90, 200]
    reqs = [random_tokens(n + 40, cfg["vocab_size"], 60 + n) for n in lens]
    want = [P.forward_logits(cfg, w32, r)[n - 1:] for r, n in zip(reqs, lens)]
    e = Engine.from_tensors(config_from_dict(cfg), w, dtype="bfloat16", max_tokens=3 * 256, max_context=256)
    got = teacher_forced(e, reqs, lens, 40)
    for i in range(3):
        rows_close(got[i], want[i], "bfloat16", f"{heads}/{kv_heads} heads of {hd}, request {i}")


@pytest.mark.parametrize("B", [1, 3, 8])
def test_reproducible_mode_gives_the_same_bits_on_every_run(models, B):
    """``reproducible=True``: the K slices of the decode products add up in a fixed order (and no prompt tile is cut
    along K), so the same requests in the same batch give bit-identical logits on every run, on another engine, and
    replayed from a graph or launched kernel by kernel; against the plain implementation they stay as close as the
    default mode, which is allowed to differ from run to run in the last bits."""
    from titan_b200 import Engine
    from titan_b200.config import config_from_dict
    cfg, w, w32 = models["hd128"]
    lens = PROMPTS[B]
    steps = 40
    reqs = [random_tokens(n + steps, cfg["vocab_size"], 4100 + 3 * n + B) for n in lens]
    want = [P.forward_logits(cfg, w32, r)[n - 1:] for r, n in zip(reqs, lens)]
    kw = dict(dtype="bfloat16", max_tokens=B * 768, max_context=768, reproducible=True)
    first = Engine.from_tensors(config_from_dict(cfg), w, decode_graphs=True, **kw)
    runs = [teacher_forced(first, reqs, lens, steps), teacher_forced(first, reqs, lens, steps)]
    assert first.graph_launches > 0
    runs.append(teacher_forced(Engine.from_tensors(config_from_dict(cfg), w, decode_graphs=True, **kw), reqs, lens, steps))
    runs.append(teacher_forced(Engine.from_tensors(config_from_dict(cfg), w, decode_graphs=False, **kw), reqs, lens, steps))
    for i in range(B):
        rows_close(runs[0][i], want[i], "bfloat16", f"batch {B}, request {i}")
        for other in runs[1:]:
            assert torch.equal(other[i], runs[0][i]), (B, i, float((other[i] - runs[0][i]).abs().max()))
