"""The engine against the plain implementation, under every way of cutting the work.
Needs a B200; each case runs in float32 (true 32-bit) and in bfloat16."""
import os

import pytest
import torch

from helpers import TINY, TOL, random_tokens, random_weights, rel_l2, rows_close, write_folder
from plain import qwen3_plain as P

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [5, 11, 17, 70], "B": [1, 7, 23, 40], "C": [30, 45, 90, 150]}
SEEDS = {"A": 0, "B": 1, "C": 2}
CASES = [(c, d) for c in "ABC" for d in ("float32", "bfloat16")]


class World:
    """One tiny model: folder, plain logits of its requests, engines by dtype."""

    def __init__(self, name, root):
        self.name, self.cfg = name, TINY[name]
        self.weights = random_weights(self.cfg, SEEDS[name], torch.bfloat16, std=0.08)
        self.folder = write_folder(os.path.join(root, name), self.cfg, self.weights)
        self.w32 = {k: v.float() for k, v in self.weights.items()}
        self.requests = [random_tokens(n, self.cfg["vocab_size"], 100 + i) for i, n in enumerate(LENGTHS[name])]
        self._plain = {}
        self._engines = {}

    def plain(self, i):
        if i not in self._plain:
            self._plain[i] = P.forward_logits(self.cfg, self.w32, self.requests[i])
        return self._plain[i]

    def engine(self, dtype, **kw):
        from titan_b200 import Engine
        key = (dtype, tuple(sorted(kw.items())))
        if key not in self._engines:
            self._engines[key] = Engine.from_pretrained(self.folder, dtype=dtype, **({"max_tokens": 1024} | kw))
        return self._engines[key]


@pytest.fixture(scope="module")
def worlds(tmp_path_factory):
    root = str(tmp_path_factory.mktemp("models"))
    return {n: World(n, root) for n in "ABC"}


def close(got, want, dtype, what=""):
    rows_close(got, want, dtype, what)          # the tensor within the bound and every row within four times the bound


@pytest.mark.parametrize("name,dtype", CASES)
def test_each_request_alone_and_whole(worlds, name, dtype):
    from titan_b200 import StepEntry
    w = worlds[name]
    e = w.engine(dtype)
    for i, toks in enumerate(w.requests):
        s = e.alloc_slot()
        logits = e.step([StepEntry(s, toks, list(range(len(toks))))])
        e.free_slot(s)
        close(logits, w.plain(i), dtype, f"request {i}")
    e.cache.check()


@pytest.mark.parametrize("name,dtype", CASES)
def test_last_32_tokens_one_by_one(worlds, name, dtype):
    from titan_b200 import StepEntry
    w = worlds[name]
    e = w.engine(dtype)
    for i, toks in enumerate(w.requests):
        if len(toks) <= 32:
            continue
        cut = len(toks) - 32
        s = e.alloc_slot()
        rows = [e.step([StepEntry(s, toks[:cut], list(range(cut)))])]
        for t in toks[cut:]:
            rows.append(e.step([StepEntry(s, [t], [0])]))
        e.free_slot(s)
        got = torch.cat(rows)
        close(got, w.plain(i), dtype, f"request {i}")
        close(got[cut:], w.plain(i)[cut:], dtype, f"request {i}, decoded part")
        close(got[cut:cut + 1], w.plain(i)[cut:cut + 1], dtype, f"request {i}, first decoded token")


@pytest.mark.parametrize("name,dtype", CASES)
def test_from_the_first_token_one_by_one(worlds, name, dtype):
    from titan_b200 import StepEntry
    w = worlds[name]
    e = w.engine(dtype)
    toks = w.requests[1][:9]
    s = e.alloc_slot()
    got = torch.cat([e.step([StepEntry(s, [t], [0])]) for t in toks])
    e.free_slot(s)
    close(got, w.plain(1)[:9], dtype)
    close(got[:1], w.plain(1)[:1], dtype, "position 0")


def replay_in_batches(e, requests, batch_size, prompt_part):
    """Batches of ``batch_size`` requests one after another: their first ``prompt_part`` of tokens in
    one step, the rest one token each; a request that is through leaves and frees its slot."""
    from titan_b200 import StepEntry
    got = {i: [] for i in range(len(requests))}
    for b0 in range(0, len(requests), batch_size):
        ids = list(range(b0, min(b0 + batch_size, len(requests))))
        slots = {i: e.alloc_slot() for i in ids}
        fed = {i: max(1, int(len(requests[i]) * prompt_part)) for i in ids}
        out = e.step([StepEntry(slots[i], requests[i][:fed[i]], list(range(fed[i]))) for i in ids])
        o = 0
        for i in ids:
            got[i].append(out[o:o + fed[i]])
            o += fed[i]
        live = list(ids)
        while True:
            for i in list(live):
                if fed[i] == len(requests[i]):
                    e.free_slot(slots.pop(i))
                    live.remove(i)
            if not live:
                break
            out = e.step([StepEntry(slots[i], [requests[i][fed[i]]], [0]) for i in live])
            for k, i in enumerate(live):
                got[i].append(out[k:k + 1])
                fed[i] += 1
    return {i: torch.cat(v) for i, v in got.items()}


@pytest.mark.parametrize("name,dtype", CASES)
def test_batches_of_unequal_lengths_with_slots_used_again(worlds, name, dtype):
    w = worlds[name]
    e = w.engine(dtype, max_slots=2, max_tokens=512, mark_freed_pages=True)     # a stale row of an earlier owner would show
    order = [3, 0, 2, 1]                               # long with short, so the short one leaves early
    reqs = [w.requests[i] for i in order]
    for part in (0.5, 1.0):
        got = replay_in_batches(e, reqs, 2, part)
        for k, i in enumerate(order):
            close(got[k], w.plain(i), dtype, f"request {i}, prompt part {part}")
        e.cache.check()
        assert e.cache.slots.free_count == 2 and e.cache.tokens_held() == 0


@pytest.mark.parametrize("name,dtype", CASES)
def test_padding_and_neighbours_change_nothing(worlds, name, dtype):
    """The same request alone and beside others: the bound is rounding, the float32 engine is bit-equal."""
    from titan_b200 import StepEntry
    w = worlds[name]
    e = w.engine(dtype)
    toks = w.requests[2]
    s = e.alloc_slot()
    alone = e.step([StepEntry(s, toks, list(range(len(toks))))])
    e.free_slot(s)
    slots = [e.alloc_slot() for _ in range(3)]
    both = e.step([StepEntry(slots[0], w.requests[3], []), StepEntry(slots[1], toks, list(range(len(toks)))),
                   StepEntry(slots[2], w.requests[0], [0])])
    for s in slots:
        e.free_slot(s)
    got = both[:len(toks)]
    if dtype == "float32":
        assert torch.equal(got, alone)
    else:
        close(got, alone.float().cpu(), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(worlds, dtype):
    """600 single-token steps: pages are added on the way, decode attention runs several splits, and
    the window of model C wraps its ring many times."""
    from titan_b200 import StepEntry
    for name in ("A", "C"):
        w = worlds[name]
        e = w.engine(dtype)
        toks = random_tokens(600, w.cfg["vocab_size"], 77)
        want = P.forward_logits(w.cfg, w.w32, toks)
        s = e.alloc_slot()
        rows = [e.step([StepEntry(s, toks[:3], [0, 1, 2])])]
        for t in toks[3:]:
            rows.append(e.step([StepEntry(s, [t], [0])]))
        e.free_slot(s)
        got = torch.cat(rows)
        close(got, want, dtype, name)
        close(got[500:], want[500:], dtype, name + " tail")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_prompt_then_continuation_chunks(worlds, dtype):
    """A prompt longer than the ring, then chunks of several tokens on a filled cache."""
    from titan_b200 import StepEntry
    w = worlds["C"]
    e = w.engine(dtype)
    toks = random_tokens(260, w.cfg["vocab_size"], 78)
    want = P.forward_logits(w.cfg, w.w32, toks)
    s = e.alloc_slot()
    rows, at = [], 0
    for n in (130, 7, 70, 1, 52):
        rows.append(e.step([StepEntry(s, toks[at:at + n], list(range(n)))]))
        at += n
    e.free_slot(s)
    close(torch.cat(rows), want, dtype)


@pytest.mark.parametrize("name,dtype", CASES)
def test_greedy_generation_through_the_entry_point(worlds, name, dtype):
    from titan_b200 import SamplerParams
    w = worlds[name]
    e = w.engine(dtype, max_batch=3)
    prompts = w.requests[:4]
    out = e.generate(prompts, max_tokens=8, params=SamplerParams.greedy(), stop_tokens=[])
    assert [r.finish_reason for r in out] == ["length"] * 4 and all(len(r.tokens) == 8 for r in out)
    for p, r in zip(prompts, out):
        seq = list(p)
        for tok in r.tokens:
            logits = P.forward_logits(w.cfg, w.w32, seq)[-1]
            top2 = torch.topk(logits, 2).values
            margin = float(top2[0] - top2[1])
            if tok != int(torch.argmax(logits)):
                # only a near-tie may be decided differently, and only by rounding
                assert dtype == "bfloat16" and float(top2[0] - logits[tok]) < 0.05 * float(logits.abs().max()), (tok, margin)
            seq.append(tok)
    e.cache.check()
    assert e.cache.slots.held_count == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_generation_stops_and_samples_reproducibly(worlds, dtype):
    from titan_b200 import SamplerParams
    w = worlds["B"]
    e = w.engine(dtype, max_batch=4)
    params = SamplerParams(temperature=0.8, top_k=0, top_p=1.0, repetition_penalty=1.0, seed=11)
    a = e.generate(w.requests, max_tokens=12, params=params, stop_tokens=[])
    b = e.generate(list(reversed(w.requests)), max_tokens=12, params=params, stop_tokens=[])
    # same seed, other batch composition: a sequence's draws depend on (seed, sequence id, step) only,
    # and the id is the request's index, so request 0 alone must repeat itself
    c = e.generate(w.requests[:1], max_tokens=12, params=params, stop_tokens=[])
    assert c[0].tokens == a[0].tokens
    assert [r.tokens for r in e.generate(w.requests, max_tokens=12, params=params, stop_tokens=[])] == [r.tokens for r in a]
    assert all(len(r.tokens) == 12 for r in b)
    # a stop token: taken from the very run that the stopped run is compared with (request 1 alone has sequence id 0)
    ref = e.generate(w.requests[1:2], max_tokens=12, params=params, stop_tokens=[])[0].tokens
    stop = ref[5]
    d = e.generate(w.requests[1:2], max_tokens=12, params=params, stop_tokens=[stop])
    assert d[0].finish_reason == "stop" and d[0].tokens == ref[:ref.index(stop)]
    kept = e.generate(w.requests[1:2], max_tokens=12, params=params, stop_tokens=[stop], include_stop=True)
    assert kept[0].finish_reason == "stop" and kept[0].tokens == ref[:ref.index(stop) + 1]


def test_step_errors_leave_the_cache_alone(worlds):
    from titan_b200 import StepEntry, StepError
    e = worlds["A"].engine("float32", max_tokens=128, max_slots=2)
    s = e.alloc_slot()
    for bad in ([StepEntry(s, [], [])], [StepEntry(s, [999], [])], [StepEntry(s, [1], [1])], [StepEntry(5, [1], [])],
                [StepEntry(s, [1], []), StepEntry(s, [2], [])], [StepEntry(s, [1] * 129, [])], []):
        with pytest.raises(StepError):
            e.step(bad)
    assert e.cache.length[s] == 0
    e.free_slot(s)
    e.cache.check()


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("C", "bfloat16"), ("B", "bfloat16")])
def test_captured_decode_steps_equal_eager_ones(worlds, name, dtype):
    """The same greedy generation with and without CUDA graphs, and with the host out of the loop."""
    from titan_b200 import SamplerParams
    w = worlds[name]
    eager = w.engine(dtype, decode_graphs=False)
    graph = w.engine(dtype, decode_graphs=True)
    prompts = w.requests
    params = SamplerParams(temperature=0.9, top_k=20, top_p=0.95, repetition_penalty=1.2, seed=5)
    for p in (SamplerParams.greedy(), params):
        a = eager.generate(prompts, max_tokens=70, params=p, stop_tokens=[])
        b = graph.generate(prompts, max_tokens=70, params=p, stop_tokens=[])
        assert [r.tokens for r in a] == [r.tokens for r in b]
    assert graph.graph_launches > 0 and eager.graph_launches == 0
    # host out of the loop: prompts, one eager step, then 20 steps on the device
    slots, first = graph.start(prompts, [SamplerParams.greedy()] * 4, [0, 1, 2, 3])
    second = graph.advance(slots, first)
    last = graph.decode_on_device(slots, 20).cpu().tolist()
    for s in slots:
        graph.finish(s)
    ref = eager.generate(prompts, max_tokens=22, params=SamplerParams.greedy(), stop_tokens=[])
    assert [r.tokens[0] for r in ref] == first and [r.tokens[1] for r in ref] == second
    assert [r.tokens[21] for r in ref] == last
    graph.cache.check()


def test_programmatic_dependent_launch_changes_no_result(worlds):
    """The same steps with kernels overlapping their predecessors' tails and fully serialised."""
    from titan_b200 import StepEntry, kernels as K
    w = worlds["C"]
    e = w.engine("float32")
    toks = w.requests[2]
    outs = []
    try:
        for on in (True, False):
            K.set_pdl(on)
            s = e.alloc_slot()
            rows = [e.step([StepEntry(s, toks[:60], list(range(60)))])]
            rows += [e.step([StepEntry(s, [t], [0])]) for t in toks[60:]]
            e.free_slot(s)
            outs.append(torch.cat(rows))
    finally:
        K.set_pdl(True)
    assert torch.equal(outs[0], outs[1])


def test_capture_survives_dead_engines_waiting_for_the_cycle_collector(worlds, monkeypatch):
    """An engine that is dropped while a reference cycle still holds it owns captured graphs and device memory
    until Python's cycle collector runs.  If that happens while another engine's decode step is being captured,
    the capture is invalidated; so the capture collects first and keeps the collector off meanwhile.  Here the
    collector is held back between engines, and the first launcher of a captured step runs a collection."""
    import gc
    from titan_b200 import Engine, SamplerParams, kernels as K
    w = worlds["A"]
    prompts = [w.requests[0], w.requests[1]]
    prepare = K.decode_prepare

    def collect_then_prepare(*a, **k):
        if torch.cuda.is_current_stream_capturing():
            gc.collect()
        return prepare(*a, **k)
    monkeypatch.setattr(K, "decode_prepare", collect_then_prepare)
    gc.collect()
    gc.disable()
    try:
        want = None
        for _ in range(3):
            e = Engine.from_pretrained(w.folder, dtype="float32", max_tokens=512)
            e.held_by_a_cycle = [e]                                   # only the cycle collector can free it
            out = [r.tokens for r in e.generate(prompts, max_tokens=6, params=SamplerParams.greedy(), stop_tokens=[])]
            assert want is None or out == want
            want = out
            del e
    finally:
        gc.enable()
        gc.collect()
