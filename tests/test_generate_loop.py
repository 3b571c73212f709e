"""The generation loop's decisions, with a scripted backend (no GPU)."""
import pytest

from titan_b200.engine.generate import GenerationRequest, generate
from titan_b200.sampling import SamplerParams


class Scripted:
    """Emits, for the sequence with id s, the tokens script[s] one after another."""
    vocab_size, max_context = 100, 40

    def __init__(self, script, max_batch=2, capacity=10_000):
        self.script, self.max_batch, self.capacity = script, max_batch, capacity
        self.live, self.log, self.next_handle, self.held = {}, [], 0, 0

    def room_for(self, counts):
        return self.held + sum(-(-n // 64) * 64 for n in counts) <= self.capacity and len(self.live) + len(counts) <= 8

    def start(self, prompts, params, sequence_ids):
        handles = []
        for p, s in zip(prompts, sequence_ids):
            h = self.next_handle
            self.next_handle += 1
            self.live[h] = [s, 0, len(p)]
            handles.append(h)
        self.log.append(("start", list(sequence_ids), [len(p) for p in prompts]))
        return handles, [self._emit(h) for h in handles]

    def advance(self, handles, tokens):
        for h, t in zip(handles, tokens):
            assert h in self.live
            self.live[h][2] += 1
            assert self.live[h][2] <= self.max_context
        self.log.append(("advance", [self.live[h][0] for h in handles], list(tokens)))
        return [self._emit(h) for h in handles]

    def finish(self, h):
        assert h in self.live, "finished twice"
        self.log.append(("finish", self.live.pop(h)[0]))

    def _emit(self, h):
        s, k, _ = self.live[h]
        self.live[h][1] += 1
        return self.script[s][k]


def req(n_prompt, max_tokens, stop=(), include_stop=False):
    return GenerationRequest(list(range(1, n_prompt + 1)), max_tokens, SamplerParams.greedy(), stop, include_stop)


def test_stop_token_is_not_emitted_and_budget_counts_the_first_token():
    b = Scripted({0: [5, 6, 9, 7], 1: [9], 2: [1, 2, 3, 4, 5]}, max_batch=3)
    out = generate(b, [req(3, 10, stop=(9,)), req(2, 10, stop=(9,)), req(4, 3, stop=(9,))])
    assert (out[0].tokens, out[0].finish_reason) == ([5, 6], "stop")
    assert (out[1].tokens, out[1].finish_reason) == ([], "stop")
    assert (out[2].tokens, out[2].finish_reason) == ([1, 2, 3], "length")
    assert not b.live


def test_include_stop():
    b = Scripted({0: [5, 9]})
    assert generate(b, [req(1, 5, stop=(9,), include_stop=True)])[0].tokens == [5, 9]


def test_shorter_sequences_leave_and_the_rest_go_on():
    b = Scripted({0: [1, 9], 1: [1, 2, 3, 9], 2: [4, 9]}, max_batch=3)
    generate(b, [req(2, 9, (9,)), req(2, 9, (9,)), req(2, 9, (9,))])
    advances = [e for e in b.log if e[0] == "advance"]
    assert [a[1] for a in advances] == [[0, 1, 2], [1], [1]]
    assert [a[2] for a in advances] == [[1, 1, 4], [2], [3]]             # the last token of each goes back in
    order = [e for e in b.log if e[0] in ("advance", "finish")]
    assert order.index(("finish", 0)) < order.index(advances[1])          # freed before the next step


def test_batches_follow_one_another_in_arrival_order():
    b = Scripted({i: [1, 9] for i in range(5)}, max_batch=2)
    out = generate(b, [req(1 + i, 4, (9,)) for i in range(5)])
    starts = [e for e in b.log if e[0] == "start"]
    assert [s[1] for s in starts] == [[0, 1], [2, 3], [4]]
    assert [s[2] for s in starts] == [[1, 2], [3, 4], [5]]
    assert all(o.tokens == [1] and o.finish_reason == "stop" for o in out)


def test_a_batch_is_cut_where_the_cache_ends():
    b = Scripted({i: [1, 9] for i in range(3)}, max_batch=3, capacity=128)
    generate(b, [req(10, 20, (9,)), req(10, 20, (9,)), req(10, 20, (9,))])
    assert [s[1] for s in b.log if s[0] == "start"] == [[0, 1], [2]]


def test_context_full_ends_with_length():
    b = Scripted({0: list(range(10, 90))})
    out = generate(b, [req(38, 50)])
    # 38 prompt tokens; tokens 1 and 2 can be fed back (positions 38, 39); the third cannot
    assert out[0].finish_reason == "length" and len(out[0].tokens) == 3


def test_zero_budget_and_bad_requests():
    b = Scripted({})
    assert generate(b, [req(3, 0)])[0].finish_reason == "length" and b.log == []
    for bad in (GenerationRequest([], 4), GenerationRequest([100], 4), GenerationRequest([1] * 41, 4)):
        with pytest.raises(ValueError):
            generate(b, [bad])
    with pytest.raises(ValueError):
        generate(b, [GenerationRequest([1], 4, SamplerParams(top_p=0.0))])


def test_everything_is_given_back_when_the_backend_fails():
    class Failing(Scripted):
        def advance(self, handles, tokens):
            raise RuntimeError("boom")
    b = Failing({0: [1, 2], 1: [1, 2]})
    with pytest.raises(RuntimeError):
        generate(b, [req(1, 5), req(1, 5)])
    assert not b.live


def test_sampler_params_defaults_are_the_references():
    p = SamplerParams()
    assert (p.temperature, p.top_p, p.top_k, p.repetition_penalty, p.seed) == (0.7, 0.9, 40, 1.1, None)
    assert p.seed_value() == 42 and SamplerParams.greedy().is_greedy() and not p.is_greedy()
    assert SamplerParams(temperature=1e-4).is_greedy()
