"""The generation loop: batches of unequal prompts, stop tokens, sequences that end early.

The loop decides; a *backend* computes.  A backend offers

    vocab_size, max_context, max_batch          (ints)
    room_for(token_counts) -> bool              would these sequences fit the cache together?
    start(prompts, params, sequence_ids) -> (handles, first_tokens)
                                                one step over all prompts, one sampled token each
    advance(handles, tokens) -> next_tokens     one token each for the sequences that go on
    finish(handle)                              give back what the sequence holds

``Engine`` is the real backend; tests drive the loop with a scripted one.

After berniehans/titan's loop (engine/engine-server/src/server.rs:213-370): the
first token is sampled from the prompt's logits and counts toward the budget
(:261-276); a stop token ends the sequence and is not emitted (:266-268,
345-348); the budget is ``max_tokens`` generated tokens (:281) and a full
context also ends it (:336-339); finish reasons "stop" and "length".  The
reference serves one request at a time; batches, early leavers and slot reuse
follow its stub scheduler's rule that finished sessions leave at once and the
others go on (engine/engine-server/src/scheduler.rs:50-70, 204-217).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

from ..sampling.params import SamplerParams


@dataclass
class GenerationRequest:
    prompt: Sequence[int]
    max_tokens: int = 512                         # engine-server/src/main.rs:515
    params: SamplerParams = field(default_factory=SamplerParams)
    stop_tokens: Sequence[int] = ()
    include_stop: bool = False


@dataclass
class GenerationResult:
    tokens: List[int]
    finish_reason: str                            # "stop" | "length"
    prompt_tokens: int = 0


def round_up(n: int, unit: int) -> int:
    return -(-n // unit) * unit


def validate_request(req: GenerationRequest, vocab_size: int, max_context: int) -> None:
    if len(req.prompt) == 0:
        raise ValueError("a prompt needs at least one token")
    if len(req.prompt) > max_context:
        raise ValueError(f"a prompt of {len(req.prompt)} tokens does not fit the context of {max_context}")
    for t in req.prompt:
        if not 0 <= int(t) < vocab_size:
            raise ValueError(f"token id {t} lies outside the vocabulary of {vocab_size}")
    if req.max_tokens < 0:
        raise ValueError("max_tokens must be >= 0")
    req.params.validate()


def plan_batch(pending: Sequence[int], requests: Sequence[GenerationRequest], backend) -> List[int]:
    """The next batch: requests in arrival order, as many as fit the batch size and the cache."""
    chosen: List[int] = []
    counts: List[int] = []
    for i in pending:
        if len(chosen) == backend.max_batch:
            break
        r = requests[i]
        need = min(len(r.prompt) + r.max_tokens, backend.max_context)
        if backend.room_for(counts + [need]):
            chosen.append(i)
            counts.append(need)
        else:
            break
    if not chosen:      # the first request does not fit with its whole budget: run it alone, the context ends it
        if not backend.room_for([len(requests[pending[0]].prompt)]):
            raise ValueError(f"the cache cannot hold a prompt of {len(requests[pending[0]].prompt)} tokens")
        chosen = [pending[0]]
    return chosen


def generate(backend, requests: Sequence[GenerationRequest], first_sequence_id: int = 0) -> List[GenerationResult]:
    """Run every request to its end, one batch after another; results in request order."""
    for r in requests:
        validate_request(r, backend.vocab_size, backend.max_context)
    results: List[Optional[GenerationResult]] = [None] * len(requests)
    pending = list(range(len(requests)))
    for i in list(pending):                       # nothing to generate: no slot is taken
        if requests[i].max_tokens == 0:
            results[i] = GenerationResult([], "length", len(requests[i].prompt))
            pending.remove(i)
    while pending:
        batch = plan_batch(pending, requests, backend)
        pending = [i for i in pending if i not in batch]
        _run_batch(backend, [requests[i] for i in batch], [first_sequence_id + i for i in batch], batch, results)
        check = getattr(backend, "check_kernels", None)
        if check is not None:
            check()                               # a kernel that gave up on a wait fails the batch loudly
    return results  # type: ignore[return-value]


def _run_batch(backend, reqs, sequence_ids, indices, results) -> None:
    handles, tokens = backend.start([list(r.prompt) for r in reqs], [r.params for r in reqs], sequence_ids)
    outs: List[List[int]] = [[] for _ in reqs]
    lengths = [len(r.prompt) for r in reqs]       # tokens in the cache
    active = list(range(len(reqs)))
    try:
        while True:
            going: List[int] = []
            for j, tok in zip(active, tokens):
                r = reqs[j]
                reason = None
                if int(tok) in r.stop_tokens:
                    if r.include_stop:
                        outs[j].append(int(tok))
                    reason = "stop"
                else:
                    outs[j].append(int(tok))
                    if len(outs[j]) >= r.max_tokens or lengths[j] + 1 > backend.max_context:
                        reason = "length"           # budget spent, or no room to feed this token back
                if reason is None:
                    going.append(j)
                else:
                    results[indices[j]] = GenerationResult(outs[j], reason, len(r.prompt))
                    backend.finish(handles[j])
                    handles[j] = None
            active = going
            if not active:
                return
            tokens = backend.advance([handles[j] for j in active], [outs[j][-1] for j in active])
            for j in active:
                lengths[j] += 1
    finally:
        for h in handles:
            if h is not None:
                backend.finish(h)
