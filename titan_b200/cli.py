"""Command line, in the manner of berniehans/titan's ``titan <SUBCOMMAND> [OPTIONS]``
(engine/engine-server/src/main.rs:361-388, 401-462).

Kept from the reference, with their names, meanings and defaults:
  subcommands  ``run`` (the reference's ``chat|run``), ``bench``, ``help``
  -m, --model <PATH>            model folder (config.json + model.safetensors); may be positional
  -c, --kv-capacity <TOKENS>    tokens the cache holds (default 2048)
  -t, --temp, --temperature     sampling temperature (default 0.7; <= 1e-4 is greedy)
  --top-p <FLOAT>               nucleus mass (default 0.9)
Added, because this library takes token ids, not text, and has options the reference reads from its
HTTP request (engine/engine-core/src/sampler.rs:13-24): --prompt-ids, --prompts-file, --max-tokens
(default 512, main.rs:515), --top-k (40), --repetition-penalty (1.1), --seed (42), --stop-ids,
--dtype, --random <config.json> (random weights from a configuration and --weights-seed),
--max-context (longest sequence; default: the model's position limit or what the cache holds) and
--max-batch (sequences per generation batch, default 64), --reproducible (the same bits on every run, slower).
Not kept: ``serve``, ``agent``, -e/--engine, -s/--speculative, --system, -p/--port: servers,
streaming, speculative decoding and text are outside this library.
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from typing import List


def _ids(text: str) -> List[int]:
    return [int(t) for t in text.replace(",", " ").split()]


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="titan_b200", description="Qwen3-dense generation on one B200: token ids in, token ids out")
    sub = ap.add_subparsers(dest="command")
    for name in ("run", "chat", "bench"):
        p = sub.add_parser(name, help={"run": "generate from prompt token ids", "chat": "alias of run",
                                       "bench": "prompt and decode throughput on three prompts"}[name])
        p.add_argument("model_pos", nargs="?", default=None, help="model folder (same as --model)")
        p.add_argument("-m", "--model", default=None)
        p.add_argument("--random", default=None, metavar="CONFIG_JSON", help="random weights for this configuration")
        p.add_argument("--weights-seed", type=int, default=0)
        p.add_argument("-c", "--kv-capacity", type=int, default=2048)
        p.add_argument("-t", "--temp", "--temperature", dest="temperature", type=float, default=0.7)
        p.add_argument("--top-p", type=float, default=0.9)
        p.add_argument("--top-k", type=int, default=40)
        p.add_argument("--repetition-penalty", type=float, default=1.1)
        p.add_argument("--seed", type=int, default=None)
        p.add_argument("--max-tokens", type=int, default=512)
        p.add_argument("--stop-ids", type=_ids, default=None, help="default: the configuration's eos_token_id")
        p.add_argument("--prompt-ids", type=_ids, action="append", default=None, help="one prompt: 1,2,3 (repeatable)")
        p.add_argument("--prompts-file", default=None, help="one prompt per line: token ids, or a JSON list")
        p.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
        p.add_argument("--max-context", type=int, default=None, help="longest sequence (prompt + generated); default: the model's limit or the cache's size")
        p.add_argument("--max-batch", type=int, default=64, help="sequences that generate together; more prompts run one batch after another")
        p.add_argument("--reproducible", action="store_true", help="bfloat16: partial sums add up in a fixed order, the same bits on every run (slower)")
    sub.add_parser("help", help="print this help")
    return ap


def _engine(args):
    from . import Engine
    from .config import config_from_dict
    model = args.model or args.model_pos
    kw = dict(dtype=args.dtype, max_tokens=args.kv_capacity, max_context=args.max_context, max_batch=args.max_batch,
              reproducible=args.reproducible)
    if args.random:
        with open(args.random) as f:
            return Engine.from_random(config_from_dict(json.load(f)), args.weights_seed, **kw)
    if not model:
        raise SystemExit("give a model folder (-m/--model) or --random <config.json>")
    return Engine.from_pretrained(model, **kw)


def _prompts(args) -> List[List[int]]:
    prompts = list(args.prompt_ids or [])
    if args.prompts_file:
        with open(args.prompts_file) as f:
            for line in f:
                line = line.strip()
                if line:
                    prompts.append(json.loads(line) if line.startswith("[") else _ids(line))
    if not prompts:
        raise SystemExit("no prompt: use --prompt-ids 1,2,3 or --prompts-file")
    return prompts


def main(argv=None) -> int:
    """Errors of the library's own kinds (configuration, weights, a step's input, a kernel's refusal) end the
    program with one line and status 1, not a traceback."""
    from .config import ConfigError
    from .engine.engine import StepError
    from .kernels import KernelError
    from .weights import WeightError
    try:
        return _main(argv)
    except (ConfigError, WeightError, StepError, KernelError, FileNotFoundError) as err:
        print(f"titan_b200: {type(err).__name__}: {err}", file=sys.stderr)
        return 1


def _main(argv=None) -> int:
    ap = build_parser()
    args = ap.parse_args(argv)
    if args.command in (None, "help"):
        ap.print_help()
        return 0
    from . import SamplerParams
    params = SamplerParams(args.temperature, args.top_p, args.top_k, args.repetition_penalty, args.seed)
    engine = _engine(args)
    if args.command == "bench":      # the reference: 3 prompts, prompt tok/s and 40-token decode tok/s (main.rs:316-355)
        import torch
        V = engine.vocab_size
        for n in (16, 128, min(1024, engine.max_context - 41)):
            prompt = [(31 * i + 7) % V for i in range(n)]
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            slots, toks = engine.start([prompt], [SamplerParams.greedy()], [0])
            torch.cuda.synchronize()
            t1 = time.perf_counter()
            for _ in range(40):
                toks = engine.advance(slots, toks)
            torch.cuda.synchronize()
            t2 = time.perf_counter()
            engine.finish(slots[0])
            print(f"prompt {n:5d} tokens: prefill {n / (t1 - t0):10.1f} tok/s   decode {40 / (t2 - t1):8.1f} tok/s")
        return 0
    t0 = time.perf_counter()
    results = engine.generate(_prompts(args), max_tokens=args.max_tokens, params=params, stop_tokens=args.stop_ids)
    dt = time.perf_counter() - t0
    for r in results:
        print(json.dumps({"tokens": r.tokens, "finish_reason": r.finish_reason, "prompt_tokens": r.prompt_tokens}))
    n = sum(len(r.tokens) for r in results)
    print(f"[titan_b200] {n} tokens in {dt:.2f} s ({n / dt:.1f} tok/s)", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
