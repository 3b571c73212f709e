"""Trace replay: feeds given token ids through the engine step by step and writes logits.

It samples nothing, and it has no forward pass, cache or loader of its own: it
drives ``Engine.step``, the step function that generation uses.  Steps come
from standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step that wants logits, ``<out>/<step>.f32`` holds them as little-endian
float32 [wanted, vocab] in the order of the entries and of their ``want``
lists.  After every step a line ``done <step>`` is printed and flushed.

berniehans/titan's nearest pieces are its teacher-forced drift gate
(engine/engine-core/tests/decode_drift_gate.rs:453-485) and its raw-logits
dumper (tools/golden_dump.py:101-144).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Dict



def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    ap.add_argument("--out", required=True, help="folder for the <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64)")
    args = ap.parse_args(argv)
    os.makedirs(args.out, exist_ok=True)

    print("[titan_b200] loading the engine (kernels are compiled on the first call)", file=sys.stderr, flush=True)
    from .engine import Engine, StepEntry
    engine = Engine.from_pretrained(args.model, dtype=args.dtype, max_tokens=args.max_tokens)
    print(f"[titan_b200] ready: {engine.spec.architecture}, {args.dtype}, cache of {engine.cache.num_pages} pages",
          file=sys.stderr, flush=True)
    slots: Dict[str, int] = {}
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = []
        for e in rec.get("entries", []):
            rid = str(e["id"])
            if rid not in slots:
                slots[rid] = engine.alloc_slot()
            entries.append(StepEntry(slots[rid], e["tokens"], e.get("want", [])))
        if entries:
            logits = engine.step(entries)
            if logits is not None:
                arr = logits.float().cpu().numpy().astype("<f4", copy=False)
                arr.tofile(os.path.join(args.out, f"{step}.f32"))
                engine.check_kernels()                 # the copy above has synchronised: a wait that gave up fails the replay
        for rid in rec.get("end", []):
            rid = str(rid)
            if rid in slots:
                engine.free_slot(slots.pop(rid))
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
