#!/usr/bin/env python3
"""Decode and prefill throughput of titan_b200 on one B200, Qwen3-8B layer sizes, random bfloat16 weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  The workload is the benchmark configuration's: sequences that hold 2,048-token
prompts in a context of 8,192, decoded one token each per step.  ``value`` is decoded tokens per second at
batch 8 (device time, CUDA events around K replays of the captured decode step that start with 2,048 tokens in
the cache, each step feeding the token the step before sampled); ``e2e`` is the same K steps, from the same
prompts run again, through the Python entry point with host tokens in and out every step (wall clock); ``prefill`` is one
2,048-token prompt; ``roofline`` divides the bytes a decode step has to read (every weight once, the
live cache) by its time.  ``points`` holds the whole stated run, 256 steps from 2,048 cached tokens, at
batch 1, 8 and 64 (tokens per second, with ``_ms`` per step and ``_frac`` of the copy bandwidth beside
each), and batch 8 at the end of the context.  The prompts are really run (no cache is filled by hand).
The step reads far more than the 126 MB L2, so no flush is needed between iterations (``config.l2``).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_8B = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=36, hidden_size=4096,
                num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288,
                vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False,
                max_position_embeddings=40960, hidden_act="silu")
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            p = json.load(f)
        p["source"] = "measured"
        return p
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs (read-only queries)."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.proc, self.index = None, index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "25", "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def fill_cache_random(engine, slots, length):
    """Set-up of the small profiling case only: give every slot ``length`` tokens of random keys and values
    without running the prompts."""
    engine.cache.reserve({s: length for s in slots})
    for s in slots:
        engine.cache.commit(s, length)
        engine.cache.state.seq_len[s] = length           # the device copy, which a real step advances itself
    for g in engine.cache.groups:
        if hasattr(g, "pool"):
            g.storage.normal_(0.0, 1.0)


def run_prompts(engine, slots, length):
    """Every slot gets a prompt of ``length`` tokens of its own, eight prompts to a step."""
    from titan_b200 import StepEntry
    V = engine.vocab_size
    for at in range(0, len(slots), 8):
        part = slots[at:at + 8]
        engine.step([StepEntry(s, [(13 * i + 977 * s + 5) % V for i in range(length)], []) for s in part])


def decode_flops_and_bytes(engine, batch, kv_len):
    spec = engine.spec
    per_token_kv = 0
    for g in engine.cache.groups:
        if hasattr(g, "pool"):
            per_token_kv += len(g.layers) * 2 * g.need.num_kv_heads * g.need.head_dim * g.storage.element_size()
    return engine.model.weight_bytes() + batch * kv_len * per_token_kv


def prefill_flops(cfg, layers, T):
    H, F, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    Q, KV = cfg["num_attention_heads"] * cfg["head_dim"], cfg["num_key_value_heads"] * cfg["head_dim"]
    linear = 2 * T * (H * (Q + 2 * KV) + Q * H + 3 * H * F) * layers
    attn = 4 * Q * (T * (T + 1) / 2) * layers        # QK^T and PV over the causal half
    return linear + attn + 2 * H * V                 # LM head on the last row


def time_decode(engine, torch, K, batch, kv_timed, steps, warmup, end_to_end=True):
    """``steps`` timed decode steps of ``batch`` sequences whose caches hold ``kv_timed`` tokens when the first
    timed step begins: prompts of ``kv_timed - warmup`` tokens are run, then ``warmup`` untimed steps.  The steps
    are timed twice, each time from freshly run prompts: on the device alone (``Engine.decode_on_device``: the
    captured step replayed ``steps`` times, every step feeding the token that the step before sampled; CUDA events),
    and end to end through ``Engine.advance`` (host token ids in, sampled host token ids out, every step; wall clock).
    Returns (device ms per step, end-to-end ms per step or None, launcher calls in the device-timed steps, bytes
    copied to and from the device per end-to-end step)."""
    from titan_b200 import SamplerParams

    def started():
        slots = [engine.alloc_slot() for _ in range(batch)]
        engine.sampler.configure(slots, [SamplerParams.greedy()] * batch, list(range(batch)))
        run_prompts(engine, slots, kv_timed - warmup)
        tokens = [(7 * i + 1) % engine.vocab_size for i in range(batch)]
        return slots, tokens

    wall_ms, h2d, d2h = None, 0, 0
    if end_to_end:                                       # first: it is the number that a user sees
        slots, tokens = started()
        try:
            for _ in range(warmup):
                tokens = engine.advance(slots, tokens)
            h2d0, d2h0 = engine.h2d_bytes, engine.d2h_bytes
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(steps):
                tokens = engine.advance(slots, tokens)   # host token ids in, sampled host token ids out
            torch.cuda.synchronize()
            wall_ms = (time.perf_counter() - t0) * 1e3 / steps
            h2d, d2h = (engine.h2d_bytes - h2d0) // steps, (engine.d2h_bytes - d2h0) // steps
        finally:
            for s in slots:
                engine.free_slot(s)
    slots, tokens = started()
    try:
        for _ in range(max(1, warmup - 2)):
            tokens = engine.advance(slots, tokens)
        engine.decode_on_device(slots, warmup - max(1, warmup - 2))     # the last warm-up steps: the replayed graph itself
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        launches0 = K.launch_count + engine.graph_launches
        start.record()
        engine.decode_on_device(slots, steps)
        stop.record()
        torch.cuda.synchronize()
        dev_ms = start.elapsed_time(stop) / steps
        return dev_ms, wall_ms, K.launch_count + engine.graph_launches - launches0, h2d, d2h
    finally:
        for s in slots:
            engine.free_slot(s)


def time_prefill(engine, torch, T, warmup, reps, chunk=None):
    """One prompt of T tokens in one step, or (chunk) in steps of ``chunk`` tokens; (median, best) ms."""
    from titan_b200 import StepEntry
    prompt = [(13 * i + 5) % engine.vocab_size for i in range(T)]
    chunk = chunk or T
    times = []
    for r in range(warmup + reps):
        s = engine.alloc_slot()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for at in range(0, T, chunk):
            part = prompt[at:at + chunk]
            engine.step([StepEntry(s, part, [len(part) - 1] if at + chunk >= T else [])])
        stop.record()
        torch.cuda.synchronize()
        engine.free_slot(s)
        if r >= warmup:
            times.append(start.elapsed_time(stop))
    return statistics.median(times), min(times)


def run_ours(args):
    import torch

    from titan_b200 import Engine, kernels as K
    from titan_b200.config import config_from_dict
    pk = peaks()
    cfg = dict(QWEN3_8B)
    cfg["num_hidden_layers"] = args.layers
    context, B, kv0 = args.context, args.batch, args.prompt_tokens
    point_steps = 0 if args.skip_points else args.point_steps
    biggest = max(B, 1 if args.skip_points else 64)
    room = max(biggest * (kv0 + max(args.steps, point_steps) + 64), 8 * context if not args.skip_points else 0)
    engine = Engine.from_random(config_from_dict(cfg), seed=2, dtype="bfloat16", max_tokens=room,
                                max_context=context, max_slots=biggest, max_batch=biggest)
    hbm = pk["hbm_gbs"]

    def measured(batch, kv_timed, steps, end_to_end=True):
        ms, wall, launches, h2d, d2h = time_decode(engine, torch, K, batch, kv_timed, steps, args.warmup, end_to_end)
        gbs = decode_flops_and_bytes(engine, batch, kv_timed + steps // 2) / (ms * 1e-3) / 1e9
        return ms, wall, launches, h2d, d2h, gbs

    clocks = ClockSampler()
    clocks.start()
    dev_ms, wall_ms, launches, h2d, d2h, achieved = measured(B, kv0, args.steps)
    clock_rec = clocks.stop()
    value = B * 1e3 / dev_ms
    e2e = B * 1e3 / wall_ms
    points = {}
    if point_steps:
        for b in (1, 8, 64):                                   # the stated run: 256 steps after 2,048-token prompts
            ms, _, _, _, _, gbs = measured(b, kv0, point_steps, end_to_end=False)
            points[f"decode_b{b}"] = round(b * 1e3 / ms, 1)
            points[f"decode_b{b}_ms"] = round(ms, 4)
            points[f"decode_b{b}_frac"] = round(gbs / hbm, 4)
        tail = context - 20 - 1                                # and batch 8 at the end of the context
        ms, _, _, _, _, gbs = measured(8, tail, 20, end_to_end=False)
        points["decode_b8_context_end"] = round(8e3 / ms, 1)
        points["decode_b8_context_end_ms"] = round(ms, 4)
        points["decode_b8_context_end_frac"] = round(gbs / hbm, 4)
        points["steps"] = point_steps
        points["kv_len_at_context_end"] = tail
    T = args.prefill_tokens
    pre_clocks = ClockSampler()
    pre_clocks.start()
    pre_ms, pre_best = time_prefill(engine, torch, T, 3, 12)       # ~0.4 s back to back: the power cap is reached
    pre_rec = pre_clocks.stop()
    chunked_ms = time_prefill(engine, torch, T, 2, 6, chunk=512)[0]    # the same prompt in chunks of 512 (continuation steps)
    flops = prefill_flops(cfg, args.layers, T)
    engine.check_kernels()                                        # raises if a bounded wait gave up anywhere
    line = {
        "metric": "decode tok/s (Qwen3-8B layer sizes, bf16, batch 8, after 2,048-token prompts)", "value": round(value, 1), "unit": "tok/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dev_ms, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights (seed 2), prompts of token ids from a fixed pattern, run through the engine",
        "config": {"model": "Qwen3-8B shape", "layers": args.layers, "layers_of_model": 36, "hidden": 4096, "heads": 32,
                   "kv_heads": 8, "head_dim": 128, "intermediate": 12288, "vocab": 151936, "global_batch": B,
                   "seq_len": context, "kv_len_at_first_timed_step": kv0, "prefill_tokens": T,
                   "parallelism": "single_gpu", "l2": "inputs_larger_than_l2", "cache_fill": "prompts_run",
                   "peaks": pk["source"], "points_steps": point_steps},
        "e2e": {"value": round(e2e, 1), "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "prefill": {"value": round(T * 1e3 / pre_ms, 1), "tokens": T, "ms": round(pre_ms, 3),
                    "frac": round(flops / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
                    "frac_of_sustained_peak": round(flops / (pre_ms * 1e-3) / (pk.get("bf16_tflops_sustained", pk["bf16_tflops"]) * 1e12), 4),
                    "best_ms": round(pre_best, 3), "in_chunks_of_512_ms": round(chunked_ms, 3), "sm_mhz": pre_rec.get("sm_mhz"), "reasons": pre_rec.get("reasons")},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm, "unit": "GB/s",
                     "frac": round(achieved / hbm, 4)},
        "points": points, "clocks": clock_rec, "kernel_error": 0,
    }
    print(json.dumps(line))
    return 0


# The further configurations of the benchmark set: other layer sizes, ragged prompts, longer contexts, sampling.
QWEN3_4B = dict(QWEN3_8B, hidden_size=2560, intermediate_size=9728, tie_word_embeddings=True)
QWEN3_32B = dict(QWEN3_8B, num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, intermediate_size=25600)
OTHER_CONFIGS = {
    4: dict(name="Qwen3-4B shape", cfg=QWEN3_4B, seed=3, batch=8, prompt_range=(512, 16384), context=32768, steps=256,
            temperature=0.0, end_of_context=True),
    5: dict(name="Qwen3-32B shape", cfg=QWEN3_32B, seed=4, batch=16, prompt_range=(256, 4096), context=8192, steps=512,
            temperature=0.7, end_of_context=False),
}


def run_other(args, which):
    """Configurations 4 and 5: unequal prompts of seeded lengths in one step (prefill tokens per second over all of
    them), then the stated number of decode steps through the Python entry point (tokens per second, bytes a step
    must read over its time), and for configuration 4 the same at the end of its 32,768-token context."""
    import random

    import torch

    from titan_b200 import Engine, SamplerParams, StepEntry, kernels as K
    from titan_b200.config import config_from_dict
    c = OTHER_CONFIGS[which]
    pk = peaks()
    cfg = dict(c["cfg"])
    layers_of_model = cfg["num_hidden_layers"]
    if args.layers != 36:
        cfg["num_hidden_layers"] = args.layers
    B, context, steps = c["batch"], c["context"], c["steps"]
    rng = random.Random(c["seed"])
    lengths = [rng.randint(*c["prompt_range"]) for _ in range(B)]
    engine = Engine.from_random(config_from_dict(cfg), seed=c["seed"], dtype="bfloat16", max_tokens=B * context,
                                max_context=context, max_slots=B, max_batch=B)
    V = engine.vocab_size
    params = SamplerParams.greedy() if c["temperature"] <= 0 else SamplerParams(c["temperature"], 1.0, 0, 1.0, c["seed"])

    def run(lengths, steps):
        slots = [engine.alloc_slot() for _ in lengths]
        try:
            engine.sampler.configure(slots, [params] * len(slots), list(range(len(slots))))
            prompts = [[(13 * i + 977 * j + 5) % V for i in range(n)] for j, n in enumerate(lengths)]
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
            torch.cuda.synchronize()
            ev[0].record()
            at = 0
            while at < len(slots):                               # prompts of up to 65,536 tokens to a step
                take, total = [], 0
                while at + len(take) < len(slots) and (not take or total + lengths[at + len(take)] <= 65536):
                    total += lengths[at + len(take)]
                    take.append(at + len(take))
                engine.step([StepEntry(slots[j], prompts[j], []) for j in take])
                at += len(take)
            ev[1].record()
            tokens = [(7 * i + 1) % V for i in range(len(slots))]
            for _ in range(max(3, args.warmup)):
                tokens = engine.advance(slots, tokens)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            ev[2].record()
            for _ in range(steps):
                tokens = engine.advance(slots, tokens)
            ev[3].record()
            torch.cuda.synchronize()
            wall = (time.perf_counter() - t0) * 1e3 / steps
            engine.check_kernels()
            held = sum(lengths) + len(lengths) * (max(3, args.warmup) + steps // 2)
            step_bytes = decode_flops_and_bytes(engine, 1, held)
            ms = ev[2].elapsed_time(ev[3]) / steps
            return dict(prefill_ms=ev[0].elapsed_time(ev[1]), ms=ms, wall_ms=wall, gbs=step_bytes / ms / 1e6, bytes=step_bytes)
        finally:
            for s in slots:
                engine.free_slot(s)
    first = run(lengths, steps)
    points = {}
    if c["end_of_context"]:
        tail_steps = 128
        tail = run([context - tail_steps - max(3, args.warmup) - 1] * B, tail_steps)
        points = {"decode_at_context_end": round(B * 1e3 / tail["ms"], 1), "decode_at_context_end_ms": round(tail["ms"], 4),
                  "decode_at_context_end_frac": round(tail["gbs"] / pk["hbm_gbs"], 4), "kv_len_at_context_end": context - tail_steps - 1,
                  "prefill_of_long_prompts_tok_s": round(B * (context - tail_steps - max(3, args.warmup) - 1) * 1e3 / tail["prefill_ms"], 1)}
    line = {
        "metric": f"decode tok/s ({c['name']}, bf16, batch {B}, unequal prompts)", "value": round(B * 1e3 / first["ms"], 1), "unit": "tok/s",
        "n_gpus": 1, "steps": steps, "warmup": max(3, args.warmup), "ms_per_step": round(first["ms"], 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": f"synthetic: random weights (seed {c['seed']}), prompts of seeded lengths and patterned ids, run through the engine",
        "config": {"model": c["name"], "layers": cfg["num_hidden_layers"], "layers_of_model": layers_of_model, "hidden": cfg["hidden_size"],
                   "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "global_batch": B, "seq_len": context,
                   "prompt_tokens_min": min(lengths), "prompt_tokens_max": max(lengths), "prompt_tokens_total": sum(lengths),
                   "temperature": c["temperature"], "parallelism": "single_gpu", "l2": "inputs_larger_than_l2", "peaks": pk["source"]},
        "e2e": {"value": round(B * 1e3 / first["wall_ms"], 1), "unit": "tok/s", "h2d_bytes_per_step": 4 * B, "d2h_bytes_per_step": 4 * B},
        "prefill": {"value": round(sum(lengths) * 1e3 / first["prefill_ms"], 1), "tokens": sum(lengths), "ms": round(first["prefill_ms"], 3)},
        "roofline": {"bound": "hbm", "achieved": round(first["gbs"], 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(first["gbs"] / pk["hbm_gbs"], 4), "bytes_per_step": first["bytes"]},
        "points": points, "device_memory_gb": round(torch.cuda.max_memory_allocated() / 1e9, 1),
    }
    print(json.dumps(line))
    return 0


def profile_case(kv=2048):
    """The small case that the ncu summaries under profiles/ are captured on: ONE layer of the benchmark's sizes;
    two 2,048-token prompts in one step each, one in four chunks of 512 (continuation steps), then two decode
    steps at batch 8 and two at batch 1 after prompts of ``kv`` tokens, CUDA graphs off so that every kernel is
    a launch of its own.  A few GB on the device."""
    import torch

    from titan_b200 import Engine, SamplerParams, StepEntry
    from titan_b200.config import config_from_dict
    cfg = dict(QWEN3_8B)
    cfg["num_hidden_layers"] = 1
    batch = 8
    engine = Engine.from_random(config_from_dict(cfg), 2, "bfloat16", max_tokens=(batch + 1) * (kv + 128) + 4096, max_context=8192,
                                max_slots=batch + 2, decode_graphs=False)
    prompt = [(13 * i + 5) % 151936 for i in range(2048)]
    for _ in range(2):
        s = engine.alloc_slot()
        engine.step([StepEntry(s, prompt, [2047])])
        engine.free_slot(s)
    s = engine.alloc_slot()
    for at in range(0, 2048, 512):
        engine.step([StepEntry(s, prompt[at:at + 512], [])])
    engine.free_slot(s)
    for b in (batch, 1):
        slots = [engine.alloc_slot() for _ in range(b)]
        engine.sampler.configure(slots, [SamplerParams.greedy()] * b, list(range(b)))
        run_prompts(engine, slots, kv)
        tokens = [1] * b
        for _ in range(2):
            tokens = engine.advance(slots, tokens)
        for s in slots:
            engine.free_slot(s)
    torch.cuda.synchronize()
    engine.check_kernels()
    print("profile case done", tokens)
    return 0


def timeline(batch, kv=2048):
    """When the CTAs of every kernel of ONE captured decode step start, pass their wait for the kernel before, see
    their first tile, finish and end (microseconds from the step's first record), for the first layers of the
    benchmark's model; and the phases of the decode attention's CTAs.  Needs the tensor-core library built with the
    timeline probe: TITAN_B200_NVCC_FLAGS=-DTB_TIMELINE python bench.py --timeline 1.  Prints text lines."""
    import numpy as np
    import torch

    from titan_b200 import Engine, SamplerParams, kernels as K
    from titan_b200.config import config_from_dict
    engine = Engine.from_random(config_from_dict(dict(QWEN3_8B)), seed=2, dtype="bfloat16", max_tokens=batch * (kv + 256), max_context=8192,
                                max_slots=batch, max_batch=batch)
    records = 200000
    buf = torch.zeros(1 + 8 * records, dtype=torch.int64, device="cuda")
    if not K.timeline_attach(buf):
        print("the kernels were built without the timeline probe: set TITAN_B200_NVCC_FLAGS=-DTB_TIMELINE and run again")
        return 1
    slots = [engine.alloc_slot() for _ in range(batch)]
    engine.sampler.configure(slots, [SamplerParams.greedy()] * batch, list(range(batch)))
    run_prompts(engine, slots, kv)
    tokens = [1] * batch
    for _ in range(6):                                   # the step is captured from the third one on
        tokens = engine.advance(slots, tokens)
    torch.cuda.synchronize()
    buf.zero_()
    torch.cuda.synchronize()
    engine.advance(slots, tokens)                       # the one step that is recorded
    torch.cuda.synchronize()
    K.timeline_attach(None)
    engine.check_kernels()
    host = buf.cpu().numpy()
    n = int(host[0])
    rec = host[1:1 + 8 * min(n, records)].reshape(-1, 8)
    if os.environ.get("TITAN_B200_TIMELINE_RAW"):        # the records themselves, for a closer look: tag, block | sm << 32, six stamps (ns)
        np.save(os.environ["TITAN_B200_TIMELINE_RAW"], rec)
    launches = []                                       # a launch = the records of one tag, in the order of their starts, a grid at a time
    for tag in np.unique(rec[:, 0]):
        r = rec[rec[:, 0] == tag]
        r = r[np.argsort(r[:, 2], kind="stable")]
        per = (tag // 100) * (tag % 100) if tag < 100000 else int((r[:, 1] & 0xffffffff).max()) + 1
        launches += [(int(tag), r[i:i + per]) for i in range(0, len(r), per)]
    launches.sort(key=lambda x: x[1][:, 2].min())
    base = launches[0][1][:, 2].min()
    us = lambda v: (int(v) - int(base)) / 1e3
    seen = lambda a: a[a > 0] if (a > 0).any() else np.array([base])
    print(f"batch {batch}, {kv} cached tokens, {n} CTAs recorded in one captured step; times in us")
    print("kernel (tiles x K slices | attention splits)  CTAs  start first..last  wait passed min..max  first tile min..max  last tile done min..max  end max")
    for tag, r in launches:
        t0, t1, t2, t3, t4 = (r[:, 2 + k] for k in range(5))
        name = f"attention, {tag - 100000} splits" if tag >= 100000 else f"product {tag // 100} x {tag % 100}"
        print(f"{name:26s} {len(r):5d}  {us(t0.min()):8.2f} {us(t0.max()):8.2f}   {us(seen(t1).min()):8.2f} {us(seen(t1).max()):8.2f}   "
              f"{us(seen(t2).min()):8.2f} {us(seen(t2).max()):8.2f}   {us(seen(t3).min()):8.2f} {us(seen(t3).max()):8.2f}   {us(seen(t4).max()):8.2f}")
        if tag >= 100000:
            t5 = r[:, 7]
            med = lambda a, b: float(np.median((a.astype(np.int64) - b.astype(np.int64))[(a > 0) & (b > 0)])) / 1e3 if ((a > 0) & (b > 0)).any() else float("nan")
            print(f"    a CTA's phases (medians): start -> wait passed {med(t1, t0):.2f}, -> queries ready {med(t2, t1):.2f}, -> pages done {med(t3, t2):.2f}, "
                  f"-> all parts here {med(t5, t3):.2f}, -> end {med(t4, t5 if (t5 > 0).any() else t3):.2f}")
        if us(t0.min()) > 320:
            break
    return 0


def micro():
    """Kernels of the benchmark's layer sizes timed alone with CUDA events (back to back, after warm-up);
    the figures that the summaries under profiles/ quote beside the ncu captures.  Prints text lines."""
    import torch

    from titan_b200 import Engine, StepEntry, kernels as K
    from titan_b200.config import config_from_dict
    K.lib()
    st = torch.cuda.current_stream().cuda_stream

    def timed(fn, n):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / n * 1e3           # microseconds

    H, F = QWEN3_8B["hidden_size"], QWEN3_8B["intermediate_size"]
    QKV = (QWEN3_8B["num_attention_heads"] + 2 * QWEN3_8B["num_key_value_heads"]) * QWEN3_8B["head_dim"]
    shapes = [("qkv", QKV, H, K.EPI_ADD, K.EPI_STORE), ("o", H, H, K.EPI_ADD, K.EPI_ADD),
              ("gate+up", 2 * F, H, K.EPI_SWIGLU, K.EPI_SWIGLU), ("down", H, F, K.EPI_ADD, K.EPI_ADD)]
    copies = 12                                       # different weights per call: more than L2 in total
    for M in (1, 8, 64):
        for name, N, Kd, epi, _ in shapes:
            ws = [torch.randn(N, Kd, device="cuda").to(torch.bfloat16) for _ in range(copies)]
            x = torch.randn(M, Kd, device="cuda").to(torch.bfloat16)
            out = torch.zeros(M, N // 2 if epi == K.EPI_SWIGLU else N, device="cuda",
                              dtype=torch.bfloat16 if epi == K.EPI_SWIGLU else torch.float32)
            us = timed(lambda: [K.gemm_tc(x, w, out, epi, st) for w in ws], 5) / copies
            print(f"decode product M={M:2d} {name:8s} {N:6d} x {Kd:5d}: {us:7.1f} us  {N * Kd * 2 / us / 1e6:5.2f} TB/s", flush=True)
            del ws
    M = 2048
    for name, N, Kd, _, epi in shapes:
        w = torch.randn(N, Kd, device="cuda").to(torch.bfloat16)
        x = torch.randn(M, Kd, device="cuda").to(torch.bfloat16)
        out = torch.zeros(M, N // 2 if epi == K.EPI_SWIGLU else N, device="cuda",
                          dtype=torch.float32 if epi == K.EPI_ADD else torch.bfloat16)
        for pair in (True, False):
            K.set_gemm_pair(pair)
            us = timed(lambda: K.gemm_tc(x, w, out, epi, st), 20)
            print(f"prompt product M={M} {name:8s} {N:6d} x {Kd:5d} {'CTA pairs' if pair else 'one CTA  '}: {us:7.1f} us  "
                  f"{2 * M * N * Kd / us / 1e6:5.0f} TFLOP/s", flush=True)
        K.set_gemm_pair(True)
    # the other kernels of a prompt, inside one layer's step: each launcher call repeated in place
    cfg = dict(QWEN3_8B)
    cfg["num_hidden_layers"] = 1
    engine = Engine.from_random(config_from_dict(cfg), 2, "bfloat16", max_tokens=8192, max_context=8192, max_slots=2, max_batch=2)
    found = {}

    def repeated(name):
        f = getattr(K, name)

        def g(*a, **k):
            found.setdefault(name, []).append(timed(lambda: f(*a, **k), 20))
        return g
    originals = {n: getattr(K, n) for n in ("qk_norm_rope", "rmsnorm", "attn_prefill_tc")}
    for n in originals:
        setattr(K, n, repeated(n))
    try:
        s = engine.alloc_slot()
        engine.step([StepEntry(s, [(13 * i + 5) % engine.vocab_size for i in range(M)], [M - 1])])
    finally:
        for n, f in originals.items():
            setattr(K, n, f)
    for n, v in found.items():
        print(f"prompt of {M} tokens, {n}: " + ", ".join(f"{x:.1f}" for x in v) + " us (rows: " +
              ("2048, 2048, 1" if n == "rmsnorm" else "2048") + ")", flush=True)
    # sampling alone: one call of the device sampler on float32 logits of the model's vocabulary
    from titan_b200.cache import SlotState
    from titan_b200.sampling import DeviceSampler, SamplerParams
    V = QWEN3_8B["vocab_size"]
    for B in (1, 8, 64):
        state = SlotState(B, "cuda")
        sampler = DeviceSampler(state, B, V, "cuda")
        slots = list(range(B))
        slot_t = torch.tensor(slots, dtype=torch.int32, device="cuda")
        logits = torch.randn(B, V, device="cuda") * 3
        line = []
        for name, p in (("greedy", SamplerParams.greedy()), ("temperature", SamplerParams(0.8, 1.0, 0, 1.0, 3)),
                        ("top_k 40", SamplerParams(0.8, 1.0, 40, 1.0, 3)), ("top_p 0.95", SamplerParams(0.8, 0.95, 0, 1.0, 3)),
                        ("top_k 40 top_p 0.95 penalty 1.1", SamplerParams(0.8, 0.95, 40, 1.1, 3))):
            sampler.configure(slots, [p] * B, slots)
            line.append(f"{name} {timed(lambda: sampler.sample(logits, slot_t, st), 50):.1f}")
        print(f"sampling, {B} rows of {V}: " + ", ".join(line) + " us", flush=True)
    print("wait errors:", K.gemm_tc_error(), K.attn_tc_error())
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=36, help="fewer than 36 only where time needs it; both numbers are reported")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--prompt-tokens", type=int, default=2048, help="tokens every sequence holds when the first timed step begins")
    ap.add_argument("--point-steps", type=int, default=256, help="decode steps of each entry of 'points'")
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--config", type=int, default=3, choices=[3, 4, 5], help="3: the benchmark configuration (default); 4, 5: the Qwen3-4B and Qwen3-32B shaped ones")
    ap.add_argument("--profile-case", action="store_true", help="run the small one-layer case used for ncu captures and exit")
    ap.add_argument("--micro", action="store_true", help="time the layer's kernels alone (CUDA events) and exit; text lines, not the JSON line")
    ap.add_argument("--timeline", type=int, default=0, metavar="BATCH", help="when the CTAs of one captured decode step's kernels start, wait and end "
                    "(needs TITAN_B200_NVCC_FLAGS=-DTB_TIMELINE); text lines, not the JSON line")
    args = ap.parse_args()
    if args.profile_case:
        return profile_case(args.prompt_tokens)
    if args.micro:
        return micro()
    if args.timeline:
        return timeline(args.timeline, args.prompt_tokens)
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "berniehans/titan is a Rust workspace (cargo is not installed) "
                          "that needs GGUF Q4_K weights and NVRTC for compute_86; it cannot be installed or run offline here"}))
        return 0
    if args.gpus != 1:
        print("titan_b200 is a single-GPU library: bench.py runs at --gpus 1 only")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.config != 3:
        return run_other(args, args.config)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
