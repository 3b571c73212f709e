"""bin/trace_run as a user runs it: a subprocess, steps on stdin, logits in files."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from helpers import TINY, TOL, random_tokens, random_weights, rel_l2, write_folder
from plain import qwen3_plain as P

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_trace(folder, dtype, out, max_tokens, steps):
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
                        "--out", out, "--max-tokens", str(max_tokens)],
                       input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done")] == [f"done {s['step']}" for s in steps]
    return p


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_three_ways(tmp_path, dtype):
    cfg = TINY["C"]
    w = random_weights(cfg, 5, torch.bfloat16, std=0.08)
    folder = write_folder(str(tmp_path / "model"), cfg, w)
    w32 = {k: v.float() for k, v in w.items()}
    V = cfg["vocab_size"]
    reqs = {"a": random_tokens(100, V, 1), "b": random_tokens(37, V, 2), "c": random_tokens(70, V, 3)}
    want = {k: P.forward_logits(cfg, w32, t).numpy() for k, t in reqs.items()}

    def read(out, step, rows):
        a = np.fromfile(os.path.join(out, f"{step}.f32"), dtype="<f4")
        assert a.size == rows * V
        return a.reshape(rows, V)

    # 1. each request alone and whole; 2. whole but the last 32, then one by one (same process: slots are reused)
    steps, n = [], 0
    for k, t in reqs.items():
        steps.append({"step": n, "entries": [{"id": k, "tokens": t, "want": list(range(len(t)))}], "end": [k]})
        n += 1
    marks = {}
    for k, t in reqs.items():
        cut = len(t) - 32
        marks[k] = n
        steps.append({"step": n, "entries": [{"id": k + "2", "tokens": t[:cut], "want": [cut - 1]}], "end": []})
        n += 1
        for j in range(cut, len(t)):
            steps.append({"step": n, "entries": [{"id": k + "2", "tokens": [t[j]], "want": [0]}],
                          "end": [k + "2"] if j == len(t) - 1 else []})
            n += 1
    out1 = str(tmp_path / "o1")
    run_trace(folder, dtype, out1, 128, steps)           # 128 tokens: one request of up to 100 at a time
    for i, k in enumerate(reqs):
        assert rel_l2(torch.from_numpy(read(out1, i, len(reqs[k]))), torch.from_numpy(want[k])) < TOL[dtype]
        cut = len(reqs[k]) - 32
        got = np.concatenate([read(out1, marks[k] + j, 1) for j in range(33)])
        assert rel_l2(torch.from_numpy(got), torch.from_numpy(want[k][cut - 1:])) < TOL[dtype]

    # 3. a batch of unequal lengths that starts together; shorter requests end earlier; a step that wants nothing
    steps = [{"step": 0, "entries": [{"id": k, "tokens": t[:20], "want": [19] if k != "b" else []} for k, t in reqs.items()], "end": []}]
    n, at = 1, 20
    while any(at < len(t) for t in reqs.values()):
        live = [k for k, t in reqs.items() if at < len(t)]
        steps.append({"step": n, "entries": [{"id": k, "tokens": [reqs[k][at]], "want": [0]} for k in live],
                      "end": [k for k in live if at == len(reqs[k]) - 1]})
        n += 1
        at += 1
    out2 = str(tmp_path / "o2")
    run_trace(folder, dtype, out2, 128 + 64 + 128, steps)
    first = read(out2, 0, 2)
    assert rel_l2(torch.from_numpy(first), torch.from_numpy(np.stack([want["a"][19], want["c"][19]]))) < TOL[dtype]
    for s in steps[1:]:
        got = read(out2, s["step"], len(s["entries"]))
        pos = 20 + s["step"] - 1
        ref = np.stack([want[e["id"]][pos] for e in s["entries"]])
        assert rel_l2(torch.from_numpy(got), torch.from_numpy(ref)) < TOL[dtype], s["step"]


def test_bad_model_folder_fails_loudly(tmp_path):
    cfg = TINY["A"]
    w = random_weights(cfg, 0)
    del w["model.norm.weight"]
    folder = write_folder(str(tmp_path / "m"), cfg, w)
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32",
                        "--out", str(tmp_path / "o"), "--max-tokens", "64"], input="", capture_output=True, text=True, timeout=600)
    assert p.returncode != 0 and "missing (1): model.norm.weight" in p.stderr
