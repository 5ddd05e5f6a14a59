"""bin/trace_run as a program: the same requests whole, with the last 32 tokens one by one,
and in batches of unequal lengths, in 32-bit and in bfloat16, against the plain implementation."""
import json
import subprocess
from pathlib import Path

import numpy as np
import pytest

import tiny
from helpers import CONFIGS, check_logits, plain_logits

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def run_trace(model_dir, dtype, out_dir, max_tokens, steps):
    text = "".join(json.dumps(s) + "\n" for s in steps)
    proc = subprocess.run([str(ROOT / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", dtype,
                           "--out", str(out_dir), "--max-tokens", str(max_tokens)],
                          input=text, capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-3000:]
    assert proc.stdout.split() == [w for s in steps for w in ("done", str(s["step"]))]
    return proc


def read(out_dir, step, vocab):
    return np.fromfile(out_dir / f"{step}.f32", dtype="<f4").reshape(-1, vocab)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b"])
def test_three_ways_of_cutting(model_dirs, tmp_path, name, dtype):
    d = model_dirs[(name, dtype)]
    cfg = CONFIGS[name]
    V = cfg["vocab_size"]
    lens = {"r0": 40, "r1": 97, "r2": 64, "r3": 33, "r4": 120}
    reqs = {k: tiny.prompt_tokens(cfg, n, 800 + i) for i, (k, n) in enumerate(lens.items())}
    want = {k: plain_logits(d, t) for k, t in reqs.items()}

    # 1. each request alone and whole
    steps = [{"step": i, "entries": [{"id": k, "tokens": t, "want": list(range(len(t)))}], "end": [k]}
             for i, (k, t) in enumerate(reqs.items())]
    run_trace(d, dtype, tmp_path / "whole", 128, steps)
    for i, k in enumerate(reqs):
        check_logits(read(tmp_path / "whole", i, V), want[k], dtype, f"{k} whole")

    # 2. the prefix whole, then the last 32 tokens one by one
    steps, expect, n = [], {}, 0
    for k, t in reqs.items():
        head = len(t) - 32
        steps.append({"step": n, "entries": [{"id": k, "tokens": t[:head], "want": [head - 1]}], "end": []})
        expect[n] = want[k][head - 1:head]
        n += 1
        for p in range(head, len(t)):
            steps.append({"step": n, "entries": [{"id": k, "tokens": [t[p]], "want": [0]}],
                          "end": [k] if p == len(t) - 1 else []})
            expect[n] = want[k][p:p + 1]
            n += 1
    run_trace(d, dtype, tmp_path / "tail", 128, steps)
    for s, w in expect.items():
        check_logits(read(tmp_path / "tail", s, V), w, dtype, f"tail step {s}")

    # 3. batches of unequal lengths, shorter requests end earlier, one batch after another;
    #    the cache holds one batch only, so pages and slots are used again
    steps, expect, n = [], {}, 0
    for batch in (["r0", "r1", "r2"], ["r3", "r4"], ["r2", "r0", "r3"]):
        pre = {k: len(reqs[k]) - (5 + 7 * i) for i, k in enumerate(batch)}   # unequal numbers of decode steps
        steps.append({"step": n, "entries": [{"id": k, "tokens": reqs[k][:pre[k]], "want": [0, pre[k] - 1]}
                                             for k in batch], "end": []})
        expect[n] = np.concatenate([want[k][[0, pre[k] - 1]] for k in batch])
        n += 1
        pos, live = dict(pre), list(batch)
        while live:
            ending = [k for k in live if pos[k] == len(reqs[k]) - 1]
            steps.append({"step": n, "entries": [{"id": k, "tokens": [reqs[k][pos[k]]], "want": [0]} for k in live],
                          "end": ending})
            expect[n] = np.stack([want[k][pos[k]] for k in live])
            n += 1
            for k in live:
                pos[k] += 1
            live = [k for k in live if k not in ending]
    run_trace(d, dtype, tmp_path / "batches", 64 * 5, steps)
    for s, w in expect.items():
        check_logits(read(tmp_path / "batches", s, V), w, dtype, f"batched step {s}")


def test_steps_without_wanted_places_write_nothing(model_dirs, tmp_path):
    d = model_dirs[("a", "float32")]
    t = tiny.prompt_tokens(tiny.TINY_A, 10, 900)
    steps = [{"step": 0, "entries": [{"id": 1, "tokens": t[:9], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": 1, "tokens": t[9:], "want": [0]}], "end": [1]}]
    run_trace(d, "float32", tmp_path / "o", 64, steps)
    assert not (tmp_path / "o" / "0.f32").exists()
    check_logits(read(tmp_path / "o", 1, 256), plain_logits(d, t)[9:], "float32")
