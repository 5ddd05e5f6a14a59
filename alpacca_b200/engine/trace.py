"""Trace replay: feeds given token ids through the model step by step and
writes the logits at the wanted places.  Nothing is sampled.

It drives the engine that generation uses (`Engine.step`, its cache, its
kernels).  The reference's nearest thing is `greedy_trace` of tests/smoke.py:743-755,
which returns the logits of every step of one sequence.

Input, one JSON object per line:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
An id seen for the first time starts a sequence (a slot is taken); `end` lists
ids whose slots are given back after the step.  For a step with wanted places
`<out>/<step>.f32` holds float32 little-endian logits [wanted, vocab], in the
order of the entries and of `want`.  After every step `done <step>` is printed
and flushed.
"""
from __future__ import annotations

import json
import sys
from pathlib import Path

import torch

from .engine import Engine
from .loading import load_model_dir, resolve_dtype
from .step import StepEntry


def replay(model_dir, dtype, out_dir, max_tokens: int, lines, out_stream) -> int:
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    max_tokens = int(max_tokens)
    if max_tokens <= 0:
        raise ValueError("--max-tokens must be positive")
    model = load_model_dir(model_dir, resolve_dtype(dtype), "cuda", max_positions=max_tokens)
    engine = Engine(model, max_tokens=max_tokens, max_slots=min(max(-(-max_tokens // 64), 1), 4096))
    slots: dict[str, int] = {}
    for line in lines:
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
            entries.append(StepEntry(slots[rid], [int(t) for t in e["tokens"]],
                                     [int(w) for w in e.get("want", [])]))
        if entries:
            logits = engine.step(entries)
            if logits.shape[0]:
                arr = logits.to(torch.float32).cpu().contiguous().numpy().astype("<f4", copy=False)
                engine.wait()          # nothing is written from a step whose kernels gave up
                arr.tofile(out_dir / f"{step}.f32")
            else:
                engine.wait()
        for rid in rec.get("end", []):
            rid = str(rid)
            if rid in slots:
                engine.free_slot(slots.pop(rid))
        out_stream.write(f"done {step}\n")
        out_stream.flush()
    return 0


def main(argv=None) -> int:
    import argparse
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for the <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64)")
    args = ap.parse_args(argv)
    try:
        return replay(args.model, args.dtype, args.out, args.max_tokens, sys.stdin, sys.stdout)
    except (RuntimeError, ValueError) as e:
        print(f"trace_run: error: {e}", file=sys.stderr)
        return 1
