#!/usr/bin/env python3
"""Decode and prefill throughput of alpacca_b200 on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--shape 1b|7b|8b]

Workloads (layer sizes, prompts and sampling as the benchmark configurations name them; random
bfloat16 weights N(0, 0.02), seeded uniform-random token ids):

  1b (default)  Llama-3.2-1B sizes, context 4096.  8 sequences, each prefilled with 512 tokens, then
                K greedy decode steps (256 unless --steps says otherwise).  Also one prompt of 2,048
                tokens (`prefill`) and decode at batch 1 and 64 (`points`).
  7b            Llama-2-7B sizes.  8 prompts with lengths uniform in [16, 1024], then 128 greedy steps.
  8b            Llama-3.1-8B sizes.  64 prompts with lengths uniform in [128, 2048], then 256 steps at
                temperature 1.0 with a seeded generator; the cache holds 4,096 tokens per sequence.

A "step" is one decode step of the whole batch.  `value` is decoded tokens per second, timed on the
device with CUDA events around exactly K steps replayed from the engine's CUDA graph (a step's sampled
token is the next step's input, on the device).  `e2e` is the same workload through the Python entry
point (`alpacca_b200.api.generate`): token ids in from host lists, token ids out to host lists, with
the per-step host traffic that serving has.  `prefill` is the 2,048-token prompt (1b) or the
workload's own unequal batch of prompts in one step (7b, 8b); `roofline` divides the bytes a decode
step must read (all weights once, plus the cache of the live requests) by the step time.  Every step
streams more bytes than the L2 holds, so nothing is flushed between timed iterations.  The default run
(1b) also times the decode of the 7b and 8b workloads, each in a child process, with their own numbers of
steps: `points.decode_7b_b8`, `points.decode_8b_b64` and `other_workloads` (--no-other-workloads leaves
them out).

`--impl reference` runs the same workload through the unmodified reference (a CPU engine for one
sequence at a time: it takes the sequences one after another) and prints the same line.

One JSON line goes to standard output.  With --gpus N > 1 it prints a line that says so and exits
with 2: this library runs on one GPU.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

LLAMA3_SCALING = {"rope_type": "llama3", "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                  "original_max_position_embeddings": 8192}
# No stop token is configured: with random weights a sequence must not end by chance.
SHAPES = {
    "1b": {
        "name": "Llama-3.2-1B shape",
        "config": {"architectures": ["LlamaForCausalLM"], "num_hidden_layers": 16, "hidden_size": 2048,
                   "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64, "intermediate_size": 8192,
                   "vocab_size": 128256, "max_position_embeddings": 131072, "rms_norm_eps": 1e-5,
                   "rope_theta": 500000.0, "rope_pairing": "neox", "rope_scaling": dict(LLAMA3_SCALING, factor=32.0),
                   "tie_word_embeddings": True, "hidden_act": "silu", "bos_token_id": 128000},
        "context": 4096, "batch": 8, "prompt_lengths": (512, 512), "steps": 256, "temperature": 0.0,
        "prefill_tokens": 2048, "points": (1, 64),
    },
    "7b": {
        "name": "Llama-2-7B shape",
        "config": {"architectures": ["LlamaForCausalLM"], "num_hidden_layers": 32, "hidden_size": 4096,
                   "num_attention_heads": 32, "num_key_value_heads": 32, "head_dim": 128, "intermediate_size": 11008,
                   "vocab_size": 32000, "max_position_embeddings": 4096, "rms_norm_eps": 1e-5,
                   "rope_theta": 10000.0, "rope_pairing": "neox", "rope_scaling": None,
                   "tie_word_embeddings": False, "hidden_act": "silu", "bos_token_id": 1},
        "context": 4096, "batch": 8, "prompt_lengths": (16, 1024), "steps": 128, "temperature": 0.0,
        "prefill_tokens": None, "points": (),
    },
    "8b": {
        "name": "Llama-3.1-8B shape",
        "config": {"architectures": ["LlamaForCausalLM"], "num_hidden_layers": 32, "hidden_size": 4096,
                   "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 14336,
                   "vocab_size": 128256, "max_position_embeddings": 131072, "rms_norm_eps": 1e-5,
                   "rope_theta": 500000.0, "rope_pairing": "neox", "rope_scaling": dict(LLAMA3_SCALING, factor=8.0),
                   "tie_word_embeddings": False, "hidden_act": "silu", "bos_token_id": 128000},
        "context": 4096, "batch": 64, "prompt_lengths": (128, 2048), "steps": 256, "temperature": 1.0,
        "prefill_tokens": None, "points": (),
    },
}
SAMPLING_SEED = 1234
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.is_file():
        try:
            d = json.loads(p.read_text())
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
        except (ValueError, KeyError):
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        out, _ = self.proc.communicate(timeout=10)
        mhz, top, reasons = [], None, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 6 or not f[0].isdigit():
                continue
            mhz.append(int(f[0]))
            top = int(f[1])
            reasons |= {n for n, v in zip(names, f[2:6]) if v.lower().startswith("active")}
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": top, "reasons": sorted(reasons)}


def workload_prompts(shape, batch, seed):
    """`batch` prompts of the workload: lengths uniform in the shape's range, uniform-random token ids."""
    import random
    rng = random.Random(seed)
    lo, hi = shape["prompt_lengths"]
    vocab = shape["config"]["vocab_size"]
    lengths = [rng.randint(lo, hi) for _ in range(batch)]
    return [[rng.randrange(vocab) for _ in range(n)] for n in lengths]


def sampler_params(shape):
    from alpacca_b200.sampling import SamplerParams
    if shape["temperature"] <= 0:
        return SamplerParams.greedy()
    # plain temperature sampling over the whole vocabulary, seeded
    return SamplerParams(temperature=shape["temperature"], top_k=0, top_p=1.0, repeat_penalty=1.0, seed=SAMPLING_SEED)


def model_bytes(model) -> int:
    """Bytes of every weight a decode step reads once (a tied embedding table counts once: it is the head;
    an untied one is read by rows only and does not count)."""
    seen, total = set(), 0
    head_is_table = model.decoder.spec.head.tied_to is not None
    stack = [model.decoder]
    while stack:
        part = stack.pop()
        stack.extend(part.children())
        if type(part).__name__ == "RotaryEncoding" or (type(part).__name__ == "TokenEmbedding" and not head_is_table):
            continue
        for v in vars(part).values():
            if hasattr(v, "data_ptr") and hasattr(v, "element_size") and v.is_cuda and v.dim() >= 1:
                if v.data_ptr() not in seen and v.dtype.is_floating_point:
                    seen.add(v.data_ptr())
                    total += v.numel() * v.element_size()
    return total


def prefill_flops(cfg, lengths) -> float:
    """Floating-point operations of one step that runs prompts of these lengths whole and asks for the
    logits of each prompt's last token."""
    E, H, K, D = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    F, L, V = cfg["intermediate_size"], cfg["num_hidden_layers"], cfg["vocab_size"]
    per_token = 2.0 * (E * (H + 2 * K) * D + H * D * E + 3 * E * F)
    attention = sum(2.0 * 2.0 * H * D * T * (T + 1) / 2.0 for T in lengths)
    return L * (sum(lengths) * per_token + attention) + len(lengths) * 2.0 * V * E


def start_batch(model, shape, batch, seed):
    """Prefills the workload's prompts in one step, samples their first tokens; returns what the decoder needs."""
    from alpacca_b200.engine.step import StepEntry
    from alpacca_b200.sampling import DeviceSampler
    eng = model.engine
    prompts = workload_prompts(shape, batch, seed)
    slots = [eng.alloc_slot() for _ in prompts]
    sampler = DeviceSampler(sampler_params(shape), eng.device)
    states = [sampler.new_state(i, p) for i, p in enumerate(prompts)]
    logits = eng.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
    first = sampler.sample(logits, states)
    decoder = model.decoder_for(sampler)
    return slots, decoder, [(s, t, st) for s, t, st in zip(slots, first, states)]


def measure_decode(model, shape, batch, steps, warmup, seed=0):
    """Device-timed decode: (tokens per second, ms per step, mean tokens held per step, kernels per step)."""
    import torch
    from alpacca_b200 import ops
    slots, decoder, live = start_batch(model, shape, batch, seed)
    try:
        warm = max(warmup, 3)
        # the pages of the whole run are reserved first, so that the warm-up steps and the timed
        # steps have the same batch shape (and the capture of its graph falls into the warm-up)
        model.engine.cache.reserve([(s, warm + steps) for s in slots])
        decoder.run(live, warm)
        before = ops.launches
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        held0 = sum(model.engine.length(s) for s in slots)
        t0.record()
        decoder.run(live, steps)
        t1.record()
        torch.cuda.synchronize()
        ops.check_tc_status()
        ms = t0.elapsed_time(t1)
        eager_launches = ops.launches - before
        per_step = getattr(decoder, "kernels_per_step", None) or (eager_launches // max(steps, 1))
        # step i reads the held0 + i * batch tokens cached so far (and appends one per sequence)
        measure_decode.last_held = held0 + batch * (steps - 1) / 2.0
        return batch * steps / (ms / 1e3), ms / steps, measure_decode.last_held, per_step
    finally:
        for s in slots:
            model.engine.free_slot(s)


def measure_e2e(model, shape, batch, steps, seed=1):
    """The same decode through the Python entry point: host token lists in, host token lists out."""
    from alpacca_b200.api import generate
    prompts = workload_prompts(shape, batch, seed)
    params = sampler_params(shape)
    generate(model, prompts, params, n_predict=8, stop_token_ids=[])     # warm-up (graphs)
    res = generate(model, prompts, params, n_predict=steps + 1, stop_token_ids=[])
    tokens = sum(r.tokens - 1 for r in res)            # the first token of each comes from the prompt step
    seconds = max(r.seconds for r in res)
    return tokens / seconds, seconds


def measure_prefill(model, prompts, runs=5):
    """Median device time (ms) of one step that runs `prompts` whole."""
    import numpy as np
    import torch
    from alpacca_b200.engine.step import StepEntry
    eng = model.engine
    prompts = [np.asarray(p, dtype=np.int32) for p in prompts]     # token ids as arrays, as a tokenizer hands them over
    times = []
    for i in range(runs + 2):
        slots = [eng.alloc_slot() for _ in prompts]
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        eng.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
        t1.record()
        eng.wait()
        for s in slots:
            eng.free_slot(s)
        if i >= 2:
            times.append(t0.elapsed_time(t1))
    return statistics.median(times)


def other_workload(name: str, timeout: float = 240.0) -> dict:
    """`python bench.py --shape NAME --only decode` in a child process; its short line, or why there is none."""
    cmd = [sys.executable, str(Path(__file__).resolve()), "--shape", name, "--only", "decode"]
    try:
        out = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout)
    except subprocess.TimeoutExpired:
        return {"unavailable": f"no result within {timeout:.0f} s"}
    lines = [ln for ln in out.stdout.splitlines() if ln.startswith("{")]
    if out.returncode != 0 or not lines:
        tail = (out.stderr or out.stdout).strip().splitlines()[-1:] or [""]
        return {"unavailable": f"exit code {out.returncode}: {tail[0][:200]}"}
    d = json.loads(lines[-1])
    return {k: d[k] for k in ("batch", "tok_s", "ms_per_step", "gb_s", "of_hbm_peak", "steps") if k in d}


def flat_config(shape, cfg, layers_full, batch, steps, weights, kv_per_token, prompts):
    lens = [len(p) for p in prompts]
    lo, hi = shape["prompt_lengths"]
    return {"model": shape["name"], "layers": cfg["num_hidden_layers"], "layers_of_config": layers_full,
            "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
            "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
            "ffn": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "global_batch": batch,
            "prompt_len": lo if lo == hi else f"uniform in [{lo}, {hi}], seeded (sum {sum(lens)})",
            "seq_len": shape["context"], "decode_steps": steps,
            "sampling": "greedy" if shape["temperature"] <= 0 else f"temperature {shape['temperature']}, seeded",
            "parallelism": "single GPU", "l2": "inputs larger than L2 (no flush)",
            "weight_bytes": weights, "kv_bytes_per_token": kv_per_token}


def metric_name(shape, batch):
    lo, hi = shape["prompt_lengths"]
    prompt = f"{lo}-token prompts" if lo == hi else f"prompts of {lo} to {hi} tokens"
    return f"decode tok/s at batch {batch} ({shape['name']}, {prompt}, context {shape['context']})"


def run_ours(args):
    import torch
    from alpacca_b200.api import Model

    assert torch.cuda.is_available(), "bench.py needs a CUDA device"
    torch.cuda.set_device(0)
    pk = peaks()
    shape = dict(SHAPES[args.shape])
    if args.only == "decode" and args.prompt_len:
        shape["prompt_lengths"] = (args.prompt_len, args.prompt_len)
        # room for the prompt, the warm-up steps and the timed steps in every slot
        shape["context"] = max(shape["context"], args.prompt_len + max(args.warmup, 3) + (args.steps or shape["steps"]) + 1)
    if args.only == "prefill" and args.prefill_tokens:
        shape["prefill_tokens"] = args.prefill_tokens
        shape["context"] = max(shape["context"], args.prefill_tokens)
    cfg = dict(shape["config"])
    layers_full = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    batch = args.batch or shape["batch"]
    if args.only == "prefill" and args.prefill_tokens and not args.batch:
        batch = 1           # one prompt: the cache is sized for it alone
    steps = args.steps or shape["steps"]
    biggest = max([batch, *shape["points"]]) if args.only == "all" else batch
    model = Model.random(cfg, seed=0, n_ctx=shape["context"], dtype="bfloat16", max_batch=biggest)
    weights = model_bytes(model)
    kv_per_token = sum(g.bytes_per_token for g in model.engine.cache.kv_groups)

    if args.only == "decode":
        tps, ms_step, _, kernels = measure_decode(model, shape, batch, steps, args.warmup)
        held = measure_decode.last_held
        gbs = (weights + held * kv_per_token) / (ms_step / 1e3) / 1e9
        print(json.dumps({"only": "decode", "shape": args.shape, "batch": batch, "steps": steps, "tok_s": round(tps, 1),
                          "ms_per_step": round(ms_step, 4), "kernels_per_step": kernels,
                          "tokens_held": int(held), "gb_s": round(gbs, 1), "of_hbm_peak": round(gbs / pk["hbm_gbs"], 3)}))
        return 0
    if shape["prefill_tokens"]:
        pre_prompts = workload_prompts(dict(shape, prompt_lengths=(shape["prefill_tokens"],) * 2), 1, seed=2)
    else:
        pre_prompts = workload_prompts(shape, batch, seed=0)        # the prompts that the decode run starts from
    if args.only == "prefill":
        pre_ms = measure_prefill(model, pre_prompts, runs=max(args.steps, 1))
        fl = prefill_flops(cfg, [len(p) for p in pre_prompts])
        print(json.dumps({"only": "prefill", "shape": args.shape, "tokens": sum(map(len, pre_prompts)),
                          "ms": round(pre_ms, 3), "tok_s": round(sum(map(len, pre_prompts)) / (pre_ms / 1e3), 1),
                          "of_bf16_peak": round(fl / (pre_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}))
        return 0

    clocks = ClockSampler()
    clocks.start()
    tps, ms_step, held_mean, kernels = measure_decode(model, shape, batch, steps, args.warmup)
    clock_info = clocks.stop()

    e2e_tps, _ = measure_e2e(model, shape, batch, steps)
    # the points: at least 64 timed steps after at least 16 untimed ones, so that a short run's figure
    # is not that of the few milliseconds after the prompt step (which runs into the power cap at batch 64)
    points = {}
    for b in shape["points"]:
        points[f"decode_b{b}"] = round(measure_decode(model, shape, b, max(steps, 64), max(args.warmup, 16),
                                                      seed=10 + b)[0], 1)
    pre_ms = measure_prefill(model, pre_prompts)
    pre_tokens = sum(map(len, pre_prompts))
    flops = prefill_flops(cfg, [len(p) for p in pre_prompts])

    # the other two workloads of the benchmark, each in a process of its own (its own memory, and a
    # failure there leaves this line whole): device-timed decode with its share of the HBM peak
    others = {}
    if args.shape == "1b" and not args.no_other_workloads and not args.layers:
        del model
        torch.cuda.empty_cache()
        for other in ("7b", "8b"):
            others[other] = other_workload(other)
            if "tok_s" in others[other]:
                points[f"decode_{other}_b{others[other]['batch']}"] = others[other]["tok_s"]

    step_bytes = weights + held_mean * kv_per_token
    achieved = step_bytes / (ms_step / 1e3) / 1e9
    from alpacca_b200.engine.decode import bucket_rows
    rows = bucket_rows(batch)
    line = {
        "metric": metric_name(shape, batch),
        "value": round(tps, 1), "unit": "tok/s", "n_gpus": 1, "steps": steps, "warmup": max(args.warmup, 3),
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: uniform-random token ids, random-init weights N(0, 0.02)",
        "impl": "ours",
        "config": flat_config(shape, cfg, layers_full, batch, steps, weights, kv_per_token,
                              workload_prompts(shape, batch, seed=0)),
        "e2e": {"value": round(e2e_tps, 1), "unit": "tok/s", "h2d_bytes_per_step": 4 * rows,
                "d2h_bytes_per_step": 4 * rows},
        "gpu_launches": int(kernels * steps),
        "prefill": {"value": round(pre_tokens / (pre_ms / 1e3), 1), "tokens": pre_tokens,
                    "ms": round(pre_ms, 3), "frac": round(flops / (pre_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "peaks": pk["source"],
                     "bytes_per_step": int(step_bytes)},
        "points": points,
        "clocks": clock_info,
    }
    if others:
        line["other_workloads"] = others
    print(json.dumps(line), flush=True)
    return 0


# ---------------------------------------------------------------------------------------------
# the reference arm

def write_reference_model(gguf, np, path, cfg, context):
    """An F32 GGUF of `cfg`'s layer sizes with random weights N(0, 0.02), written with the reference's own writer."""
    E, H, K, D = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    F, V, L = cfg["intermediate_size"], cfg["vocab_size"], cfg["num_hidden_layers"]
    w = gguf.GGUFWriter(path, "llama")
    for key, typ, val in (("general.name", gguf.T_STRING, "bench"), ("llama.context_length", gguf.T_UINT32, context),
                          ("llama.embedding_length", gguf.T_UINT32, E), ("llama.block_count", gguf.T_UINT32, L),
                          ("llama.feed_forward_length", gguf.T_UINT32, F),
                          ("llama.attention.head_count", gguf.T_UINT32, H),
                          ("llama.attention.head_count_kv", gguf.T_UINT32, K),
                          ("llama.attention.layer_norm_rms_epsilon", gguf.T_FLOAT32, cfg["rms_norm_eps"]),
                          ("llama.rope.dimension_count", gguf.T_UINT32, D), ("llama.vocab_size", gguf.T_UINT32, V),
                          ("llama.rope.freq_base", gguf.T_FLOAT32, cfg["rope_theta"]),
                          ("tokenizer.ggml.model", gguf.T_STRING, "llama")):
        w.add(key, typ, val)
    w.add_array("tokenizer.ggml.tokens", gguf.T_STRING, [f"t{i}" for i in range(V)])
    w.add_array("tokenizer.ggml.scores", gguf.T_FLOAT32, [0.0] * V)
    w.add_array("tokenizer.ggml.token_type", gguf.T_INT32, [1] * V)
    rng = np.random.default_rng(0)

    def mat(name, shape):
        n = int(np.prod(shape))
        w.add_raw_tensor(name, shape, "F32", (rng.standard_normal(n, dtype=np.float32) * 0.02).tobytes())

    ones = np.ones(E, np.float32).tobytes()
    mat("token_embd.weight", (E, V))
    for i in range(L):
        p = f"blk.{i}."
        w.add_raw_tensor(p + "attn_norm.weight", (E,), "F32", ones)
        mat(p + "attn_q.weight", (E, H * D))
        mat(p + "attn_k.weight", (E, K * D))
        mat(p + "attn_v.weight", (E, K * D))
        mat(p + "attn_output.weight", (H * D, E))
        w.add_raw_tensor(p + "ffn_norm.weight", (E,), "F32", ones)
        mat(p + "ffn_gate.weight", (E, F))
        mat(p + "ffn_up.weight", (E, F))
        mat(p + "ffn_down.weight", (F, E))
    w.add_raw_tensor("output_norm.weight", (E,), "F32", ones)
    if not cfg.get("tie_word_embeddings"):
        mat("output.weight", (E, V))
    w.write()


def run_reference(args):
    """The unmodified reference (installed into baseline/_ref) through its own public API.

    It is a CPU engine for one sequence at a time and has no batch: it takes the workload's sequences
    one after another (`reset`, `prefill`, then the decode loop), which is how its user serves several
    requests.  `value` is decoded tokens over the time of the hand-timed `forward` + `sample` loop,
    `e2e` the same through its own generation loop (`alpacca.chat.generate`, whose clock starts after
    the prompt), `prefill` one prompt of 2,048 tokens.
    """
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "alpacca" / "model.py").is_file():
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref holds no installed reference "
                          "(pip install --no-index --no-build-isolation --target baseline/_ref <the reference's source tree>)"}))
        return 0
    sys.path.insert(0, str(ref))
    try:
        import numpy as np
        from alpacca import chat, gguf
        from alpacca.model import Model
        from alpacca.sample import Sampler, SamplerParams
    except Exception as e:  # noqa: BLE001
        print(json.dumps({"impl": "reference", "unavailable": f"reference does not import: {e}"}))
        return 0
    import tempfile
    shape = SHAPES[args.shape]
    if args.shape != "1b":
        print(json.dumps({"impl": "reference", "unavailable": f"the reference arm runs the 1b workload only "
                          f"(float32 weights of the {args.shape} sizes on the host and minutes per prompt)"}))
        return 0
    cfg = dict(shape["config"])
    layers_full = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    batch = args.batch or shape["batch"]
    steps = min(args.steps or shape["steps"], 32)
    warm = max(args.warmup, 3)
    prompts = workload_prompts(shape, batch, seed=0)
    greedy = dict(temperature=0.0, top_k=0, top_p=1.0, repeat_penalty=1.0, seed=1)
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "bench.gguf")
        write_reference_model(gguf, np, path, cfg, shape["context"])
        model = Model.load(path, n_ctx=shape["context"], progress=False)
        # the timed loop by hand: prompt, warm-up steps, then `steps` steps, for each sequence in turn
        decode_s = 0.0
        per_seq = []
        for prompt in prompts:
            model.reset()
            sampler = Sampler(SamplerParams(**greedy))
            logits = model.prefill(prompt)
            for _ in range(warm):
                logits = model.forward(sampler.sample(logits))
            t0 = time.perf_counter()
            for _ in range(steps):
                logits = model.forward(sampler.sample(logits))
            per_seq.append(time.perf_counter() - t0)
            decode_s += per_seq[-1]
        # the same through the reference's own generation loop
        e2e_tokens, e2e_s = 0, 0.0
        for prompt in prompts:
            model.reset()
            res = chat.generate(model, list(prompt), SamplerParams(**greedy), n_predict=steps + 1)
            e2e_tokens += res.tokens - 1           # the first token comes from the prompt step
            e2e_s += res.seconds
        model.reset()
        long_prompt = workload_prompts(dict(shape, prompt_lengths=(shape["prefill_tokens"],) * 2), 1, seed=2)[0]
        t0 = time.perf_counter()
        model.prefill(long_prompt)
        prefill_s = time.perf_counter() - t0
    lo, _ = shape["prompt_lengths"]
    print(json.dumps({
        "metric": metric_name(shape, batch), "impl": "reference",
        "value": round(batch * steps / decode_s, 2), "unit": "tok/s", "n_gpus": args.gpus,
        "device": "cpu (the reference has no GPU path)", "steps": steps, "warmup": warm,
        "ms_per_step": round(decode_s / steps * 1e3, 2), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp32 (the reference has no reduced-precision dense path)",
        "data": "synthetic: uniform-random token ids, random-init weights N(0, 0.02)",
        "config": {"model": shape["name"], "layers": cfg["num_hidden_layers"], "layers_of_config": layers_full,
                   "global_batch": batch, "prompt_len": lo, "seq_len": shape["context"], "decode_steps": steps,
                   "sampling": "greedy", "parallelism": "CPU; the sequences of the batch one after another (the "
                   "reference has no batch and no GPU path)"},
        "e2e": {"value": round(e2e_tokens / e2e_s, 2), "unit": "tok/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0, "through": "alpacca.chat.generate"},
        "gpu_launches": 0,
        "points": {"decode_b1": round(steps / per_seq[0], 2)},
        "prefill": {"value": round(len(long_prompt) / prefill_s, 1), "tokens": len(long_prompt),
                    "ms": round(prefill_s * 1e3, 1)}}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=0, help="decode steps to time (0: the workload's own number)")
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--shape", default="1b", choices=sorted(SHAPES), help="which benchmark workload")
    ap.add_argument("--batch", type=int, default=0, help="another batch size than the workload's (0: its own)")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration (0: all)")
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill"],
                    help="measure one part only and print a short line (for profiling runs)")
    ap.add_argument("--no-other-workloads", action="store_true",
                    help="the default run also times the decode of the 7b and 8b workloads (in child processes, "
                         "into `points` and `other_workloads`); this leaves them out")
    ap.add_argument("--prompt-len", type=int, default=0,
                    help="with --only decode: equal prompts of this many tokens instead of the workload's")
    ap.add_argument("--prefill-tokens", type=int, default=0,
                    help="with --only prefill: one prompt of this many tokens instead of the workload's")
    args = ap.parse_args()
    n = int(os.environ.get("WORLD_SIZE", args.gpus))
    if args.gpus > 1 or n > 1:
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps({"impl": args.impl, "n_gpus": max(args.gpus, n),
                              "unsupported": "alpacca_b200 is a single-GPU library; bench.py runs with --gpus 1 only"}))
        return 2
    return run_reference(args) if args.impl == "reference" else run_ours(args)


if __name__ == "__main__":
    raise SystemExit(main())
