#!/usr/bin/env python3
"""Decode and prefill throughput of alpacca_b200 on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

The workload is the Llama-3.2-1B shape with random bfloat16 weights: every
sequence is prefilled with 512 uniform-random tokens, then K decode steps
(one token per sequence per step, greedy) are timed.  A "step" is one decode
step of the whole batch.  `value` is decoded tokens per second at batch 8,
timed on the device with CUDA events around exactly K steps replayed from the
engine's CUDA graph (the sampled token of a step is the next step's input, on
the device).  `e2e` is the same workload through the Python entry point
(`alpacca_b200.api.generate`): token ids in from host lists, token ids out to
host lists, with the per-step host traffic that serving has.  `prefill` is one
2,048-token prompt; `points` are decode at batch 1 and 64; `roofline` divides
the bytes a decode step must read (all weights once, plus the cache of the
live requests) by the step time.  Every step streams more bytes than the L2
holds, so nothing is flushed between timed iterations.

One JSON line goes to standard output.  With --gpus N > 1 it prints a line
that says so and exits with 2: this library runs on one GPU.
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

# layer sizes of the Llama-3.2-1B shape
LLAMA_1B = {
    "architectures": ["LlamaForCausalLM"], "num_hidden_layers": 16, "hidden_size": 2048,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64, "intermediate_size": 8192,
    "vocab_size": 128256, "max_position_embeddings": 131072, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_pairing": "neox",
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "tie_word_embeddings": True, "hidden_act": "silu", "bos_token_id": 128000, "eos_token_id": 128001,
}
CONTEXT = 4096
PROMPT = 512
PREFILL_TOKENS = 2048
REFERENCE_DECODE_B1 = 10.1     # tok/s of the reference's own code at this shape on a CPU (its only number here)
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


def random_prompts(n, length, vocab, seed):
    import random
    rng = random.Random(seed)
    return [[rng.randrange(vocab) for _ in range(length)] for _ in range(n)]


def model_bytes(model) -> int:
    """Bytes of every weight a decode step reads once (the embedding table counts once: it is the head)."""
    seen, total = set(), 0
    stack = [model.decoder]
    while stack:
        part = stack.pop()
        stack.extend(part.children())
        for v in vars(part).values():
            if hasattr(v, "data_ptr") and hasattr(v, "element_size") and v.is_cuda and v.dim() >= 1:
                if v.data_ptr() not in seen and v.dtype.is_floating_point and not _is_rope_table(part, v):
                    seen.add(v.data_ptr())
                    total += v.numel() * v.element_size()
    return total


def _is_rope_table(part, tensor) -> bool:
    return type(part).__name__ == "RotaryEncoding"


def prefill_flops(cfg, T) -> float:
    E, H, K, D = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    F, L, V = cfg["intermediate_size"], cfg["num_hidden_layers"], cfg["vocab_size"]
    per_token = 2.0 * (E * (H + 2 * K) * D + H * D * E + 3 * E * F)
    attention = 2.0 * 2.0 * H * D * T * (T + 1) / 2.0
    return L * (T * per_token + attention) + 2.0 * V * E


def start_batch(model, batch, seed):
    """Prefills `batch` prompts, samples their first tokens; returns what the decoder needs."""
    from alpacca_b200.engine.step import StepEntry
    from alpacca_b200.sampling import DeviceSampler, SamplerParams
    eng = model.engine
    prompts = random_prompts(batch, PROMPT, model.config.vocab_size, seed)
    slots = [eng.alloc_slot() for _ in prompts]
    sampler = DeviceSampler(SamplerParams.greedy(), eng.device)
    states = [sampler.new_state(i, p) for i, p in enumerate(prompts)]
    logits = eng.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
    first = sampler.sample(logits, states)
    decoder = model.decoder_for(sampler)
    return slots, decoder, [(s, t, st) for s, t, st in zip(slots, first, states)]


def measure_decode(model, batch, steps, warmup, seed=0):
    """Device-timed decode: (tokens per second, ms per step, mean context, kernels per step)."""
    import torch
    from alpacca_b200 import ops
    slots, decoder, live = start_batch(model, batch, seed)
    try:
        # the pages of the whole run are reserved first, so that the warm-up steps and the timed
        # steps have the same batch shape (and the capture of its graph falls into the warm-up)
        model.engine.cache.reserve([(s, max(warmup, 3) + steps) for s in slots])
        decoder.run(live, max(warmup, 3))
        before = ops.launches
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ctx0 = model.engine.length(slots[0])
        t0.record()
        decoder.run(live, steps)
        t1.record()
        torch.cuda.synchronize()
        ms = t0.elapsed_time(t1)
        eager_launches = ops.launches - before
        per_step = getattr(decoder, "kernels_per_step", None) or (eager_launches // max(steps, 1))
        return batch * steps / (ms / 1e3), ms / steps, ctx0 + (steps - 1) / 2.0, per_step
    finally:
        for s in slots:
            model.engine.free_slot(s)


def measure_e2e(model, batch, steps, seed=1):
    """The same decode through the Python entry point: host token lists in, host token lists out."""
    from alpacca_b200.api import generate
    from alpacca_b200.sampling import SamplerParams
    prompts = random_prompts(batch, PROMPT, model.config.vocab_size, seed)
    generate(model, prompts, SamplerParams.greedy(), n_predict=8, stop_token_ids=[])     # warm-up (graphs)
    res = generate(model, prompts, SamplerParams.greedy(), n_predict=steps + 1, stop_token_ids=[])
    tokens = sum(r.tokens - 1 for r in res)            # the first token of each comes from the prompt step
    seconds = max(r.seconds for r in res)
    return tokens / seconds, seconds


def measure_prefill(model, runs=5, seed=2):
    import torch
    from alpacca_b200.engine.step import StepEntry
    eng = model.engine
    prompt = random_prompts(1, PREFILL_TOKENS, model.config.vocab_size, seed)[0]
    times = []
    for i in range(runs + 2):
        slot = eng.alloc_slot()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        eng.step([StepEntry(slot, prompt, [len(prompt) - 1])])
        t1.record()
        torch.cuda.synchronize()
        eng.free_slot(slot)
        if i >= 2:
            times.append(t0.elapsed_time(t1))
    return statistics.median(times)


def run_ours(args):
    import torch
    from alpacca_b200.api import Model

    assert torch.cuda.is_available(), "bench.py needs a CUDA device"
    torch.cuda.set_device(0)
    pk = peaks()
    cfg = dict(LLAMA_1B)
    layers_full = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    model = Model.random(cfg, seed=0, n_ctx=CONTEXT, dtype="bfloat16", max_batch=max(64, args.batch or 0))
    weights = model_bytes(model)
    kv_per_token = sum(g.bytes_per_token for g in model.engine.cache.kv_groups)

    if args.only == "decode":
        tps, ms_step, _, kernels = measure_decode(model, args.batch, args.steps, args.warmup)
        print(json.dumps({"only": "decode", "batch": args.batch, "tok_s": round(tps, 1),
                          "ms_per_step": round(ms_step, 4), "kernels_per_step": kernels}))
        return 0
    if args.only == "prefill":
        pre_ms = measure_prefill(model, runs=max(args.steps, 1))
        print(json.dumps({"only": "prefill", "tokens": PREFILL_TOKENS, "ms": round(pre_ms, 3)}))
        return 0

    clocks = ClockSampler()
    clocks.start()
    tps, ms_step, ctx_mean, kernels = measure_decode(model, args.batch, args.steps, args.warmup)
    clock_info = clocks.stop()

    e2e_tps, _ = measure_e2e(model, args.batch, args.steps)
    points = {}
    for b in (1, 64):
        points[f"decode_b{b}"] = round(measure_decode(model, b, min(args.steps, 128), args.warmup, seed=10 + b)[0], 1)
    pre_ms = measure_prefill(model)
    flops = prefill_flops(cfg, PREFILL_TOKENS)

    step_bytes = weights + args.batch * ctx_mean * kv_per_token
    achieved = step_bytes / (ms_step / 1e3) / 1e9
    from alpacca_b200.engine.decode import bucket_rows
    rows = bucket_rows(args.batch)
    line = {
        "metric": "decode tok/s at batch 8 (Llama-3.2-1B shape, 512-token prompts, context 4096)",
        "value": round(tps, 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "vs_reference_cpu_b1": round(points["decode_b1"] / REFERENCE_DECODE_B1, 1),
        "dtype": "bf16", "data": "synthetic: uniform-random token ids, random-init weights N(0, 0.02)",
        "impl": "ours",
        "config": {"model": "Llama-3.2-1B shape", "layers": cfg["num_hidden_layers"], "layers_of_config": layers_full,
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "ffn": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "global_batch": args.batch,
                   "prompt_len": PROMPT, "seq_len": CONTEXT, "decode_steps": args.steps, "sampling": "greedy",
                   "parallelism": "single GPU", "l2": "inputs larger than L2 (no flush)",
                   "weight_bytes": weights, "kv_bytes_per_token": kv_per_token},
        "e2e": {"value": round(e2e_tps, 1), "unit": "tok/s", "h2d_bytes_per_step": 4 * rows,
                "d2h_bytes_per_step": 4 * rows},
        "gpu_launches": int(kernels * args.steps),
        "prefill": {"value": round(PREFILL_TOKENS / (pre_ms / 1e3), 1), "tokens": PREFILL_TOKENS,
                    "ms": round(pre_ms, 3), "frac": round(flops / (pre_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "peaks": pk["source"]},
        "points": points,
        "clocks": clock_info,
    }
    print(json.dumps(line), flush=True)
    return 0


def run_reference(args):
    """The unmodified reference (installed into baseline/_ref) through its own public API.

    It is a CPU engine for one sequence at a time, so its arm is decode at batch 1 after a 512-token
    prompt at the same layer sizes; `config.global_batch` says so.
    """
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "alpacca" / "model.py").is_file():
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref holds no installed reference "
                          "(pip install --no-index --no-build-isolation --target baseline/_ref <the reference's source tree>)"}))
        return 0
    sys.path.insert(0, str(ref))
    try:
        import numpy as np
        from alpacca import gguf
        from alpacca.model import Model
        from alpacca.sample import Sampler, SamplerParams
    except Exception as e:  # noqa: BLE001
        print(json.dumps({"impl": "reference", "unavailable": f"reference does not import: {e}"}))
        return 0
    import tempfile
    cfg = dict(LLAMA_1B)
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    steps = min(args.steps, 32)
    E, H, K, D = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    F, V, L = cfg["intermediate_size"], cfg["vocab_size"], cfg["num_hidden_layers"]
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "bench.gguf")
        w = gguf.GGUFWriter(path, "llama")
        for key, typ, val in (("general.name", gguf.T_STRING, "bench"), ("llama.context_length", gguf.T_UINT32, CONTEXT),
                              ("llama.embedding_length", gguf.T_UINT32, E), ("llama.block_count", gguf.T_UINT32, L),
                              ("llama.feed_forward_length", gguf.T_UINT32, F),
                              ("llama.attention.head_count", gguf.T_UINT32, H),
                              ("llama.attention.head_count_kv", gguf.T_UINT32, K),
                              ("llama.attention.layer_norm_rms_epsilon", gguf.T_FLOAT32, 1e-5),
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

        mat("token_embd.weight", (E, V))
        for i in range(L):
            p = f"blk.{i}."
            w.add_raw_tensor(p + "attn_norm.weight", (E,), "F32", np.ones(E, np.float32).tobytes())
            mat(p + "attn_q.weight", (E, H * D))
            mat(p + "attn_k.weight", (E, K * D))
            mat(p + "attn_v.weight", (E, K * D))
            mat(p + "attn_output.weight", (H * D, E))
            w.add_raw_tensor(p + "ffn_norm.weight", (E,), "F32", np.ones(E, np.float32).tobytes())
            mat(p + "ffn_gate.weight", (E, F))
            mat(p + "ffn_up.weight", (E, F))
            mat(p + "ffn_down.weight", (F, E))
        w.add_raw_tensor("output_norm.weight", (E,), "F32", np.ones(E, np.float32).tobytes())
        w.write()
        model = Model.load(path, n_ctx=CONTEXT, progress=False)
        prompt = random_prompts(1, PROMPT, V, 0)[0]
        sampler = Sampler(SamplerParams(temperature=0.0, seed=1))
        t0 = time.perf_counter()
        logits = model.prefill(prompt)
        prefill_s = time.perf_counter() - t0
        for _ in range(max(args.warmup, 3)):
            logits = model.forward(sampler.sample(logits))
        t0 = time.perf_counter()
        for _ in range(steps):
            logits = model.forward(sampler.sample(logits))
        sec = time.perf_counter() - t0
    print(json.dumps({
        "metric": "decode tok/s (Llama-3.2-1B shape, 512-token prompt, context 4096)", "impl": "reference",
        "value": round(steps / sec, 2), "unit": "tok/s", "n_gpus": args.gpus, "device": "cpu (the reference has no GPU path)", "steps": steps, "warmup": max(args.warmup, 3),
        "ms_per_step": round(sec / steps * 1e3, 2), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp32 (the reference has no reduced-precision dense path)", "data": "synthetic",
        "config": {"model": "Llama-3.2-1B shape", "layers": L, "global_batch": 1, "prompt_len": PROMPT,
                   "seq_len": CONTEXT, "parallelism": "CPU, one sequence at a time (the reference has no batch "
                   "and no GPU path)"},
        "prefill": {"value": round(PROMPT / prefill_s, 1), "tokens": PROMPT, "ms": round(prefill_s * 1e3, 1)}}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration (0: all)")
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill"],
                    help="measure one part only and print a short line (for profiling runs)")
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
