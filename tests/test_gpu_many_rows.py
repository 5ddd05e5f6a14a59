"""Decode steps of the sizes that serving runs: 8, 12, 20 and 64 sequences of unequal lengths.

Between 9 and 16 rows the narrow products keep the skinny kernel and the wide ones go to the library;
from 17 rows all products are the library's; a batch shape has more rows than live sequences (20 in a
shape of 24), and the rows without a sequence hold whatever they hold; with many (sequence, head) pairs
the decode attention takes its small CTAs.  Each of these is run here through the engine, step by step
and replayed from the CUDA graph, in 32-bit and in bfloat16, against the plain implementation; then
longer generations in which sequences end at different steps, so that the shape's rows empty and a
smaller shape takes over, and a second batch that takes the slots of the first.
"""
import numpy as np
import pytest

import plain_llama as plain
import tiny
from helpers import CONFIGS, check_logits, plain_logits, plain_model

pytestmark = pytest.mark.gpu

DTYPES = ("float32", "bfloat16")
ROWS = (8, 12, 20, 64)


def unequal_prompts(cfg, n, seed, longest=90):
    """n prompts whose lengths differ: 1, a page's edge, and lengths spread up to `longest`."""
    special = [1, 64, 63, 65, 2]
    lens = [special[i] if i < len(special) else 3 + (i * 37) % (longest - 3) for i in range(n)]
    return [tiny.prompt_tokens(cfg, m, seed + i) for i, m in enumerate(lens)]


def load(model_dir, dtype, n, tokens_each=192):
    from alpacca_b200.api import Model
    return Model.load(model_dir, dtype=dtype, max_batch=n, max_tokens=n * tokens_each)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n", ROWS)
@pytest.mark.parametrize("name", ["B", "C", "D", "E", "D-streamed", "E-streamed"])
def test_logits_of_every_decode_step(model_dirs, name, n, dtype, monkeypatch):
    """The prompts in one step, then four single-token steps through `Engine.step` and four replayed
    from the graph (which feeds on its own sampled tokens): the logits of every step against the
    plain implementation's for the sequence as it stands.  "streamed": the decode attention that
    streams the cache takes every step; without it the other decode kernel does.
    ("C" has five KV heads: 64 sequences are 320 (sequence, KV head) pairs, more than the device has
    processors, so the other decode kernel takes its small CTAs, several per processor.)"""
    from alpacca_b200 import ops
    from alpacca_b200.engine.decode import bucket_rows
    if name.endswith("-streamed"):
        if dtype != "bfloat16":
            pytest.skip("the streamed kernel is a bfloat16 kernel")
        name = name[0]
        monkeypatch.setattr(ops, "STREAM_MIN_BYTES", 0)
        launched = []
        real = ops.attention_stream
        monkeypatch.setattr(ops, "attention_stream", lambda *a, **k: (launched.append(1), real(*a, **k))[1])
    else:
        launched = None
        monkeypatch.setattr(ops, "STREAM_MIN_BYTES", float("inf"))     # the other decode kernel takes every step
    from alpacca_b200.engine.step import StepEntry
    from alpacca_b200.sampling import DeviceSampler, SamplerParams
    d = model_dirs[(name, dtype)]
    cfg = CONFIGS[name]
    prompts = unequal_prompts(cfg, n, 1000 + n)
    model = load(d, dtype, n)
    eng = model.engine
    sampler = DeviceSampler(SamplerParams.greedy(), eng.device)
    slots = [eng.alloc_slot() for _ in prompts]
    states = [sampler.new_state(i, p) for i, p in enumerate(prompts)]
    seqs = [list(p) for p in prompts]
    rows = []          # per step: float32 logits [n, V] as the engine gave them
    logits = eng.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
    rows.append(logits.cpu().numpy())
    toks = sampler.sample(logits, states)
    for _ in range(4):                                  # step by step
        for q, t in zip(seqs, toks):
            q.append(t)
        logits = eng.step([StepEntry(s, [t], [0]) for s, t in zip(slots, toks)])
        rows.append(logits.cpu().numpy())
        toks = sampler.sample(logits, states)
    dec = model.decoder_for(sampler)
    assert type(dec).__name__ == "GraphDecoder"
    live = [(s, t, st) for s, t, st in zip(slots, toks, states)]
    for _ in range(4):                                  # replayed; nothing runs ahead without `more`
        for q, (_, t, _) in zip(seqs, live):
            q.append(t)
        toks = dec.step(live)
        assert dec.shape.rows == bucket_rows(n) and dec.shape.logits.shape[0] == dec.shape.rows
        rows.append(dec.shape.logits[:n].cpu().numpy())
        assert [int(x) for x in np.argmax(rows[-1], axis=1)] == toks, "the graph sampled from other logits"
        live = [(s, t, st) for (s, _, st), t in zip(live, toks)]
    for b, q in enumerate(seqs):
        want = plain_logits(d, q)
        first = len(prompts[b]) - 1
        for i, r in enumerate(rows):
            check_logits(r[b], want[first + i], dtype,
                         f"{name} {n} sequences, seq {b} ({len(prompts[b])} tokens), step {i}")
    for s in slots:
        eng.free_slot(s)
    eng.cache.check()
    eng.wait()
    assert launched is None or len(launched) >= 4 * len(model.decoder.spec.layers), "the streamed kernel did not run"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n", (20, 64))
@pytest.mark.parametrize("name", ["B", "D-streamed"])
def test_sequences_that_end_at_different_steps(model_dirs, name, n, dtype, monkeypatch):
    """A long generation of n sequences in which many end early by a stop token, so that rows of the
    batch shape empty and smaller shapes take over, and then twice as many requests as a batch holds,
    so that a second batch takes the slots of the first: replayed from graphs and step by step give the
    same tokens in 32-bit; in bfloat16 every token is the plain model's choice within the tolerance."""
    from alpacca_b200 import ops
    from alpacca_b200.api import generate
    from alpacca_b200.sampling import SamplerParams
    from test_gpu_generate import margin_ok
    if name.endswith("-streamed"):          # the streamed decode attention takes every step, rows that empty included
        if dtype != "bfloat16":
            pytest.skip("the streamed kernel is a bfloat16 kernel")
        name = name[0]
        monkeypatch.setattr(ops, "STREAM_MIN_BYTES", 0)
    d = model_dirs[(name, dtype)]
    cfg = CONFIGS[name]
    prompts = unequal_prompts(cfg, n, 2000 + n, longest=60)
    model = load(d, dtype, n, tokens_each=128)
    params = SamplerParams.greedy()
    model.use_graphs = False
    free = generate(model, prompts, params, n_predict=40, stop_token_ids=[])
    # tokens that end a third of the sequences at different steps
    stops = sorted({free[i].token_ids[min(5 + (i * 7) % 30, len(free[i].token_ids) - 1)]
                    for i in range(0, n, 3) if free[i].token_ids})
    out = {}
    for graphs in (True, False):
        model.use_graphs = graphs
        res = generate(model, prompts + prompts, params, n_predict=40, stop_token_ids=stops)
        out[graphs] = [(r.token_ids, r.finish_reason) for r in res]
        assert model.engine.cache.slots.n_held == 0
        model.engine.cache.check()
        assert out[graphs][:n] == out[graphs][n:], "the second batch, in slots used before, gave other tokens"
    ends = {len(t) for t, _ in out[True]}
    assert len(ends) > 4 and any(r == "stop" for _, r in out[True]), "the sequences should end at different steps"
    if dtype == "float32":
        assert out[True] == out[False]
        pm = plain_model(str(d))
        for b in (0, 1, n // 2, n - 1):
            eos = cfg["eos_token_id"]
            ending = set(stops) | set(eos if isinstance(eos, list) else [eos])
            want, _ = plain.generate(pm, prompts[b], 40, stop=ending)
            assert out[True][b][0] == [t for t in want if t not in ending]
    else:
        for kind in (True, False):
            for b in (0, 1, n // 2, n - 1):
                assert margin_ok(d, prompts[b], out[kind][b][0], dtype), (kind, b)
