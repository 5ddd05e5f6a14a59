"""Generation through the Python entry point and the command line, against the plain loop."""
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

import plain_llama as plain
import tiny
from helpers import CONFIGS, plain_model

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def margin_ok(model_dir, prompt, tokens, dtype):
    """Every generated token is the plain model's argmax for the same prefix, or as close to it as two
    logits can be swapped by the engine's allowed error (each may be off by the tolerance)."""
    from helpers import logit_tolerances
    pm = plain_model(str(model_dir))
    seq = list(prompt)
    for t in tokens:
        row = pm.logits(seq)[-1]
        if row[t] < row.max() - 2 * logit_tolerances(row, dtype)[0]:
            return False
        seq.append(t)
    return True


@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b", "B"])
def test_greedy_generation_of_an_unequal_batch(model_dirs, name, dtype, graphs):
    from alpacca_b200.api import Model, generate
    from alpacca_b200.sampling import SamplerParams
    d = model_dirs[(name, dtype)]
    cfg = CONFIGS[name]
    lens = (5, 11, 17) if name == "a" else (1, 9, 33, 70)
    prompts = [tiny.prompt_tokens(cfg, n, 700 + i) for i, n in enumerate(lens)]
    model = Model.load(d, dtype=dtype, max_batch=4)
    assert model.use_graphs, "the Llama model's decode steps are captured in CUDA graphs"
    model.use_graphs = graphs
    res = generate(model, prompts, SamplerParams.greedy(), n_predict=8, stop_token_ids=[])
    stops = set(model.decoder.spec.stop_token_ids)
    for p, r in zip(prompts, res):
        want, _ = plain.generate(plain_model(str(d)), p, 8, stop=stops)
        if dtype == "float32":
            kept = [t for t in want if t not in stops]
            assert r.token_ids == kept and r.tokens == len(want)
        assert margin_ok(d, p, r.token_ids, dtype)
        assert r.finish_reason in ("length", "stop") and r.prompt_tokens == len(p)
    one = generate(model, prompts[1], SamplerParams.greedy(), n_predict=8)
    assert one.token_ids == res[1].token_ids, "a request alone and in a batch must give the same tokens"
    # more requests than a batch holds: batches one after another
    many = generate(model, prompts * 3, SamplerParams.greedy(), n_predict=4)
    assert [r.token_ids for r in many[:len(prompts)]] == [r.token_ids[:4] for r in res]
    assert [r.token_ids for r in many[len(prompts):2 * len(prompts)]] == [r.token_ids[:4] for r in res]
    assert model.engine.cache.slots.n_held == 0


def test_graph_steps_beyond_the_context_are_refused(model_dirs):
    """Replaying more steps than a sequence has positions left would write past its pages and read past
    the rotation tables: the decoder refuses before it launches, and leaves the lengths as they were."""
    from alpacca_b200.api import Model
    from alpacca_b200.cache import CacheFull
    from alpacca_b200.engine.step import StepEntry
    from alpacca_b200.sampling import DeviceSampler, SamplerParams
    d = model_dirs[("a", "bfloat16")]
    model = Model.load(d, dtype="bfloat16", n_ctx=32, max_batch=2)
    eng = model.engine
    sampler = DeviceSampler(SamplerParams.greedy(), eng.device)
    p = tiny.prompt_tokens(tiny.TINY_A, 20, 770)
    slot = eng.alloc_slot()
    st = sampler.new_state(0, p)
    tok = sampler.sample(eng.step([StepEntry(slot, p, [19])]), [st])[0]
    dec = model.decoder_for(sampler)
    live = [(slot, tok, st)]
    dec.run(live, 10)                       # positions 20 .. 29
    assert eng.length(slot) == 30
    with pytest.raises(CacheFull, match="context window full"):
        dec.run(live, 3)                    # 30, 31 are left: three steps do not fit
    assert eng.length(slot) == 30
    dec.run(live, 2)
    assert eng.length(slot) == 32
    eng.free_slot(slot)


def test_stop_token_and_context_end_sequences(model_dirs):
    from alpacca_b200.api import Model, generate
    from alpacca_b200.sampling import SamplerParams
    d = model_dirs[("a", "float32")]
    p = tiny.prompt_tokens(tiny.TINY_A, 6, 710)
    model = Model.load(d, dtype="float32", n_ctx=16)
    free = generate(model, p, SamplerParams.greedy(), n_predict=6)
    assert free.tokens == 6
    stopped = generate(model, p, SamplerParams.greedy(), n_predict=6, stop_token_ids=[free.token_ids[2]])
    assert stopped.token_ids == free.token_ids[:2] and stopped.tokens == 3 and stopped.finish_reason == "stop"
    full = generate(model, p, SamplerParams.greedy(), n_predict=-1)       # until the 16 positions are used
    assert len(p) + full.tokens <= 16 and full.finish_reason in ("context", "length", "stop")


@pytest.mark.parametrize("graphs", [True, False])
def test_temperature_sampling_is_seeded_and_batch_independent(model_dirs, graphs):
    from alpacca_b200.api import Model, generate
    from alpacca_b200.sampling import SamplerParams
    d = model_dirs[("b", "float32")]
    prompts = [tiny.prompt_tokens(tiny.TINY_B, n, 720 + i) for i, n in enumerate((1, 9, 33, 70))]
    model = Model.load(d, dtype="float32", max_batch=4)
    model.use_graphs = graphs
    params = SamplerParams(temperature=0.8, top_k=0, top_p=1.0, repeat_penalty=1.0, seed=11)
    a = generate(model, prompts, params, n_predict=12, stop_token_ids=[])
    b = generate(model, prompts, params, n_predict=12, stop_token_ids=[])
    assert [r.token_ids for r in a] == [r.token_ids for r in b]
    c = generate(model, prompts, SamplerParams(temperature=0.8, top_k=0, top_p=1.0, repeat_penalty=1.0, seed=12),
                 n_predict=12)
    assert [r.token_ids for r in a] != [r.token_ids for r in c]
    # the plain loop with the same seed and stream gives the same tokens
    stops = set(model.decoder.spec.stop_token_ids)
    for i in (0, 2):
        want, _ = plain.generate(plain_model(str(d)), prompts[i], 12, temperature=0.8, seed=11, stream=i, stop=stops)
        assert a[i].token_ids == [t for t in want if t not in stops]


def test_reference_style_single_sequence_calls(model_dirs):
    from alpacca_b200.api import Model
    d = model_dirs[("c", "float32")]
    toks = tiny.prompt_tokens(tiny.TINY_C, 20, 730)
    want = plain_model(str(d)).logits(toks)
    model = Model.load(d, dtype="float32")
    got = model.prefill(toks[:15]).cpu().numpy()
    assert np.abs(got - want[14]).max() < 5e-5 and model.n_past == 15
    for p in range(15, 20):
        got = model.forward(toks[p]).cpu().numpy()
        assert np.abs(got - want[p]).max() < 5e-5
    model.reset()
    assert model.n_past == 0
    assert "LlamaForCausalLM" in model.describe()


@pytest.mark.parametrize("dtype,tol", [("float32", 5e-5), ("bfloat16", None)])
def test_prefill_keeps_the_longest_common_prefix(model_dirs, dtype, tol):
    """As tests/smoke.py:974-997 of the reference: only what follows the shared prefix is run, a prompt
    that is held in full runs its last token again, and a prompt that diverges gives the logits of a
    fresh sequence (the cache behind the shared prefix was given back)."""
    from alpacca_b200.api import Model
    from helpers import check_logits
    d = model_dirs[("c", dtype)]
    ids = tiny.prompt_tokens(tiny.TINY_C, 200, 760)
    base, longer, diverged = ids[:70], ids[:70] + ids[70:150], ids[:70] + ids[160:190]
    model = Model.load(d, dtype=dtype)
    pages = model.engine.cache.kv_groups[0].pages
    model.prefill(base)
    assert model.last_prefill_forwarded == len(base)
    got = model.prefill(longer).cpu().numpy()
    assert model.last_prefill_forwarded == len(longer) - len(base) and model.n_past == len(longer)
    check_logits(got, plain_model(str(d)).logits(longer)[-1], dtype, "suffix on a cached prefix")
    again = model.prefill(longer).cpu().numpy()
    assert model.last_prefill_forwarded == 1 and model.n_past == len(longer)
    assert np.abs(again - got).max() <= (tol or 4e-2)
    assert pages.n_held == 3
    got = model.prefill(diverged).cpu().numpy()
    assert model.last_prefill_forwarded == len(diverged) - len(base)
    assert model.cached_ids == diverged and model.n_past == len(diverged) and pages.n_held == 2
    fresh = Model.load(d, dtype=dtype).prefill(diverged).cpu().numpy()
    assert np.abs(got - fresh).max() <= (tol or 4e-2)
    check_logits(got, plain_model(str(d)).logits(diverged)[-1], dtype, "a prompt that diverges")
    got = model.prefill(ids[100:130]).cpu().numpy()           # nothing shared: from position 0
    assert model.last_prefill_forwarded == 30 and model.n_past == 30 and pages.n_held == 1
    check_logits(got, plain_model(str(d)).logits(ids[100:130])[-1], dtype, "nothing shared")
    model.engine.cache.check()


def test_command_line(model_dirs):
    d = model_dirs[("a", "float32")]
    p = tiny.prompt_tokens(tiny.TINY_A, 5, 740)
    cmd = [sys.executable, "-m", "alpacca_b200", "run", str(d), " ".join(map(str, p)), "/", "7 8 9",
           "-n", "6", "--temp", "0", "--repeat-penalty", "1.0", "--dtype", "float32", "--seed", "1"]
    out = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr
    lines = out.stdout.strip().splitlines()
    assert len(lines) == 2 and "tokens," in out.stderr
    want, _ = plain.generate(plain_model(str(d)), p, 6, stop={2})
    assert [int(t) for t in lines[0].split()] == [t for t in want if t != 2]
    bad = subprocess.run([sys.executable, "-m", "alpacca_b200", "run", str(d), "hello"], cwd=ROOT,
                         capture_output=True, text=True, timeout=600)
    assert bad.returncode == 1 and "alpacca_b200: error:" in bad.stderr


def test_graph_and_eager_decoding_agree_over_many_steps(model_dirs):
    """Long generation with the reference's default sampler options (top-k, top-p, repeat penalty):
    decode steps replayed from CUDA graphs give the tokens of the step-by-step path, across page
    boundaries, while sequences end at different times."""
    from alpacca_b200.api import Model, generate
    from alpacca_b200.sampling import SamplerParams
    d = model_dirs[("c", "float32")]
    prompts = [tiny.prompt_tokens(tiny.TINY_C, n, 750 + i) for i, n in enumerate((3, 60, 130, 17, 64))]
    model = Model.load(d, dtype="float32", max_batch=5)
    params = SamplerParams(seed=5)
    model.use_graphs = False
    free = generate(model, prompts, params, n_predict=150, stop_token_ids=[])
    stops = [free[0].token_ids[40], free[2].token_ids[90], free[4].token_ids[120]]
    out = {}
    for graphs in (True, False):
        model.use_graphs = graphs
        res = generate(model, prompts, params, n_predict=150, stop_token_ids=stops)
        out[graphs] = [(r.token_ids, r.finish_reason) for r in res]
        assert model.engine.cache.slots.n_held == 0
    assert out[True] == out[False]
    assert len({len(t) for t, _ in out[True]}) > 1, "the sequences should end at different times"
    assert out[False][1][0] == free[1].token_ids[:len(out[False][1][0])]


def runs_len_hint(trace, prompts):
    """Lengths of sequences 0 and 2 after the prompt and len(trace) - 1 fed tokens."""
    return [len(prompts[0]) + len(trace) - 1, len(prompts[2]) + len(trace) - 1]


def test_a_step_that_ran_ahead_is_given_up_cleanly(model_dirs):
    """The graph decoder starts the next step early when it is told who comes back.  A caller that
    comes back with other sequences, or other tokens, than forecast gets what it asked for: the early
    step is dropped, lengths and device state are put right, and the tokens are those of the plain
    step-by-step decoder."""
    import torch
    from alpacca_b200.api import Model
    from alpacca_b200.engine.decode import EagerDecoder
    from alpacca_b200.engine.step import StepEntry
    from alpacca_b200.sampling import DeviceSampler, SamplerParams
    d = model_dirs[("b", "bfloat16")]
    prompts = [tiny.prompt_tokens(tiny.TINY_B, n, 900 + i) for i, n in enumerate((5, 70, 33))]
    runs = {}
    for kind in ("graph", "eager"):
        model = Model.load(d, dtype="bfloat16", max_batch=4)
        eng = model.engine
        sampler = DeviceSampler(SamplerParams.greedy(), eng.device)
        dec = model.decoder_for(sampler) if kind == "graph" else EagerDecoder(eng, sampler)
        slots = [eng.alloc_slot() for _ in prompts]
        states = [sampler.new_state(i, p) for i, p in enumerate(prompts)]
        logits = eng.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
        toks = sampler.sample(logits, states)
        trace = [list(toks)]
        live = [(s, t, st) for s, t, st in zip(slots, toks, states)]
        for step in range(12):
            toks = dec.step(live, more=[True] * len(live), stop=())
            trace.append(list(toks))
            live = [(s, t, st) for (s, _, st), t in zip(live, toks)]
            if step == 3:            # one sequence leaves although it was forecast to stay
                eng.free_slot(live[1][0])
                live = [live[0], live[2]]
            if step == 7:            # another token than the sampled one is fed
                live[0] = (live[0][0], (live[0][1] + 1) % tiny.TINY_B["vocab_size"], live[0][2])
        if kind == "graph":
            assert [eng.length(s) for s, _, _ in live] > runs_len_hint(trace, prompts)
            dec.settle(live)         # steps that run ahead are in the lengths until they are given up
        runs[kind] = (trace, [eng.length(s) for s, _, _ in live])
        for s, _, _ in live:
            eng.free_slot(s)
        assert eng.cache.slots.n_held == 0
        torch.cuda.synchronize()
    assert runs["graph"] == runs["eager"]
