"""The engine against the plain implementation, in 32-bit and in bfloat16:
whole requests, the last 32 tokens one by one, unequal batches one after another
with slots used again, long decoding, the first tokens of a sequence."""
import numpy as np
import pytest
import torch

import tiny
from helpers import CONFIGS, check_logits, plain_logits

pytestmark = pytest.mark.gpu

DTYPES = ("float32", "bfloat16")
NAMES = ("a", "b", "c", "d", "e", "B", "C", "D", "E")     # upper case: weights N(0, 0.1), sharp attention


def make_engine(model_dir, dtype, max_tokens=64 * 24, max_slots=8, max_positions=None):
    from alpacca_b200.engine import Engine
    from alpacca_b200.engine.loading import load_model_dir
    model = load_model_dir(model_dir, dtype=dtype, device="cuda", max_positions=max_positions)
    return Engine(model, max_tokens=max_tokens, max_slots=max_slots)


def lengths_for(name):
    top = CONFIGS[name]["max_position_embeddings"]
    return [n for n in (1, 9, 33, 70, 63, 64, 65, 127, 128, 200, 331, 600) if n <= top]     # 600: ten pages


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_each_request_alone_and_whole(model_dirs, name, dtype):
    from alpacca_b200.engine import StepEntry
    d = model_dirs[(name, dtype)]
    eng = make_engine(d, dtype)
    for i, n in enumerate(lengths_for(name)):
        toks = tiny.prompt_tokens(CONFIGS[name], n, 100 + i)
        slot = eng.alloc_slot()
        got = eng.step([StepEntry(slot, toks, list(range(n)))]).cpu().numpy()
        check_logits(got, plain_logits(d, toks), dtype, f"{name} whole n={n}")
        eng.free_slot(slot)
        eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_last_32_tokens_one_by_one(model_dirs, name, dtype):
    from alpacca_b200.engine import StepEntry
    d = model_dirs[(name, dtype)]
    eng = make_engine(d, dtype)
    for i, n in enumerate((33, 100)):
        toks = tiny.prompt_tokens(CONFIGS[name], n, 200 + i)
        want = plain_logits(d, toks)
        slot = eng.alloc_slot()
        head = n - 32
        got = eng.step([StepEntry(slot, toks[:head], [head - 1])]).cpu().numpy()
        check_logits(got[0], want[head - 1], dtype, f"{name} prefix of {n}")
        for p in range(head, n):
            got = eng.step([StepEntry(slot, [toks[p]], [0])]).cpu().numpy()
            check_logits(got[0], want[p], dtype, f"{name} n={n} token {p} fed alone")
        eng.free_slot(slot)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_one_after_another(model_dirs, name, dtype):
    """Batches of unequal prompts; every request is fed some more tokens one by one and the
    shorter ones end earlier; the next batch takes the slots and pages that came back."""
    from alpacca_b200.engine import StepEntry
    d = model_dirs[(name, dtype)]
    cfg = CONFIGS[name]
    # room for one batch only, so that the second and third batches must reuse pages
    eng = make_engine(d, dtype, max_tokens=64 * 7, max_slots=4)     # 7 pages: each batch fits, two do not
    top = cfg["max_position_embeddings"]
    batches = [[(5, 3), (70, 9), (17, 1), (33, 12)], [(1, 20), (64, 2), (40, 6)], [(63, 4), (2, 2), (90, 11), (9, 0)]]
    if top >= 512:      # long prompts too: steps of 128 tokens and more take the tcgen05 attention
        batches.append([(150, 3), (129, 1), (60, 2)])
    seen_slots = set()
    for bi, batch in enumerate(batches):
        reqs = []
        for ri, (n_prompt, n_more) in enumerate(batch):
            total = min(n_prompt + n_more, top)
            toks = tiny.prompt_tokens(cfg, total, 300 + 10 * bi + ri)
            reqs.append({"toks": toks, "prompt": min(n_prompt, total), "slot": eng.alloc_slot(),
                         "want": plain_logits(d, toks)})
        if bi:
            assert {r["slot"] for r in reqs} & seen_slots, "later batches must reuse slots"
        seen_slots |= {r["slot"] for r in reqs}
        got = eng.step([StepEntry(r["slot"], r["toks"][:r["prompt"]], [r["prompt"] - 1]) for r in reqs])
        got = got.cpu().numpy()
        for row, r in enumerate(reqs):
            check_logits(got[row], r["want"][r["prompt"] - 1], dtype, f"{name} batch {bi} prompt of req {row}")
            r["pos"] = r["prompt"]
        live = [r for r in reqs if r["pos"] < len(r["toks"])]
        for r in reqs:
            if r not in live:
                eng.free_slot(r["slot"])
        while live:
            got = eng.step([StepEntry(r["slot"], [r["toks"][r["pos"]]], [0]) for r in live]).cpu().numpy()
            nxt = []
            for row, r in enumerate(live):
                check_logits(got[row], r["want"][r["pos"]], dtype,
                             f"{name} batch {bi} decode pos {r['pos']} (batch of {len(live)})")
                r["pos"] += 1
                if r["pos"] < len(r["toks"]):
                    nxt.append(r)
                else:
                    eng.free_slot(r["slot"])
            live = nxt
            eng.cache.check()
        assert eng.cache.slots.n_held == 0 and eng.cache.kv_groups[0].pages.n_held == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["c", "C"])
def test_long_decoding(model_dirs, name, dtype):
    """A short prompt and then hundreds of single-token steps across several pages."""
    from alpacca_b200.engine import StepEntry
    d = model_dirs[(name, dtype)]
    eng = make_engine(d, dtype, max_tokens=64 * 6)
    toks = tiny.prompt_tokens(CONFIGS[name], 330, 400)
    want = plain_logits(d, toks)
    slot = eng.alloc_slot()
    eng.step([StepEntry(slot, toks[:3], [])])
    for p in range(3, len(toks)):
        got = eng.step([StepEntry(slot, [toks[p]], [0])])
        if p % 7 == 0 or p in (63, 64, 65, 127, 128, 129, 255, 256, 257, len(toks) - 1):
            check_logits(got.cpu().numpy()[0], want[p], dtype, f"long decode pos {p}")
    eng.free_slot(slot)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_first_tokens_of_a_sequence(model_dirs, name, dtype):
    """A sequence that starts with a single token and grows one token at a time from
    position 0, in a batch with a longer one."""
    from alpacca_b200.engine import StepEntry
    d = model_dirs[(name, dtype)]
    eng = make_engine(d, dtype)
    a = tiny.prompt_tokens(CONFIGS[name], 6, 500)
    b = tiny.prompt_tokens(CONFIGS[name], 40, 501)
    wa, wb = plain_logits(d, a), plain_logits(d, b)
    sa, sb = eng.alloc_slot(), eng.alloc_slot()
    got = eng.step([StepEntry(sa, a[:1], [0]), StepEntry(sb, b[:35], [0, 34])]).cpu().numpy()
    check_logits(got[0], wa[0], dtype, "first token alone")
    check_logits(got[1], wb[0], dtype, "first token of the longer one")
    check_logits(got[2], wb[34], dtype, "last prompt token of the longer one")
    for p in range(1, 6):
        got = eng.step([StepEntry(sa, [a[p]], [0]), StepEntry(sb, [b[34 + p]], [0])]).cpu().numpy()
        check_logits(got[0], wa[p], dtype, f"short sequence pos {p}")
        check_logits(got[1], wb[34 + p], dtype, f"long sequence pos {34 + p}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["b", "B"])
def test_padding_and_batch_do_not_change_a_result(model_dirs, name, dtype):
    """The same request alone, in a batch, and cut into uneven steps gives the same logits
    (equal up to rounding; in 32-bit the kernels make them equal to the last bit)."""
    from alpacca_b200.engine import StepEntry
    from helpers import logit_tolerances
    d = model_dirs[(name, dtype)]
    eng = make_engine(d, dtype)
    toks = tiny.prompt_tokens(CONFIGS[name], 75, 600)
    other = tiny.prompt_tokens(CONFIGS[name], 120, 601)
    s = eng.alloc_slot()
    alone = eng.step([StepEntry(s, toks, list(range(75)))]).cpu().numpy()
    eng.free_slot(s)
    s1, s2 = eng.alloc_slot(), eng.alloc_slot()
    both = eng.step([StepEntry(s1, other, [119]), StepEntry(s2, toks, list(range(75)))]).cpu().numpy()[1:]
    eng.free_slot(s1)
    eng.free_slot(s2)
    s = eng.alloc_slot()
    cut = [eng.step([StepEntry(s, toks[a:b], list(range(b - a)))]).cpu().numpy()
           for a, b in ((0, 10), (10, 11), (11, 64), (64, 75))]
    cut = np.concatenate(cut)
    if dtype == "float32":
        assert np.array_equal(alone, both), "a batch neighbour changed 32-bit logits"
        assert np.abs(alone - cut).max() <= 2e-6 * max(1.0, np.abs(alone).max())
    else:
        tol = logit_tolerances(alone, dtype)[0]
        assert np.abs(alone - both).max() <= tol and np.abs(alone - cut).max() <= tol
    check_logits(cut, plain_logits(d, toks), dtype, "cut into steps")


@pytest.mark.parametrize("name", ["b", "e", "B", "E"])
def test_norms_inside_the_products_change_no_result(model_dirs, name, monkeypatch):
    """Steps of a few rows run the RMS norms inside the products before and after them.  With that
    switched off the same logits come out, within bfloat16 rounding, from more kernels."""
    from alpacca_b200 import ops
    from alpacca_b200.engine import StepEntry
    d = model_dirs[(name, "bfloat16")]
    cfg = CONFIGS[name]
    seqs = [tiny.prompt_tokens(cfg, n, 700 + i) for i, n in enumerate((30, 9, 17))]
    want = [plain_logits(d, s) for s in seqs]
    runs = {}
    for defer in (True, False):
        monkeypatch.setattr(ops, "DEFER_NORM", defer)
        eng = make_engine(d, "bfloat16")
        slots = [eng.alloc_slot() for _ in seqs]
        eng.step([StepEntry(slot, s[:-6], []) for slot, s in zip(slots, seqs)])
        before, got = ops.launches, []
        for p in range(6, 0, -1):
            got.append(eng.step([StepEntry(slot, [s[-p]], [0]) for slot, s in zip(slots, seqs)]).cpu().numpy())
        runs[defer] = (np.stack(got), ops.launches - before)
        for i, p in enumerate(range(6, 0, -1)):
            for b in range(len(seqs)):
                check_logits(got[i][b], want[b][len(seqs[b]) - p], "bfloat16", f"{name} defer={defer} step {i} seq {b}")
    assert runs[True][1] < runs[False][1], "the norms still ran as kernels of their own"
    from helpers import logit_tolerances
    assert np.abs(runs[True][0] - runs[False][0]).max() <= logit_tolerances(runs[False][0], "bfloat16")[0]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["B", "D", "E"])
def test_only_a_sequence_s_own_positions_are_written(model_dirs, name, dtype, monkeypatch):
    """Canaries: the whole cache holds a huge value before the run.  After prompts of unequal lengths,
    single-token steps and steps replayed from a graph whose shape has more rows than sequences, exactly
    positions 0 .. length-1 of each sequence's own pages hold keys and values, in every layer and head,
    and everything else still holds the canary: no kernel wrote beside its place (a padded row, a page of
    another sequence, a position past the end), and none read one (the logits are the plain model's)."""
    from alpacca_b200 import ops
    from alpacca_b200.api import Model
    from alpacca_b200.engine import StepEntry
    from alpacca_b200.sampling import DeviceSampler, SamplerParams
    CANARY = 1.0e30
    d = model_dirs[(name, dtype)]
    cfg = CONFIGS[name]
    if dtype == "bfloat16":
        monkeypatch.setattr(ops, "STREAM_MIN_BYTES", 0)        # the streamed decode attention where it can run
    model = Model.load(d, dtype=dtype, max_batch=8, max_tokens=64 * 24)
    eng = model.engine
    for grp in eng.cache.kv_groups:
        grp.k.fill_(CANARY)
        grp.v.fill_(CANARY)
    prompts = [tiny.prompt_tokens(cfg, n, 1100 + i) for i, n in enumerate((1, 63, 64, 65, 130))]
    slots = [eng.alloc_slot() for _ in prompts]
    sampler = DeviceSampler(SamplerParams.greedy(), eng.device)
    states = [sampler.new_state(i, p) for i, p in enumerate(prompts)]
    seqs = [list(p) for p in prompts]
    logits = eng.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
    toks = sampler.sample(logits, states)
    for _ in range(2):                                  # step by step
        for q, t in zip(seqs, toks):
            q.append(t)
        logits = eng.step([StepEntry(s, [t], [0]) for s, t in zip(slots, toks)])
        toks = sampler.sample(logits, states)
    dec = model.decoder_for(sampler)                    # five sequences in a shape of eight rows
    live = [(s, t, st) for s, t, st in zip(slots, toks, states)]
    for _ in range(3):
        for q, (_, t, _) in zip(seqs, live):
            q.append(t)
        toks = dec.step(live)
        live = [(s, t, st) for (s, _, st), t in zip(live, toks)]
    last = dec.shape.logits[:len(seqs)].cpu().numpy()
    eng.wait()
    assert np.isfinite(last).all()
    for b, q in enumerate(seqs):
        check_logits(last[b], plain_logits(d, q)[-1], dtype, f"{name} canaries, sequence {b}")
    for grp in eng.cache.kv_groups:
        own = torch.zeros(grp.n_pages, 64, dtype=torch.bool)
        for s in slots:
            pages = grp.page_lists[s]
            for pos in range(eng.length(s)):
                own[pages[pos // 64], pos % 64] = True
        for what, t in (("keys", grp.k), ("values", grp.v)):
            written = (t != CANARY).cpu()               # [entry, page, head, position, dim]
            everywhere = written.all(dim=4).all(dim=2).all(dim=0)
            anywhere = written.any(dim=4).any(dim=2).any(dim=0)
            assert torch.equal(anywhere, own), f"{what}: {int((anywhere & ~own).sum())} places written that no sequence owns"
            assert torch.equal(everywhere, own), f"{what}: {int((own & ~everywhere).sum())} owned places not written in full"
    for s in slots:
        eng.free_slot(s)
