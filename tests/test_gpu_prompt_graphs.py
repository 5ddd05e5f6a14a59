"""Prompt steps replayed from CUDA graphs: the second step of a shape (the same numbers of new and held
tokens per sequence) is captured, later ones replay it with their own token ids, slots, pages and wanted
places.  Every step's logits against the plain implementation, in both precisions; what is in the cache
afterwards serves single-token steps as usual."""
import numpy as np
import pytest
import torch

import tiny
from helpers import CONFIGS, check_logits, plain_logits

pytestmark = pytest.mark.gpu


def make_engine(model_dir, dtype, **kw):
    from alpacca_b200.engine import Engine
    from alpacca_b200.engine.loading import load_model_dir
    return Engine(load_model_dir(model_dir, dtype=dtype, device="cuda"), **kw)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "B", "D", "E"])
def test_steps_of_one_shape_with_other_tokens_slots_and_places(model_dirs, name, dtype):
    from alpacca_b200.engine import StepEntry
    d = model_dirs[(name, dtype)]
    cfg = CONFIGS[name]
    eng = make_engine(d, dtype, max_tokens=64 * 30, max_slots=12)
    assert eng.step_graphs
    top = cfg["max_position_embeddings"]
    lens = [n for n in (70, 5, 33) if n <= top] + ([200] if top >= 512 else [])
    parked = []
    for rnd in range(5):
        # other slots and pages every round: a slot is parked before the round's are taken
        parked.append(eng.alloc_slot())
        eng.step([StepEntry(parked[-1], tiny.prompt_tokens(cfg, 3 + rnd, 50 + rnd), [])])
        toks = [tiny.prompt_tokens(cfg, n + 2, 1000 + 10 * rnd + j) for j, n in enumerate(lens)]
        wants = [[(rnd * 7 + j) % n, n - 1] for j, n in enumerate(lens)]
        slots = [eng.alloc_slot() for _ in lens]
        got = eng.step([StepEntry(s, t[:n], w) for s, t, n, w in zip(slots, toks, lens, wants)]).cpu().numpy()
        assert (len(eng._graphs) > 0) == (rnd >= 1), "the second step of a shape is captured"
        at = 0
        for t, n, w in zip(toks, lens, wants):
            check_logits(got[at:at + 2], plain_logits(d, t)[w], dtype, f"{name} round {rnd} prompt of {n}")
            at += 2
        # the cache that the (replayed) step left serves the next tokens
        for p in range(2):
            got = eng.step([StepEntry(s, [t[n + p]], [0]) for s, t, n in zip(slots, toks, lens)]).cpu().numpy()
            for j, (t, n) in enumerate(zip(toks, lens)):
                check_logits(got[j], plain_logits(d, t)[n + p], dtype, f"{name} round {rnd} token {p} after {n}")
        for s in slots:
            eng.free_slot(s)
    for s in parked:
        eng.free_slot(s)
    eng.cache.check()
    eng.wait()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_second_chunk_on_a_held_prefix_and_every_row_wanted(model_dirs, dtype):
    """Shapes with tokens held before the step (a prompt's second chunk) and with every row's logits
    wanted; a step of another shape in between takes its own way."""
    from alpacca_b200.engine import StepEntry
    d = model_dirs[("D", dtype)]
    cfg = CONFIGS["D"]
    eng = make_engine(d, dtype, max_tokens=64 * 30, max_slots=8)
    for rnd in range(4):
        t = tiny.prompt_tokens(cfg, 300, 2000 + rnd)
        want = plain_logits(d, t)
        s = eng.alloc_slot()
        eng.step([StepEntry(s, t[:130], [])])
        got = eng.step([StepEntry(s, t[130:], list(range(170)))]).cpu().numpy()
        check_logits(got, want[130:], dtype, f"round {rnd}: second chunk, every row")
        other = eng.alloc_slot()
        u = tiny.prompt_tokens(cfg, 40 + rnd, 2100 + rnd)
        got = eng.step([StepEntry(other, u, [len(u) - 1])]).cpu().numpy()
        check_logits(got[0], plain_logits(d, u)[-1], dtype, f"round {rnd}: a step of another shape")
        eng.free_slot(s)
        eng.free_slot(other)
    assert len(eng._graphs) == 2      # the first chunk's shape and the second chunk's
    eng.wait()


def test_long_prompts_through_the_tensor_core_kernels(model_dirs):
    """A shape long enough for the tcgen05 attention and (at real widths) the tcgen05 product: replays of a
    1,100-token prompt with other tokens agree with the step-by-step run of the same tokens exactly."""
    from alpacca_b200.engine import StepEntry
    d = model_dirs[("E", "bfloat16")]
    cfg = dict(CONFIGS["E"])
    eng = make_engine(d, "bfloat16", max_tokens=64 * 40, max_slots=4)
    ref = make_engine(d, "bfloat16", max_tokens=64 * 40, max_slots=4)
    ref.step_graphs = False
    for rnd in range(4):
        t = tiny.prompt_tokens(cfg, 500, 3000 + rnd)
        a, b = eng.alloc_slot(), ref.alloc_slot()
        got = eng.step([StepEntry(a, t, [0, 250, 499])])
        want = ref.step([StepEntry(b, t, [0, 250, 499])])
        assert torch.equal(got, want), f"round {rnd}: replayed and issued steps differ"
        eng.free_slot(a)
        ref.free_slot(b)
    assert len(eng._graphs) == 1 and len(ref._graphs) == 0
    eng.wait()
