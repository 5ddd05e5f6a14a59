"""Sequences of several thousand tokens: a batch of four unequal prompts (100 to 5,000 tokens: block
tables of 2 to 79 pages, the prompt step's attention over dozens of key tiles), then 24 tokens fed one by
one, against the plain implementation; the same decode steps through the streamed decode attention; and
generation from these prompts replayed from CUDA graphs against the step-by-step decoder."""
import pytest
import torch

import plain_llama as plain
import tiny
from helpers import check_logits

pytestmark = pytest.mark.gpu

LENGTHS = [5000, 100, 2500, 4097]
FED = 24


@pytest.fixture(scope="module")
def long_dirs(tmp_path_factory):
    from alpacca_b200.engine.loading import write_random_model_dir
    root = tmp_path_factory.mktemp("long")
    cfg = dict(tiny.TINY_D, max_position_embeddings=8192)
    return cfg, {name: write_random_model_dir(root / name, cfg, 77, dtype=dt, std=0.1)
                 for name, dt in (("float32", torch.float32), ("bfloat16", torch.bfloat16))}


@pytest.fixture(scope="module")
def long_requests(long_dirs):
    cfg, dirs = long_dirs
    toks = [tiny.prompt_tokens(cfg, n + FED, 900 + j) for j, n in enumerate(LENGTHS)]
    want = {}
    for name, d in dirs.items():
        pm = plain.PlainLlama.from_dir(str(d))
        want[name] = [pm.logits(t) for t in toks]
    return toks, want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompts_of_thousands_of_tokens_and_the_steps_after_them(long_dirs, long_requests, dtype):
    from alpacca_b200 import ops
    from alpacca_b200.engine import Engine, StepEntry
    from alpacca_b200.engine.loading import load_model_dir
    _, dirs = long_dirs
    toks, want = long_requests
    want = want[dtype]
    eng = Engine(load_model_dir(dirs[dtype], dtype=dtype, device="cuda"), max_tokens=64 * 200, max_slots=6)
    for streamed in ((False, True) if dtype == "bfloat16" else (False,)):
        floor = ops.STREAM_MIN_BYTES
        ops.STREAM_MIN_BYTES = 0 if streamed else float("inf")     # every decode step takes the one kernel or the other
        eng.forget_graphs()         # steps captured with the one kernel are not replayed for the other
        try:
            slots = [eng.alloc_slot() for _ in toks]
            got = eng.step([StepEntry(s, t[:n], [0, n // 2, n - 1]) for s, t, n in zip(slots, toks, LENGTHS)])
            got = got.cpu().numpy()
            for j, n in enumerate(LENGTHS):
                check_logits(got[3 * j:3 * j + 3], want[j][[0, n // 2, n - 1]], dtype, f"prompt of {n} tokens")
            for p in range(FED):
                got = eng.step([StepEntry(slots[j], [toks[j][LENGTHS[j] + p]], [0]) for j in range(4)]).cpu().numpy()
                for j in range(4):
                    check_logits(got[j], want[j][LENGTHS[j] + p], dtype,
                                 f"token {p} after {LENGTHS[j]}" + (" (streamed)" if streamed else ""))
            eng.wait()
        finally:
            ops.STREAM_MIN_BYTES = floor
        for s in slots:
            eng.free_slot(s)
        eng.cache.check()


def test_generation_from_long_prompts_replayed_from_graphs(long_dirs, long_requests):
    """In 32-bit, where the two decoders add in the same order whatever the width of their block tables
    (the graph's is rounded up to its shape's): the same tokens."""
    from alpacca_b200.api import Model, generate
    from alpacca_b200.sampling import SamplerParams
    _, dirs = long_dirs
    toks, _ = long_requests
    prompts = [t[:n] for t, n in zip(toks, LENGTHS)]
    model = Model.load(dirs["float32"], dtype="float32", n_ctx=8192, max_batch=4)
    out = {}
    for graphs in (True, False):
        model.use_graphs = graphs
        res = generate(model, prompts, SamplerParams(temperature=0.7, seed=3), n_predict=70, stop_token_ids=[])
        out[graphs] = [r.token_ids for r in res]
        assert all(len(t) == 70 for t in out[graphs]) and model.engine.cache.slots.n_held == 0
    assert out[True] == out[False]


def test_bfloat16_generation_from_long_prompts_stays_within_the_plain_model_s_margin(long_dirs, long_requests):
    """In bfloat16 the graph's attention cuts a sequence into other chunks than the step-by-step path (its
    block table is wider), so the two may round differently: each greedy token of the graph decoder is
    held to the plain model's logits for the sequence as it stands instead."""
    from alpacca_b200.api import Model, generate
    from alpacca_b200.sampling import SamplerParams
    from test_gpu_generate import margin_ok
    _, dirs = long_dirs
    toks, _ = long_requests
    prompts = [t[:n] for t, n in zip(toks, LENGTHS)][1:3]        # 100 and 2,500 tokens
    model = Model.load(dirs["bfloat16"], dtype="bfloat16", n_ctx=8192, max_batch=4)
    assert model.use_graphs
    res = generate(model, prompts, SamplerParams.greedy(), n_predict=6, stop_token_ids=[])
    for p, r in zip(prompts, res):
        assert len(r.token_ids) == 6 and margin_ok(dirs["bfloat16"], p, r.token_ids, "bfloat16")
