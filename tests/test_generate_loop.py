"""The generation loop's decisions, with stand-ins for the engine and the sampler (CPU)."""
import pytest
import torch

from alpacca_b200.engine.generate import generate_requests, plan_batches

V = 50


class FakeEngine:
    """Keeps the books of slots and lengths; its logits point at (last token + 1) % V, so greedy
    generation counts upwards from the prompt's last token."""

    def __init__(self, max_positions=32, max_slots=4, pages=8):
        self.max_positions, self.max_slots, self.pages = max_positions, max_slots, pages
        self.lengths, self.free, self.steps, self.freed = {}, list(range(max_slots)), [], []

    def alloc_slot(self):
        s = self.free.pop(0)
        self.lengths[s] = 0
        return s

    def free_slot(self, s):
        assert s in self.lengths, "slot freed twice"
        del self.lengths[s]
        self.free.append(s)
        self.freed.append(s)

    def length(self, s):
        return self.lengths[s]

    def room_for(self, counts):
        used = sum(-(-n // 64) for n in self.lengths.values())
        return len(counts) <= len(self.free) and sum(-(-n // 64) for n in counts) <= self.pages - used

    def step(self, entries):
        self.steps.append([(e.slot, list(e.tokens)) for e in entries])
        out = torch.zeros(len(entries), V)
        for r, e in enumerate(entries):
            assert e.want == [len(e.tokens) - 1]
            self.lengths[e.slot] += len(e.tokens)
            assert self.lengths[e.slot] <= self.max_positions
            out[r, (e.tokens[-1] + 1) % V] = 1.0
        return out


class GreedySampler:
    class State:
        def __init__(self, stream, prompt):
            self.stream, self.seen = stream, list(prompt)

    def new_state(self, stream, prompt):
        return self.State(stream, prompt)

    def sample(self, logits, states):
        assert logits.shape[0] == len(states)
        toks = logits.argmax(-1).tolist()
        for s, t in zip(states, toks):
            s.seen.append(t)
        return toks


def run(prompts, n_predict=-1, stop=(), engine=None, **kw):
    engine = engine or FakeEngine()
    res = generate_requests(engine, GreedySampler(), prompts, n_predict, stop, **kw)
    assert engine.lengths == {} and sorted(engine.free) == list(range(engine.max_slots)), "slots were lost"
    return res, engine


def test_budget_and_last_token_not_forwarded():
    res, eng = run([[3, 4]], n_predict=3)
    assert res[0].token_ids == [5, 6, 7] and res[0].tokens == 3 and res[0].finish_reason == "length"
    # one prompt step and two decode steps: the third token is never fed back (alpacca/chat.py:176-177)
    assert [len(s) for s in eng.steps] == [1, 1, 1] and eng.steps[-1][0][1] == [6]


def test_stop_token_is_counted_not_returned_not_forwarded():
    res, eng = run([[3, 4]], n_predict=10, stop=(7,))
    assert res[0].token_ids == [5, 6] and res[0].tokens == 3 and res[0].finish_reason == "stop"
    assert eng.steps[-1][0][1] == [6]


def test_unequal_prompts_run_as_one_batch_and_end_at_different_times():
    res, eng = run([[1], [10, 11, 12], [20, 21]], n_predict=6, stop=(14, 25))
    assert [r.token_ids for r in res] == [[2, 3, 4, 5, 6, 7], [13], [22, 23, 24]]
    assert [r.finish_reason for r in res] == ["length", "stop", "stop"]
    assert [r.prompt_tokens for r in res] == [1, 3, 2]
    # all prompts in the first step, together
    assert [len(t) for _, t in eng.steps[0]] == [1, 3, 2]
    # live sequences per step shrink as requests end; nothing joins
    assert [len(s) for s in eng.steps] == [3, 3, 2, 2, 1, 1]
    # a finished request gives its slot back at once, before the batch is over
    assert eng.freed[0] == 1


def test_context_limit_ends_a_sequence():
    eng = FakeEngine(max_positions=6)
    res, eng = run([[1, 2, 3, 4]], engine=eng)            # n_predict -1: until the context is full
    # sampling needs a free position (alpacca/chat.py:161): positions 4 and 5 are filled, then it ends
    assert res[0].token_ids == [5, 6] and res[0].finish_reason in ("context", "length")
    res, _ = run([[1, 2, 3, 4, 5, 6]], n_predict=5, engine=FakeEngine(max_positions=6))
    assert res[0].tokens == 0 and res[0].finish_reason == "context"
    with pytest.raises(ValueError, match="exceeds the context"):
        run([[1] * 7], engine=FakeEngine(max_positions=6))


def test_requests_beyond_a_batch_run_in_later_batches_with_reused_slots():
    eng = FakeEngine(max_slots=2)
    res, eng = run([[i] for i in range(5)], n_predict=2, engine=eng, max_batch=2)
    assert [r.token_ids for r in res] == [[i + 1, i + 2] for i in range(5)]
    firsts = [s for s in eng.steps if len(s[0][1]) == 1 and s[0][1][0] in (0, 2, 4)]
    assert [len(s) for s in firsts] == [2, 2, 1]            # batches of 2, 2, 1, one after another
    assert set(slot for s in eng.steps for slot, _ in s) == {0, 1}


def test_batches_respect_the_cache():
    # 8 pages of 64: prompts of 100 with 100 more tokens need 4 pages each
    assert plan_batches([100] * 5, 100, 1000, 8, lambda c: sum(-(-n // 64) for n in c) <= 8) == [[0, 1], [2, 3], [4]]
    assert plan_batches([10, 10, 10], 5, 1000, 2, lambda c: True) == [[0, 1], [2]]
    with pytest.raises(ValueError, match="even alone"):
        plan_batches([600], 100, 1000, 8, lambda c: sum(-(-n // 64) for n in c) <= 8)


def test_empty_prompt_takes_bos():
    res, eng = run([[]], n_predict=1, bos_token_id=9)
    assert eng.steps[0][0][1] == [9] and res[0].token_ids == [10]
    with pytest.raises(ValueError, match="BOS"):
        run([[]], n_predict=1)


def test_on_token_and_slot_release_on_error():
    seen = []
    run([[1], [5]], n_predict=2, on_token=lambda i, t: seen.append((i, t)))
    assert seen == [(0, 2), (1, 6), (0, 3), (1, 7)]

    class Boom(FakeEngine):
        def step(self, entries):
            if len(self.steps) == 2:
                raise RuntimeError("boom")
            return super().step(entries)
    eng = Boom()
    with pytest.raises(RuntimeError):
        generate_requests(eng, GreedySampler(), [[1], [2]], 5, ())
    assert eng.lengths == {}, "slots must come back when a step fails"


def test_the_loop_tells_the_decoder_who_comes_back():
    """`more` and `stop` let a decoder know, from a step's tokens alone, which sequences the loop
    brings to the next step (it may start that step early): the forecast must be exact, whatever
    ends a sequence (budget, context, stop token)."""
    from alpacca_b200.engine.decode import EagerDecoder

    class Forecasting(EagerDecoder):
        forecast = None
        calls = 0

        def step(self, live, more=None, stop=()):
            assert more is not None and len(more) == len(live)
            if self.forecast is not None:
                assert [(slot, tok) for slot, tok, _ in live] == self.forecast
            tokens = super().step(live)
            self.forecast = [(slot, t) for (slot, _, _), t, m in zip(live, tokens, more) if m and t not in stop]
            type(self).calls += 1
            return tokens

    for kw in (dict(n_predict=5, stop=()), dict(n_predict=-1, stop=()), dict(n_predict=9, stop=(9, 14))):
        eng = FakeEngine(max_positions=12)
        dec = Forecasting(eng, GreedySampler())
        res = generate_requests(eng, dec.sampler, [[3, 4], [7], [10, 11, 12, 13, 1]], kw["n_predict"], kw["stop"],
                                decoder=dec)
        assert dec.forecast == [], "the last step must forecast that nobody comes back"
        assert eng.lengths == {}
        assert [r.finish_reason for r in res] != []
    assert Forecasting.calls > 10
