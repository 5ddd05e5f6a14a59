"""The generation loop above the step function.

For one sequence the reference's loop is (alpacca/chat.py:140-182): feed the
prompt, then sample -> count -> stop token? -> budget? -> forward.  A stop token
is counted but neither returned nor fed back (:165-166); the last sampled
token is not forwarded (:176-177); sampling needs a free position
(`n_past < n_ctx`, :161); an empty prompt becomes [bos] (:145-148).

Here the same loop runs for a batch: the prompts of a batch, of unequal
lengths, go through one step; then every live sequence gets one token per
step; a sequence that ends gives its slot back at once and the others go on;
when the batch is done the next requests form the next batch, until none are
left.  Nothing joins a batch that has started.

The loop decides; it does not compute.  It needs of the engine only
`alloc_slot`, `free_slot`, `step`, `length`, `max_positions` and `room_for`
(and `wait`, if it has one),
and of the sampler only `new_state` and `sample`, so its decisions are tested
on the CPU with stand-ins for both.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field

from .step import StepEntry


@dataclass
class GenerationResult:
    token_ids: list = field(default_factory=list)   # generated tokens, without a final stop token
    tokens: int = 0                # tokens sampled, a final stop token included (alpacca/chat.py:163-166)
    seconds: float = 0.0           # from the end of the prompt step to this sequence's end
    finish_reason: str = ""        # "stop" | "length" | "context"
    prompt_tokens: int = 0

    @property
    def tok_per_sec(self) -> float:
        return self.tokens / self.seconds if self.seconds > 0 else 0.0


def _budget(prompt_len: int, n_predict: int, max_positions: int) -> int:
    # alpacca/chat.py:158: n_predict if > 0, else what the context has left
    return n_predict if n_predict and n_predict > 0 else max(max_positions - prompt_len, 0)


def plan_batches(prompt_lens, n_predict: int, max_positions: int, max_batch: int, room_for) -> list[list[int]]:
    """Splits the requests, in order, into batches that the cache can hold to their end.

    `room_for(token_counts)` says whether sequences of these final lengths fit
    together.  A request that does not even fit alone is an error.
    """
    batches, cur = [], []
    for i, n in enumerate(prompt_lens):
        if n > max_positions:
            raise ValueError(f"request {i}: prompt of {n} tokens exceeds the context of {max_positions}")
        worst = [min(prompt_lens[j] + _budget(prompt_lens[j], n_predict, max_positions), max_positions)
                 for j in cur + [i]]
        if cur and (len(cur) >= max_batch or not room_for(worst)):
            batches.append(cur)
            cur, worst = [], worst[-1:]
        if not cur and not room_for(worst):
            raise ValueError(f"request {i}: {worst[0]} tokens do not fit into the cache even alone")
        cur.append(i)
    if cur:
        batches.append(cur)
    return batches


def generate_requests(engine, sampler, prompts, n_predict: int = -1, stop_token_ids=(), max_batch: int = 8,
                      bos_token_id=None, on_token=None, timer=time.perf_counter,
                      decoder=None) -> list[GenerationResult]:
    """Generates for every prompt (a list of token ids); returns results in the order of the prompts.

    `on_token(request index, token)` is called for every token that is kept.  `decoder` runs the
    single-token steps (`step(live, more, stop) -> tokens`, see engine/decode.py); by default every
    step is one `engine.step` and one `sampler.sample`.
    """
    if decoder is None:
        from .decode import EagerDecoder
        decoder = EagerDecoder(engine, sampler)
    prompts = [list(p) for p in prompts]
    for i, p in enumerate(prompts):
        if not p:
            if bos_token_id is None or bos_token_id < 0:
                raise ValueError(f"request {i}: empty prompt and the model has no BOS token")
            prompts[i] = [int(bos_token_id)]
    stop = set(int(t) for t in stop_token_ids)
    max_pos = engine.max_positions
    results = [GenerationResult(prompt_tokens=len(p)) for p in prompts]
    for batch in plan_batches([len(p) for p in prompts], n_predict, max_pos, max_batch, engine.room_for):
        slots = {i: engine.alloc_slot() for i in batch}
        states = {i: sampler.new_state(i, prompts[i]) for i in batch}
        budgets = {i: _budget(len(prompts[i]), n_predict, max_pos) for i in batch}
        live = list(batch)
        try:
            logits = engine.step([StepEntry(slots[i], prompts[i], [len(prompts[i]) - 1]) for i in live])
            if hasattr(engine, "wait"):
                engine.wait()       # the clock starts when the prompt has been evaluated (alpacca/chat.py:153-157)
            t0 = timer()
            # tokens in the cache after the prompt; with k tokens sampled and all but the last fed
            # back a sequence holds base + k - 1 (the decoder may already be a step further)
            base = {i: engine.length(slots[i]) for i in live}

            def finish(i, reason):
                results[i].finish_reason = reason
                results[i].seconds = timer() - t0
                engine.free_slot(slots.pop(i))

            # a sequence whose prompt already fills the context cannot sample at all
            rows = []
            for r, i in enumerate(live):
                if engine.length(slots[i]) >= max_pos:
                    finish(i, "context")
                elif budgets[i] <= 0:
                    finish(i, "length")
                else:
                    rows.append(r)
            if len(rows) != len(live):
                live = [live[r] for r in rows]
                logits = logits[rows].contiguous() if rows else None
            tokens = sampler.sample(logits, [states[i] for i in live]) if live else []
            while live:
                entries, nxt = [], []
                for i, tok in zip(live, tokens):
                    res = results[i]
                    res.tokens += 1
                    if tok in stop:
                        finish(i, "stop")
                        continue
                    res.token_ids.append(tok)
                    if on_token is not None:
                        on_token(i, tok)
                    if res.tokens >= budgets[i]:
                        finish(i, "length")
                    elif base[i] + res.tokens >= max_pos:
                        finish(i, "context")
                    else:
                        entries.append((slots[i], tok, states[i]))
                        nxt.append(i)
                live = nxt
                if live:
                    # whether a sequence has room for one more step after this one (the two tests
                    # above, one token further), unless a stop token ends it
                    more = [results[i].tokens + 1 < budgets[i] and base[i] + results[i].tokens + 1 < max_pos
                            for i in live]
                    tokens = decoder.step(entries, more, stop)
        finally:
            for s in slots.values():
                engine.free_slot(s)
    return results
