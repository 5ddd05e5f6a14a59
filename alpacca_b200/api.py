"""The Python entry point, in the reference's manner.

The reference is used as (tests/real_model_test.py:35-41, tests/bench.py:75-95):

    model = Model.load(path, n_ctx)
    result = generate(model, prompt_ids, SamplerParams(...), n_predict)
    logits = model.prefill(ids); logits = model.forward(id); model.reset()

The same names are here.  `generate` also takes a list of prompts and then
returns a list of results; prompts and results are token ids (there is no
tokenizer in this library).
"""
from __future__ import annotations

import time

import torch

from .engine.engine import Engine
from .engine.generate import GenerationResult, generate_requests
from .engine.loading import load_model_dir, random_model, resolve_dtype
from .engine.step import StepEntry
from .sampling import DeviceSampler, SamplerParams

DEFAULT_CTX = 4096   # alpacca/model.py:332: min(trained context, 4096) when no context is asked for


class Model:
    """A loaded model with its engine and cache."""

    def __init__(self, decoder, n_ctx: int, max_batch: int = 8, max_tokens: int | None = None):
        self.decoder = decoder
        self.config = decoder.config
        self.n_ctx = int(n_ctx)
        self.max_batch = int(max_batch)
        tokens = int(max_tokens) if max_tokens else self.max_batch * (-(-self.n_ctx // 64) * 64)
        self.engine = Engine(decoder, max_tokens=tokens, max_slots=max(self.max_batch, 1),
                             max_positions=self.n_ctx)
        self.load_seconds = 0.0
        # decode steps are replayed from CUDA graphs when every part of the model allows it
        self.use_graphs = self.engine.device.type == "cuda" and decoder.all_capturable()
        self._decoders: dict = {}
        self._slot = None            # the single sequence of prefill()/forward()/reset()
        self.cached_ids: list[int] = []
        self.last_prefill_forwarded = 0    # tokens the last prefill() ran (alpacca/model.py:612,628)

    # -- loading -----------------------------------------------------------
    @staticmethod
    def _context(n_ctx: int, trained: int) -> int:
        return min(n_ctx, trained) if n_ctx else min(trained, DEFAULT_CTX)

    @classmethod
    def load(cls, path, n_ctx: int = 0, progress: bool = True, dtype="bfloat16", max_batch: int = 8,
             max_tokens: int | None = None, device="cuda") -> "Model":
        """Loads a model folder (config.json + model.safetensors).  `n_ctx` as in the
        reference: 0 = min(trained context, 4096), else min(n_ctx, trained context)."""
        from .config import load_config
        t0 = time.time()
        trained = load_config(path).max_positions or DEFAULT_CTX
        ctx = cls._context(n_ctx, trained)
        decoder = load_model_dir(path, resolve_dtype(dtype), device, max_positions=ctx)
        m = cls(decoder, ctx, max_batch, max_tokens)
        m.load_seconds = time.time() - t0
        return m

    @classmethod
    def random(cls, config, seed: int = 0, n_ctx: int = 0, dtype="bfloat16", max_batch: int = 8,
               max_tokens: int | None = None, device="cuda") -> "Model":
        """A model of `config` (a dict of config.json keys or a typed configuration) with random weights."""
        from .config import config_from_dict
        t0 = time.time()
        if isinstance(config, dict):
            config = config_from_dict(config)
        ctx = cls._context(n_ctx, config.max_positions or DEFAULT_CTX)
        decoder = random_model(config, seed, resolve_dtype(dtype), device, max_positions=ctx)
        m = cls(decoder, ctx, max_batch, max_tokens)
        m.load_seconds = time.time() - t0
        return m

    # -- the reference's single-sequence calls -------------------------------------
    @property
    def n_past(self) -> int:
        return self.engine.length(self._slot) if self._slot is not None else 0

    def reset(self) -> None:
        if self._slot is not None:
            self.engine.free_slot(self._slot)
        self._slot = None
        self.cached_ids = []
        self.last_prefill_forwarded = 0

    def prefill(self, tokens) -> torch.Tensor | None:
        """Feeds prompt tokens to the single sequence; float32 logits [vocab] of the last one.

        As in the reference (alpacca/model.py:610-641): the longest common prefix of `tokens` and
        what the sequence holds is kept, the cache is truncated to it and only the rest is run; a
        prompt that is held in full runs its last token again.  `last_prefill_forwarded` counts the
        tokens that were run.  A model whose cache cannot be truncated starts the sequence anew."""
        tokens = [int(t) for t in tokens]
        self.last_prefill_forwarded = 0
        if not tokens:
            return None
        if len(tokens) > self.n_ctx:
            raise RuntimeError(f"context window full ({self.n_ctx} tokens)")
        n = 0
        if self._slot is not None:
            top = min(len(tokens), len(self.cached_ids))
            while n < top and tokens[n] == self.cached_ids[n]:
                n += 1
            if n == len(tokens):
                n = len(tokens) - 1
            if n != self.n_past:
                try:
                    self.engine.truncate(self._slot, n)
                except ValueError:
                    n = 0
                    self.reset()
        if self._slot is None:
            self._slot = self.engine.alloc_slot()
        del self.cached_ids[n:]
        suffix = tokens[n:]
        logits = self.engine.step([StepEntry(self._slot, suffix, [len(suffix) - 1])])
        self.engine.wait()       # the reference's prefill returns when the prompt has been evaluated
        self.cached_ids.extend(suffix)
        self.last_prefill_forwarded = len(suffix)
        return logits[0]

    def forward(self, token: int) -> torch.Tensor:
        """One more token of the single sequence; float32 logits [vocab]."""
        if self._slot is None:
            self._slot = self.engine.alloc_slot()
        if self.n_past >= self.n_ctx:
            raise RuntimeError(f"context window full ({self.n_ctx} tokens)")
        logits = self.engine.step([StepEntry(self._slot, [int(token)], [0])])
        self.cached_ids.append(int(token))
        return logits[0]

    def decoder_for(self, sampler):
        """The decoder of single-token steps for this sampler's options (graphs are captured per
        batch shape and per set of options, and kept)."""
        from .engine.decode import EagerDecoder, GraphDecoder
        if not self.use_graphs:
            return EagerDecoder(self.engine, sampler)
        p = sampler.params
        key = (p.temperature, p.top_k, p.top_p, p.repeat_penalty if p.penalizes else 1.0,
               p.repeat_last_n if p.penalizes else 0)
        dec = self._decoders.get(key)
        if dec is None:
            dec = self._decoders[key] = GraphDecoder(self.engine, sampler)
        dec.reset(sampler)
        return dec

    def describe(self) -> str:
        c, d = self.config, self.decoder
        dt = {torch.bfloat16: "bfloat16", torch.float32: "float32"}[d.opts.dtype]
        return (f"{c.architecture} | {len(d.spec.layers)} layers | {d.n_params() / 1e6:.0f}M params | "
                f"vocab {d.spec.vocab_size} | ctx {self.n_ctx} | {dt} | {self.engine.describe()}")


def generate(model: Model, prompt_ids, params: SamplerParams | None = None, n_predict: int = -1,
             stream=None, stop_token_ids=None):
    """Generates until a stop token, `n_predict` tokens or a full context.

    `prompt_ids`: one prompt (list of ints) -> one GenerationResult; a list of
    prompts -> a list of results, run as batches of up to `model.max_batch`.
    `stream(request index, token)` is called for each kept token.
    Stop tokens are the model's `eos_token_id` plus `stop_token_ids`.
    """
    params = params or SamplerParams()
    single = len(prompt_ids) == 0 or not isinstance(prompt_ids[0], (list, tuple))
    prompts = [prompt_ids] if single else list(prompt_ids)
    stop = set(model.decoder.spec.stop_token_ids) | set(stop_token_ids or ())
    sampler = DeviceSampler(params, model.engine.device)
    results = generate_requests(model.engine, sampler, prompts, n_predict, stop, model.max_batch,
                                bos_token_id=model.config.bos_token if model.config is not None else None, on_token=stream,
                                decoder=model.decoder_for(sampler))
    return results[0] if single else results


__all__ = ["Model", "generate", "GenerationResult", "SamplerParams"]
