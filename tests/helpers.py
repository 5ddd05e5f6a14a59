"""Shared by the GPU tests: tolerances and a cache of plain models."""
from __future__ import annotations

import functools

import numpy as np

import plain_llama as plain
import tiny

CONFIGS = {"a": tiny.TINY_A, "b": tiny.TINY_B, "c": tiny.TINY_C, "d": tiny.TINY_D, "e": tiny.TINY_E,
           # the same configurations with weights N(0, 0.1) (see conftest.model_dirs)
           "B": tiny.TINY_B, "C": tiny.TINY_C, "D": tiny.TINY_D, "E": tiny.TINY_E}

# Allowed |engine - plain| on logits.  The plain implementation is float64 on the stored weights.
# float32: absolute; rounding of float32 sums over at most a few hundred terms, logits of order 1.
# bfloat16: a share of the spread (standard deviation) of the plain logits that are compared,
# since activations are rounded to 8 bits of mantissa between the kernels and the error grows with
# the values.  The largest errors measured over all tests of the suite (conftest's error report) are
# 0.123 of the spread for a single logit and 0.027 for the mean, both at the N(0, 0.1) models, whose
# sharp softmax passes on the rounding of the scores; the shares allowed are about 2.4 and 2.2 times
# those (every kernel adds in a fixed order, so a run repeats its errors exactly; the room is for
# other tile sizes on a GPU with another number of processors).
LOGIT_TOL = {"float32": 5e-5}
LOGIT_MEAN_TOL = {"float32": 1e-5}
BF16_MAX_SHARE = 0.30
BF16_MEAN_SHARE = 0.06

SEEN: dict = {}     # (label without its numbers, dtype) -> (largest max/std, largest mean/std, count)


def logit_tolerances(want, dtype: str):
    """(largest, mean) allowed |difference| against the plain logits `want`."""
    if dtype == "bfloat16":
        spread = float(np.asarray(want, np.float64).std())
        return BF16_MAX_SHARE * spread, BF16_MEAN_SHARE * spread
    return LOGIT_TOL[dtype], LOGIT_MEAN_TOL[dtype]


@functools.lru_cache(maxsize=None)
def plain_model(model_dir: str) -> plain.PlainLlama:
    return plain.PlainLlama.from_dir(model_dir)


@functools.lru_cache(maxsize=None)
def _plain_logits(model_dir: str, tokens: tuple) -> np.ndarray:
    return plain_model(model_dir).logits(list(tokens))


def plain_logits(model_dir, tokens) -> np.ndarray:
    """Float64 logits [T, V] of the whole sequence (cached per sequence)."""
    return _plain_logits(str(model_dir), tuple(int(t) for t in tokens))


def check_logits(got, want, dtype: str, what: str = "") -> None:
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    assert got.shape == want.shape, f"{what}: shape {got.shape} != {want.shape}"
    assert np.isfinite(got).all(), f"{what}: logits are not finite"
    diff = np.abs(got - want)
    worst = np.unravel_index(np.argmax(diff), diff.shape)
    tol, mean_tol = logit_tolerances(want, dtype)
    spread = max(float(want.std()), 1e-30)
    key = ("".join(c for c in what if not c.isdigit()), dtype)
    old = SEEN.get(key, (0.0, 0.0, 0))
    SEEN[key] = (max(old[0], diff.max() / spread), max(old[1], diff.mean() / spread), old[2] + 1)
    assert diff.max() <= tol, (f"{what}: max |diff| {diff.max():.3e} at {worst} (allowed {tol:.2e}, "
                               f"mean {diff.mean():.3e}, spread of the logits {spread:.3e})")
    assert diff.mean() <= mean_tol, f"{what}: mean |diff| {diff.mean():.3e} (allowed {mean_tol:.2e})"


def load_part(part, seed=0, dtype="float32", std=0.3):
    """Gives a part random weights; returns them as float64 arrays by name."""
    import torch
    from alpacca_b200.weights import Fetcher, RandomSource
    dt = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
    src = RandomSource(part.param_specs(), seed, dt, std=std)
    part.load(Fetcher(src, "cuda", dt))
    return {n: src.get(n).double().numpy() for n in src.table()}


class PartHarness:
    """A cache and step contexts for running one mixer (or block) alone."""

    def __init__(self, cache_specs, dtype="float32", max_tokens=64 * 16, max_slots=4, max_positions=1024):
        import torch
        from alpacca_b200.cache import SequenceCache
        from alpacca_b200.engine.step import ContextBuilder
        dt = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
        self.cache = SequenceCache(cache_specs, max_tokens, max_slots, max_positions, dt, torch.device("cuda"))
        self.builder = ContextBuilder("cuda")

    def step(self, seqs):
        """seqs: list of (slot, number of new tokens).  Returns the context; call `done` afterwards."""
        from alpacca_b200.engine.step import StepEntry
        entries = [StepEntry(s, [0] * n, []) for s, n in seqs]
        self.cache.reserve([(s, n) for s, n in seqs])
        ctx = self.builder.build(entries, [self.cache.length(s) for s, _ in seqs], self.cache)
        self._pending = [(s, n) for s, n in seqs]
        return ctx

    def done(self):
        self.cache.commit(self._pending)
