"""Shared by the GPU tests: tolerances and a cache of plain models."""
from __future__ import annotations

import functools

import numpy as np

import plain_llama as plain
import tiny

CONFIGS = {"a": tiny.TINY_A, "b": tiny.TINY_B, "c": tiny.TINY_C}

# Largest allowed |engine - plain| on logits.  The plain implementation is float64 on the stored
# weights.  float32: rounding of float32 sums over at most a few hundred terms, logits of order 1.
# bfloat16: activations are rounded to 8 bits of mantissa between the kernels (relative 2^-9 each,
# some dozens of roundings along the path, logits of order 1).
LOGIT_TOL = {"float32": 5e-5, "bfloat16": 6e-2}
# mean |difference| must be far below the maximum allowed
LOGIT_MEAN_TOL = {"float32": 1e-5, "bfloat16": 1.2e-2}


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
    assert diff.max() <= LOGIT_TOL[dtype], (f"{what}: max |diff| {diff.max():.3e} at {worst} "
                                            f"(allowed {LOGIT_TOL[dtype]:.1e}, mean {diff.mean():.3e})")
    assert diff.mean() <= LOGIT_MEAN_TOL[dtype], f"{what}: mean |diff| {diff.mean():.3e}"
