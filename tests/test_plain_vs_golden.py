"""The plain implementation against the outputs of jtiro232/Alpacca's own model code
(tests/golden/*.npz, made by tests/golden/make_golden.py on the CPU)."""
import sys
from pathlib import Path

import numpy as np
import pytest

import plain_llama as plain

GOLDEN = Path(__file__).resolve().parent / "golden"
sys.path.insert(0, str(GOLDEN))
from make_golden import CASES, golden_weights  # noqa: E402


@pytest.mark.parametrize("name", sorted(CASES))
def test_plain_matches_the_reference(name):
    cfg, seed, n_tok = CASES[name]
    g = np.load(GOLDEN / f"{name}.npz")
    assert len(g["tokens"]) == n_tok
    model = plain.PlainLlama(cfg, golden_weights(cfg, seed))
    got = model.logits(g["tokens"].tolist())
    # the reference computes in float32 (NumPy path): agreement to float32 rounding
    assert np.abs(got - g["logits_token_by_token"]).max() < 2e-6
    assert np.abs(got[-1] - g["logits_batch_last"]).max() < 2e-6
