"""What a step refuses on the host, before anything is launched (no device needed: the check reads
only the vocabulary size)."""
from types import SimpleNamespace

import numpy as np
import pytest

from alpacca_b200.engine.engine import Engine
from alpacca_b200.engine.step import StepEntry


def check(entries, vocab=10):
    return Engine._check(SimpleNamespace(vocab_size=vocab), entries)


def test_good_entries_come_back_as_int32_arrays():
    arrays = check([StepEntry(0, [1, 2, 9], [0, 2]), StepEntry(3, np.array([0, 5]), [])])
    assert [a.dtype for a in arrays] == [np.int32, np.int32]
    assert arrays[0].tolist() == [1, 2, 9] and arrays[1].tolist() == [0, 5]


@pytest.mark.parametrize("entries,needle", [
    ([], "at least one sequence"),
    ([StepEntry(0, [1], [0]), StepEntry(0, [2], [0])], "appears twice"),
    ([StepEntry(0, [], [])], "at least one token"),
    ([StepEntry(0, [1, 10], [0])], "token id 10 lies outside the vocabulary of 10"),
    ([StepEntry(0, [3, -1], [0])], "token id -1 lies outside"),
    ([StepEntry(0, [1.5, 2.0], [0])], "integers"),
    ([StepEntry(0, [[1, 2]], [0])], "flat list"),
    ([StepEntry(0, [1, 2], [2])], "wanted place 2 is not among its 2 tokens"),
    ([StepEntry(0, [1, 2], [-1])], "wanted place -1"),
])
def test_faulty_entries_are_refused(entries, needle):
    with pytest.raises(ValueError, match=needle):
        check(entries)


def test_an_engine_cannot_have_more_positions_than_its_model_was_built_for():
    """Tables indexed by position (the rotation's angles) have as many rows as the model was built for;
    an engine that let sequences grow beyond them would have the kernels read past their end."""
    import torch
    from alpacca_b200.parts.base import BuildOptions
    model = SimpleNamespace(opts=BuildOptions(dtype=torch.float32, device="cpu", max_positions=128),
                            cache_entry_specs=lambda: [], spec=SimpleNamespace(vocab_size=10))
    eng = Engine(model, max_tokens=256, max_slots=2)
    assert eng.max_positions == 128
    assert Engine(model, max_tokens=256, max_slots=2, max_positions=64).max_positions == 64
    with pytest.raises(ValueError, match="built\\s+for 128"):
        Engine(model, max_tokens=256, max_slots=2, max_positions=129)
