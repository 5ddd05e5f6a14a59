import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
for p in (str(ROOT), str(ROOT / "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    # a run on a machine without a GPU that did not deselect the gpu tests skips them
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """Model folders of the tiny configurations, written by the package's random-weights
    mode into a temporary folder: model_dirs[(name, dtype)] -> path."""
    import torch
    import tiny
    from alpacca_b200.engine.loading import write_random_model_dir

    root = tmp_path_factory.mktemp("models")
    out = {}
    # lower case: weights N(0, 0.02) as the benchmark configurations prescribe.  Upper case: the same
    # configuration with weights N(0, 0.1): scores of order 1, so that attention is sharp and a wrong
    # key, page, position or rotation moves the logits by a large share of their spread.
    for name, cfg, seed, std in (("a", tiny.TINY_A, 0, 0.02), ("b", tiny.TINY_B, 1, 0.02), ("c", tiny.TINY_C, 2, 0.02),
                                 ("d", tiny.TINY_D, 3, 0.02), ("e", tiny.TINY_E, 4, 0.02),
                                 ("B", tiny.TINY_B, 11, 0.1), ("C", tiny.TINY_C, 12, 0.1),
                                 ("D", tiny.TINY_D, 13, 0.1), ("E", tiny.TINY_E, 14, 0.1)):
        for dt_name, dt in (("float32", torch.float32), ("bfloat16", torch.bfloat16)):
            out[(name, dt_name)] = write_random_model_dir(root / f"{name}_{dt_name}", cfg, seed, dtype=dt, std=std)
    return out


def pytest_sessionfinish(session, exitstatus):
    """With ALPACCA_B200_ERROR_REPORT=<file>: the largest logit errors seen by `helpers.check_logits`,
    as shares of the logits' spread, one line per (test label stem, dtype).  The tolerances in
    helpers.py are set from such a report."""
    import os
    path = os.environ.get("ALPACCA_B200_ERROR_REPORT")
    if not path:
        return
    try:
        import helpers
    except Exception:
        return
    with open(path, "w") as f:
        for (stem, dtype), (mx, mean, n) in sorted(helpers.SEEN.items()):
            f.write(f"{dtype:9s} max/std {mx:.3e} mean/std {mean:.3e} n {n:5d}  {stem}\n")
