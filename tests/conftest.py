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
    for name, cfg, seed in (("a", tiny.TINY_A, 0), ("b", tiny.TINY_B, 1), ("c", tiny.TINY_C, 2),
                            ("d", tiny.TINY_D, 3), ("e", tiny.TINY_E, 4)):
        for dt_name, dt in (("float32", torch.float32), ("bfloat16", torch.bfloat16)):
            out[(name, dt_name)] = write_random_model_dir(root / f"{name}_{dt_name}", cfg, seed, dtype=dt)
    return out
