"""Shared fixtures.  Tests marked ``gpu`` need a B200; everything else runs on the CPU."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """Random-weight model folders of the tiny configurations, made once per session in a
    temporary place: ``model_folders(name, store_dtype)`` -> path."""
    import torch
    from helpers import TINY, sharpen_for
    from xinfer_b200.weights import write_random_model
    made = {}

    def get(name: str, store_dtype=torch.float32) -> str:
        key = (name, store_dtype)
        if key not in made:
            d = tmp_path_factory.mktemp(f"model_{name}_{str(store_dtype).split('.')[-1]}")
            cfg, seed = TINY[name]
            write_random_model(str(d), cfg, seed, dtype=store_dtype, override=sharpen_for(cfg))
            made[key] = str(d)
        return made[key]

    return get
