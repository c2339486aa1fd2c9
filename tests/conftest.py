import os
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
for p in (ROOT, HERE):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        # the GPU tests go through every head size: the library with all of them, built once
        if any("gpu" in item.keywords for item in items):
            from crane_b200.csrc import build
            build.build_kernels()
        return
    skip = pytest.mark.skip(reason="no CUDA device here")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """Tiny model folders with random weights, made on demand:
    model_folders(name, dtype) -> path."""
    import tiny_configs
    from crane_b200.weights.random_init import write_model_folder
    made = {}

    def get(name: str, dtype: str) -> str:
        key = (name, dtype)
        if key not in made:
            d = tmp_path_factory.mktemp(f"{name}_{dtype}")
            spec = tiny_configs.TINY[name]
            write_model_folder(str(d), spec["config"], spec["seed"], dtype, std=spec["std"],
                               norm_std=spec["norm_std"])
            made[key] = str(d)
        return made[key]
    return get
