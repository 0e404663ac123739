import pathlib
import sys

import pytest

ROOT = pathlib.Path(__file__).resolve().parent.parent
for entry in (ROOT / "zig-cu-kernels_b200", ROOT):
    if str(entry) not in sys.path:
        sys.path.insert(0, str(entry))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def golden():
    import numpy as np

    folder = ROOT / "tests" / "golden"
    return {name: np.load(folder / f"{name}.npz") for name in ("quantizers", "gemm", "norm")}
