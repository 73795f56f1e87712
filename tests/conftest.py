import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (B200, sm_100a); run with -m gpu")
    # the CPU oracles are small: a few threads are plenty, and on a host whose cores are shared with other jobs a
    # thread per visible core makes every CPU tensor operation crawl
    import torch
    torch.set_num_threads(max(1, min(torch.get_num_threads(), 8)))


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

    return np.load(os.path.join(ROOT, "tests", "golden", "nf4_dequant_golden.npz"))
