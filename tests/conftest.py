import importlib
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = ROOT / "tests" / "golden"

# parity bars: max|a-b| / max|b| per output tensor
TOL_FP32 = 1e-4
TOL_BF16 = 2e-2


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def pkg():
    return importlib.import_module("dhammic-ai_b200")


@pytest.fixture(scope="session")
def cabi():
    build = importlib.import_module("dhammic-ai_b200.build")
    build.build()
    mod = importlib.import_module("dhammic-ai_b200._cabi")
    mod.load()
    return mod


@pytest.fixture(scope="session", autouse=True)
def _check_device_status(request):
    """On a GPU box every operator call is followed by the library's bounded-wait status check."""
    if torch.cuda.is_available():
        importlib.import_module("dhammic-ai_b200").set_check_status(True)
    yield


@pytest.fixture(scope="session")
def oracle():
    from oracle import ssd_oracle
    return ssd_oracle


def load_golden(name):
    d = np.load(GOLDEN / name, allow_pickle=True)
    return {k: d[k] for k in d.files}


def rel_err(a, b):
    a = a.detach().double().cpu()
    b = b.detach().double().cpu()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))
