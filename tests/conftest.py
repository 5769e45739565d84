import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def oracle():
    """The CPU oracle (test infrastructure): compiled on first use."""
    from oracle import api
    api.build()
    return api


@pytest.fixture(scope="session")
def kat():
    import json
    return json.loads((ROOT / "tests" / "golden" / "reference_kat.json").read_text())


@pytest.fixture(scope="session")
def libb2q():
    """The product library; built in-tree if the .so is missing."""
    from oxicuda_b200 import _build, _lib
    _build.build()
    return _lib.lib()


@pytest.fixture(scope="session")
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from oxicuda_b200 import _build
    _build.build()
    torch.cuda.set_device(0)
    return torch.device("cuda:0")


@pytest.fixture
def switches(monkeypatch):
    """Sets B2Q_* experiment switches for one test: the library reads them when a handle is created, so the cached
    default handles are dropped before the test body runs and again after it."""
    from oxicuda_b200 import _lib

    def set_(**kw):
        for k, v in kw.items():
            monkeypatch.setenv(k, str(v))
        _lib.reset_default_handles()

    yield set_
    monkeypatch.undo()
    _lib.reset_default_handles()
