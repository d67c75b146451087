import importlib
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box with -m gpu)")


@pytest.fixture(scope="session")
def pkg():
    """The product package (its directory name is not a valid identifier, hence importlib)."""
    return importlib.import_module("qwen38-5080_b200")


@pytest.fixture(scope="session")
def oracle():
    from oracle import ref_attention
    return ref_attention


@pytest.fixture(scope="session")
def golden():
    import json
    import numpy as np
    data = np.load(ROOT / "tests" / "golden" / "attn_golden.npz")
    meta = json.loads(bytes(data["meta_json"]).decode())
    return data, meta


@pytest.fixture(scope="session")
def producer_golden():
    """Fixtures made by transformers' own q_norm / k_norm / rotary functions (tests/golden/make_golden_producer.py)."""
    import json
    import numpy as np
    data = np.load(ROOT / "tests" / "golden" / "producer_golden.npz")
    meta = json.loads(bytes(data["meta_json"]).decode())
    return data, meta


@pytest.fixture(scope="session")
def cuda_device():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("a gpu-marked test was selected but no CUDA device is visible")
    return torch.device("cuda:0")
