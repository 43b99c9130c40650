import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        has_cuda = torch.cuda.is_available()
    except Exception:
        has_cuda = False
    if has_cuda:
        return
    skip = pytest.mark.skip(reason="no CUDA device in this process")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def pkg():
    from __graft_entry__ import build, load_package
    build()
    return load_package()


@pytest.fixture(scope="session")
def orc():
    from __graft_entry__ import load_oracle
    o = load_oracle()
    o.build()
    return o


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    d = ROOT / "tests" / "golden"
    return {p.stem: np.load(p) for p in d.glob("*.npz")}


def golden_cases(npz, prefix):
    """Yield dicts of the arrays of every case under `prefix` (module/class)."""
    count = int(npz[prefix + "/__count__"])
    for i in range(count):
        head = f"{prefix}/{i}/"
        case = {k[len(head):]: npz[k] for k in npz.files if k.startswith(head)}
        # the reference loads every float array as Constant<float> (tfcc/test/blas.cpp:40-43)
        yield i, {k: (v.astype(np.float32) if v.dtype == np.float64 and k != "expect" else v)
                  for k, v in case.items()}
