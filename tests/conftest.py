"""Shared fixtures.  Tests that need a GPU carry @pytest.mark.gpu; everything else runs on CPU."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import __graft_entry__ as entry  # noqa: E402

TOL = 1e-4  # relative tolerance of the fp32 parity contract


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100)")


@pytest.fixture(scope="session")
def pkg():
    p = entry.load_package()
    if not os.path.exists(p.LIB_PATH):
        p.build()
    p.load_library()
    return p


@pytest.fixture(scope="session")
def oracle():
    o = entry.load_oracle()
    o.lib()
    return o


@pytest.fixture(scope="session")
def ctx(pkg):
    import torch

    if not torch.cuda.is_available():
        pytest.fail("a gpu-marked test ran without a CUDA device; the library has no CPU path")
    c = pkg.Context(0)
    yield c
    c.close()


@pytest.fixture(scope="session")
def dev():
    import torch

    return torch.device("cuda:0")


def to_dev(a, dev):
    import torch

    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)
