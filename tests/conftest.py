"""Shared fixtures.  Tests marked `gpu` need a B200; everything else runs on CPU."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def port():
    """The plain-C restatement of the reference algorithms (oracle/port.c)."""
    from oracle import oracle
    return oracle.load_port()


@pytest.fixture(scope="session")
def ref():
    """The reference Thrust itself (OpenMP backend) where oracle/_ref has been built."""
    from oracle import oracle
    o = oracle.load_ref()
    if o is None:
        pytest.skip("oracle/_ref/liboracle_ref.so is not built (needs the reference checkout)")
    return o


@pytest.fixture(scope="session")
def oracles():
    """Every oracle available: the port always, the reference build when present."""
    from oracle import oracle
    out = [oracle.load_port()]
    r = oracle.load_ref()
    if r is not None:
        out.append(r)
    return out


@pytest.fixture(scope="session")
def golden():
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden_v1.npz")
    return np.load(path)


@pytest.fixture(scope="session")
def tb():
    """The product: thrust_b200 over the C ABI.  Fails loudly if the CUDA library is missing."""
    import torch
    if not torch.cuda.is_available():
        pytest.fail("a `gpu` test was started without a CUDA device")
    import thrust_b200
    thrust_b200._lib.load()
    return thrust_b200
