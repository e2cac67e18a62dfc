"""Shared test set-up: paths, the `gpu` marker, the CPU checkers and the golden vectors."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "p40-kernel_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN = os.path.join(ROOT, "tests", "golden", "pq2_golden.npz")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def port():
    """This repository's C restatement of the reference host path."""
    from oracle.build_oracle import build_oracle
    from oracle.oracle import Oracle
    build_oracle()
    return Oracle("port")


@pytest.fixture(scope="session")
def ref():
    """The reference's own headers, compiled here when a checkout is mounted, else the prebuilt
    library that travelled with the tree; skipped when neither exists."""
    from oracle.build_oracle import build_reference
    from oracle.oracle import Oracle
    if build_reference() is None:
        pytest.skip("oracle/_ref is not built and no reference checkout is mounted")
    return Oracle("reference")


@pytest.fixture(scope="session")
def golden():
    return dict(np.load(GOLDEN))


@pytest.fixture(scope="session")
def gpu():
    """torch + the CUDA library, for tests marked gpu.  A missing library is an error, not a skip."""
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import bonsai_b200
    bonsai_b200.lib()
    torch.cuda.set_device(0)
    return bonsai_b200
