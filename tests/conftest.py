import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
for _p in (str(ROOT), str(ROOT / "tests")):
    if _p not in sys.path:
        sys.path.insert(0, _p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    from oracle.pyoracle import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def reference():
    from oracle.pyoracle import Reference
    try:
        return Reference()
    except FileNotFoundError as e:  # neither the checkout nor a prebuilt library
        pytest.skip(str(e))


@pytest.fixture(scope="session")
def reference_gpu():
    """The unmodified reference GPU code, prebuilt where the reference checkout was present."""
    from oracle.pyoracle import ReferenceGpu
    try:
        return ReferenceGpu()
    except FileNotFoundError as e:
        pytest.skip(str(e))


@pytest.fixture(scope="session")
def capi():
    from nv_embedding_cache_b200 import capi as _capi
    return _capi


@pytest.fixture(scope="session")
def torch_cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("this test is marked gpu but no CUDA device is visible")
    torch.cuda.set_device(0)
    return torch
