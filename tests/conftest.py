import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def _has_gpu() -> bool:
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _has_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def oracle():
    from tests import oracle_binding
    return oracle_binding.load()


@pytest.fixture(scope="session")
def ctx_factory():
    """Creates (and caches per mode) contexts bound to cuda:0."""
    import torch
    from breeze_tts_cpp_b200 import ops
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    cache = {}

    def make(mode: str):
        if mode not in cache:
            cache[mode] = ops.Context(mode, device=0, workspace_bytes=32 << 20)
        return cache[mode]

    yield make
    for c in cache.values():
        c.close()


@pytest.fixture(scope="session")
def reference_kernels():
    """The reference's own CUDA kernels (oracle/_ref/libttsref.so); skipped where they were not built."""
    from tests import oracle_binding
    lib = oracle_binding.load_reference()
    if lib is None:
        pytest.skip("oracle/_ref/libttsref.so is not built")
    return lib
