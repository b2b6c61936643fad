"""pytest configuration: the `gpu` marker and shared fixtures."""
import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")
    config.addinivalue_line("markers", "multigpu: needs at least 2 CUDA devices")
    config.addinivalue_line("markers", "slow: spawns torchrun ranks on CPU, 15-25 s each "
                                       "(quick loop: -m 'not gpu and not slow')")


def pytest_collection_modifyitems(config, items):
    try:
        import torch

        ngpu = torch.cuda.device_count() if torch.cuda.is_available() else 0
    except Exception:
        ngpu = 0
    skip_gpu = pytest.mark.skip(reason="no CUDA device")
    skip_multi = pytest.mark.skip(reason="needs >= 2 CUDA devices")
    for item in items:
        if "gpu" in item.keywords and ngpu == 0:
            item.add_marker(skip_gpu)
        if "multigpu" in item.keywords and ngpu < 2:
            item.add_marker(skip_multi)


@pytest.fixture(scope="session")
def native_lib():
    """The native library; on a GPU machine its absence is a failure, not a skip."""
    from commbench_b200 import _native

    if not _native.available():
        from commbench_b200 import _build

        _build.build()
    return _native.load()
