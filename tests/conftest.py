import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with `-m gpu`)")


@pytest.fixture(scope="session")
def built_lib():
    """The C-ABI library, built in-tree if missing or stale (nvcc cross-compiles without a GPU)."""
    from muxserve_b200 import build
    build.build()
    from muxserve_b200 import _lib
    return _lib.lib()


@pytest.fixture(scope="session")
def ref_classes():
    """(KVStorage, BatchScheduler) of the compiled reference, or skip when it was never built."""
    from oracle import build_ref
    classes = build_ref.load_ref()
    if classes is None and build_ref.build_ref():
        classes = build_ref.load_ref()
    if classes is None:
        pytest.skip("compiled reference (oracle/_ref) not available")
    return classes
