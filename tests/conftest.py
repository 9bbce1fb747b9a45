import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

# kernels compiled at run time are kept on disk between processes: the tests use a directory of their own
if "DB2_RTC_CACHE" not in os.environ:
    import atexit
    import shutil
    import tempfile
    os.environ["DB2_RTC_CACHE"] = tempfile.mkdtemp(prefix="db2_rtc_cache_")
    atexit.register(shutil.rmtree, os.environ["DB2_RTC_CACHE"], ignore_errors=True)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with `pytest -m gpu`)")


def _have_gpu() -> bool:
    try:
        from daphne_b200 import lib
        return lib.device_count() > 0
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _have_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for it in items:
        if "gpu" in it.keywords:
            it.add_marker(skip)


@pytest.fixture(scope="session")
def ctx():
    from daphne_b200.kernels import Context
    c = Context(0)
    yield c
    c.close()
