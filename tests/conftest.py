"""pytest configuration: the `gpu` marker and one-time builds of the checker and the CUDA library."""
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    """GPU tests are skipped, not failed, where no device exists."""
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session", autouse=True)
def built_artifacts():
    """The oracle (rebuilt by make when stale) and the CUDA library (rebuilt when a source or header is newer than
    its object, so the tests never run against a stale binary)."""
    subprocess.run(["make", "-C", str(ROOT / "oracle"), "-s"], check=True)
    import shutil
    from richengine_b200 import build, lib
    if shutil.which("nvcc") or not lib.LIBRARY_PATH.exists():  # no compiler on this machine: test the library as shipped
        build.build()
    yield


def pytest_report_header(config):
    from richengine_b200 import lib
    path = lib.LIBRARY_PATH
    if not path.exists():
        return f"librichkv: {path} (not built yet)"
    import datetime
    stamp = datetime.datetime.fromtimestamp(path.stat().st_mtime).isoformat(timespec="seconds")
    return f"librichkv: {path} built {stamp}, {path.stat().st_size} bytes"
