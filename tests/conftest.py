import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")
    _build_library_if_missing()


def _build_library_if_missing():
    """The package refuses to import without its CUDA library; build it (nvcc, no GPU needed) when it is not
    there, so that a fresh checkout can run the tests.  (Only when missing: file times do not survive every way
    of copying a tree, and a rebuild takes minutes.)  Loaded by path: importing the package itself needs the
    library."""
    import importlib.util

    spec = importlib.util.spec_from_file_location("_moa_b200_build", os.path.join(ROOT, "moa_b200", "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    if os.path.exists(mod.LIB):
        return
    try:
        mod.build()
    except Exception as exc:     # no nvcc on this machine: the tests that need the package will say so
        print(f"[conftest] could not build libmoa_b200.so: {exc}", file=sys.stderr)


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN
