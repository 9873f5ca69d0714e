import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def native_lib():
    """The built native library; builds it when nvcc is present and it is out of date."""
    from attention_b200 import abi, build
    import shutil
    if shutil.which("nvcc"):
        build.build()
    return abi.lib()
