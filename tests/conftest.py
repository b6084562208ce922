import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a)")
    config.addinivalue_line("markers", "captures_graph: the test captures operator calls in a CUDA graph, so the "
                                       "synchronising status check after every call is left off")


def pytest_runtest_setup(item):
    # GPU tests run the operators in checked mode: after every call the device status words are read and a bounded
    # wait that gave up (or an inconsistent cu_seqlens) fails the test instead of passing with partial outputs.
    if item.get_closest_marker("gpu") is not None:
        os.environ["KDA_B200_CHECK"] = "0" if item.get_closest_marker("captures_graph") is not None else "1"


@pytest.fixture(scope="session")
def golden_dir():
    return os.path.join(ROOT, "tests", "golden")
