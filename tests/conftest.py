import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")
# a checkout of the reference, if any: KVB_REFERENCE_ROOT, else a directory named "reference" beside this repository
REFERENCE_ROOT = os.environ.get("KVB_REFERENCE_ROOT") or os.path.join(os.path.dirname(ROOT), "reference")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the GPU box)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import kvarn_oracle

    kvarn_oracle.build()
    return kvarn_oracle
