import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "xstar-infer_b200"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) device")


@pytest.fixture(scope="session")
def oracle():
    from oracle import moe_oracle

    moe_oracle.build()
    return moe_oracle
