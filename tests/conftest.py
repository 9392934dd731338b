import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 box)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as o

    o.lib()
    o.set_rows_at_once(True)  # eight K-quant rows per pass: bit-identical to the row-by-row loop (checked in test_oracle_kat.py)
    return o
