import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def ctx():
    """One context for the whole GPU session.  No skip: on a GPU box a missing library or device is a failure."""
    import jgpt_b200

    c = jgpt_b200.Context(0)
    yield c
    c.close()
