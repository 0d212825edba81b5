import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import spy_oracle

    spy_oracle.lib()
    return spy_oracle


@pytest.fixture(scope="session")
def ref():
    """The reference's own CPU path (oracle/_ref/libspy_ref.so); tests that need it are skipped where it was not built."""
    from oracle import spy_ref

    if not spy_ref.available():
        pytest.skip("oracle/_ref/libspy_ref.so not built (reference checkout absent)")
    spy_ref.lib()
    return spy_ref


@pytest.fixture(scope="session")
def tmp_models(tmp_path_factory):
    return tmp_path_factory.mktemp("models")
