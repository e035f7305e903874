import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def port_oracle():
    from oracle import binding
    return binding.port()


@pytest.fixture(scope="session")
def ref_oracle():
    from oracle import binding
    r = binding.ref()
    if r is None:
        pytest.skip("oracle/_ref/libtnns_ref.so not built (reference sources absent)")
    return r


@pytest.fixture(scope="session")
def checker():
    """The reference's own objects when they were built, else the restatement."""
    from oracle import binding
    return binding.best()


@pytest.fixture(scope="session")
def gpu_ctx():
    import fastertnn_b200 as ft
    ctx = ft.Context(0)
    yield ctx
    ctx.close()
