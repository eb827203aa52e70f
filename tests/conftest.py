import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def _host_impls():
    """The reference's integer tests are run against two implementations with one API:
    the CPU oracle and the product's C++ host layer reached through the C-ABI."""
    from oracle import ref_host

    impls = {"oracle": ref_host}
    try:
        from dmlx_b200 import host as product_host

        impls["product"] = product_host
    except Exception as e:  # library not built: the product leg fails loudly in its own test
        impls["product"] = e
    return impls


@pytest.fixture(params=["oracle", "product"])
def H(request):
    impl = _host_impls()[request.param]
    if isinstance(impl, Exception):
        pytest.fail(f"product host layer unavailable: {impl!r}")
    return impl
