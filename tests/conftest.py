import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    from oracle_lib import OracleOnly
    return OracleOnly()


@pytest.fixture(scope="session")
def ref():
    from oracle_lib import Ref
    if not Ref.available():
        pytest.skip("oracle/_ref/libgai_ref.so not built (reference sources not mounted)")
    return Ref()


@pytest.fixture(autouse=True)
def _gpu_tests_use_exact_weight_values(request):
    """GPU parity tests compare tightly against the oracle computing with the exact
    dequantised weight values (the reference's CUDA semantics); closeness to the
    fp16-rounding CPU path is asserted separately at the activation tolerance
    (tests/test_gpu_linear.py, tests/test_gpu_dropin.py)."""
    if request.node.get_closest_marker("gpu") is None:
        yield
        return
    from oracle_lib import OracleOnly
    o = OracleOnly()
    o.set_weight_rounding(False)
    yield
    o.set_weight_rounding(True)
