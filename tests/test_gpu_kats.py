"""The reference's known-answer tests run through the C ABI on the GPU."""
import pytest

import kat_runner

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from znn_b200 import ops as _ops
    _ops.init(0)
    return _ops


@pytest.mark.parametrize("name", kat_runner.CASES)
def test_cuda_matches_reference_kat(ops, name):
    kat_runner.run_case(ops, name)
