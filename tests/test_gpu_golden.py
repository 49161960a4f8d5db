"""GPU parity, part 1: every fixture produced by the reference's CPU executor, run through the public
API (Var facade -> executor -> C ABI -> sm_100a kernels). Bit-exact for gathers / integer work,
|d| <= 1e-5*|ref| + 1e-5*max|ref| for floating point."""
import pytest

from tests import golden_cases as G

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def backend():
    from tests.product_backend import ProductBackend
    return ProductBackend()


@pytest.mark.parametrize("case", G.CASES, ids=G.case_ids())
def test_cuda_matches_reference(case, backend):
    got, want, exact = G.run_case(case, backend)
    G.check(got, want, exact)
