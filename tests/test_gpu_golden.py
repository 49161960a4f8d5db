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


_GATHERS = [c for c in G.CASES if c["op"] in ("reindex", "getitem", "broadcast", "conv", "pool2d")]


@pytest.mark.parametrize("case", _GATHERS, ids=[c["name"] for c in _GATHERS])
def test_compiled_reindex_matches_reference(case, backend, monkeypatch):
    """The same gather fixtures with every affine reindex compiled for its op instance at first sight (a failed
    compilation is an error in this mode) instead of run by the ahead-of-time kernels."""
    monkeypatch.setenv("B200JT_REINDEX_JIT", "2")
    got, want, exact = G.run_case(case, backend)
    G.check(got, want, exact)
