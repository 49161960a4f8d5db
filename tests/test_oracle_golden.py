"""Pins the CPU oracle to the reference: every fixture made by the reference's CPU executor must be
reproduced by oracle/meta_ops_ref.py (bit-exact for gathers / integer work, 1e-5 mixed otherwise)."""
import numpy as np
import pytest

from oracle import meta_ops_ref as oracle
from tests import golden_cases as G


class OracleBackend:
    def __getattr__(self, name):
        return getattr(oracle, name)

    @staticmethod
    def reindex_bf16_bits(bits, shape, indexes, fill):
        # a gather moves bit patterns; fill = bf16(fill) (exact for the small integers used)
        x = (bits.astype(np.uint32) << 16).view(np.float32)
        y = oracle.reindex(x, shape, indexes, fill)
        return (y.view(np.uint32) >> 16).astype(np.uint16)


@pytest.mark.parametrize("case", G.CASES, ids=G.case_ids())
def test_oracle_matches_reference(case):
    got, want, exact = G.run_case(case, OracleBackend())
    G.check(got, want, exact)
