"""Pins the oracle's host table builders to the reference's OWN functions, compiled from
the reference sources into oracle/_ref/ (skipped when that library is not built)."""
import numpy as np
import pytest

from ckks_llm_b200 import params
from oracle import ref as R

pytestmark = pytest.mark.skipif(not R.available(), reason="reference driver library not built")


def test_roots_match_reference_search(oracle):
    moduli = params.REF_LOGN16_Q + params.REF_LOGN16_P + params.REF_LOGN16_T
    moduli += params.ntt_primes(50, 1 << 17, 6) + params.ntt_primes(60, 1 << 17, 3)
    for q in moduli:
        assert oracle.find_psi(1 << 17, q) == R.find_psi(1 << 17, q), hex(q)
    for q in params.ntt_primes(36, 1 << 13, 3):
        assert oracle.find_psi(1 << 13, q) == R.find_psi(1 << 13, q), hex(q)


@pytest.mark.parametrize("n,q", [(4096, params.REF_LOGN16_Q[0]), (1 << 16, params.REF_LOGN16_T[0]),
                                 (256, params.REF_LOGN16_Q[1])])
def test_tables_match_reference_builders(oracle, n, q):
    psi = R.find_psi(2 * n, q)
    ref_tabs = R.fill_tables(psi, q, n)
    T = oracle.NttTables(n, [q])
    for mine, theirs in zip([T.psi[0], T.psiinv[0], T.psi_shoup[0], T.psiinv_shoup[0]], ref_tabs):
        assert np.array_equal(mine, theirs)
