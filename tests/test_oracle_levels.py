"""CPU checks of the oracle's restatement of the two level changes around the PCMM
(Scheme_23::rescaleAndEqual, Bootstrapper::modUpQ0toQL) against plain integer arithmetic."""
import numpy as np

from ckks_llm_b200 import params


def _crt_poly(rng, q, n):
    """Random integer polynomial below prod(q) and its residues [len(q)][n]."""
    Q = 1
    for v in q:
        Q *= int(v)
    m = [int(rng.integers(0, 2**62)) * int(rng.integers(0, 2**62)) % Q for _ in range(n)]
    res = np.array([[c % int(v) for c in m] for v in q], dtype=np.uint64)
    return m, res


def test_rescale_divides_by_the_last_limb(oracle):
    n, L, l = 64, 3, 3
    p = params.ntt_primes(41, 2 * n, 1)
    q = params.ntt_primes(40, 2 * n, L + 1)
    T = oracle.NttTables(n, p + q)
    rng = np.random.default_rng(0)
    polys = [_crt_poly(rng, q, n) for _ in range(2)]
    cipher = np.stack([r for _, r in polys])                       # [2][L+1][n], coefficients
    oracle.ntt_batch(cipher.reshape(-1), T, 0, len(p), 2, l + 1, L + 1)
    out = oracle.rescale(cipher.copy(), T, len(p), L, l)
    oracle.ntt_batch(out.reshape(-1), T, 0, len(p), 2, l, L + 1, inverse=True)   # limbs < l back to coefficients
    for c, (m, _) in enumerate(polys):
        for i in range(l):
            exp = [((v - v % q[l]) // q[l]) % q[i] for v in m]
            assert out[c, i].tolist() == exp
        assert out[c, l].tolist() == [v % q[l] for v in m]         # the last limb is left as coefficients


def test_modup_q0_to_ql_lifts_centred(oracle):
    n, L, target = 64, 4, 3
    p = params.ntt_primes(41, 2 * n, 1)
    q = params.ntt_primes(40, 2 * n, L + 1)
    T = oracle.NttTables(n, p + q)
    rng = np.random.default_rng(1)
    x0 = rng.integers(0, q[0], size=(2, n), dtype=np.uint64)
    x0[0, :4] = [0, q[0] // 2, q[0] // 2 + 1, q[0] - 1]
    cipher = np.zeros((2, L + 1, n), dtype=np.uint64)
    cipher[:, 0] = x0
    oracle.ntt_batch(cipher.reshape(-1), T, 0, len(p), 2, 1, L + 1)
    scale_up = 37
    out = oracle.modup_q0_to_ql(cipher.copy(), T, len(p), L, target, scale_up)
    oracle.ntt_batch(out.reshape(-1), T, 0, len(p), 2, target + 1, L + 1, inverse=True)
    assert np.array_equal(out[:, 0], x0)
    for c in range(2):
        for i in range(target):
            qi = q[i + 1]
            exp = [((int(v) - q[0] + qi * scale_up) % 2**64) % qi if int(v) > q[0] // 2 else int(v) % qi
                   for v in x0[c]]
            assert out[c, i + 1].tolist() == exp
    assert not out[:, target + 1:].any()
