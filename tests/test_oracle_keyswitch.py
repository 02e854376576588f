"""CPU checks of the oracle's restatement of the key-switch chain (external product, T -> [p | q]
conversion, ModDown) against plain integer arithmetic."""
import numpy as np

import helpers as H
from ckks_llm_b200 import params


def _setup(oracle, n=64, p_num=2, q_num=4, t_num=3):
    p = params.ntt_primes(41, 2 * n, p_num)
    q = params.ntt_primes(40, 2 * n, q_num)
    t = params.ntt_primes(60, 2 * n, t_num)
    return p, q, t, oracle.KeySwitchTables(p, q, t)


def test_external_product_is_a_digit_sum(oracle):
    n, gamma, l = 64, 3, 3
    p, q, t, KT = _setup(oracle)
    rng = np.random.default_rng(0)
    R = (len(p) + len(q) + gamma - 1) // gamma
    cb = (l + 1 + len(p) - 1) // len(p)
    dnum = len(q) // len(p)
    cipher = np.stack([H.uniform_residues(rng, t, (n,)) for _ in range(cb)])
    swk = np.stack([H.uniform_residues(rng, t, (n,)) for _ in range(2 * dnum * R)]).reshape(2, dnum, R, len(t), n)
    out = oracle.external_product_t(cipher, swk, n, KT, l, gamma)
    blocks = (len(p) + l + 1 + gamma - 1) // gamma
    for h in range(2):
        for blk in range(R):
            for k, tk in enumerate(t):
                exp = [sum(int(cipher[i, k, x]) * int(swk[h, i, blk, k, x]) for i in range(cb)) % tk if blk < blocks else 0
                       for x in range(n)]
                assert out[h, blk, k].tolist() == exp


def test_modup_t_to_pql_returns_the_centred_value(oracle):
    n, gamma, l = 64, 3, 2
    p, q, t, KT = _setup(oracle)
    T = 1
    for v in t:
        T *= v
    rng = np.random.default_rng(1)
    R = (len(p) + len(q) + gamma - 1) // gamma
    blocks = (len(p) + l + 1 + gamma - 1) // gamma
    vals = [[[int(rng.integers(-2**62, 2**62)) * int(rng.integers(1, 2**62)) % (T // 2) - T // 4 for _ in range(n)]
             for _ in range(blocks)] for _ in range(2)]
    inp = np.zeros((2, R, len(t), n), dtype=np.uint64)
    for c in range(2):
        for b in range(blocks):
            for k, tk in enumerate(t):
                inp[c, b, k] = [v % tk for v in vals[c][b]]
    out = oracle.modup_t_to_pql(inp, n, KT, l, gamma, 2)
    pq = p + q
    for c in range(2):
        for r in range(len(p) + l + 1):
            assert out[c, r].tolist() == [v % pq[r] for v in vals[c][r // gamma]]
        assert not out[c, len(p) + l + 1:blocks * gamma].any()


def test_moddown_subtracts_the_p_part(oracle):
    n, gamma, l = 64, 3, 3
    for p_num in (1, 2):
        p, q, t, KT = _setup(oracle, p_num=p_num)
        P = 1
        for v in p:
            P *= v
        rng = np.random.default_rng(2 + p_num)
        R = (len(p) + len(q) + gamma - 1) // gamma
        pq = p + q
        inp = np.zeros((2, R * len(t), n), dtype=np.uint64)
        for c in range(2):
            inp[c, :len(pq)] = H.uniform_residues(rng, pq, (n,))
        out = oracle.moddown_pql_to_ql(inp, n, KT, l, gamma, 2)
        for c in range(2):
            for i in range(l + 1):
                qi = q[i]
                exp = []
                for x in range(n):
                    if p_num == 1:
                        part = int(inp[c, 0, x]) % qi
                    else:
                        part = sum((int(inp[c, j, x]) * pow(P // p[j], -1, p[j]) % p[j]) * (P // p[j]) for j in range(p_num)) % qi
                    exp.append((int(inp[c, p_num + i, x]) - part) * pow(P, -1, qi) % qi)
                assert out[c, i].tolist() == exp


def _automorphism(f, e, q):
    """f(X^e) modulo X^n + 1 and q, e odd."""
    n = len(f)
    g = [0] * n
    for j, v in enumerate(f):
        k = j * e % (2 * n)
        if k < n:
            g[k] = (g[k] + int(v)) % q
        else:
            g[k - n] = (g[k - n] - int(v)) % q
    return np.array(g, dtype=np.uint64)


def test_rotation_map_and_reversal_are_the_galois_automorphisms(oracle):
    """In the NTT domain the reference rotates by permuting words and conjugates by reversing them
    (poly_arithmetic.cuh:581-596, :666-674).  The oracle's maps must be the automorphisms X -> X^(5^r) and
    X -> X^-1 of the coefficient domain."""
    n = 64
    q = params.ntt_primes(40, 2 * n, 1)
    T = oracle.NttTables(n, q)
    rng = np.random.default_rng(3)
    f = H.uniform_residues(rng, q, (n,))[0]

    def ntt(x):
        y = np.ascontiguousarray(x, dtype=np.uint64).copy()
        oracle.ntt_batch(y, T, 0, 0, 1, 1, 1)
        return y

    F = ntt(f)
    for rot in (1, 2, 7, 31, 32):
        dst = oracle.rotation_map(n, rot)
        assert sorted(dst.tolist()) == list(range(n))
        out = np.zeros_like(F)
        out[dst] = F
        assert np.array_equal(out, ntt(_automorphism(f, pow(5, rot, 2 * n), q[0]))), rot
    assert np.array_equal(F[::-1], ntt(_automorphism(f, 2 * n - 1, q[0])))


def test_conjugate_and_rotate_compose_the_chain(oracle):
    """conjugate_23 / leftRotate_23 = index map, chain, addition (KeySwitch_23.cuh:433-470, :548-581)."""
    n, gamma, l = 64, 3, 3
    p, q, t, KT = _setup(oracle)
    T = oracle.NttTables(n, p + q + t)
    rng = np.random.default_rng(5)
    R = (len(p) + len(q) + gamma - 1) // gamma
    dnum = len(q) // len(p)
    c = np.stack([H.uniform_residues(rng, q, (n,)) for _ in range(2)])
    key = np.stack([H.uniform_residues(rng, t, (n,)) for _ in range(2 * dnum * R)]).reshape(2, dnum, R, len(t), n)
    got = oracle.conjugate(c, key, T, KT, l, gamma)
    sw = oracle.keyswitch(np.ascontiguousarray(c[0, :l + 1, ::-1]), key, T, KT, l, gamma)
    for i in range(l + 1):
        assert np.array_equal(got[0, i], sw[0, i])
        assert got[1, i].tolist() == [(int(a) + int(b)) % q[i] for a, b in zip(sw[1, i], c[1, i, ::-1])]
    rot = 9
    got = oracle.rotate(c, key, rot, T, KT, l, gamma)
    sw = oracle.keyswitch(np.ascontiguousarray(c[0, :l + 1]), key, T, KT, l, gamma)
    dst = oracle.rotation_map(n, rot)
    for i in range(l + 1):
        assert np.array_equal(got[0, i][dst], sw[0, i])
        assert got[1, i][dst].tolist() == [(int(a) + int(b)) % q[i] for a, b in zip(sw[1, i], c[1, i])]
