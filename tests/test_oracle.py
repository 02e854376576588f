"""CPU tests of the oracle itself: ordering convention, inverses, exact big-integer
cross-checks, and the end-to-end decrypt check of configuration 1."""
import numpy as np
import pytest

import helpers as H
from ckks_llm_b200 import params


def test_root_search_matches_reference_anchors(oracle):
    # generators and 2^17-th roots the reference's search yields for its ring-pack moduli
    q0, q1 = params.REF_LOGN16_Q[0], params.REF_LOGN16_Q[1]
    assert oracle.lib().orc_find_primitive_root(q0) == 3
    assert oracle.find_psi(1 << 17, q0) == 292045007481771
    assert oracle.lib().orc_find_primitive_root(q1) == 13
    assert oracle.find_psi(1 << 17, q1) == 24070355809704


@pytest.mark.parametrize("n", [16, 64, 256, 1024])
def test_ntt_order_and_roundtrip(oracle, n):
    moduli = params.ntt_primes(50, 2 * n, 2) + params.ntt_primes(60, 2 * n, 1)
    T = oracle.NttTables(n, moduli)
    rng = np.random.default_rng(n)
    a = H.uniform_residues(rng, moduli, (n,))[None].copy()      # [1][3][n]
    d = a.copy()
    oracle.ntt_batch(d, T, 0, 0, 1, 3, 3)
    for i, q in enumerate(moduli):
        bf = oracle.ntt_bruteforce(a[0, i], q, int(T.psi_root[i]))
        assert np.array_equal(bf, d[0, i])          # out[j] = a(psi^(2*bitrev(j)+1))
        assert d[0, i].max() < q
    oracle.ntt_batch(d, T, 0, 0, 1, 3, 3, inverse=True)
    assert np.array_equal(d, a)


def test_ntt_is_negacyclic_convolution(oracle):
    n = 64
    q = params.ntt_primes(50, 2 * n, 1)[0]
    T = oracle.NttTables(n, [q])
    rng = np.random.default_rng(7)
    a = rng.integers(0, q, n, dtype=np.uint64)
    s = rng.integers(-1, 2, n).astype(np.int64)
    s_res = np.where(s >= 0, s, s + np.int64(q)).astype(np.uint64)
    ref = oracle.negacyclic_mul_small(a, s, q)
    A = a[None, None].copy(); S = s_res[None, None].copy()
    oracle.ntt_batch(A, T, 0, 0, 1, 1, 1); oracle.ntt_batch(S, T, 0, 0, 1, 1, 1)
    P = np.array([(int(x) * int(y)) % q for x, y in zip(A[0, 0], S[0, 0])], dtype=np.uint64)[None, None].copy()
    oracle.ntt_batch(P, T, 0, 0, 1, 1, 1, inverse=True)
    assert np.array_equal(P[0, 0], ref)


def test_ntt_batch_addressing(oracle):
    # limb offset and modulus offset: only the addressed limbs change
    n = 64
    moduli = params.ntt_primes(40, 2 * n, 4)
    T = oracle.NttTables(n, moduli)
    rng = np.random.default_rng(3)
    data = rng.integers(0, min(moduli), (2, 5, n), dtype=np.uint64)
    d = data.copy()
    oracle.ntt_batch(d, T, 1, 2, 2, 2, 5)           # limbs 1,2 of each poly with moduli 2,3
    for p in range(2):
        for l in range(5):
            if l in (1, 2):
                exp = oracle.ntt_bruteforce(data[p, l], moduli[l + 1], int(T.psi_root[l + 1]))
                assert np.array_equal(d[p, l], exp)
            else:
                assert np.array_equal(d[p, l], data[p, l])


def test_modup_matches_exact_crt(oracle):
    n, alpha, t_num = 64, 3, 4
    q = params.ntt_primes(50, 2 * n, 7)
    t = params.ntt_primes(60, 2 * n, t_num)
    l, batch = 6, 2                                  # digits of 3, 3 and 1 limbs
    rng = np.random.default_rng(11)
    inp = np.stack([H.uniform_residues(rng, q, (n,)) for _ in range(batch)])
    out = oracle.modup(inp, n, q, t, alpha, l, batch)
    assert out.shape == (batch, 3, t_num, n)
    exact = 0
    for b in range(batch):
        for blk in range(3):
            idx = list(range(blk * alpha, min(blk * alpha + alpha, l + 1)))
            Q = 1
            for j in idx:
                Q *= q[j]
            for x in range(n):
                val = 0
                for j in idx:
                    Qh = Q // q[j]
                    val += (int(inp[b, j, x]) * pow(Qh, -1, q[j]) % q[j]) * Qh
                val %= Q
                for k in range(t_num):
                    got = int(out[b, blk, k, x])
                    assert got < t[k]
                    # the float overflow count may be one short when the sum of fractions is
                    # within rounding of an integer: allow the lift to be off by one Q
                    assert got in ((val % t[k]), ((val + Q) % t[k]), ((val - Q) % t[k]))
                    exact += got == val % t[k]
    assert exact == batch * 3 * n * t_num


def test_ppmm_matches_python_bigint(oracle):
    rng = np.random.default_rng(5)
    M, K, Cw = 5, 7, 12
    q = params.ntt_primes(50, 1 << 13, 3)
    W = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    W[0, 0] = 0.0                 # w == 0 takes the a = q branch
    W[1, 1] = -0.0
    X = np.stack([H.uniform_residues(rng, q, (Cw,)) for _ in range(K)])
    for scaler in (float(1 << 30), float(q[1])):
        got = oracle.ppmm(W, X, q, scaler)
        exp = H.ppmm_python(W, X, q, scaler)
        assert np.array_equal(got, exp)


def test_ppmm_single_limb_has_no_rescale(oracle):
    rng = np.random.default_rng(6)
    q = params.ntt_primes(36, 1 << 13, 1)
    W = rng.uniform(-1, 1, (3, 4)).astype(np.float32)
    X = np.stack([H.uniform_residues(rng, q, (8,)) for _ in range(4)])
    got = oracle.ppmm(W, X, q, float(1 << 20))
    assert np.array_equal(got, H.ppmm_python(W, X, q, float(1 << 20)))


def test_rescale_wrap_semantics(oracle):
    # out_last > r + q_i is possible only when q_last > q_i; the reference lets the 64-bit
    # sum wrap (PPMM_kernel.cuh:244).  Force it with a tiny first modulus.
    q = [97, (1 << 40) + 15]      # moduli need not be NTT-friendly for the multiply
    W = np.array([[1.0]], dtype=np.float32)
    X = np.array([[[5], [(1 << 40) - 3]]], dtype=np.uint64)        # [K=1][limbs=2][C=1]
    got = oracle.ppmm(W, X, q, 1.0)
    exp = H.ppmm_python(W, X, q, 1.0)
    assert np.array_equal(got, exp)
    assert int(got[0, 1, 0]) == (1 << 40) - 3


def test_config1_end_to_end_decrypt(oracle):
    """Configuration 1: N=2^12, three 36-bit limbs, W 64x64 at 2^30, 64 tokens, ternary
    secret, sigma 3.2, seed 0: decrypted PPMM output vs fp64 matmul within 2^-20."""
    N, N1, k = 1 << 12, 64, 64
    moduli = H.cfg1_moduli()
    rng = np.random.default_rng(0)
    W = rng.uniform(-1, 1, (64, 64)).astype(np.float32)
    Xf = rng.uniform(-1, 1, (64, 64))                       # [feature][token]
    delta = float(1 << 30)
    msg = H.encode_coeffs(H.pack_message(Xf, k), delta, moduli)
    s = H.sparse_ternary(rng, N, 192)
    a, b = H.rlwe_encrypt(oracle, rng, msg, s, moduli)
    mlwe = oracle.rlwe_decompose(a, b, N1, k, 64, moduli)    # [64][3][k+1][N1]
    X = mlwe.reshape(64, 3, (k + 1) * N1)
    out = oracle.ppmm(W, X, moduli, delta)
    s_mlwe = oracle.ring_down(s, N1, k)
    expect = W.astype(np.float64) @ Xf                       # [m][token]
    scale_out = delta * delta / moduli[-1]
    worst = 0.0
    for m in range(64):
        dec = oracle.mlwe_decrypt(out[m, 0].reshape(k + 1, N1), s_mlwe, moduli[0])
        vals = H.centered(dec, moduli[0]) / scale_out
        worst = max(worst, np.abs(vals - expect[m]).max())
    rel = worst / np.abs(expect).max()
    assert rel < 2.0 ** -20, rel
