"""CPU check that the restated MLWE -> RLWE packing is the inverse of the decomposition at the
level of decrypted messages: encrypt, decompose into k MLWE ciphertexts, pack, decrypt."""
import numpy as np

import helpers as H
from ckks_llm_b200 import params


def test_decompose_then_pack_decrypts_to_the_message(oracle):
    N1, k = 32, 32
    N = N1 * k
    q0 = params.ntt_primes(50, 2 * N, 1)[0]
    p = params.ntt_primes(51, 2 * N, 1)[0]
    T = oracle.NttTables(N, [p, q0])
    rng = np.random.default_rng(0)
    s = H.sparse_ternary(rng, N, 64)
    vals = rng.uniform(-1, 1, N)
    delta = float(1 << 30)
    msg = H.encode_coeffs(vals, delta, [q0])
    a, b = H.rlwe_encrypt(oracle, rng, msg, s, [q0])
    mlwe = oracle.rlwe_decompose(a, b, N1, k, k, [q0])[:, 0]             # [k][(k+1)][N1]
    keys = H.repacking_keys(oracle, rng, s, N1, k, p, q0, T)
    packed, stages = oracle.mlwe_packing(mlwe, keys, N1, k, p, q0, T)      # NTT domain, mod q0
    sub = oracle.NttTables(N, [q0])
    coeff = packed[:, None, :].copy()
    oracle.ntt_batch(coeff, sub, 0, 0, 2, 1, 1, inverse=True)
    A, B = coeff[0, 0], coeff[1, 0]
    dec = (B + oracle.negacyclic_mul_small(A, s, q0)) % np.uint64(q0)
    got = H.centered(dec, q0) / delta
    assert np.abs(got - vals).max() < 2.0 ** -20
    # stage sanity: the embedding puts ciphertext i, coefficient g at g*k + i
    assert stages["embed"][k, 1, 5 * k + 3] == mlwe[3, k, 5]
