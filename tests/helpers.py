"""Seeded input generators shared by the tests, the smoke check and the benchmark.

All randomness comes from numpy's PCG64 with explicit seeds (the reference's drivers are
unseeded: src/ckks/include/Utils.cuh:134-135), so every run sees the same words.
"""
import numpy as np

from ckks_llm_b200 import params


def uniform_residues(rng, moduli, shape_tail):
    """[len(moduli), *shape_tail] uint64 with limb i uniform in [0, q_i)."""
    out = np.empty((len(moduli),) + tuple(shape_tail), dtype=np.uint64)
    for i, q in enumerate(moduli):
        out[i] = rng.integers(0, int(q), size=shape_tail, dtype=np.uint64)
    return out


def cfg1_moduli():
    """Config 1: the three largest 36-bit primes = 1 mod 2^13."""
    return params.ntt_primes(36, 1 << 13, 3)


def sparse_ternary(rng, n, h):
    """Ternary secret of Hamming weight h (the reference samples h=192:
    test_rlwe_decomp.cu:23)."""
    s = np.zeros(n, dtype=np.int64)
    pos = rng.choice(n, size=h, replace=False)
    s[pos] = rng.choice(np.array([-1, 1], dtype=np.int64), size=h)
    return s


def encode_coeffs(vals, scale, moduli):
    """Coefficient encoding: data = (long)(v*scale); residue = data>=0 ? data : q+data
    (src/ckks/include/Encoder.cuh:68-78)."""
    data = np.trunc(np.asarray(vals, dtype=np.float64) * scale).astype(np.int64)
    out = np.empty((len(moduli), len(data)), dtype=np.uint64)
    for i, q in enumerate(moduli):
        out[i] = np.where(data >= 0, data, data + np.int64(q)).astype(np.uint64)
    return out


def rlwe_encrypt(oracle, rng, msg_res, s, moduli, sigma=3.2):
    """(a, b = -a*s + m + e) per limb in the coefficient domain; a uniform, e rounded
    Gaussian.  Decryption is b + a*s, the convention of the MLWE decryption
    (src/ckks/include/pcmm/PCMM_Scheme.cuh:546-554)."""
    limbs, n = msg_res.shape
    e = np.rint(rng.normal(0.0, sigma, size=n)).astype(np.int64)
    a = uniform_residues(rng, moduli, (n,))
    b = np.empty_like(a)
    for i, q in enumerate(moduli):
        a_s = oracle.negacyclic_mul_small(a[i], s, q)
        e_res = np.where(e >= 0, e, e + np.int64(q)).astype(np.uint64)
        b[i] = (msg_res[i] + e_res + (np.uint64(q) - a_s)) % np.uint64(q)
    return a, b


def centered(res, q):
    """Residues -> signed representatives in (-q/2, q/2] as float64."""
    r = res.astype(np.float64)
    return np.where(res > np.uint64(q // 2), r - float(q), r)


def pack_message(x_feat_tok, k):
    """Feature n, token t -> RLWE coefficient n + t*k (test_rlwe_decomp.cu:92-98)."""
    n_feat, n_tok = x_feat_tok.shape
    out = np.zeros(k * n_tok, dtype=np.float64)
    for t in range(n_tok):
        out[t * k: t * k + n_feat] = x_feat_tok[:, t]
    return out


def ppmm_python(W, X, q, scaler):
    """Independent big-integer PPMM for tiny shapes (Python ints), following
    PPMM_kernel.cuh:12-31,213-249 literally."""
    M, K = W.shape
    limbs = len(q)
    Cw = X.shape[-1]
    out = np.zeros((M, limbs, Cw), dtype=np.uint64)
    w = [[int(np.float64(W[m, n]) * np.float64(scaler)) for n in range(K)] for m in range(M)]
    for m in range(M):
        last = None
        for i in range(limbs - 1, -1, -1):
            qi = int(q[i])
            r = []
            for c in range(Cw):
                acc = 0
                for n in range(K):
                    a = w[m][n] if w[m][n] > 0 else qi + w[m][n]
                    acc += a * int(X[n][i][c])
                r.append((acc % (1 << 128)) % qi)
            if i == limbs - 1:
                last = r
                out[m, i] = np.array(r, dtype=np.uint64)
            else:
                inv = pow(int(q[limbs - 1]), -1, qi)
                res = []
                for c in range(Cw):
                    tmp = (r[c] + qi - last[c]) % (1 << 64)
                    res.append(tmp * inv % qi)
                out[m, i] = np.array(res, dtype=np.uint64)
    return out


def repacking_keys(oracle, rng, s, N1, k, p, q0, tables, sigma=3.2):
    """Repacking keys of PCMM_Scheme::addRepakcingKey (PCMM_Scheme.cuh:152-223): for every MLWE
    secret component i, (a_i, b_i = -a_i*s + e_i + p*iota(s_i)) over the limbs [p, q0] in the NTT
    domain, iota placing coefficient j at j*k (:149).  Returns [k][2][2][N]."""
    N = N1 * k
    mods = [p, q0]
    s_mlwe = oracle.ring_down(s, N1, k)                       # [k][N1]
    s_res = np.stack([np.where(s >= 0, s, s + np.int64(m)).astype(np.uint64) for m in mods])[None].copy()
    oracle.ntt_batch(s_res, tables, 0, 0, 1, 2, 2)            # s in the NTT domain, both limbs
    keys = np.zeros((k, 2, 2, N), dtype=np.uint64)
    for i in range(k):
        e = np.rint(rng.normal(0.0, sigma, size=N)).astype(np.int64)
        iota = np.zeros(N, dtype=np.int64)
        iota[::k] = s_mlwe[i]
        msg = np.zeros((1, 2, N), dtype=np.uint64)
        for m, mod in enumerate(mods):
            t = (e.astype(object) + int(p) * iota.astype(object)) % int(mod)
            msg[0, m] = np.array(t, dtype=np.uint64)
        oracle.ntt_batch(msg, tables, 0, 0, 1, 2, 2)
        for m, mod in enumerate(mods):
            a = rng.integers(0, mod, N, dtype=np.uint64)
            a_s = np.array([(int(x) * int(y)) % int(mod) for x, y in zip(a, s_res[0, m])], dtype=np.uint64)
            keys[i, 0, m] = a
            keys[i, 1, m] = (msg[0, m] + np.uint64(mod) - a_s) % np.uint64(mod)
    return keys
