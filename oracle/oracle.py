"""ctypes front end of the CPU oracle (oracle/ckks_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
benchmark's CPU-baseline leg.  The product package never imports this module.
"""
import ctypes as C
import os

import numpy as np

from .build import LIB, build_oracle

_U64P = np.ctypeslib.ndpointer(dtype=np.uint64, flags="C_CONTIGUOUS")
_I64P = np.ctypeslib.ndpointer(dtype=np.int64, flags="C_CONTIGUOUS")
_F32P = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")

_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB):
            build_oracle()
        L = C.CDLL(LIB)
        L.orc_num_threads.restype = C.c_int
        L.orc_set_threads.argtypes = [C.c_int]
        for name in ("orc_mulmod", "orc_powmod"):
            getattr(L, name).restype = C.c_uint64
            getattr(L, name).argtypes = [C.c_uint64] * 3
        L.orc_invmod.restype = C.c_uint64
        L.orc_invmod.argtypes = [C.c_uint64] * 2
        L.orc_shoup.restype = C.c_uint64
        L.orc_shoup.argtypes = [C.c_uint64] * 2
        L.orc_find_primitive_root.restype = C.c_uint64
        L.orc_find_primitive_root.argtypes = [C.c_uint64]
        L.orc_find_mth_root.restype = C.c_uint64
        L.orc_find_mth_root.argtypes = [C.c_uint64, C.c_uint64]
        L.orc_barrett_mu.argtypes = [C.c_uint64, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]
        L.orc_fill_tables.argtypes = [C.c_uint64, C.c_uint64, C.c_uint32, _U64P, _U64P, _U64P, _U64P]
        L.orc_ntt_batch.argtypes = [_U64P, C.c_uint32, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                    _U64P, _U64P, _U64P, C.c_int]
        L.orc_ntt_bruteforce.argtypes = [_U64P, _U64P, C.c_uint32, C.c_uint64, C.c_uint64]
        L.orc_modup.argtypes = [_U64P, _U64P, C.c_uint32, _U64P, C.c_int, _U64P, C.c_int, C.c_int,
                                C.c_int, C.c_int]
        L.orc_ppmm.argtypes = [_F32P, C.POINTER(C.c_void_p), _U64P, C.c_int, C.c_int, C.c_long,
                               C.c_int, _U64P, C.c_double, C.c_int, C.c_int]
        L.orc_rlwe_decompose.argtypes = [_U64P, _U64P, C.POINTER(C.c_void_p), C.c_long, C.c_int,
                                         C.c_int, C.c_int, C.c_int, _U64P]
        L.orc_ring_down.argtypes = [_I64P, _I64P, C.c_long, C.c_int, C.c_int]
        L.orc_mlwe_decrypt.argtypes = [_U64P, _I64P, _U64P, C.c_int, C.c_int, C.c_uint64]
        L.orc_negacyclic_mul_small.argtypes = [_U64P, _I64P, _U64P, C.c_long, C.c_uint64]
        L.orc_pack_embed.argtypes = [C.POINTER(C.c_void_p), _U64P, C.c_long, C.c_int, C.c_int, C.c_int,
                                     C.c_uint64, C.c_uint64]
        L.orc_pack_keymac.argtypes = [_U64P, _U64P, _U64P, C.c_long, C.c_int, _U64P]
        L.orc_pack_moddown.argtypes = [_U64P, _U64P, _U64P, C.c_long, C.c_uint64, C.c_uint64]
        L.orc_external_product_t.argtypes = [_U64P, _U64P, _U64P, C.c_uint32, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                             _U64P]
        L.orc_modup_t_to_pql.argtypes = [_U64P, _U64P, C.c_uint32] + [C.c_int] * 6 + [_U64P] * 7
        L.orc_moddown_pql_to_ql.argtypes = [_U64P, _U64P, C.c_uint32] + [C.c_int] * 6 + [_U64P] * 6
        L.orc_tensor_product.argtypes = [_U64P, _U64P, _U64P, _U64P, _U64P, C.c_uint32, C.c_int, C.c_int, _U64P]
        L.orc_add_switched.argtypes = [_U64P, _U64P, _U64P, C.c_uint32, C.c_int, C.c_int, _U64P]
        L.orc_mod_to_qi.argtypes = [_U64P, _U64P, C.c_uint32, C.c_int, C.c_int, _U64P]
        L.orc_rescale_combine.argtypes = [_U64P, _U64P, C.c_uint32, C.c_int, C.c_int, _U64P, _U64P, _U64P]
        L.orc_modup_q0_to_ql.argtypes = [_U64P, C.c_uint32, C.c_int, C.c_int, _U64P, C.c_int]
        _lib = L
    return _lib


def num_threads():
    return lib().orc_num_threads()


def set_threads(n):
    lib().orc_set_threads(int(n))


def find_psi(two_n, q):
    """2N-th root of unity the reference would pick (Utils.cuh:99-109)."""
    return int(lib().orc_find_mth_root(int(two_n), int(q)))


def barrett_mu(q):
    hi, lo = C.c_uint64(), C.c_uint64()
    lib().orc_barrett_mu(int(q), C.byref(hi), C.byref(lo))
    return hi.value, lo.value


class NttTables:
    """psi tables [mod][n] for a list of moduli, the layout of
    psi_table_device / psiinv_table_device (Context_23.cuh:481-521)."""

    def __init__(self, n, moduli):
        self.n = int(n)
        self.moduli = np.ascontiguousarray(moduli, dtype=np.uint64)
        k = len(self.moduli)
        self.psi_root = np.zeros(k, dtype=np.uint64)
        self.psi = np.zeros((k, n), dtype=np.uint64)
        self.psiinv = np.zeros((k, n), dtype=np.uint64)
        self.psi_shoup = np.zeros((k, n), dtype=np.uint64)
        self.psiinv_shoup = np.zeros((k, n), dtype=np.uint64)
        for i, q in enumerate(self.moduli):
            r = find_psi(2 * n, int(q))
            if r == 2 ** 64 - 1:
                raise ValueError(f"modulus {int(q)} is not 1 mod {2 * n}")
            self.psi_root[i] = r
            lib().orc_fill_tables(r, int(q), n, self.psi[i], self.psiinv[i],
                                  self.psi_shoup[i], self.psiinv_shoup[i])


def ntt_batch(data, tables, start_limb_off, start_mod_idx, poly_num, mod_num, poly_mod_len,
              inverse=False):
    """In-place batched transform, arguments as Context_23::ToNTTInplace /
    FromNTTInplace (Context_23.cuh:847-889)."""
    assert data.dtype == np.uint64 and data.flags.c_contiguous
    tab = tables.psiinv if inverse else tables.psi
    tabs = tables.psiinv_shoup if inverse else tables.psi_shoup
    lib().orc_ntt_batch(data.reshape(-1), tables.n, start_limb_off, start_mod_idx, poly_num,
                        mod_num, poly_mod_len, tables.moduli, tab.reshape(-1), tabs.reshape(-1),
                        1 if inverse else 0)
    return data


def ntt_bruteforce(a, q, psi):
    a = np.ascontiguousarray(a, dtype=np.uint64)
    out = np.zeros_like(a)
    lib().orc_ntt_bruteforce(a, out, len(a), int(q), int(psi))
    return out


def modup(inp, n, q, t, alpha, l, batch):
    """modUpQjtoT_23 (BasisConv.cuh:84-179): in [batch][q_num][n] ->
    out [batch][blocks][t_num][n]."""
    q = np.ascontiguousarray(q, dtype=np.uint64)
    t = np.ascontiguousarray(t, dtype=np.uint64)
    blocks = (l + 1 + alpha - 1) // alpha
    out = np.zeros((batch, blocks, len(t), n), dtype=np.uint64)
    lib().orc_modup(out.reshape(-1), np.ascontiguousarray(inp).reshape(-1), n, q, len(q), t,
                    len(t), alpha, l, batch)
    return out


def ppmm(W, X, q, scaler, m0=0, m1=None):
    """PPMM (PPMM_kernel.cuh:93-252).  W fp32 [M][K]; X uint64 [K][limbs][C] (one
    contiguous array, or a list of K arrays [limbs][C]); returns [M][limbs][C] with
    rows outside [m0, m1) left zero."""
    W = np.ascontiguousarray(W, dtype=np.float32)
    M, K = W.shape
    q = np.ascontiguousarray(q, dtype=np.uint64)
    limbs = len(q)
    rows = [np.ascontiguousarray(X[n], dtype=np.uint64) for n in range(K)]
    Cw = rows[0].shape[-1]
    assert all(r.shape == (limbs, Cw) for r in rows)
    ptrs = (C.c_void_p * K)(*[r.ctypes.data for r in rows])
    out = np.zeros((M, limbs, Cw), dtype=np.uint64)
    m1 = M if m1 is None else m1
    lib().orc_ppmm(W, ptrs, out.reshape(-1), M, K, Cw, limbs, q, float(scaler), m0, m1)
    return out


def rlwe_decompose(rlwe_a, rlwe_b, N1, k, mlwe_num, q):
    """rlweCipherDecompose_kernel (PCMM_Scheme.cuh:51-88) on coefficient-domain
    limbs [limbs][N]; returns [mlwe_num][limbs][k+1][N1]."""
    q = np.ascontiguousarray(q, dtype=np.uint64)
    limbs, N = rlwe_a.shape
    out = np.zeros((mlwe_num, limbs, k + 1, N1), dtype=np.uint64)
    ptrs = (C.c_void_p * mlwe_num)(*[out[i].ctypes.data for i in range(mlwe_num)])
    lib().orc_rlwe_decompose(np.ascontiguousarray(rlwe_a).reshape(-1),
                             np.ascontiguousarray(rlwe_b).reshape(-1), ptrs, N, N1, k, mlwe_num,
                             limbs, q)
    return out


def ring_down(S, N1, k):
    S = np.ascontiguousarray(S, dtype=np.int64)
    out = np.zeros_like(S)
    lib().orc_ring_down(S, out, len(S), N1, k)
    return out.reshape(k, N1)


def mlwe_decrypt(ct_limb, s_mlwe, q):
    """ct_limb [(k+1)][N1] for one limb -> message residues [N1]."""
    kp1, N1 = ct_limb.shape
    m = np.zeros(N1, dtype=np.uint64)
    lib().orc_mlwe_decrypt(np.ascontiguousarray(ct_limb).reshape(-1),
                           np.ascontiguousarray(s_mlwe, dtype=np.int64).reshape(-1), m, N1,
                           kp1 - 1, int(q))
    return m


def negacyclic_mul_small(a, s, q):
    a = np.ascontiguousarray(a, dtype=np.uint64)
    c = np.zeros_like(a)
    lib().orc_negacyclic_mul_small(a, np.ascontiguousarray(s, dtype=np.int64), c, len(a), int(q))
    return c


def mlwe_packing(mlwe, keys, N1, k, p, q0, tables):
    """PCMM_Scheme::mlweCipherPacking (PCMM_Scheme.cuh:362-430) for ring-pack moduli {p | q0, q1}.

    mlwe: [mlwe_num][(k+1)][N1] limb-0 words of the MLWE ciphertexts; keys: [k][2][2][N] repacking
    keys (a, b) x (p, q0) in the NTT domain; tables: NttTables over [p, q0].  Returns the packed
    RLWE ciphertext (a, b) mod q0 in the NTT domain plus the intermediate stages."""
    mlwe = np.ascontiguousarray(mlwe, dtype=np.uint64)
    keys = np.ascontiguousarray(keys, dtype=np.uint64)
    mlwe_num = mlwe.shape[0]
    N = N1 * k
    E = np.zeros((k + 1, 2, N), dtype=np.uint64)
    ptrs = (C.c_void_p * mlwe_num)(*[mlwe[i].ctypes.data for i in range(mlwe_num)])
    lib().orc_pack_embed(ptrs, E.reshape(-1), N, N1, k, mlwe_num, int(p), int(q0))
    stages = {"embed": E.copy()}
    ntt_batch(E, tables, 0, 0, k, 2, 2)                      # the k a-polynomials only (:401)
    O = np.zeros((2, 2, N), dtype=np.uint64)
    lib().orc_pack_keymac(E.reshape(-1), keys.reshape(-1), O.reshape(-1), N, k,
                          np.array([p, q0], dtype=np.uint64))
    stages["keymac"] = O.copy()
    ntt_batch(O, tables, 0, 0, 2, 2, 2, inverse=True)        # :416
    out = np.zeros((2, N), dtype=np.uint64)
    lib().orc_pack_moddown(O.reshape(-1), out[0], out[1], N, int(p), int(q0))
    stages["moddown"] = out.copy()
    out[1] = (out[1] + E[k, 1]) % np.uint64(q0)              # + embedded b, coefficient domain (:426)
    res = out[:, None, :].copy()                             # [2][1 limb][N]
    sub = NttTables.__new__(NttTables)
    sub.n, sub.moduli = tables.n, tables.moduli[1:2].copy()
    sub.psi, sub.psiinv = tables.psi[1:2].copy(), tables.psiinv[1:2].copy()
    sub.psi_shoup, sub.psiinv_shoup = tables.psi_shoup[1:2].copy(), tables.psiinv_shoup[1:2].copy()
    ntt_batch(res, sub, 0, 0, 2, 1, 1)                       # :428
    return res[:, 0, :], stages


def rescale(cipher, tables, p_num, L, l):
    """Scheme_23::rescaleAndEqual (Scheme_23.cuh:368-385) on a cipher buffer [2][L+1][n] (modified in
    place and returned); tables cover the moduli [p | q | ...]."""
    n = tables.n
    cipher = np.ascontiguousarray(cipher, dtype=np.uint64)
    flat = cipher.reshape(-1)
    q = np.ascontiguousarray(tables.moduli[p_num:p_num + L + 1])
    ntt_batch(flat, tables, l, p_num + l, 2, 1, L + 1, inverse=True)
    buf = np.zeros_like(flat)
    lib().orc_mod_to_qi(buf, flat, n, L + 1, l, q)
    ntt_batch(buf, tables, 0, p_num, 2, l, L + 1)
    qinv = np.array([pow(int(q[l]), -1, int(q[i])) for i in range(l)], dtype=np.uint64)
    qinv_s = np.array([(int(qinv[i]) << 64) // int(q[i]) for i in range(l)], dtype=np.uint64)
    lib().orc_rescale_combine(flat, buf, n, L + 1, l, q, qinv, qinv_s)
    return cipher


def modup_q0_to_ql(cipher, tables, p_num, L, target_level, scale_up):
    """Bootstrapper::modUpQ0toQL (bootstrapping/Bootstrapper.cuh:192-209) on a level-0 cipher buffer
    [2][L+1][n] (modified in place and returned)."""
    n = tables.n
    cipher = np.ascontiguousarray(cipher, dtype=np.uint64)
    flat = cipher.reshape(-1)
    q = np.ascontiguousarray(tables.moduli[p_num:p_num + L + 1])
    ntt_batch(flat, tables, 0, p_num, 2, 1, L + 1, inverse=True)
    lib().orc_modup_q0_to_ql(flat, n, L + 1, target_level, q, int(scale_up))
    ntt_batch(flat, tables, 0, p_num, 2, target_level + 1, L + 1)
    return cipher


class KeySwitchTables:
    """Constants of the key-switch chain computed with Python integers (definitions of
    Context_23::preComputeOnCPU, Context_23.cuh:60-192 and :286-351)."""

    def __init__(self, p, q, t):
        p, q, t = [int(v) for v in p], [int(v) for v in q], [int(v) for v in t]
        self.p, self.q, self.t = p, q, t
        pq = p + q
        T = 1
        for v in t:
            T *= v
        P = 1
        for v in p:
            P *= v
        u = lambda xs: np.array(xs, dtype=np.uint64)
        shoup = lambda x, m: (x << 64) // m
        self.pq = u(pq)
        self.tv = u(t)
        inv = [pow(T // ti, -1, ti) for ti in t]
        self.t_hat_inv, self.t_hat_inv_shoup = u(inv), u([shoup(a, m) for a, m in zip(inv, t)])
        self.t_hat_mod_r = u([[(T // ti) % r for ti in t] for r in pq]).reshape(-1)
        self.half_t = u([(T // 2) % m for m in pq + t])
        self.t_mod_pq = u([T % r for r in pq])
        inv = [pow(P // pj, -1, pj) for pj in p]
        self.p_hat_inv, self.p_hat_inv_shoup = u(inv), u([shoup(a, m) for a, m in zip(inv, p)])
        self.p_hat_mod_q = u([[(P // pj) % qi for pj in p] for qi in q]).reshape(-1)
        inv = [pow(P, -1, qi) for qi in q]
        self.p_inv_mod_q, self.p_inv_mod_q_shoup = u(inv), u([shoup(a, m) for a, m in zip(inv, q)])


def external_product_t(cipher_t, swk, n, KT, l, gamma):
    """Context_23::external_product_T (ExternalProduct.cuh:7-97): cipher_t [cipher_blocks][t_num][n], swk
    [2][dnum][R][t_num][n] -> out [2][R][t_num][n] (blocks beyond the level stay zero)."""
    p_num, q_num, t_num = len(KT.p), len(KT.q), len(KT.t)
    R = (p_num + q_num + gamma - 1) // gamma
    cb = (l + 1 + p_num - 1) // p_num
    blocks = (p_num + l + 1 + gamma - 1) // gamma
    out = np.zeros((2, R, t_num, n), dtype=np.uint64)
    lib().orc_external_product_t(out.reshape(-1), np.ascontiguousarray(cipher_t, dtype=np.uint64).reshape(-1),
                                 np.ascontiguousarray(swk, dtype=np.uint64).reshape(-1), n, t_num, R, cb, blocks,
                                 q_num // p_num, KT.tv)
    return out


def modup_t_to_pql(inp, n, KT, l, gamma, batch):
    """Context_23::modUpTtoPQl_23 (BasisConv.cuh:183-248): in [batch][R][t_num][n] -> out of the same shape with
    limb i of [p | q_0..q_l] at flat limb offset i of its half."""
    p_num, q_num, t_num = len(KT.p), len(KT.q), len(KT.t)
    R = (p_num + q_num + gamma - 1) // gamma
    out = np.zeros((batch, R * t_num, n), dtype=np.uint64)
    lib().orc_modup_t_to_pql(out.reshape(-1), np.ascontiguousarray(inp, dtype=np.uint64).reshape(-1), n, p_num, q_num,
                             t_num, l, gamma, batch, KT.pq, KT.tv, KT.t_hat_inv, KT.t_hat_inv_shoup, KT.t_hat_mod_r,
                             KT.half_t, KT.t_mod_pq)
    return out


def moddown_pql_to_ql(inp, n, KT, l, gamma, batch):
    """Context_23::modDownPQltoQl_23 (BasisConv.cuh:251-347): in as written by modup_t_to_pql -> out
    [batch][q_num][n], limbs 0..l."""
    p_num, q_num, t_num = len(KT.p), len(KT.q), len(KT.t)
    out = np.zeros((batch, q_num, n), dtype=np.uint64)
    lib().orc_moddown_pql_to_ql(out.reshape(-1), np.ascontiguousarray(inp, dtype=np.uint64).reshape(-1), n, p_num, q_num,
                                t_num, l, gamma, batch, KT.pq, KT.p_hat_inv, KT.p_hat_inv_shoup, KT.p_hat_mod_q,
                                KT.p_inv_mod_q, KT.p_inv_mod_q_shoup)
    return out


def keyswitch(inp, swk, tables, KT, l, gamma):
    """The chain of Scheme_23::mult_23 between the tensor product and the final addition
    (KeySwitch_23.cuh:219-232): inp [l+1][n] (NTT domain) -> out [2][q_num][n] (NTT domain, limbs 0..l).
    tables: NttTables over [p | q | t]."""
    n = tables.n
    p_num, q_num, t_num = len(KT.p), len(KT.q), len(KT.t)
    R = (p_num + q_num + gamma - 1) // gamma
    cb = (l + 1 + p_num - 1) // p_num
    blocks = (p_num + l + 1 + gamma - 1) // gamma
    coef = np.zeros((q_num, n), dtype=np.uint64)
    coef[:l + 1] = inp
    ntt_batch(coef.reshape(-1), tables, 0, p_num, 1, l + 1, q_num, inverse=True)
    dig = modup(coef[None], n, KT.q, KT.t, p_num, l, 1)[0]                     # [cb][t_num][n]
    ntt_batch(dig.reshape(-1), tables, 0, p_num + q_num, cb, t_num, t_num)
    ext = external_product_t(dig, swk, n, KT, l, gamma)
    for h in range(2):
        ntt_batch(ext[h].reshape(-1), tables, 0, p_num + q_num, blocks, t_num, t_num, inverse=True)
    pq = modup_t_to_pql(ext, n, KT, l, gamma, 2)
    out = moddown_pql_to_ql(pq, n, KT, l, gamma, 2)
    ntt_batch(out.reshape(-1), tables, 0, p_num, 2, l + 1, q_num)
    return out


def tensor_product(c1, c2, n, q, l):
    """compute_c0c1c2 (poly_arithmetic.cuh:787-824): c1, c2 [2][q_num][n] -> (a1b2+a2b1, a1a2, b1b2), each [q_num][n]."""
    q_num = len(q)
    outs = [np.zeros((q_num, n), dtype=np.uint64) for _ in range(3)]
    lib().orc_tensor_product(outs[0].reshape(-1), outs[1].reshape(-1), outs[2].reshape(-1),
                             np.ascontiguousarray(c1, dtype=np.uint64).reshape(-1),
                             np.ascontiguousarray(c2, dtype=np.uint64).reshape(-1), n, q_num, l + 1,
                             np.ascontiguousarray(q, dtype=np.uint64))
    return outs


def mult(c1, c2, rlk, tables, KT, l, gamma):
    """Scheme_23::mult_23 (KeySwitch_23.cuh:192-236): c1, c2 [2][q_num][n] in the NTT domain -> result
    [2][q_num][n], limbs 0..l."""
    n = tables.n
    axbx, axax, bxbx = tensor_product(c1, c2, n, KT.q, l)
    res = keyswitch(axax[:l + 1], rlk, tables, KT, l, gamma)
    lib().orc_add_switched(res.reshape(-1), axbx.reshape(-1), bxbx.reshape(-1), n, len(KT.q), l + 1,
                           np.array(KT.q, dtype=np.uint64))
    return res


def _bitrev(x, bits):
    x = np.asarray(x, dtype=np.int64)
    r = np.zeros_like(x)
    for b in range(bits):
        r |= ((x >> b) & 1) << (bits - 1 - b)
    return r


def rotation_map(n, rot_slots):
    """Destination index of every NTT-domain word under sk_and_poly_LeftRot_ntt_kernel
    (poly_arithmetic.cuh:581-596): pow = rotGroups[n/2 - rot_slots] with rotGroups[i] = 5^i mod 2n
    (Context_23.cuh:648-659); word j, which holds the value at the odd power 2*bitrev(j)+1, goes to the
    position that holds the power pow*(2*bitrev(j)+1) mod 2n."""
    logn = n.bit_length() - 1
    power = pow(5, n // 2 - rot_slots, 2 * n)
    j = np.arange(n, dtype=np.int64)
    t = 2 * _bitrev(j, logn) + 1
    t = (((power * t) & (2 * n - 1)) - 1) >> 1
    return _bitrev(t, logn)


def conjugate(cipher, conj_key, tables, KT, l, gamma):
    """Scheme_23::conjugate_23 (KeySwitch_23.cuh:433-470): both polynomials reversed in the NTT domain
    (sk_and_poly_conjugate_kernel, poly_arithmetic.cuh:666-674), the chain on the reversed a with the
    conjugation key, the reversed b added to the b half (poly_add_batch_device).  cipher [2][q_num][n]."""
    q_num = len(KT.q)
    cipher = np.ascontiguousarray(cipher, dtype=np.uint64).reshape(2, q_num, tables.n)
    ac = np.ascontiguousarray(cipher[0, :l + 1, ::-1])
    bc = cipher[1, :l + 1, ::-1]
    res = keyswitch(ac, conj_key, tables, KT, l, gamma)
    for i in range(l + 1):
        qi = np.uint64(KT.q[i])
        s = res[1, i] + bc[i]
        res[1, i] = np.where(s >= qi, s - qi, s)
    return res


def rotate(cipher, rot_key, rot_slots, tables, KT, l, gamma):
    """Scheme_23::leftRotate_23 (KeySwitch_23.cuh:548-581): the chain on a with the rotation key, b added to
    the b half, then both halves permuted in the NTT domain (sk_and_poly_LeftRot_ntt_double,
    poly_arithmetic.cuh:581-603).  cipher [2][q_num][n]."""
    n, q_num = tables.n, len(KT.q)
    cipher = np.ascontiguousarray(cipher, dtype=np.uint64).reshape(2, q_num, n)
    sw = keyswitch(np.ascontiguousarray(cipher[0, :l + 1]), rot_key, tables, KT, l, gamma)
    for i in range(l + 1):
        qi = np.uint64(KT.q[i])
        s = sw[1, i] + cipher[1, i]
        sw[1, i] = np.where(s >= qi, s - qi, s)
    dst = rotation_map(n, rot_slots)
    res = np.zeros_like(sw)
    res[:, :l + 1, dst] = sw[:, :l + 1, :]
    return res
