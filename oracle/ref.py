"""ctypes front end of oracle/_ref/libref_driver.so: the REAL reference's host table
builders and CUDA kernels (see oracle/ref_driver.cu).  TEST INFRASTRUCTURE ONLY."""
import ctypes as C
import os

import numpy as np

from .build_ref import LIB, build_ref

_U64P = np.ctypeslib.ndpointer(dtype=np.uint64, flags="C_CONTIGUOUS")
_F32P = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_lib = None


def available():
    return build_ref() is not None and os.path.exists(LIB)


def lib():
    global _lib
    if _lib is None:
        if not available():
            raise RuntimeError("reference driver library is not built")
        L = C.CDLL(LIB)
        L.ref_find_mth_root.restype = C.c_uint64
        L.ref_find_mth_root.argtypes = [C.c_uint64, C.c_uint64]
        L.ref_fill_tables.argtypes = [C.c_uint64, C.c_uint64, C.c_uint, _U64P, _U64P, _U64P, _U64P]
        L.ref_ntt.argtypes = [_U64P, C.c_int, _U64P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]
        L.ref_modup.argtypes = [_U64P, _U64P, C.c_int, _U64P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                _U64P, _U64P, _U64P, _U64P]
        L.ref_ppmm.argtypes = [_F32P, _U64P, _U64P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _U64P,
                               C.c_double, _U64P, _U64P]
        L.ref_rescale_stage.argtypes = [_U64P, _U64P, C.c_int, _U64P, C.c_int, C.c_int, C.c_int, C.c_int, _U64P, _U64P]
        L.ref_modup_q0_to_ql.argtypes = [_U64P, C.c_int, _U64P, C.c_int, C.c_int, C.c_int, C.c_int]
        L.ref_keyswitch_stage.argtypes = [_U64P, _U64P, _U64P, C.c_int, _U64P] + [C.c_int] * 6 + [_U64P] * 10
        if hasattr(L, "ref_tensor_product"):
            L.ref_tensor_product.argtypes = [_U64P, _U64P, _U64P, C.c_int, _U64P, C.c_int, C.c_int, C.c_int, C.c_int]
        if hasattr(L, "ref_galois"):
            L.ref_galois.argtypes = [_U64P, _U64P, C.c_int, _U64P, C.c_int, C.c_int, C.c_int, C.c_long, C.c_int]
        L.ref_decompose.argtypes = [_U64P, _U64P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _U64P]
        _lib = L
    return _lib


def find_psi(two_n, q):
    return int(lib().ref_find_mth_root(int(two_n), int(q)))


def fill_tables(psi, q, n):
    out = [np.zeros(n, dtype=np.uint64) for _ in range(4)]
    lib().ref_fill_tables(int(psi), int(q), int(n), *out)
    return out  # psi, psiinv, psi_shoup, psiinv_shoup


def ntt(data, logN, pqt, start_poly_idx, start_mod_idx, poly_num, mod_num, poly_mod_len, inverse=False):
    d = np.ascontiguousarray(data, dtype=np.uint64).copy()
    pqt = np.ascontiguousarray(pqt, dtype=np.uint64)
    rc = lib().ref_ntt(d.reshape(-1), logN, pqt, len(pqt), start_poly_idx, start_mod_idx, poly_num, mod_num,
                       poly_mod_len, int(inverse))
    if rc:
        raise RuntimeError(f"ref_ntt failed with {rc}")
    return d


def modup(inp, logN, p, q, t, l, batch, tables):
    """tables = (hat_inv, hat_inv_shoup, hat_mod_t, blk_mod_t) for level l."""
    pqt = np.ascontiguousarray(list(p) + list(q) + list(t), dtype=np.uint64)
    alpha = len(p)
    blocks = (l + 1 + alpha - 1) // alpha
    out = np.zeros((batch, blocks, len(t), 1 << logN), dtype=np.uint64)
    rc = lib().ref_modup(out.reshape(-1), np.ascontiguousarray(inp, dtype=np.uint64).reshape(-1), logN, pqt,
                         len(p), len(q), len(t), l, batch, *[np.ascontiguousarray(x, dtype=np.uint64) for x in tables])
    if rc:
        raise RuntimeError(f"ref_modup failed with {rc}")
    return out


def ppmm(W, X, N1, rank, q, scaler, qinv, qinv_shoup):
    W = np.ascontiguousarray(W, dtype=np.float32)
    X = np.ascontiguousarray(X, dtype=np.uint64)
    M, K = W.shape
    limbs = len(q)
    out = np.zeros((M, limbs, (rank + 1) * N1), dtype=np.uint64)
    rc = lib().ref_ppmm(W, X.reshape(-1), out.reshape(-1), M, K, N1, rank, limbs,
                        np.ascontiguousarray(q, dtype=np.uint64), float(scaler),
                        np.ascontiguousarray(qinv, dtype=np.uint64), np.ascontiguousarray(qinv_shoup, dtype=np.uint64))
    if rc:
        raise RuntimeError(f"ref_ppmm failed with {rc}")
    return out


def decompose(rlwe, logN, N1, rank, mlwe_num, L, l, q):
    """rlwe [2][L+1][N] coefficient domain -> [mlwe_num][l+1][(rank+1)*N1] by the reference kernel."""
    rlwe = np.ascontiguousarray(rlwe, dtype=np.uint64)
    out = np.zeros((mlwe_num, l + 1, (rank + 1) * N1), dtype=np.uint64)
    rc = lib().ref_decompose(rlwe.reshape(-1), out.reshape(-1), logN, N1, rank, mlwe_num, L, l,
                             np.ascontiguousarray(q, dtype=np.uint64))
    if rc:
        raise RuntimeError(f"ref_decompose failed with {rc}")
    return out


def _pack_fns():
    L = lib()
    if not hasattr(L, "ref_pack_embed"):
        return None
    L.ref_pack_embed.argtypes = [_U64P, _U64P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_uint64, C.c_uint64]
    L.ref_pack_keymac.argtypes = [_U64P, _U64P, _U64P, C.c_int, C.c_int, C.c_int, C.c_uint64, C.c_uint64]
    L.ref_pack_moddown.argtypes = [_U64P, _U64P, C.c_int, C.c_uint64, C.c_uint64]
    return L


def pack_embed(mlwe, logN, N1, rank, p, q0):
    """mlwe [num][(rank+1)*N1] -> E [(rank+1)][2][N] by mlweCipherEmbedding_new_kernel."""
    L = _pack_fns()
    mlwe = np.ascontiguousarray(mlwe, dtype=np.uint64)
    E = np.zeros((rank + 1, 2, 1 << logN), dtype=np.uint64)
    rc = L.ref_pack_embed(mlwe.reshape(-1), E.reshape(-1), logN, N1, rank, mlwe.shape[0], int(p), int(q0))
    if rc:
        raise RuntimeError(f"ref_pack_embed failed with {rc}")
    return E


def pack_keymac(E_ntt, keys, logN, N1, rank, p, q0):
    L = _pack_fns()
    O = np.zeros((2, 2, 1 << logN), dtype=np.uint64)
    rc = L.ref_pack_keymac(np.ascontiguousarray(E_ntt, dtype=np.uint64).reshape(-1),
                           np.ascontiguousarray(keys, dtype=np.uint64).reshape(-1), O.reshape(-1), logN, N1, rank,
                           int(p), int(q0))
    if rc:
        raise RuntimeError(f"ref_pack_keymac failed with {rc}")
    return O


def pack_moddown(O, logN, p, q0):
    L = _pack_fns()
    out = np.zeros((2, 1 << logN), dtype=np.uint64)
    rc = L.ref_pack_moddown(np.ascontiguousarray(O, dtype=np.uint64).reshape(-1), out.reshape(-1), logN, int(p), int(q0))
    if rc:
        raise RuntimeError(f"ref_pack_moddown failed with {rc}")
    return out


def rescale(cipher, logN, pq, p_num, L, l):
    """Scheme_23::rescaleAndEqual's sequence (Scheme_23.cuh:368-385) with the reference's own kernels and
    transform launchers on a cipher buffer [2][L+1][N]; returns the buffer afterwards."""
    pq = np.ascontiguousarray(pq, dtype=np.uint64)
    q = [int(v) for v in pq[p_num:]]
    c = ntt(np.ascontiguousarray(cipher, dtype=np.uint64).reshape(2, L + 1, -1), logN, pq, l, p_num + l, 2, 1, L + 1,
            inverse=True).reshape(-1)
    buf = np.zeros_like(c)
    qinv = np.array([pow(q[l], -1, q[i]) for i in range(l)], dtype=np.uint64)
    qinv_s = np.array([(int(qinv[i]) << 64) // q[i] for i in range(l)], dtype=np.uint64)
    rc = lib().ref_rescale_stage(c, buf, logN, pq, p_num, L + 1, l, 0, qinv, qinv_s)
    assert rc == 0, rc
    buf = ntt(buf.reshape(2, L + 1, -1), logN, pq, 0, p_num, 2, l, L + 1).reshape(-1)
    rc = lib().ref_rescale_stage(c, buf, logN, pq, p_num, L + 1, l, 1, qinv, qinv_s)
    assert rc == 0, rc
    return c.reshape(2, L + 1, -1)


def modup_q0_to_ql(cipher, logN, pq, p_num, L, target_level, scale_up):
    """Bootstrapper::modUpQ0toQL's sequence (bootstrapping/Bootstrapper.cuh:192-209) with the reference's kernel
    and transform launchers."""
    pq = np.ascontiguousarray(pq, dtype=np.uint64)
    c = ntt(np.ascontiguousarray(cipher, dtype=np.uint64).reshape(2, L + 1, -1), logN, pq, 0, p_num, 2, 1, L + 1,
            inverse=True).reshape(-1)
    rc = lib().ref_modup_q0_to_ql(c, logN, pq, p_num, L + 1, target_level, int(scale_up))
    assert rc == 0, rc
    return ntt(c.reshape(2, L + 1, -1), logN, pq, 0, p_num, 2, target_level + 1, L + 1)


def keyswitch_stage(stage, inp, aux, logN, KT, l, gamma):
    """One kernel of the key-switch chain through the reference's launcher: stage 0 external_product_T
    (inp = digits over T, aux = key), 1 modUpTtoPQl_23, 2 modDownPQltoQl_23.  KT: oracle.KeySwitchTables."""
    p_num, q_num, t_num = len(KT.p), len(KT.q), len(KT.t)
    n = 1 << logN
    R = (p_num + q_num + gamma - 1) // gamma
    out = np.zeros((2, q_num, n) if stage == 2 else (2, R, t_num, n), dtype=np.uint64)
    pqt = np.array(KT.p + KT.q + KT.t, dtype=np.uint64)
    aux = np.zeros(1, dtype=np.uint64) if aux is None else np.ascontiguousarray(aux, dtype=np.uint64).reshape(-1)
    rc = lib().ref_keyswitch_stage(out.reshape(-1), np.ascontiguousarray(inp, dtype=np.uint64).reshape(-1), aux, logN, pqt,
                                   p_num, q_num, t_num, l, gamma, stage, KT.t_hat_inv, KT.t_hat_inv_shoup, KT.t_hat_mod_r,
                                   KT.half_t, KT.t_mod_pq, KT.p_hat_inv, KT.p_hat_inv_shoup, KT.p_hat_mod_q,
                                   KT.p_inv_mod_q, KT.p_inv_mod_q_shoup)
    if rc:
        raise RuntimeError(f"ref_keyswitch_stage failed with {rc}")
    return out


def tensor_product(c1, c2, logN, pq, p_num, l):
    """compute_c0c1c2 as mult_23 calls it: returns [3][q_num][N] = (a1b2+a2b1, a1a2, b1b2)."""
    c1 = np.ascontiguousarray(c1, dtype=np.uint64)
    q_num, n = c1.shape[1], c1.shape[2]
    out = np.zeros((3, q_num, n), dtype=np.uint64)
    rc = lib().ref_tensor_product(out.reshape(-1), c1.copy().reshape(-1), np.ascontiguousarray(c2, dtype=np.uint64).reshape(-1),
                                  logN, np.ascontiguousarray(pq, dtype=np.uint64), p_num, q_num, l, 0)
    assert rc == 0, rc
    return out


def add_switched(cipher, axbx, logN, pq, p_num, l):
    """cipher_add_axbx_batch_device as mult_23 calls it: cipher [2][q_num][N] += axbx [2][q_num][N] (ax then bx)."""
    c = np.ascontiguousarray(cipher, dtype=np.uint64).copy()
    q_num = c.shape[1]
    dummy = np.zeros(1, dtype=np.uint64)
    rc = lib().ref_tensor_product(dummy, c.reshape(-1), np.ascontiguousarray(axbx, dtype=np.uint64).reshape(-1), logN,
                                  np.ascontiguousarray(pq, dtype=np.uint64), p_num, q_num, l, 1)
    assert rc == 0, rc
    return c


def galois(cipher, logN, pq, p_num, l, mode, rot_slots=0, into=None):
    """The reference's own kernels for the steps conjugate_23 and leftRotate_23 add around the chain, on a
    Ciphertext buffer [2][q_num][N]: mode 0 = sk_and_poly_conjugate of both halves, mode 1 =
    sk_and_poly_LeftRot_ntt_double by rot_slots, mode 2 = poly_add_batch_device of the b half onto `into`."""
    c = np.ascontiguousarray(cipher, dtype=np.uint64)
    q_num = c.shape[1]
    out = np.zeros_like(c) if into is None else np.ascontiguousarray(into, dtype=np.uint64).copy()
    rc = lib().ref_galois(out.reshape(-1), c.reshape(-1), logN, np.ascontiguousarray(pq, dtype=np.uint64), p_num, q_num, l,
                          int(rot_slots), mode)
    assert rc == 0, rc
    return out
