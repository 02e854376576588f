"""Pins the oracle AND the library to the REAL reference kernels run on this GPU.

oracle/_ref/libref_driver.so holds the reference's own NTT, ModUp and PPMM kernels,
compiled for sm_100a from the reference sources (oracle/ref_driver.cu).  The tests are
skipped when that library was not built."""
import ctypes as C

import numpy as np
import pytest
import torch

import helpers as H
from ckks_llm_b200 import capi, params
from ckks_llm_b200.host import Context_23, PCMM_Context, PCMM_Scheme, as_u64_tensor, to_u64_numpy
from oracle import ref as R

R_ = R        # the key-switch test uses R for the block count

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not R.available(), reason="reference driver library not built")]


@pytest.mark.parametrize("logN", [14, 16])
def test_reference_ntt_kernels(oracle, cuda_device, logN):
    N = 1 << logN
    if logN == 16:
        pqt = params.REF_LOGN16_P[:1] + params.REF_LOGN16_Q[:3] + params.REF_LOGN16_T[:2]
    else:
        pqt = params.ntt_primes(50, 2 * N, 4) + params.ntt_primes(60, 2 * N, 2)
    rng = np.random.default_rng(logN)
    polys = 2
    data = np.stack([H.uniform_residues(rng, pqt, (N,)) for _ in range(polys)])
    ref_fwd = R.ntt(data, logN, pqt, 0, 0, polys, len(pqt), len(pqt))
    T = oracle.NttTables(N, pqt)
    orc = data.copy()
    oracle.ntt_batch(orc, T, 0, 0, polys, len(pqt), len(pqt))
    assert np.array_equal(orc, ref_fwd)                       # oracle == reference kernels
    ctx = Context_23(logN, [], pqt, [])
    d = as_u64_tensor(data, ctx.device)
    ctx.ToNTTInplace(d, 0, 0, polys, len(pqt), len(pqt))
    assert np.array_equal(to_u64_numpy(d), ref_fwd)           # library == reference kernels
    ref_inv = R.ntt(data, logN, pqt, 0, 0, polys, len(pqt), len(pqt), inverse=True)
    orc = data.copy()
    oracle.ntt_batch(orc, T, 0, 0, polys, len(pqt), len(pqt), inverse=True)
    assert np.array_equal(orc, ref_inv)
    d = as_u64_tensor(data, ctx.device)
    ctx.FromNTTInplace(d, 0, 0, polys, len(pqt), len(pqt))
    assert np.array_equal(to_u64_numpy(d), ref_inv)
    ctx.close()


def test_reference_modup_kernel(oracle, cuda_device):
    logN, N = 14, 1 << 14
    p = params.ntt_primes(51, 2 * N, 4)
    q = params.ntt_primes(50, 2 * N, 10)
    t = params.ntt_primes(60, 2 * N, 6)
    l, batch, alpha = 9, 2, 4
    rng = np.random.default_rng(5)
    inp = np.stack([H.uniform_residues(rng, q, (N,)) for _ in range(batch)])
    blocks = (l + 1 + alpha - 1) // alpha
    hat_inv = np.zeros(blocks * alpha, dtype=np.uint64)
    hat_inv_s = np.zeros_like(hat_inv)
    hat_mod_t = np.zeros(blocks * len(t) * alpha, dtype=np.uint64)
    blk_mod_t = np.zeros(blocks * len(t), dtype=np.uint64)
    qa, ta = np.array(q, dtype=np.uint64), np.array(t, dtype=np.uint64)
    L = oracle.lib()
    L.orc_modup_tables.argtypes = [np.ctypeslib.ndpointer(np.uint64), C.c_int, np.ctypeslib.ndpointer(np.uint64),
                                   C.c_int, C.c_int, C.c_int] + [np.ctypeslib.ndpointer(np.uint64)] * 4
    L.orc_modup_tables(qa, len(q), ta, len(t), alpha, l, hat_inv, hat_inv_s, hat_mod_t, blk_mod_t)
    # The reference only ever converts one polynomial per call (batch_size 1 at every call
    # site); for a batch index b > 0 its kernel indexes the Qblk-mod-t table with an extra
    # offset of b*Qj_blockNum*t_num (BasisConv.cuh:142,153) and so reads another level's row.
    # Each polynomial is therefore pinned as a batch of one.
    ref_out = np.concatenate([R.modup(inp[b:b + 1], logN, p, q, t, l, 1, (hat_inv, hat_inv_s, hat_mod_t, blk_mod_t))
                              for b in range(batch)])
    assert np.array_equal(oracle.modup(inp, N, q, t, alpha, l, batch), ref_out)
    ctx = Context_23(logN, p, q, t)
    out = torch.empty(batch * blocks * len(t) * N, dtype=torch.int64, device=ctx.device)
    ctx.modUpQjtoT_23(out, as_u64_tensor(inp, ctx.device), l, batch)
    assert np.array_equal(to_u64_numpy(out).reshape(ref_out.shape), ref_out)
    ctx.close()


@pytest.mark.parametrize("limbs", [2, 3])
def test_reference_ppmm_kernel(oracle, cuda_device, limbs):
    """pcmm_cuda_core_kernel<128> of the reference at its native moduli {q0,q1(,q2)} and
    scaler = q1, against the oracle and both library paths."""
    q = params.REF_LOGN16_Q[:limbs]
    N1, rank, M, K = 64, 7, 64, 128
    rng = np.random.default_rng(limbs)
    W = rng.uniform(-0.1, 0.1, (M, K)).astype(np.float32)
    W[3, 3] = 0.0
    X = np.stack([H.uniform_residues(rng, q, ((rank + 1) * N1,)) for _ in range(K)])
    scaler = float(q[1])
    qinv = [pow(q[-1], -1, qi) if i < limbs - 1 else 0 for i, qi in enumerate(q)]
    qinv_s = [(v << 64) // qi for v, qi in zip(qinv, q)]
    ref_out = R.ppmm(W, X, N1, rank, q, scaler, qinv, qinv_s)
    assert np.array_equal(oracle.ppmm(W, X, q, scaler), ref_out)
    pc = PCMM_Context(N1, rank, [], q)
    for algo in (capi.PCMM_SIMT, capi.PCMM_TENSOR):
        got = PCMM_Scheme(pc, algo=algo).PPMM_host(W, X, M, K, N1, K, scaler)
        assert np.array_equal(got, ref_out), algo
    pc.close()


def test_reference_rescale_kernels(oracle, cuda_device):
    """mod_to_qi + rescaleAndEqual_new_kernel with the reference's transform launchers
    (Scheme_23.cuh:339-385) == oracle == library."""
    from ckks_llm_b200.host import Ciphertext, Scheme_23
    logN, N = 14, 1 << 14
    p = params.ntt_primes(51, 2 * N, 2)
    q = params.ntt_primes(50, 2 * N, 3) + params.ntt_primes(60, 2 * N, 2)     # mixed widths, the last limb is 60-bit
    L, l = len(q) - 1, len(q) - 1
    rng = np.random.default_rng(21)
    cipher = np.stack([H.uniform_residues(rng, q, (N,)) for _ in range(2)])
    ref = R.rescale(cipher, logN, p + q, len(p), L, l)
    T = oracle.NttTables(N, p + q)
    orc = oracle.rescale(cipher.copy(), T, len(p), L, l)
    assert np.array_equal(orc, ref)
    ctx = Context_23(logN, p, q, [])
    ct = Ciphertext(N, L, l, N // 2, 1.0, cipher=as_u64_tensor(cipher.reshape(-1), ctx.device))
    Scheme_23(ctx).rescaleAndEqual(ct)
    assert np.array_equal(to_u64_numpy(ct.cipher_device).reshape(2, L + 1, N), ref)
    ctx.close()


def test_reference_modup_q0_to_ql_kernel(oracle, cuda_device):
    """modUpQ0toQL_kernel with the reference's transform launchers (bootstrapping/Bootstrapper.cuh:192-209)
    == oracle == library."""
    from ckks_llm_b200.host import Bootstrapper, Ciphertext
    logN, N = 14, 1 << 14
    p = params.ntt_primes(51, 2 * N, 1)
    q = params.ntt_primes(60, 2 * N, 1) + params.ntt_primes(50, 2 * N, 4)     # a wide q0 and narrower upper limbs
    L, target = len(q) - 1, 3
    precision = 1 << 50
    scale_up = q[0] // precision
    rng = np.random.default_rng(22)
    cipher = np.stack([H.uniform_residues(rng, q, (N,)) for _ in range(2)])
    ref = R.modup_q0_to_ql(cipher, logN, p + q, len(p), L, target, scale_up)
    T = oracle.NttTables(N, p + q)
    orc = oracle.modup_q0_to_ql(cipher.copy(), T, len(p), L, target, scale_up)
    assert np.array_equal(orc, ref)
    ctx = Context_23(logN, p, q, [])
    ct = Ciphertext(N, L, 0, N // 2, 1.0, cipher=as_u64_tensor(cipher.reshape(-1), ctx.device))
    Bootstrapper(ctx, precision).modUpQ0toQL(ct, target)
    assert np.array_equal(to_u64_numpy(ct.cipher_device).reshape(2, L + 1, N), ref)
    ctx.close()


@pytest.mark.parametrize("p_num,q_num,t_num,gamma,l", [(2, 6, 4, 3, 5), (1, 5, 3, 3, 3), (3, 9, 5, 4, 7)])
def test_reference_keyswitch_kernels(oracle, cuda_device, p_num, q_num, t_num, gamma, l):
    """external_product_T, modUpTtoPQl_23 and modDownPQltoQl_23 through the reference's own launchers
    (ExternalProduct.cuh:83-97, BasisConv.cuh:237-248, :327-347) == oracle == library."""
    logN, N = 12, 1 << 12
    p = params.ntt_primes(51, 2 * N, p_num)
    q = params.ntt_primes(50, 2 * N, q_num)
    t = params.ntt_primes(60, 2 * N, t_num)
    KT = oracle.KeySwitchTables(p, q, t)
    ctx = Context_23(logN, p, q, t, gamma=gamma)
    dev = ctx.device
    R = (p_num + q_num + gamma - 1) // gamma
    cb, dnum = (l + 1 + p_num - 1) // p_num, q_num // p_num
    rng = np.random.default_rng(31 + p_num)
    cipher = np.stack([H.uniform_residues(rng, t, (N,)) for _ in range(cb)])
    swk = np.stack([H.uniform_residues(rng, t, (N,)) for _ in range(2 * dnum * R)]).reshape(2, dnum, R, t_num, N)
    ref = R_.keyswitch_stage(0, cipher, swk, logN, KT, l, gamma)
    assert np.array_equal(oracle.external_product_t(cipher, swk, N, KT, l, gamma), ref)
    out = torch.zeros(2 * R * t_num * N, dtype=torch.int64, device=dev)
    ctx.external_product_T(out, as_u64_tensor(cipher, dev), as_u64_tensor(swk, dev), l)
    assert np.array_equal(to_u64_numpy(out).reshape(2, R, t_num, N), ref)

    inp = np.stack([H.uniform_residues(rng, t, (N,)) for _ in range(2 * R)]).reshape(2, R, t_num, N)
    ref = R_.keyswitch_stage(1, inp, None, logN, KT, l, gamma)
    assert np.array_equal(oracle.modup_t_to_pql(inp, N, KT, l, gamma, 2).reshape(ref.shape), ref)
    for algo in ("tensor", "simt"):
        ctx.set_modup_algo(algo)
        out = torch.zeros(2 * R * t_num * N, dtype=torch.int64, device=dev)
        ctx.modUpTtoPQl_23(out, as_u64_tensor(inp, dev), l, 2)
        assert np.array_equal(to_u64_numpy(out).reshape(ref.shape), ref), algo
    ctx.set_modup_algo("auto")

    pqin = np.zeros((2, R * t_num, N), dtype=np.uint64)
    for c in range(2):
        pqin[c, :p_num + q_num] = H.uniform_residues(rng, p + q, (N,))
    ref = R_.keyswitch_stage(2, pqin, None, logN, KT, l, gamma)
    assert np.array_equal(oracle.moddown_pql_to_ql(pqin, N, KT, l, gamma, 2)[:, :l + 1], ref[:, :l + 1])
    out = torch.zeros(2 * q_num * N, dtype=torch.int64, device=dev)
    ctx.modDownPQltoQl_23(out, as_u64_tensor(pqin, dev), l, 2)
    assert np.array_equal(to_u64_numpy(out).reshape(2, q_num, N)[:, :l + 1], ref[:, :l + 1])
    ctx.close()


def test_reference_tensor_product_and_addition(oracle, cuda_device):
    """compute_c0c1c2 and cipher_add_axbx_batch_device (poly_arithmetic.cuh:787-824, :155-172) == oracle."""
    if not hasattr(R_.lib(), "ref_tensor_product"):
        pytest.skip("reference driver built without the tensor-product entry")
    logN, N, l = 12, 1 << 12, 3
    p = params.ntt_primes(51, 2 * N, 2)
    q = params.ntt_primes(50, 2 * N, 3) + params.ntt_primes(60, 2 * N, 2)
    rng = np.random.default_rng(41)
    c1 = np.stack([H.uniform_residues(rng, q, (N,)) for _ in range(2)])
    c2 = np.stack([H.uniform_residues(rng, q, (N,)) for _ in range(2)])
    c1[:, :, 0] = c2[:, :, 0] = np.array(q, dtype=np.uint64) - np.uint64(1)
    ref = R_.tensor_product(c1, c2, logN, p + q, len(p), l)
    orc = oracle.tensor_product(c1, c2, N, q, l)
    for i in range(3):
        assert np.array_equal(orc[i][:l + 1], ref[i][:l + 1])
    summed = R_.add_switched(c1, np.stack([ref[0], ref[2]]), logN, p + q, len(p), l)
    exp = c1.copy()
    oracle.lib().orc_add_switched(exp.reshape(-1), np.ascontiguousarray(ref[0]).reshape(-1), np.ascontiguousarray(ref[2]).reshape(-1),
                                  N, len(q), l + 1, np.array(q, dtype=np.uint64))
    assert np.array_equal(exp, summed)


def test_reference_conjugation_and_rotation_steps(oracle, cuda_device):
    """sk_and_poly_conjugate, sk_and_poly_LeftRot_ntt_double and poly_add_batch_device (poly_arithmetic.cuh:666-680,
    :581-603, :395-399) == the oracle's index maps and addition, at the two ring sizes the reference runs."""
    if not hasattr(R_.lib(), "ref_galois"):
        pytest.skip("reference driver built without the conjugation / rotation entry")
    for logN, rots in ((12, (1, 5, 1000, 2048)), (14, (3, 8191))):
        N, l = 1 << logN, 2
        p = params.ntt_primes(51, 2 * N, 1)
        q = params.ntt_primes(50, 2 * N, 4)
        rng = np.random.default_rng(50 + logN)
        c = np.stack([H.uniform_residues(rng, q, (N,)) for _ in range(2)])
        rev = R_.galois(c, logN, p + q, len(p), l, 0)
        assert np.array_equal(rev[:, :l + 1], c[:, :l + 1, ::-1]) and not rev[:, l + 1:].any()
        for rot in rots:
            out = R_.galois(c, logN, p + q, len(p), l, 1, rot_slots=rot)
            exp = np.zeros_like(c)
            exp[:, :l + 1, oracle.rotation_map(N, rot)] = c[:, :l + 1]
            assert np.array_equal(out, exp), rot
        other = np.stack([H.uniform_residues(rng, q, (N,)) for _ in range(2)])
        other[1, :, 0] = c[1, :, 0] = np.array(q, dtype=np.uint64) - np.uint64(1)
        summed = R_.galois(c, logN, p + q, len(p), l, 2, into=other)
        exp = other.copy()
        for i in range(l + 1):
            exp[1, i] = ((other[1, i].astype(object) + c[1, i].astype(object)) % q[i]).astype(np.uint64)
        assert np.array_equal(summed, exp)
