"""GPU parity of the key-switch chain (external product over T, T -> [p | q] conversion, ModDown and the
whole chain of Scheme_23::mult_23) against the CPU oracle, through the reference-shaped mirrors."""
import numpy as np
import pytest
import torch

import helpers as H
from ckks_llm_b200 import params
from ckks_llm_b200.host import Context_23, as_u64_tensor, to_u64_numpy

pytestmark = pytest.mark.gpu


def _setup(oracle, logN, p_num, q_num, t_num, gamma, q_bits=50, t_bits=60):
    N = 1 << logN
    p = params.ntt_primes(q_bits + 1, 2 * N, p_num)
    q = params.ntt_primes(q_bits, 2 * N, q_num)
    t = params.ntt_primes(t_bits, 2 * N, t_num)
    ctx = Context_23(logN, p, q, t, gamma=gamma)
    return N, p, q, t, ctx, oracle.KeySwitchTables(p, q, t)


def _shapes(p, q, t, l, gamma):
    R = (len(p) + len(q) + gamma - 1) // gamma
    return R, (l + 1 + len(p) - 1) // len(p), len(q) // len(p), (len(p) + l + 1 + gamma - 1) // gamma


CASES = [(12, 2, 6, 4, 3, 5), (12, 3, 9, 5, 4, 8), (13, 1, 5, 3, 3, 2), (12, 2, 6, 4, 3, 0), (12, 4, 8, 8, 5, 6)]


@pytest.mark.parametrize("logN,p_num,q_num,t_num,gamma,l", CASES)
def test_chain_stages(oracle, cuda_device, logN, p_num, q_num, t_num, gamma, l):
    N, p, q, t, ctx, KT = _setup(oracle, logN, p_num, q_num, t_num, gamma)
    R, cb, dnum, blocks = _shapes(p, q, t, l, gamma)
    rng = np.random.default_rng(logN * 100 + l)
    dev = ctx.device
    # external product
    cipher = np.stack([H.uniform_residues(rng, t, (N,)) for _ in range(cb)])
    swk = np.stack([H.uniform_residues(rng, t, (N,)) for _ in range(2 * dnum * R)]).reshape(2, dnum, R, t_num, N)
    exp = oracle.external_product_t(cipher, swk, N, KT, l, gamma)
    out = torch.zeros(2 * R * t_num * N, dtype=torch.int64, device=dev)
    ctx.external_product_T(out, as_u64_tensor(cipher, dev), as_u64_tensor(swk, dev), l)
    assert np.array_equal(to_u64_numpy(out).reshape(2, R, t_num, N), exp)
    # T -> [p | q]: any residues, and values at the centring boundaries
    inp = np.stack([H.uniform_residues(rng, t, (N,)) for _ in range(2 * R)]).reshape(2, R, t_num, N)
    inp[0, 0, :, 0] = 0
    inp[0, 0, :, 1] = np.array(t, dtype=np.uint64) - np.uint64(1)
    inp[0, 0, :, 2] = KT.half_t[len(p) + len(q):]
    exp = oracle.modup_t_to_pql(inp, N, KT, l, gamma, 2)
    for algo in ("tensor", "simt", "auto"):          # the tcgen05 byte-plane contraction and the 64-bit CUDA-core kernel
        ctx.set_modup_algo(algo)
        out = torch.zeros(2 * R * t_num * N, dtype=torch.int64, device=dev)
        ctx.modUpTtoPQl_23(out, as_u64_tensor(inp, dev), l, 2)
        ctx.check()
        assert np.array_equal(to_u64_numpy(out).reshape(2, R * t_num, N), exp), algo
    # ModDown
    pqin = np.zeros((2, R * t_num, N), dtype=np.uint64)
    for c in range(2):
        pqin[c, :len(p) + len(q)] = H.uniform_residues(rng, p + q, (N,))
    exp = oracle.moddown_pql_to_ql(pqin, N, KT, l, gamma, 2)
    out = torch.zeros(2 * len(q) * N, dtype=torch.int64, device=dev)
    ctx.modDownPQltoQl_23(out, as_u64_tensor(pqin, dev), l, 2)
    assert np.array_equal(to_u64_numpy(out).reshape(2, len(q), N), exp)
    ctx.close()


@pytest.mark.parametrize("logN,p_num,q_num,t_num,gamma,l", [(12, 2, 6, 4, 3, 5), (13, 3, 9, 5, 4, 6), (14, 1, 4, 3, 3, 3)])
def test_whole_chain(oracle, cuda_device, logN, p_num, q_num, t_num, gamma, l):
    N, p, q, t, ctx, KT = _setup(oracle, logN, p_num, q_num, t_num, gamma)
    R, cb, dnum, blocks = _shapes(p, q, t, l, gamma)
    rng = np.random.default_rng(7 + logN)
    T = oracle.NttTables(N, p + q + t)
    inp = H.uniform_residues(rng, q[:l + 1], (N,))
    swk = np.stack([H.uniform_residues(rng, t, (N,)) for _ in range(2 * dnum * R)]).reshape(2, dnum, R, t_num, N)
    exp = oracle.keyswitch(inp, swk, T, KT, l, gamma)
    out = torch.zeros(2 * len(q) * N, dtype=torch.int64, device=ctx.device)
    ctx.keyswitch(out, as_u64_tensor(inp, ctx.device), as_u64_tensor(swk, ctx.device), l)
    got = to_u64_numpy(out).reshape(2, len(q), N)
    assert np.array_equal(got[:, :l + 1], exp[:, :l + 1])
    ctx.close()


@pytest.mark.parametrize("logN,p_num,q_num,t_num,gamma,l", [(12, 2, 6, 4, 3, 5), (13, 1, 4, 3, 3, 2)])
def test_mult_23(oracle, cuda_device, logN, p_num, q_num, t_num, gamma, l):
    """Ciphertext x ciphertext with relinearisation through the Scheme_23 mirror, the result aliasing an operand."""
    from ckks_llm_b200.host import Ciphertext, Scheme_23
    N, p, q, t, ctx, KT = _setup(oracle, logN, p_num, q_num, t_num, gamma)
    R, cb, dnum, blocks = _shapes(p, q, t, l, gamma)
    rng = np.random.default_rng(11 + logN)
    T = oracle.NttTables(N, p + q + t)
    c1 = np.stack([H.uniform_residues(rng, q, (N,)) for _ in range(2)])
    c2 = np.stack([H.uniform_residues(rng, q, (N,)) for _ in range(2)])
    c1[0, :, :2] = (np.array(q, dtype=np.uint64) - np.uint64(1))[:, None]           # largest residues in every product
    c1[1, :, :2] = c2[0, :, :2] = c2[1, :, :2] = c1[0, :, :2]
    rlk = np.stack([H.uniform_residues(rng, t, (N,)) for _ in range(2 * dnum * R)]).reshape(2, dnum, R, t_num, N)
    exp = oracle.mult(c1, c2, rlk, T, KT, l, gamma)
    L = len(q) - 1
    sch = Scheme_23(ctx)
    a = Ciphertext(N, L, l, N // 2, 2.0 ** 40, cipher=as_u64_tensor(c1.reshape(-1), ctx.device))
    b = Ciphertext(N, L, l + 0, N // 2, 2.0 ** 30, cipher=as_u64_tensor(c2.reshape(-1), ctx.device))
    with pytest.raises(ValueError):
        sch.mult_23(a, a, b)                                                          # no key yet
    sch.rlk_23 = as_u64_tensor(rlk.reshape(-1), ctx.device)
    sch.mult_23(a, a, b)                                                              # result over the first operand
    got = to_u64_numpy(a.cipher_device).reshape(2, len(q), N)
    assert np.array_equal(got[:, :l + 1], exp[:, :l + 1])
    assert np.array_equal(got[:, l + 1:], c1[:, l + 1:])                              # limbs above the level untouched
    assert a.l == l and a.scale == 2.0 ** 70
    zero = Ciphertext(N, L, 0, N // 2, 1.0, cipher=as_u64_tensor(c2.reshape(-1), ctx.device))
    with pytest.raises(ValueError):
        sch.mult_23(a, a, zero)
    ctx.close()


@pytest.mark.parametrize("logN,p_num,q_num,t_num,gamma,l", [(12, 2, 6, 4, 3, 5), (13, 1, 4, 3, 3, 2)])
def test_conjugate_and_rotate(oracle, cuda_device, logN, p_num, q_num, t_num, gamma, l):
    """conjugate_23 and leftRotate_23 through the Scheme_23 mirror, out of place and in place, against the oracle."""
    from ckks_llm_b200.host import Ciphertext, Scheme_23
    N, p, q, t, ctx, KT = _setup(oracle, logN, p_num, q_num, t_num, gamma)
    R, cb, dnum, blocks = _shapes(p, q, t, l, gamma)
    rng = np.random.default_rng(21 + logN)
    T = oracle.NttTables(N, p + q + t)
    c = np.stack([H.uniform_residues(rng, q, (N,)) for _ in range(2)])
    c[:, :, :2] = (np.array(q, dtype=np.uint64) - np.uint64(1))[None, :, None]
    key = np.stack([H.uniform_residues(rng, t, (N,)) for _ in range(2 * dnum * R)]).reshape(2, dnum, R, t_num, N)
    L = len(q) - 1
    sch = Scheme_23(ctx)
    src = Ciphertext(N, L, l, N // 2, 2.0 ** 40, cipher=as_u64_tensor(c.reshape(-1), ctx.device))
    res = Ciphertext(N, L, L, N // 2, 1.0, cipher=torch.zeros(2 * len(q) * N, dtype=torch.int64, device=ctx.device))
    with pytest.raises(ValueError):
        sch.conjugate_23(res, src)                                                    # no key yet
    with pytest.raises(ValueError):
        sch.leftRotate_23(res, src, 3)
    kd = as_u64_tensor(key.reshape(-1), ctx.device)
    sch.ConjKey_23 = kd
    exp = oracle.conjugate(c, key, T, KT, l, gamma)
    sch.conjugate_23(res, src)
    got = to_u64_numpy(res.cipher_device).reshape(2, len(q), N)
    assert np.array_equal(got[:, :l + 1], exp[:, :l + 1]) and not got[:, l + 1:].any()
    assert res.l == l and res.scale == 2.0 ** 40
    assert np.array_equal(to_u64_numpy(src.cipher_device).reshape(c.shape), c)        # the source is untouched
    for rot in (1, N // 2, 37):
        sch.rotKey_vec_23[rot] = kd
        exp = oracle.rotate(c, key, rot, T, KT, l, gamma)
        sch.leftRotate_23(res, src, rot)
        got = to_u64_numpy(res.cipher_device).reshape(2, len(q), N)
        assert np.array_equal(got[:, :l + 1], exp[:, :l + 1]), rot
    inplace = Ciphertext(N, L, l, N // 2, 1.0, cipher=as_u64_tensor(c.reshape(-1), ctx.device))
    sch.leftRotateAndEqual_23(inplace, 37)
    got = to_u64_numpy(inplace.cipher_device).reshape(2, len(q), N)
    assert np.array_equal(got[:, :l + 1], exp[:, :l + 1]) and np.array_equal(got[:, l + 1:], c[:, l + 1:])
    inplace = Ciphertext(N, L, l, N // 2, 1.0, cipher=as_u64_tensor(c.reshape(-1), ctx.device))
    sch.conjugateAndEqual_23(inplace)
    exp = oracle.conjugate(c, key, T, KT, l, gamma)
    assert np.array_equal(to_u64_numpy(inplace.cipher_device).reshape(2, len(q), N)[:, :l + 1], exp[:, :l + 1])
    L_ = ctx.lib
    assert L_.ckks_b200_rotate(ctx._h, res.cipher_device.data_ptr(), src.cipher_device.data_ptr(), kd.data_ptr(), 0, l, gamma,
                               None) != 0                                             # outside the rotation group table
    ctx.close()
