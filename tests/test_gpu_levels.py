"""GPU parity of the two level changes around the PCMM (Scheme_23::rescaleAndEqual,
Bootstrapper::modUpQ0toQL) against the CPU oracle, through the reference-shaped mirrors."""
import numpy as np
import pytest
import torch

import helpers as H
from ckks_llm_b200 import params
from ckks_llm_b200.capi import CkksB200Error
from ckks_llm_b200.host import Bootstrapper, Ciphertext, Context_23, Scheme_23, as_u64_tensor, to_u64_numpy

pytestmark = pytest.mark.gpu


def _setup(oracle, logN, p_num, q_num, q_bits, seed):
    N = 1 << logN
    p = params.ntt_primes(q_bits + 1, 2 * N, p_num)
    q = params.ntt_primes(q_bits, 2 * N, q_num)
    ctx = Context_23(logN, p, q, [])
    T = oracle.NttTables(N, p + q)
    return N, p, q, ctx, T, np.random.default_rng(seed)


@pytest.mark.parametrize("logN,q_num,l,q_bits", [(12, 4, 3, 50), (13, 6, 2, 59), (14, 5, 4, 36), (16, 4, 1, 50)])
def test_rescale(oracle, cuda_device, logN, q_num, l, q_bits):
    N, p, q, ctx, T, rng = _setup(oracle, logN, 2, q_num, q_bits, seed=logN)
    L = q_num - 1
    cipher = np.stack([H.uniform_residues(rng, q, (N,)) for _ in range(2)])       # [2][L+1][N], any residues
    cipher[0, :, :3] = 0
    cipher[1, :, :3] = (np.array(q, dtype=np.uint64) - np.uint64(1))[:, None]
    exp = oracle.rescale(cipher.copy(), T, len(p), L, l)
    ct = Ciphertext(N, L, l, N // 2, 2.0 ** 40, cipher=as_u64_tensor(cipher.reshape(-1), ctx.device))
    Scheme_23(ctx).rescaleAndEqual(ct)
    got = to_u64_numpy(ct.cipher_device).reshape(2, L + 1, N)
    assert np.array_equal(got, exp)                   # every limb, the coefficient-domain last one included
    assert ct.l == l - 1 and ct.scale == 2.0 ** 40 / q[l]
    ctx.close()


@pytest.mark.parametrize("logN,q_num,target,q_bits", [(12, 5, 4, 50), (13, 4, 1, 59), (16, 6, 5, 50)])
def test_modup_q0_to_ql(oracle, cuda_device, logN, q_num, target, q_bits):
    N, p, q, ctx, T, rng = _setup(oracle, logN, 1, q_num, q_bits, seed=100 + logN)
    L = q_num - 1
    cipher = np.stack([H.uniform_residues(rng, q, (N,)) for _ in range(2)])
    coeff0 = rng.integers(0, q[0], size=(2, N), dtype=np.uint64)
    coeff0[0, :4] = [0, q[0] // 2, q[0] // 2 + 1, q[0] - 1]
    cipher[:, 0] = coeff0
    oracle.ntt_batch(cipher.reshape(-1), T, 0, len(p), 2, 1, L + 1)
    precision = 1 << (q_bits - 10)
    scale_up = q[0] // precision
    exp = oracle.modup_q0_to_ql(cipher.copy(), T, len(p), L, target, scale_up)
    ct = Ciphertext(N, L, 0, N // 2, 2.0 ** 40, cipher=as_u64_tensor(cipher.reshape(-1), ctx.device))
    Bootstrapper(ctx, precision).modUpQ0toQL(ct, target)
    got = to_u64_numpy(ct.cipher_device).reshape(2, L + 1, N)
    assert np.array_equal(got, exp)                   # limbs above the target keep what they held
    assert ct.l == target
    # the reference returns at once for a ciphertext that is not at level 0 (Bootstrapper.cuh:194)
    before = ct.cipher_device.clone()
    Bootstrapper(ctx, precision).modUpQ0toQL(ct, target)
    assert torch.equal(before, ct.cipher_device)
    ctx.close()


def test_level_arguments_are_checked(oracle, cuda_device):
    N, p, q, ctx, T, rng = _setup(oracle, 12, 1, 3, 50, seed=7)
    buf = torch.zeros(2 * 3 * N, dtype=torch.int64, device=ctx.device)
    ct = Ciphertext(N, 2, 0, N // 2, 1.0, cipher=buf)
    with pytest.raises(CkksB200Error):
        Scheme_23(ctx).rescaleAndEqual(ct)            # level 0 has no limb to divide by
    with pytest.raises(CkksB200Error):
        Bootstrapper(ctx, 1 << 40).modUpQ0toQL(ct, 3)  # beyond L
    ctx.close()


def test_batched_forms_equal_single_calls(oracle, cuda_device):
    """Three ciphertexts in one pool: the batched level changes give what the oracle gives for each alone."""
    logN, q_num, q_bits = 13, 5, 50
    N, p, q, ctx, T, rng = _setup(oracle, logN, 1, q_num, q_bits, seed=77)
    L, l, B = q_num - 1, 3, 3
    pool = np.stack([np.stack([H.uniform_residues(rng, q, (N,)) for _ in range(2)]) for _ in range(B)])   # [B][2][L+1][N]
    exp = np.stack([oracle.rescale(pool[b].copy(), T, len(p), L, l) for b in range(B)])
    dev = as_u64_tensor(pool.reshape(-1), ctx.device)
    words = 2 * (L + 1) * N
    cts = [Ciphertext(N, L, l, N // 2, 2.0 ** 40, cipher=dev[b * words:(b + 1) * words]) for b in range(B)]
    Scheme_23(ctx).rescaleAndEqual_batch(cts)
    assert np.array_equal(to_u64_numpy(dev).reshape(pool.shape), exp)
    assert all(c.l == l - 1 for c in cts)
    with pytest.raises(ValueError):
        Scheme_23(ctx).rescaleAndEqual_batch([cts[0], cts[2]])                   # not adjacent
    # level 0 -> target
    target, precision = 4, 1 << (q_bits - 10)
    pool0 = np.stack([np.stack([H.uniform_residues(rng, q, (N,)) for _ in range(2)]) for _ in range(B)])
    exp0 = np.stack([oracle.modup_q0_to_ql(pool0[b].copy(), T, len(p), L, target, q[0] // precision) for b in range(B)])
    dev0 = as_u64_tensor(pool0.reshape(-1), ctx.device)
    cts0 = [Ciphertext(N, L, 0, N // 2, 1.0, cipher=dev0[b * words:(b + 1) * words]) for b in range(B)]
    Bootstrapper(ctx, precision).modUpQ0toQL_batch(cts0, target)
    assert np.array_equal(to_u64_numpy(dev0).reshape(pool0.shape), exp0)
    assert all(c.l == target for c in cts0)
    ctx.close()
