"""GPU parity of the Q-digit -> T basis conversion against the CPU oracle."""
import numpy as np
import pytest

import helpers as H
from ckks_llm_b200 import params
from ckks_llm_b200.host import Context_23, as_u64_tensor, to_u64_numpy
import torch

pytestmark = pytest.mark.gpu


def _run(oracle, logN, alpha, q_num, t_num, l, batch, seed, q_bits=50, t_bits=60, algos=("tensor", "simt", "auto"),
         edge=False, exact_count=False):
    """Both kernels (the tcgen05 byte-plane product and the 64-bit CUDA-core one) against the oracle."""
    N = 1 << logN
    p = params.ntt_primes(q_bits + 1, 2 * N, alpha)
    q = params.ntt_primes(q_bits, 2 * N, q_num)
    t = params.ntt_primes(t_bits, 2 * N, t_num)
    ctx = Context_23(logN, p, q, t)
    if exact_count:
        ctx.test_exact_count()
    rng = np.random.default_rng(seed)
    inp = np.stack([H.uniform_residues(rng, q, (N,)) for _ in range(batch)])
    if edge:
        # extreme residues: zeros, q-1 everywhere (overflow count at its maximum), single ones
        qa = np.array(q, dtype=np.uint64)
        inp[0, :, 0] = 0
        inp[0, :, 1] = qa - np.uint64(1)
        inp[0, :, 2] = 1
        inp[0, :, 3] = 0
        inp[0, 0, 3] = 1
        inp[0, :, 4:132] = (qa - np.uint64(1))[:, None]
    blocks = (l + 1 + alpha - 1) // alpha
    exp = oracle.modup(inp, N, q, t, alpha, l, batch)
    for algo in algos:
        ctx.set_modup_algo(algo)
        out = torch.full((batch * blocks * t_num * N,), -1, dtype=torch.int64, device=ctx.device)
        ctx.modUpQjtoT_23(out, as_u64_tensor(inp, ctx.device), l, batch)
        ctx.check()
        got = to_u64_numpy(out).reshape(batch, blocks, t_num, N)
        assert np.array_equal(got, exp), algo
        host = ctx.modUpQjtoT_23_host(inp, l, batch)
        assert np.array_equal(host, exp), algo
    ctx.close()


def test_reference_parameter_shape(oracle, cuda_device):
    # the reference's own logN=16 set: alpha=4, 8 target limbs (Params.cuh:118-165)
    _run(oracle, 13, 4, 12, 8, 11, 2, seed=1)


def test_ragged_last_digit_and_low_level(oracle, cuda_device):
    _run(oracle, 12, 4, 10, 3, 8, 3, seed=2)      # digits of 4, 4, 1 limbs
    _run(oracle, 12, 3, 7, 2, 0, 1, seed=3)       # level 0: one digit of one limb


def test_config3_shape(oracle, cuda_device):
    """Configuration 3: N=2^16, 24 Q-limbs (50-bit), alpha=8 -> 3 digits, 12 target limbs
    (60-bit); a reduced batch keeps the CPU oracle to seconds (full batch is timed in bench)."""
    _run(oracle, 16, 8, 24, 12, 23, 4, seed=0)


def test_extreme_residues(oracle, cuda_device):
    _run(oracle, 12, 8, 16, 12, 15, 2, seed=4, edge=True)
    _run(oracle, 12, 4, 8, 5, 6, 1, seed=5, edge=True)         # ragged digit, odd target count


def test_digit_sizes_off_the_mma_step(oracle, cuda_device):
    """alpha that is not a multiple of four pads the contraction with zero rows."""
    _run(oracle, 12, 5, 10, 4, 9, 2, seed=6)
    _run(oracle, 12, 2, 6, 16, 5, 1, seed=7)                    # sixteen targets fill the accumulator columns
    _run(oracle, 12, 11, 22, 3, 21, 1, seed=8)


def test_wide_q_limbs(oracle, cuda_device):
    _run(oracle, 12, 4, 8, 6, 7, 2, seed=9, q_bits=59, t_bits=61)


def test_narrow_targets(oracle, cuda_device):
    """Targets below 2^49: the quotient of the 81-bit sum no longer fits 32 bits, the kernel's general form runs."""
    _run(oracle, 12, 4, 8, 4, 7, 2, seed=11, t_bits=44, algos=("tensor", "simt"))
    _run(oracle, 12, 4, 8, 8, 7, 1, seed=12, q_bits=58, t_bits=42, algos=("tensor", "simt"))


def test_overflow_count_from_divisions(oracle, cuda_device):
    """The tensor-core kernel takes the overflow count from a sum of products with reciprocals and falls back to the
    reference's IEEE divisions only next to an integer, which random inputs do not reach: the test switch sends every
    coefficient down the division path, for both ways of forming rb_j, extreme residues included."""
    _run(oracle, 12, 8, 16, 12, 15, 2, seed=13, algos=("tensor",), edge=True, exact_count=True)
    _run(oracle, 12, 4, 10, 3, 8, 2, seed=14, algos=("tensor",), exact_count=True)
    _run(oracle, 12, 4, 8, 6, 7, 2, seed=15, q_bits=59, t_bits=61, algos=("tensor",), edge=True, exact_count=True)


def test_tensor_kernel_refuses_what_it_cannot_reduce(oracle, cuda_device):
    """Targets outside [2^40, 2^62) go to the CUDA-core kernel; insisting on tensor cores is an error."""
    from ckks_llm_b200.capi import CkksB200Error
    N = 1 << 12
    p = params.ntt_primes(31, 2 * N, 2)
    q = params.ntt_primes(30, 2 * N, 4)
    t = params.ntt_primes(36, 2 * N, 3)
    ctx = Context_23(12, p, q, t)
    rng = np.random.default_rng(10)
    inp = np.stack([H.uniform_residues(rng, q, (N,))])
    exp = oracle.modup(inp, N, q, t, 2, 3, 1)
    assert np.array_equal(ctx.modUpQjtoT_23_host(inp, 3, 1), exp)         # auto -> CUDA cores
    ctx.set_modup_algo("tensor")
    with pytest.raises(CkksB200Error):
        ctx.modUpQjtoT_23_host(inp, 3, 1)
    ctx.close()


def test_wait_that_runs_out_is_reported_and_the_context_stays_usable(oracle, cuda_device):
    """The bounded wait of the tensor-core kernel: with the test switch one tile's completion signal is left out and the
    threads waiting for it give up after about a millisecond.  The kernel returns by itself (nothing faults or hangs),
    the check reports the time-out once, and the next conversion on the same context is exact."""
    logN, alpha, q_num, t_num, l, batch = 12, 4, 8, 6, 7, 2
    N = 1 << logN
    p = params.ntt_primes(51, 2 * N, alpha)
    q = params.ntt_primes(50, 2 * N, q_num)
    t = params.ntt_primes(60, 2 * N, t_num)
    ctx = Context_23(logN, p, q, t)
    ctx.set_modup_algo("tensor")
    rng = np.random.default_rng(7)
    inp = np.stack([H.uniform_residues(rng, q, (N,)) for _ in range(batch)])
    d_in = as_u64_tensor(inp, ctx.device)
    blocks = (l + 1 + alpha - 1) // alpha
    out = torch.empty(batch * blocks * t_num * N, dtype=torch.int64, device=ctx.device)
    ctx.set_wait_budget(2_000_000)
    ctx.test_withhold_commit()
    ctx.modUpQjtoT_23(out, d_in, l, batch)
    with pytest.raises(Exception) as e:
        ctx.check()
    assert e.value.status == 7 and "site 10" in e.value.message          # CKKS_B200_ERR_TIMEOUT, group 0's wait
    ctx.check()                                                           # reported once
    ctx.set_wait_budget(0)
    ctx.modUpQjtoT_23(out, d_in, l, batch)
    ctx.check()
    assert np.array_equal(to_u64_numpy(out).reshape(batch, blocks, t_num, N), oracle.modup(inp, N, q, t, alpha, l, batch))
    ctx.close()
