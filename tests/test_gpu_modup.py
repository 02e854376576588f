"""GPU parity of the Q-digit -> T basis conversion against the CPU oracle."""
import numpy as np
import pytest

import helpers as H
from ckks_llm_b200 import params
from ckks_llm_b200.host import Context_23, as_u64_tensor, to_u64_numpy
import torch

pytestmark = pytest.mark.gpu


def _run(oracle, logN, alpha, q_num, t_num, l, batch, seed, q_bits=50, t_bits=60):
    N = 1 << logN
    p = params.ntt_primes(q_bits + 1, 2 * N, alpha)
    q = params.ntt_primes(q_bits, 2 * N, q_num)
    t = params.ntt_primes(t_bits, 2 * N, t_num)
    ctx = Context_23(logN, p, q, t)
    rng = np.random.default_rng(seed)
    inp = np.stack([H.uniform_residues(rng, q, (N,)) for _ in range(batch)])
    blocks = (l + 1 + alpha - 1) // alpha
    out = torch.full((batch * blocks * t_num * N,), -1, dtype=torch.int64, device=ctx.device)
    ctx.modUpQjtoT_23(out, as_u64_tensor(inp, ctx.device), l, batch)
    got = to_u64_numpy(out).reshape(batch, blocks, t_num, N)
    exp = oracle.modup(inp, N, q, t, alpha, l, batch)
    assert np.array_equal(got, exp)
    host = ctx.modUpQjtoT_23_host(inp, l, batch)
    assert np.array_equal(host, exp)
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
