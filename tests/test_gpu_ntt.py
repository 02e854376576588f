"""GPU parity of the batched NTT / INTT against the CPU oracle, through the C ABI."""
import numpy as np
import pytest
import torch

import helpers as H
from ckks_llm_b200 import capi, params
from ckks_llm_b200.host import Context_23, as_u64_tensor, to_u64_numpy

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("logN", [12, 13, 14, 15, 16])
def test_forward_inverse_bit_exact(oracle, cuda_device, logN):
    N = 1 << logN
    q = params.ntt_primes(50, 2 * N, 3) + params.ntt_primes(60, 2 * N, 1) + params.ntt_primes(36, 2 * N, 1)
    ctx = Context_23(logN, [], q, [])
    T = oracle.NttTables(N, q)
    for i in range(len(q)):
        assert ctx.psi(i) == int(T.psi_root[i])
        assert np.array_equal(ctx.psi_table(i), T.psi[i])
        assert np.array_equal(ctx.psi_table(i, inverse=True), T.psiinv[i])
    rng = np.random.default_rng(logN)
    polys = 3
    data = np.stack([H.uniform_residues(rng, q, (N,)) for _ in range(polys)])   # [3][5][N]
    d = as_u64_tensor(data, ctx.device)
    ctx.ToNTTInplace(d, 0, 0, polys, len(q), len(q))
    got = to_u64_numpy(d)
    exp = data.copy()
    oracle.ntt_batch(exp, T, 0, 0, polys, len(q), len(q))
    assert np.array_equal(got, exp)
    ctx.FromNTTInplace(d, 0, 0, polys, len(q), len(q))
    assert np.array_equal(to_u64_numpy(d), data)                 # bit-exact round trip
    # inverse alone, from an arbitrary (not transformed) input
    d2 = as_u64_tensor(data, ctx.device)
    ctx.FromNTTInplace(d2, 0, 0, polys, len(q), len(q))
    exp2 = data.copy()
    oracle.ntt_batch(exp2, T, 0, 0, polys, len(q), len(q), inverse=True)
    assert np.array_equal(to_u64_numpy(d2), exp2)
    ctx.close()


def test_small_n_against_brute_force(oracle, cuda_device):
    logN, N = 12, 4096
    q = params.ntt_primes(50, 2 * N, 1)
    ctx = Context_23(logN, [], q, [])
    rng = np.random.default_rng(1)
    a = rng.integers(0, q[0], N, dtype=np.uint64)
    d = as_u64_tensor(a[None, None], ctx.device)
    ctx.ToNTTInplace(d, 0, 0, 1, 1, 1)
    assert np.array_equal(to_u64_numpy(d)[0, 0], oracle.ntt_bruteforce(a, q[0], ctx.psi(0)))
    ctx.close()


def test_limb_and_modulus_offsets(oracle, cuda_device):
    """start_poly_idx is a limb offset inside each polynomial and start_mod_idx an index
    into [p|q|t] (ntt_60bit.cuh:446-458); untouched limbs must stay untouched."""
    logN, N = 13, 1 << 13
    p = params.ntt_primes(51, 2 * N, 2)
    q = params.ntt_primes(50, 2 * N, 4)
    t = params.ntt_primes(60, 2 * N, 2)
    ctx = Context_23(logN, p, q, t)
    allmods = p + q + t
    T = oracle.NttTables(N, allmods)
    rng = np.random.default_rng(2)
    polys, plen = 2, 6
    data = rng.integers(0, 1 << 35, (polys, plen, N), dtype=np.uint64)
    d = as_u64_tensor(data, ctx.device)
    ctx.ToNTTInplace(d, 1, 3, polys, 4, plen)        # limbs 1..4 with moduli 3..6
    exp = data.copy()
    oracle.ntt_batch(exp, T, 1, 3, polys, 4, plen)
    got = to_u64_numpy(d)
    assert np.array_equal(got, exp)
    assert np.array_equal(got[:, 0], data[:, 0]) and np.array_equal(got[:, 5], data[:, 5])
    ctx.close()


def test_config2_full_size_roundtrip_and_sample(oracle, cuda_device):
    """Configuration 2: N=2^16, 40 limbs of 50-bit primes, 16 ciphertexts x 2 polys."""
    logN, N = 16, 1 << 16
    q = params.ntt_primes(50, 2 * N, 40)
    ctx = Context_23(logN, [], q, [])
    polys = 32
    g = torch.Generator(device="cpu").manual_seed(0)
    data = np.empty((polys, 40, N), dtype=np.uint64)
    rng = np.random.default_rng(0)
    for i, qi in enumerate(q):
        data[:, i, :] = rng.integers(0, qi, (polys, N), dtype=np.uint64)
    d = as_u64_tensor(data, ctx.device)
    ctx.ToNTTInplace(d, 0, 0, polys, 40, 40)
    fwd = to_u64_numpy(d)
    # oracle on a sample of polynomials (all limbs), full round trip on everything
    T = oracle.NttTables(N, q)
    for p in (0, 17, 31):
        exp = data[p:p + 1].copy()
        oracle.ntt_batch(exp, T, 0, 0, 1, 40, 40)
        assert np.array_equal(fwd[p], exp[0])
    for i, qi in enumerate(q):
        assert fwd[:, i].max() < qi
    ctx.FromNTTInplace(d, 0, 0, polys, 40, 40)
    assert np.array_equal(to_u64_numpy(d), data)
    ctx.close()


def test_host_buffer_entry_points(oracle, cuda_device):
    logN, N = 12, 4096
    q = params.ntt_primes(45, 2 * N, 2)
    ctx = Context_23(logN, [], q, [])
    T = oracle.NttTables(N, q)
    rng = np.random.default_rng(4)
    data = H.uniform_residues(rng, q, (N,))[None].copy()
    h = data.copy()
    ctx.ToNTTInplace_host(h, 0, 0, 1, 2, 2)
    exp = data.copy()
    oracle.ntt_batch(exp, T, 0, 0, 1, 2, 2)
    assert np.array_equal(h, exp)
    ctx.FromNTTInplace_host(h, 0, 0, 1, 2, 2)
    assert np.array_equal(h, data)
    ctx.close()


def test_argument_errors(cuda_device):
    N = 4096
    q = params.ntt_primes(45, 2 * N, 2)
    ctx = Context_23(12, [], q, [])
    d = torch.zeros(2 * N, dtype=torch.int64, device=ctx.device)
    with pytest.raises(capi.CkksB200Error) as e:
        ctx.ToNTTInplace(d, 0, 1, 1, 2, 2)           # moduli 1..2 but only 2 exist
    assert e.value.status == capi.ERR_ARG
    with pytest.raises(capi.CkksB200Error):
        ctx.ToNTTInplace(d, 1, 0, 1, 2, 2)           # limb offset + count exceeds poly_mod_len
    ctx.ToNTTInplace(d, 0, 0, 0, 2, 2)               # empty batch is a no-op
    with pytest.raises(capi.CkksB200Error):
        Context_23(12, [], [q[0] + 2], [])           # not a prime = 1 mod 2N
    ctx.close()


@pytest.mark.parametrize("logN", [12, 14, 16])
def test_extreme_residues(oracle, cuda_device, logN):
    """Inputs that push the lazily reduced intermediate values of the transforms to their bounds: every residue q-1,
    residues alternating between 0 and q-1 at every stride, single spikes.  Moduli just below 2^50 (the FP64 back
    end at its widest), one just below 2^57 and one of 60 bits (the two integer back ends)."""
    N = 1 << logN
    q = params.ntt_primes(50, 2 * N, 2) + params.ntt_primes(57, 2 * N, 1) + params.ntt_primes(60, 2 * N, 1)
    ctx = Context_23(logN, [], q, [])
    T = oracle.NttTables(N, q)
    qa = np.array(q, dtype=np.uint64)[:, None]
    x = np.arange(N, dtype=np.uint64)[None, :]
    pats = [np.broadcast_to(qa - np.uint64(1), (len(q), N)).copy()]
    for b in range(0, logN, 3):
        pats.append(np.where((x >> np.uint64(b)) & np.uint64(1), qa - np.uint64(1), np.uint64(0)).astype(np.uint64))
    spike = np.zeros((len(q), N), dtype=np.uint64)
    spike[:, 0] = (qa - np.uint64(1))[:, 0]
    spike[:, N - 1] = 1
    pats.append(spike)
    data = np.stack(pats)
    n = len(pats)
    for inverse in (False, True):
        d = as_u64_tensor(data, ctx.device)
        (ctx.FromNTTInplace if inverse else ctx.ToNTTInplace)(d, 0, 0, n, len(q), len(q))
        exp = data.copy()
        oracle.ntt_batch(exp, T, 0, 0, n, len(q), len(q), inverse=inverse)
        assert np.array_equal(to_u64_numpy(d), exp), inverse
    ctx.close()
