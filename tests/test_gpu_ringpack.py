"""GPU parity of the RLWE -> MLWE decomposition against the oracle and the reference kernel."""
import numpy as np
import pytest
import torch

import helpers as H
from ckks_llm_b200 import capi, params
from ckks_llm_b200.host import (Ciphertext, Context_23, MLWECiphertext, PCMM_Context, PCMM_Scheme, as_u64_tensor,
                                to_u64_numpy)
from oracle import ref as R

pytestmark = pytest.mark.gpu


def _setup(logN, N1, L, seed, p_num=1):
    N = 1 << logN
    p = params.ntt_primes(51, 2 * N, p_num)
    q = params.ntt_primes(50, 2 * N, L + 1)
    ctx = Context_23(logN, p, q, [])
    rng = np.random.default_rng(seed)
    rlwe = np.stack([H.uniform_residues(rng, q, (N,)), H.uniform_residues(rng, q, (N,))])     # [2][L+1][N]
    return N, q, ctx, rlwe


@pytest.mark.parametrize("logN,N1,mlwe_num", [(12, 64, 64), (12, 64, 16), (13, 32, 5), (15, 128, 8)])
def test_decompose_coefficient_domain(oracle, cuda_device, logN, N1, mlwe_num):
    L = l = 2
    N, q, ctx, rlwe = _setup(logN, N1, L, seed=logN + mlwe_num)
    k = N // N1
    pc = PCMM_Context(N1, k, [], q)
    sch = PCMM_Scheme(pc, context=ctx)
    ct = Ciphertext(N, L, l, N // 2, 1.0, cipher=as_u64_tensor(rlwe, ctx.device).reshape(-1))
    mlwe = [MLWECiphertext(N1, L, l, k, 1.0) for _ in range(mlwe_num + 2)]
    sch.rlweCipherDecompose(ct, mlwe, mlwe_num, 2, ntt_domain=False)
    exp = oracle.rlwe_decompose(rlwe[0], rlwe[1], N1, k, mlwe_num, q)          # [num][limbs][k+1][N1]
    for i in range(mlwe_num):
        got = to_u64_numpy(mlwe[i + 2].cipher_device).reshape(L + 1, k + 1, N1)
        assert np.array_equal(got, exp[i]), i
    assert np.array_equal(to_u64_numpy(ct.cipher_device).reshape(rlwe.shape), rlwe)     # input untouched
    assert not to_u64_numpy(mlwe[0].cipher_device).any()                                 # offset respected
    pc.close(); ctx.close()


def test_decompose_from_ntt_domain_and_level(oracle, cuda_device):
    """The reference's call: ciphertext at rest in the NTT domain, level l below L."""
    logN, N1, L, l = 13, 64, 3, 1
    N, q, ctx, rlwe = _setup(logN, N1, L, seed=7, p_num=2)
    k = N // N1
    T = oracle.NttTables(N, ctx.pVec + ctx.qVec)
    ntt = rlwe.copy()
    oracle.ntt_batch(ntt, T, 0, ctx.p_num, 2, l + 1, L + 1)            # limbs 0..l of a and b into the NTT domain
    pc = PCMM_Context(N1, k, [], q[:l + 1])
    sch = PCMM_Scheme(pc, context=ctx)
    ct = Ciphertext(N, L, l, N // 2, 1.0, cipher=as_u64_tensor(ntt, ctx.device).reshape(-1))
    mlwe = [MLWECiphertext(N1, l, l, k, 1.0) for _ in range(4)]
    sch.rlweCipherDecompose(ct, mlwe, 4, 0)
    exp = oracle.rlwe_decompose(rlwe[0, :l + 1], rlwe[1, :l + 1], N1, k, 4, q[:l + 1])
    for i in range(4):
        assert np.array_equal(to_u64_numpy(mlwe[i].cipher_device).reshape(l + 1, k + 1, N1), exp[i])
    assert np.array_equal(to_u64_numpy(ct.cipher_device).reshape(ntt.shape), ntt)      # back in the NTT domain
    pc.close(); ctx.close()


def test_decompose_error_message(cuda_device, capsys):
    N, q, ctx, rlwe = _setup(12, 64, 0, seed=1)
    pc = PCMM_Context(64, 64, [], q)
    sch = PCMM_Scheme(pc, context=ctx)
    ct = Ciphertext(N, 0, 0, N // 2, 1.0, cipher=as_u64_tensor(rlwe, ctx.device).reshape(-1))
    mlwe = [MLWECiphertext(64, 0, 0, 64, 1.0) for _ in range(65)]
    sch.rlweCipherDecompose(ct, mlwe, 65, 0)
    assert "extract number muse <= mlwe_rank" in capsys.readouterr().out
    pc.close(); ctx.close()


@pytest.mark.skipif(not R.available(), reason="reference driver library not built")
def test_decompose_matches_reference_kernel(oracle, cuda_device):
    """rlweCipherDecompose_kernel<256> of the reference (N=2^15, N1=128, rank 256)."""
    if not hasattr(R.lib(), "ref_decompose"):
        pytest.skip("reference driver built without the decomposition entry")
    logN, N1, L, l = 15, 128, 1, 1
    N, q, ctx, rlwe = _setup(logN, N1, L, seed=3, p_num=0)
    k = N // N1
    pc = PCMM_Context(N1, k, [], q)
    sch = PCMM_Scheme(pc, context=ctx)
    ct = Ciphertext(N, L, l, N // 2, 1.0, cipher=as_u64_tensor(rlwe, ctx.device).reshape(-1))
    for mlwe_num in (8, 128, 256):            # gaps 32 (word-by-word kernel), 2 and 1 (the kernel that shares RLWE words)
        ref_out = R.decompose(rlwe, logN, N1, k, mlwe_num, L, l, q)
        exp = oracle.rlwe_decompose(rlwe[0], rlwe[1], N1, k, mlwe_num, q).reshape(ref_out.shape)
        assert np.array_equal(exp, ref_out)
        mlwe = [MLWECiphertext(N1, L, l, k, 1.0) for _ in range(mlwe_num)]
        sch.rlweCipherDecompose(ct, mlwe, mlwe_num, 0, ntt_domain=False)
        for i in range(mlwe_num):
            assert np.array_equal(to_u64_numpy(mlwe[i].cipher_device).reshape(l + 1, -1), ref_out[i]), (mlwe_num, i)
    pc.close(); ctx.close()


def test_packing_bit_exact_and_decrypts(oracle, cuda_device):
    """mlweCipherPacking on the GPU: every word equal to the oracle's, and the packed RLWE
    ciphertext decrypts to the message that went through decompose -> pack."""
    N1, k = 64, 64
    logN, N = 12, 4096
    q = params.ntt_primes(50, 2 * N, 2)                       # q0, q1 (q1 only sizes the buffers)
    p = params.ntt_primes(51, 2 * N, 2)                       # the LAST p is the ring-pack prime
    ctx = Context_23(logN, p, q, [])
    T = oracle.NttTables(N, [p[-1], q[0]])
    rng = np.random.default_rng(4)
    s = H.sparse_ternary(rng, N, 64)
    vals = rng.uniform(-1, 1, N)
    delta = float(1 << 30)
    a, b = H.rlwe_encrypt(oracle, rng, H.encode_coeffs(vals, delta, q[:1]), s, q[:1])
    for mlwe_num in (k, 16):
        mlwe = oracle.rlwe_decompose(a, b, N1, k, mlwe_num, q[:1])[:, 0]          # [num][(k+1)][N1]
        keys = H.repacking_keys(oracle, np.random.default_rng(5), s, N1, k, p[-1], q[0], T)
        exp, stages = oracle.mlwe_packing(mlwe, keys, N1, k, p[-1], q[0], T)
        pc = PCMM_Context(N1, k, [p[-1]], q)
        sch = PCMM_Scheme(pc, context=ctx)
        sch.addRepakcingKey(as_u64_tensor(keys, ctx.device).reshape(-1))
        L = 1
        cts = [MLWECiphertext(N1, L, 0, k, delta, cipher=as_u64_tensor(
            np.concatenate([mlwe[i].reshape(-1), np.zeros((k + 1) * N1, dtype=np.uint64)]), ctx.device)) for i in range(mlwe_num)]
        out = Ciphertext(N, L, L, N // 2, 1.0)
        sch.mlweCipherPacking(out, cts, mlwe_num, 0)
        got = to_u64_numpy(out.cipher_device).reshape(2, L + 1, N)
        assert np.array_equal(got[:, 0], exp)
        assert out.l == 0 and out.scale == delta
        if mlwe_num == k:
            sub = oracle.NttTables(N, q[:1])
            coeff = got[:, :1].copy()
            oracle.ntt_batch(coeff, sub, 0, 0, 2, 1, 1, inverse=True)
            dec = (coeff[1, 0] + oracle.negacyclic_mul_small(coeff[0, 0], s, q[0])) % np.uint64(q[0])
            assert np.abs(H.centered(dec, q[0]) / delta - vals).max() < 2.0 ** -20
        pc.close()
    ctx.close()


@pytest.mark.skipif(not R.available(), reason="reference driver library not built")
def test_packing_stages_match_reference_kernels(oracle, cuda_device):
    """mlweCipherEmbedding_new_kernel, mlweCipherMultRepackingKey_kernel<256> and
    ringpacking_ModDown_kernel of the reference (N=2^15, N1=128, rank 256) against the oracle's
    stages, and the library's end result against the oracle's."""
    if R._pack_fns() is None:
        pytest.skip("reference driver built without the packing entries")
    import ctypes as C
    logN, N1, k = 15, 128, 256
    N = 1 << logN
    q0 = params.REF_LOGN16_Q[0]                 # the reference's own q0 and special prime (both = 1 mod 2^17)
    p = params.REF_LOGN16_P[-1]
    rng = np.random.default_rng(8)
    mlwe_num = 32
    mlwe = rng.integers(0, q0, (mlwe_num, (k + 1) * N1), dtype=np.uint64)
    keys = np.empty((k, 2, 2, N), dtype=np.uint64)
    keys[:, :, 0] = rng.integers(0, p, (k, 2, N), dtype=np.uint64)
    keys[:, :, 1] = rng.integers(0, q0, (k, 2, N), dtype=np.uint64)
    T = oracle.NttTables(N, [p, q0])
    exp, stages = oracle.mlwe_packing(mlwe.reshape(mlwe_num, k + 1, N1), keys, N1, k, p, q0, T)
    E_ref = R.pack_embed(mlwe, logN, N1, k, p, q0)
    assert np.array_equal(E_ref, stages["embed"])
    E_ntt = stages["embed"][:k].copy()
    oracle.ntt_batch(E_ntt, T, 0, 0, k, 2, 2)
    O_ref = R.pack_keymac(E_ntt, keys, logN, N1, k, p, q0)
    assert np.array_equal(O_ref, stages["keymac"])
    O_c = stages["keymac"].copy()
    oracle.ntt_batch(O_c, T, 0, 0, 2, 2, 2, inverse=True)
    assert np.array_equal(R.pack_moddown(O_c, logN, p, q0), stages["moddown"])
    # the library end to end on the same inputs
    ctx = Context_23(logN, [p], [q0, params.REF_LOGN16_Q[1]], [])
    pc = PCMM_Context(N1, k, [p], [q0, params.REF_LOGN16_Q[1]])
    sch = PCMM_Scheme(pc, context=ctx)
    sch.addRepakcingKey(as_u64_tensor(keys, ctx.device).reshape(-1))
    cts = [MLWECiphertext(N1, 0, 0, k, 1.0, cipher=as_u64_tensor(mlwe[i], ctx.device)) for i in range(mlwe_num)]
    out = Ciphertext(N, 1, 1, N // 2, 1.0)
    sch.mlweCipherPacking(out, cts, mlwe_num, 0)
    assert np.array_equal(to_u64_numpy(out.cipher_device).reshape(2, 2, N)[:, 0], exp)
    pc.close(); ctx.close()


@pytest.mark.parametrize("logN,N1,parts,M", [
    (12, 64, [(64, 0)], 40),                     # one source, every ciphertext of it (gap 1)
    (12, 64, [(32, 0), (16, 32), (5, 48)], 70),  # three sources with gaps 2, 4 and 12; 53 ciphertexts, ragged K block
    (13, 32, [(128, 0), (256, 128)], 130),       # the pipeline's pattern: one source half taken, one whole
    (12, 64, [(64, 0), (36, 64)], 33),           # whole K blocks per source, the last one ragged
    (12, 32, [(128, 0)], 16),                    # rank 128: eight row blocks of polynomials per tile column
    (12, 128, [(32, 0), (16, 32), (32, 48)], 24),  # rank 32: K blocks of 64 made of runs of 16 from different sources
])
def test_decompose_and_ppmm_in_one_call(oracle, cuda_device, logN, N1, parts, M):
    """The multiply that reads RLWE ciphertexts through the decomposition's index map gives, word for word,
    what rlweCipherDecompose followed by PPMM gives (and what the oracle gives for the two steps)."""
    L = l = 2
    N = 1 << logN
    k = N // N1
    q = params.ntt_primes(50, 2 * N, L + 1)
    ctx = Context_23(logN, params.ntt_primes(51, 2 * N, 1), q, [])
    rng = np.random.default_rng(logN * 100 + len(parts))
    K = sum(n for n, _ in parts)
    W = rng.uniform(-0.1, 0.1, (M, K)).astype(np.float32)
    scaler = float(1 << 30)
    pc = PCMM_Context(N1, k, [], q)
    sch = PCMM_Scheme(pc, context=ctx)
    rlwes, cts, exp_X = [], [], [None] * K
    for num, off in parts:
        rl = np.stack([H.uniform_residues(rng, q, (N,)), H.uniform_residues(rng, q, (N,))])
        rlwes.append(rl)
        cts.append(Ciphertext(N, L, l, N // 2, 1.0, cipher=as_u64_tensor(rl, ctx.device).reshape(-1)))
        dec = oracle.rlwe_decompose(rl[0], rl[1], N1, k, num, q)
        for i in range(num):
            exp_X[off + i] = dec[i].reshape(L + 1, -1)
    Wd = torch.from_numpy(W).to(ctx.device)
    sources = [(ct, num, off) for ct, (num, off) in zip(cts, parts)]
    mlwe = [MLWECiphertext(N1, L, l, k, 1.0) for _ in range(K)]
    fused = to_u64_numpy(sch.decomposeAndPPMM(Wd, sources, mlwe, M, K, N1, K, scaler=scaler, ntt_domain=False,
                                              copy_back=False)).copy()
    sch.check()
    for ct, rl in zip(cts, rlwes):
        assert np.array_equal(to_u64_numpy(ct.cipher_device).reshape(rl.shape), rl)       # sources untouched
    for ct, (num, off) in zip(cts, parts):
        sch.rlweCipherDecompose(ct, mlwe, num, off, ntt_domain=False)
    two_step = to_u64_numpy(sch.PPMM(Wd, mlwe, M, K, N1, K, scaler=scaler, copy_back=False))
    assert np.array_equal(fused, two_step)
    exp = oracle.ppmm(W, np.stack(exp_X), q, scaler)
    assert np.array_equal(fused, exp)
    # the same in three column ranges (a shard's view): the middle one starts and ends inside rows of polynomials
    C_ = (k + 1) * N1
    sch.ppmm_output.zero_()
    cuts = [0, 32 * 3, 32 * ((C_ // 32) - 2), C_]
    for a, b in zip(cuts[:-1], cuts[1:]):
        sch.decomposeAndPPMM(Wd, sources, mlwe, M, K, N1, K, scaler=scaler, col_begin=a, col_end=b, ntt_domain=False,
                             copy_back=False)
    sch.check()
    assert np.array_equal(to_u64_numpy(sch.ppmm_output[:exp.size]).reshape(exp.shape), exp)
    pc.close(); ctx.close()


def test_decompose_and_ppmm_from_ntt_domain_with_copy_back(oracle, cuda_device):
    """Sources at rest in the NTT domain: transformed back for the multiply and forward again afterwards, and the
    first limb of result row i lands in ciphertext i as after PPMM."""
    logN, N1, L = 12, 64, 1
    N, l = 1 << logN, 1
    k = N // N1
    q = params.ntt_primes(50, 2 * N, L + 1)
    ctx = Context_23(logN, params.ntt_primes(51, 2 * N, 1), q, [])
    rng = np.random.default_rng(77)
    rl = np.stack([H.uniform_residues(rng, q, (N,)), H.uniform_residues(rng, q, (N,))])
    T = oracle.NttTables(N, ctx.pVec + ctx.qVec)
    ntt = rl.copy()
    oracle.ntt_batch(ntt, T, 0, ctx.p_num, 2, l + 1, L + 1)
    K = M = 64
    W = rng.uniform(-0.1, 0.1, (M, K)).astype(np.float32)
    pc = PCMM_Context(N1, k, [], q)
    sch = PCMM_Scheme(pc, context=ctx)
    ct = Ciphertext(N, L, l, N // 2, 1.0, cipher=as_u64_tensor(ntt, ctx.device).reshape(-1))
    mlwe = [MLWECiphertext(N1, L, l, k, 1.0) for _ in range(K)]
    out = to_u64_numpy(sch.decomposeAndPPMM(torch.from_numpy(W).to(ctx.device), [(ct, K, 0)], mlwe, M, K, N1, K,
                                            scaler=float(1 << 30)))
    sch.check()
    X = oracle.rlwe_decompose(rl[0], rl[1], N1, k, K, q).reshape(K, L + 1, -1)
    exp = oracle.ppmm(W, X, q, float(1 << 30))
    assert np.array_equal(out, exp)
    assert np.array_equal(to_u64_numpy(ct.cipher_device).reshape(ntt.shape), ntt)          # back in the NTT domain
    for i in range(K):
        assert np.array_equal(to_u64_numpy(mlwe[i].cipher_device).reshape(L + 1, -1)[0], exp[i, 0])
    pc.close(); ctx.close()


def test_decompose_and_ppmm_rejects_gaps_and_overlaps(cuda_device):
    N, q, ctx, rlwe = _setup(12, 64, 1, seed=5)
    pc = PCMM_Context(64, 64, [], q)
    L_ = capi.load()
    ct = as_u64_tensor(rlwe, ctx.device).reshape(-1)
    W = torch.zeros((8, 64), dtype=torch.float32, device=ctx.device)
    out = torch.empty(8 * 2 * 65 * 64, dtype=torch.int64, device=ctx.device)

    def call(parts, K=64):
        arr = (capi.RlweSource * len(parts))()
        for j, (num, off) in enumerate(parts):
            arr[j].d_rlwe, arr[j].L, arr[j].mlwe_num, arr[j].offset = ct.data_ptr(), 1, num, off
        return L_.ckks_b200_pcmm_ppmm_rlwe(pc._h, W.data_ptr(), arr, len(parts), out.data_ptr(), 8, K, 64, K, 1.0, 0, 65 * 64, None)

    assert call([(32, 0)]) == capi.ERR_ARG                      # ciphertexts 32..63 filled by no source
    assert call([(64, 0), (8, 8)]) == capi.ERR_ARG              # filled twice
    assert call([(65, 0)], K=65) == capi.ERR_SHAPE              # more than the rank from one source
    assert call([(64, 0)]) == capi.OK
    torch.cuda.synchronize()
    pc.close(); ctx.close()
