"""GPU parity of PPMM (tensor-core and CUDA-core paths) against the CPU oracle."""
import numpy as np
import pytest
import torch

import helpers as H
from ckks_llm_b200 import capi, params
from ckks_llm_b200.host import MLWECiphertext, PCMM_Context, PCMM_Scheme, as_u64_tensor, to_u64_numpy

pytestmark = pytest.mark.gpu

ALGOS = [capi.PCMM_SIMT, capi.PCMM_TENSOR]


def _ciphers(rng, q, K, N1, rank, device):
    Cw = (rank + 1) * N1
    X = np.stack([H.uniform_residues(rng, q, (Cw,)) for _ in range(K)])     # [K][limbs][C]
    cts = [MLWECiphertext(N1, len(q) - 1, len(q) - 1, rank, float(1 << 49),
                          cipher=as_u64_tensor(X[n], device).reshape(-1)) for n in range(K)]
    return X, cts


def _run(oracle, algo, q, M, K, N1, rank, scaler, seed, wdist="uniform", rows=None):
    pc = PCMM_Context(N1, rank, [], q)
    sch = PCMM_Scheme(pc, algo=algo)
    rng = np.random.default_rng(seed)
    if wdist == "uniform":
        W = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    else:
        W = rng.normal(0, 0.02, (M, K)).astype(np.float32)
    W[0, 0] = 0.0
    X, cts = _ciphers(rng, q, K, N1, rank, pc.device)
    Wd = torch.from_numpy(W).to(pc.device)
    out = sch.PPMM(Wd, cts, M, K, N1, K, scaler=scaler, copy_back=False)
    sch.check()
    got = to_u64_numpy(out)
    rows = range(M) if rows is None else rows
    for m in rows:
        exp = oracle.ppmm(W, X, q, scaler, m0=m, m1=m + 1)
        assert np.array_equal(got[m], exp[m]), (m, algo)
    pc.close()
    return got


@pytest.mark.parametrize("algo", ALGOS, ids=["simt", "tensor"])
def test_config1_shape(oracle, cuda_device, algo):
    """Configuration 1 shape: N1=64, rank 64, 64x64 weights at 2^30, three 36-bit limbs."""
    _run(oracle, algo, H.cfg1_moduli(), 64, 64, 64, 64, float(1 << 30), seed=0)


@pytest.mark.parametrize("algo", ALGOS, ids=["simt", "tensor"])
def test_reference_native_two_limbs(oracle, cuda_device, algo):
    """The reference's own setting: q_ringpack = {q0, q1} of its logN=16 chain, scaler = q1
    (scale 2^49), weights uniform +-0.1 (test_rlwe_decomp.cu:36-37,83-86)."""
    q = params.REF_LOGN16_Q[:2]
    pc_scaler = float(q[1])
    rng = np.random.default_rng(1)
    M = K = 128
    N1, rank = 128, 7
    pc = PCMM_Context(N1, rank, [], q)
    sch = PCMM_Scheme(pc, algo=algo)
    W = rng.uniform(-0.1, 0.1, (M, K)).astype(np.float32)
    X, cts = _ciphers(rng, q, K, N1, rank, pc.device)
    assert sch.scaler_for(float(1 << 49)) == pc_scaler
    out = sch.PPMM(torch.from_numpy(W).to(pc.device), cts, M, K, N1, K, copy_back=True)
    sch.check()
    got = to_u64_numpy(out)
    exp = oracle.ppmm(W, X, q, pc_scaler)
    assert np.array_equal(got, exp)
    # copy-back: limb 0 of row i replaces ciphertext i (PPMM_kernel.cuh:345-348)
    Cw = (rank + 1) * N1
    for i in (0, 5, K - 1):
        assert np.array_equal(to_u64_numpy(cts[i].cipher_device)[:Cw], exp[i, 0])
    pc.close()


@pytest.mark.parametrize("algo", ALGOS, ids=["simt", "tensor"])
def test_ragged_shapes(oracle, cuda_device, algo):
    """M and K that are not multiples of the tile sizes, four limbs."""
    q = params.ntt_primes(50, 1 << 13, 4)
    _run(oracle, algo, q, 40, 72, 32, 3, float(1 << 40), seed=2, wdist="normal")
    _run(oracle, algo, q[:1], 130, 100, 64, 1, float(1 << 40), seed=3, wdist="normal")


@pytest.mark.parametrize("algo", ALGOS, ids=["simt", "tensor"])
def test_wide_moduli_and_weights(oracle, cuda_device, algo):
    """60-bit limbs and 2^40-scaled weights exercise the widest plane configuration."""
    q = params.ntt_primes(60, 1 << 13, 2)
    _run(oracle, algo, q, 32, 64, 32, 1, float(1 << 40), seed=4)


def test_bert_shape_sampled_rows(oracle, cuda_device):
    """Configuration 4 geometry at reduced limb count: K=768, N1=128, rank 512 would need
    8 GB per operand at 20 limbs; 2 limbs keep it to 0.8 GB.  Tensor path vs CUDA-core path
    on every word, and vs the oracle on sampled rows."""
    q = params.ntt_primes(50, 1 << 17, 2)
    N1, rank, M, K = 128, 512, 768, 768
    pc = PCMM_Context(N1, rank, [], q)
    rng = np.random.default_rng(0)
    W = rng.normal(0, 0.02, (M, K)).astype(np.float32)
    Cw = (rank + 1) * N1
    Xd = torch.empty((K, 2, Cw), dtype=torch.int64, device=pc.device)
    g = torch.Generator(device=pc.device).manual_seed(0)
    for i, qi in enumerate(q):
        Xd[:, i, :] = torch.randint(0, qi, (K, Cw), generator=g, device=pc.device, dtype=torch.int64)
    cts = [MLWECiphertext(N1, 1, 1, rank, 1.0, cipher=Xd[n].reshape(-1)) for n in range(K)]
    Wd = torch.from_numpy(W).to(pc.device)
    outs = {}
    for algo in ALGOS:
        sch = PCMM_Scheme(pc, algo=algo)
        o = sch.PPMM(Wd, cts, M, K, N1, K, scaler=float(1 << 40), copy_back=False)
        sch.check()
        outs[algo] = o.clone()
    assert torch.equal(outs[capi.PCMM_SIMT], outs[capi.PCMM_TENSOR])
    X = to_u64_numpy(Xd)
    got = to_u64_numpy(outs[capi.PCMM_TENSOR])
    for m in (0, 383, 767):
        exp = oracle.ppmm(W, X, q, float(1 << 40), m0=m, m1=m + 1)
        assert np.array_equal(got[m], exp[m])
    pc.close()


def test_llama_contraction_depth(oracle, cuda_device):
    """Configuration 5 contraction: K = 4096 at 2^40-scaled weights and 50-bit limbs is the
    deepest sum the s32 accumulators take with five weight planes (5*4096*255^2 < 2^31).
    Reduced to 256 rows, N1=32, rank 3, 3 limbs; every word vs the CUDA-core path, sampled
    rows vs the oracle."""
    q = params.ntt_primes(50, 1 << 17, 3)
    N1, rank, M, K = 32, 3, 256, 4096
    Cw = (rank + 1) * N1
    rng = np.random.default_rng(5)
    W = rng.normal(0, 0.02, (M, K)).astype(np.float32)
    pc = PCMM_Context(N1, rank, [], q)
    X, cts = _ciphers(rng, q, K, N1, rank, pc.device)
    Wd = torch.from_numpy(W).to(pc.device)
    outs = {}
    for algo in ALGOS:
        sch = PCMM_Scheme(pc, algo=algo)
        outs[algo] = sch.PPMM(Wd, cts, M, K, N1, K, scaler=float(1 << 40), copy_back=False).clone()
        sch.check()
    assert torch.equal(outs[capi.PCMM_SIMT], outs[capi.PCMM_TENSOR])
    got = to_u64_numpy(outs[capi.PCMM_TENSOR])
    for m in (0, 100, 255):
        assert np.array_equal(got[m], oracle.ppmm(W, X, q, float(1 << 40), m0=m, m1=m + 1)[m])
    pc.close()


def test_column_range(oracle, cuda_device):
    """Only the requested column range is written (the unit multi-GPU sharding uses)."""
    q = params.ntt_primes(50, 1 << 13, 2)
    N1, rank, M, K = 64, 3, 64, 64
    Cw = (rank + 1) * N1
    rng = np.random.default_rng(9)
    W = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    for algo in ALGOS:
        pc = PCMM_Context(N1, rank, [], q)
        sch = PCMM_Scheme(pc, algo=algo)
        X, cts = _ciphers(np.random.default_rng(9), q, K, N1, rank, pc.device)
        sch.ppmm_output = torch.full((M * 2 * Cw,), -1, dtype=torch.int64, device=pc.device)
        out = sch.PPMM(torch.from_numpy(W).to(pc.device), cts, M, K, N1, K, scaler=float(1 << 30),
                       col_begin=64, col_end=160, copy_back=False)
        sch.check()
        got = to_u64_numpy(out)
        exp = oracle.ppmm(W, X, q, float(1 << 30))
        assert np.array_equal(got[:, :, 64:160], exp[:, :, 64:160])
        assert (got[:, :, :64] == np.uint64(2 ** 64 - 1)).all() and (got[:, :, 160:] == np.uint64(2 ** 64 - 1)).all()
        pc.close()


def test_peer_output_buffers_receive_the_same_words(oracle, cuda_device):
    """The epilogue's extra stores into other GPUs' output buffers, exercised with two more buffers on this GPU:
    each must end up with exactly the words of the local output, inside the column range only."""
    q = params.ntt_primes(50, 1 << 13, 3)
    N1, rank, M, K = 64, 3, 150, 96              # M spans two 128-row tiles; the second ends inside a 32-row group
    Cw = (rank + 1) * N1
    rng = np.random.default_rng(12)
    W = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    pc = PCMM_Context(N1, rank, [], q)
    sch = PCMM_Scheme(pc, algo=capi.PCMM_TENSOR)
    X, cts = _ciphers(np.random.default_rng(12), q, K, N1, rank, pc.device)
    peers = [torch.full((M * len(q) * Cw,), -1, dtype=torch.int64, device=pc.device) for _ in range(2)]
    pc.set_peer_outputs([t.data_ptr() for t in peers])
    sch.ppmm_output = torch.full((M * len(q) * Cw,), -1, dtype=torch.int64, device=pc.device)
    out = sch.PPMM(torch.from_numpy(W).to(pc.device), cts, M, K, N1, K, scaler=float(1 << 30), col_begin=32, col_end=224,
                   copy_back=False)
    sch.check()
    got = to_u64_numpy(out)
    exp = oracle.ppmm(W, X, q, float(1 << 30))
    assert np.array_equal(got[:, :, 32:224], exp[:, :, 32:224])
    for t in peers:
        assert torch.equal(t, sch.ppmm_output)
    # the CUDA-core algorithm does not write peers and says so
    sch.algo = capi.PCMM_SIMT
    with pytest.raises(capi.CkksB200Error):
        sch.PPMM(torch.from_numpy(W).to(pc.device), cts, M, K, N1, K, scaler=float(1 << 30), copy_back=False)
    pc.set_peer_outputs([])
    sch.PPMM(torch.from_numpy(W).to(pc.device), cts, M, K, N1, K, scaler=float(1 << 30), copy_back=False)
    pc.close()


def test_shape_rules_and_errors(cuda_device, capsys):
    q = params.ntt_primes(50, 1 << 13, 2)
    pc = PCMM_Context(64, 3, [], q)
    sch = PCMM_Scheme(pc)
    cts = [MLWECiphertext(64, 1, 1, 3, 1.0) for _ in range(4)]
    W = torch.zeros((4, 4), dtype=torch.float32, device=pc.device)
    assert sch.PPMM(W, cts, 4, 4, 32, 4, scaler=1.0) is None          # mat_K != N1
    assert "matrix K should be equal to N1!" in capsys.readouterr().out
    assert sch.PPMM(W, cts, 4, 4, 64, 3, scaler=1.0) is None          # mat_N != mlwe_num
    assert "matrix N should be equal to mlwe number!" in capsys.readouterr().out
    Wbad = torch.full((4, 4), float("inf"), dtype=torch.float32, device=pc.device)
    with pytest.raises(capi.CkksB200Error) as e:
        sch.PPMM(Wbad, cts, 4, 4, 64, 4, scaler=1.0)
    assert e.value.status == capi.ERR_RANGE
    pc.close()


def test_host_buffer_entry_point(oracle, cuda_device):
    q = H.cfg1_moduli()
    rng = np.random.default_rng(12)
    N1, rank, M, K = 64, 1, 32, 32
    W = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    X = np.stack([H.uniform_residues(rng, q, ((rank + 1) * N1,)) for _ in range(K)])
    pc = PCMM_Context(N1, rank, [], q)
    for algo in ALGOS:
        got = PCMM_Scheme(pc, algo=algo).PPMM_host(W, X, M, K, N1, K, float(1 << 30))
        assert np.array_equal(got, oracle.ppmm(W, X, q, float(1 << 30)))
    pc.close()


def test_config1_decrypt_through_gpu(oracle, cuda_device):
    """Configuration 1 end to end with the GPU multiply in the middle: decrypted output
    within 2^-20 of the fp64 matmul, residues bit-exact vs the oracle."""
    N, N1, k = 1 << 12, 64, 64
    moduli = H.cfg1_moduli()
    rng = np.random.default_rng(0)
    W = rng.uniform(-1, 1, (64, 64)).astype(np.float32)
    Xf = rng.uniform(-1, 1, (64, 64))
    delta = float(1 << 30)
    msg = H.encode_coeffs(H.pack_message(Xf, k), delta, moduli)
    s = H.sparse_ternary(rng, N, 192)
    a, b = H.rlwe_encrypt(oracle, rng, msg, s, moduli)
    X = oracle.rlwe_decompose(a, b, N1, k, 64, moduli).reshape(64, 3, (k + 1) * N1)
    pc = PCMM_Context(N1, k, [], moduli)
    out = PCMM_Scheme(pc, algo=capi.PCMM_TENSOR).PPMM_host(W, X, 64, 64, N1, 64, delta)
    assert np.array_equal(out, oracle.ppmm(W, X, moduli, delta))
    s_mlwe = oracle.ring_down(s, N1, k)
    expect = W.astype(np.float64) @ Xf
    scale_out = delta * delta / moduli[-1]
    worst = 0.0
    for m in range(64):
        dec = oracle.mlwe_decrypt(out[m, 0].reshape(k + 1, N1), s_mlwe, moduli[0])
        worst = max(worst, np.abs(H.centered(dec, moduli[0]) / scale_out - expect[m]).max())
    assert worst / np.abs(expect).max() < 2.0 ** -20
    pc.close()


def test_prepared_weights_and_graph_replay(oracle, cuda_device):
    """Weights scaled and sliced once (ckks_b200_pcmm_prepare_weights), then multiplies with a null weight pointer:
    same words as the per-call form on both algorithms, and the call, which then contains no host wait, can be
    recorded into a CUDA graph and replayed on new ciphertext words."""
    q = params.ntt_primes(50, 1 << 13, 3)
    N1, rank, M, K = 64, 3, 96, 80
    Cw = (rank + 1) * N1
    rng = np.random.default_rng(31)
    W = rng.normal(0, 0.02, (M, K)).astype(np.float32)
    scaler = float(1 << 40)
    pc = PCMM_Context(N1, rank, [], q)
    X = np.stack([H.uniform_residues(rng, q, (Cw,)) for _ in range(K)])
    Xd = as_u64_tensor(X, pc.device)                                    # one buffer: the ciphertexts sit at one stride
    cts = [MLWECiphertext(N1, 2, 2, rank, 1.0, cipher=Xd[n].reshape(-1)) for n in range(K)]
    Wd = torch.from_numpy(W).to(pc.device)
    exp = oracle.ppmm(W, X, q, scaler)
    for algo in ALGOS:
        sch = PCMM_Scheme(pc, algo=algo)
        sch.prepare_weights(Wd, M, K, scaler)
        out = sch.PPMM(None, cts, M, K, N1, K, scaler=scaler, copy_back=False)
        sch.check()
        assert np.array_equal(to_u64_numpy(out), exp), algo
        # another shape or scaler than the prepared one is an argument error, not a wrong product
        with pytest.raises(capi.CkksB200Error) as e:
            sch.PPMM(None, cts, M, K, N1, K, scaler=2 * scaler, copy_back=False)
        assert e.value.status == capi.ERR_ARG
    sch = PCMM_Scheme(pc, algo=capi.PCMM_TENSOR)
    sch.prepare_weights(Wd, M, K, scaler)
    sch.PPMM(None, cts, M, K, N1, K, scaler=scaler, copy_back=False)     # warm: workspaces exist
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            out = sch.PPMM(None, cts, M, K, N1, K, scaler=scaler, copy_back=False)
    X2 = np.stack([H.uniform_residues(rng, q, (Cw,)) for _ in range(K)])
    Xd.copy_(as_u64_tensor(X2, pc.device))
    out.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert np.array_equal(to_u64_numpy(out), oracle.ppmm(W, X2, q, scaler))
    # a multiply that brings its own weights replaces the prepared ones
    sch.PPMM(Wd, cts, M, K, N1, K, scaler=scaler, copy_back=False)
    with pytest.raises(capi.CkksB200Error):
        sch.PPMM(None, cts, M, K, N1, K, scaler=scaler, copy_back=False)
    del graph
    pc.close()


def test_deep_contraction_is_cut_into_passes(oracle, cuda_device):
    """K = 11008, the depth of the LLaMA down-projection (configuration 5's second weight transposed): with five weight
    planes one pass of s32 accumulators holds 6592 of it, so the tensor-core path runs two passes and adds the partial
    sums in 128 bits.  Every word against the oracle."""
    q = params.ntt_primes(50, 1 << 17, 2)
    N1, rank, M, K = 32, 1, 40, 11008
    Cw = (rank + 1) * N1
    rng = np.random.default_rng(41)
    W = rng.normal(0, 0.02, (M, K)).astype(np.float32)
    pc = PCMM_Context(N1, rank, [], q)
    X = np.stack([H.uniform_residues(rng, q, (Cw,)) for _ in range(K)])
    Xd = as_u64_tensor(X, pc.device)
    cts = [MLWECiphertext(N1, 1, 1, rank, 1.0, cipher=Xd[n].reshape(-1)) for n in range(K)]
    Wd = torch.from_numpy(W).to(pc.device)
    exp = oracle.ppmm(W, X, q, float(1 << 40))
    for algo in (capi.PCMM_TENSOR, capi.PCMM_AUTO):
        sch = PCMM_Scheme(pc, algo=algo)
        out = sch.PPMM(Wd, cts, M, K, N1, K, scaler=float(1 << 40), copy_back=False)
        sch.check()
        assert np.array_equal(to_u64_numpy(out), exp)
    pc.close()


def test_cuda_core_path_refuses_what_could_wrap(oracle, cuda_device):
    """The 64-bit kernel keeps the reference's unchecked 128-bit accumulator; where K products of two 60-bit factors
    could wrap it the call is refused, while the tensor-core path (exact signed sums) computes the product."""
    q = params.ntt_primes(60, 1 << 13, 2)
    N1, rank, M, K = 32, 1, 8, 512
    rng = np.random.default_rng(43)
    W = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    pc = PCMM_Context(N1, rank, [], q)
    X, cts = _ciphers(rng, q, K, N1, rank, pc.device)
    Wd = torch.from_numpy(W).to(pc.device)
    with pytest.raises(capi.CkksB200Error) as e:
        PCMM_Scheme(pc, algo=capi.PCMM_SIMT).PPMM(Wd, cts, M, K, N1, K, scaler=float(1 << 40), copy_back=False)
    assert e.value.status == capi.ERR_UNSUPPORTED
    sch = PCMM_Scheme(pc, algo=capi.PCMM_TENSOR)
    out = sch.PPMM(Wd, cts, M, K, N1, K, scaler=float(1 << 40), copy_back=False)
    sch.check()
    # below the wrap the reference's formula and the exact sum agree, so the oracle (which wraps like the reference)
    # is the exact product here: 512 * 2^60 * 2^40 < 2^128
    assert np.array_equal(to_u64_numpy(out), oracle.ppmm(W, X, q, float(1 << 40)))
    pc.close()


def test_wait_that_runs_out_is_reported_once_and_the_handle_stays_usable(oracle, cuda_device):
    """The bounded device-side waits: with the test switch the operand feed of every CTA stops before tile 5 and the
    wait for that tile gives up after a budget of about a millisecond.  The kernel returns by itself (nothing faults or
    hangs), the record survives a second multiply, the check reports it once with the site of the wait, and the
    handle multiplies correctly afterwards."""
    q = params.ntt_primes(50, 1 << 13, 3)
    N1, rank, M, K = 64, 3, 256, 1024                # 16 K blocks per tile: tile 5 is in the middle of the first one
    rng = np.random.default_rng(47)
    W = rng.normal(0, 0.02, (M, K)).astype(np.float32)
    pc = PCMM_Context(N1, rank, [], q)
    sch = PCMM_Scheme(pc, algo=capi.PCMM_TENSOR)
    X, cts = _ciphers(rng, q, K, N1, rank, pc.device)
    Wd = torch.from_numpy(W).to(pc.device)
    exp = oracle.ppmm(W, X, q, float(1 << 40))
    pc.set_wait_budget(2_000_000)
    pc.test_withhold_stage(5)
    sch.PPMM(Wd, cts, M, K, N1, K, scaler=float(1 << 40), copy_back=False)        # gives up
    out = sch.PPMM(Wd, cts, M, K, N1, K, scaler=float(1 << 40), copy_back=False)  # a normal multiply before any check
    with pytest.raises(capi.CkksB200Error) as e:
        sch.check()
    # sites 4 and 5 are the waits of the instruction issuer and of the epilogue warps for the tile that never came
    assert e.value.status == capi.ERR_TIMEOUT and ("site 4" in e.value.message or "site 5" in e.value.message)
    assert np.array_equal(to_u64_numpy(out), exp)     # the second multiply was not disturbed by the first
    sch.check()                                       # reported once
    pc.set_wait_budget(0)
    out = sch.PPMM(Wd, cts, M, K, N1, K, scaler=float(1 << 40), copy_back=False)
    sch.check()
    assert np.array_equal(to_u64_numpy(out), exp)
    pc.close()


def test_row_owner_buffers_receive_their_rows_only(oracle, cuda_device):
    """ckks_b200_pcmm_set_row_owners with three 'ranks' whose buffers all live on this GPU: every buffer ends up with
    the rows of its owner's run, all requested columns of them, and nothing else."""
    q = params.ntt_primes(50, 1 << 13, 3)
    N1, rank, M, K = 64, 3, 150, 96
    Cw = (rank + 1) * N1
    rng = np.random.default_rng(53)
    W = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    pc = PCMM_Context(N1, rank, [], q)
    sch = PCMM_Scheme(pc, algo=capi.PCMM_TENSOR)
    X, cts = _ciphers(rng, q, K, N1, rank, pc.device)
    world, me = 3, 1
    bufs = [torch.full((M * len(q) * Cw,), -1, dtype=torch.int64, device=pc.device) for _ in range(world)]
    sch.ppmm_output = bufs[me]
    pc.set_row_owners([b.data_ptr() if r != me else 0 for r, b in enumerate(bufs)], me)
    c0, c1 = 32, 224
    sch.PPMM(torch.from_numpy(W).to(pc.device), cts, M, K, N1, K, scaler=float(1 << 30), col_begin=c0, col_end=c1, copy_back=False)
    sch.check()
    exp = oracle.ppmm(W, X, q, float(1 << 30))
    untouched = np.uint64(2 ** 64 - 1)
    covered = 0
    for r in range(world):
        got = to_u64_numpy(bufs[r]).reshape(M, len(q), Cw)
        b, e = pc.row_owner_range(M, world, r)
        covered += e - b
        assert np.array_equal(got[b:e, :, c0:c1], exp[b:e, :, c0:c1])
        mask = np.ones(got.shape, dtype=bool)
        mask[b:e, :, c0:c1] = False
        assert (got[mask] == untouched).all()
    assert covered == M
    assert pc.row_owner_range(M, world, 0) == (0, 64) and pc.row_owner_range(M, world, 2) == (128, 150)
    pc.set_row_owners([], 0)
    pc.close()


def test_rlwe_host_entry_point(oracle, cuda_device):
    """ckks_b200_pcmm_ppmm_rlwe_host: RLWE ciphertexts in host memory in, product in host memory out, equal to the
    oracle's decomposition followed by its PPMM."""
    N, N1, k = 1 << 12, 64, 64
    q = params.ntt_primes(50, 2 * N, 2)
    rng = np.random.default_rng(59)
    M, K = 48, 96                                       # 64 ciphertexts from the first source, 32 (gap 2) from the second
    W = rng.uniform(-0.1, 0.1, (M, K)).astype(np.float32)
    rl = [np.stack([H.uniform_residues(rng, q, (N,)) for _ in range(2)]) for _ in range(2)]      # [2][2][N] each
    Xd = np.concatenate([oracle.rlwe_decompose(rl[0][0], rl[0][1], N1, k, 64, q).reshape(64, 2, -1),
                         oracle.rlwe_decompose(rl[1][0], rl[1][1], N1, k, 32, q).reshape(32, 2, -1)])
    pc = PCMM_Context(N1, k, [], q)
    got = PCMM_Scheme(pc).PPMM_rlwe_host(W, [(rl[0], 1, 64, 0), (rl[1], 1, 32, 64)], M, K, N1, K, float(1 << 30))
    assert np.array_equal(got, oracle.ppmm(W, Xd, q, float(1 << 30)))
    pc.close()


def test_config5_geometry_column_range(oracle, cuda_device):
    """BASELINE configuration 5 at its stated geometry: N1 = 2048, rank 32 (67584 words per ciphertext and limb),
    24 limbs of 50-bit primes, 4096 x 4096 weights ~N(0, 0.02) at 2^40.  One 256-column range of the product (the unit
    a GPU of the 8-way split works on) is computed from seeded ciphertext words and compared with the oracle on sampled
    rows, all 24 limbs of them.  The ciphertext and output buffers have their full row pitch, as in the sharded job;
    only the columns of the range are filled and read."""
    N1, rank, M, K, limbs = 2048, 32, 4096, 4096, 24
    Cw = (rank + 1) * N1
    q = params.ntt_primes(50, 1 << 17, limbs)
    c0, c1 = 33 * N1 - 512, 33 * N1 - 256              # inside the b polynomial, not aligned to its start
    torch.cuda.empty_cache()
    free, _ = torch.cuda.mem_get_info()
    need = 8 * limbs * Cw * (K + M)
    assert free > need * 1.05, f"the test needs {need / 2**30:.0f} GiB of device memory, {free / 2**30:.0f} are free"
    pc = PCMM_Context(N1, rank, [], q)
    dev = pc.device
    Xd = torch.empty((K, limbs, Cw), dtype=torch.int64, device=dev)
    g = torch.Generator(device=dev).manual_seed(5)
    for i, qi in enumerate(q):
        Xd[:, i, c0:c1] = torch.randint(0, qi, (K, c1 - c0), generator=g, device=dev, dtype=torch.int64)
    rng = np.random.default_rng(5)
    W = rng.normal(0, 0.02, (M, K)).astype(np.float32)
    cts = [MLWECiphertext(N1, limbs - 1, limbs - 1, rank, 1.0, cipher=Xd[n].reshape(-1)) for n in range(K)]
    sch = PCMM_Scheme(pc, algo=capi.PCMM_TENSOR)
    sch.ppmm_output = torch.empty(M * limbs * Cw, dtype=torch.int64, device=dev)
    out = sch.PPMM(torch.from_numpy(W).to(dev), cts, M, K, N1, K, scaler=float(1 << 40), col_begin=c0, col_end=c1,
                   copy_back=False)
    sch.check()
    Xs = to_u64_numpy(Xd[:, :, c0:c1].contiguous())
    for m in (0, 1, 2047, 2048, 4095):
        got = to_u64_numpy(out[m, :, c0:c1].contiguous())
        assert np.array_equal(got, oracle.ppmm(W, Xs, q, float(1 << 40), m0=m, m1=m + 1)[m]), m
    del out, cts, Xd
    sch.ppmm_output = None
    pc.close()
    torch.cuda.empty_cache()


def _pack_features(x_feat_tok, k, gap):
    """Feature i, token t -> RLWE coefficient i*gap + t*k: the comb ciphertext i of rlweCipherDecompose extracts
    (PCMM_Scheme.cuh:67-73; gap = k / mlwe_num)."""
    n_feat, n_tok = x_feat_tok.shape
    out = np.zeros(k * n_tok, dtype=np.float64)
    for t in range(n_tok):
        out[t * k: t * k + n_feat * gap: gap] = x_feat_tok[:, t]
    return out


def test_config4_decrypt_through_gpu(oracle, cuda_device):
    """BASELINE configuration 4 end to end on a reduced limb count: activations ~N(0,1) clipped to [-8, 8] for 128 tokens
    x 768 features, encoded at 2^40 into two RLWE ciphertexts of N = 2^16 (512 + 256 features, as Bert.cuh:249-254 cuts
    them), encrypted, decomposed into 768 MLWE ciphertexts (N1 = 128, rank 512), multiplied by 768 x 768 weights
    ~N(0, 0.02) at 2^40 on the tensor cores over three 50-bit limbs, decrypted.  Residues of sampled rows equal the
    oracle's; every decrypted output is within 2^-20 of the fp64 product, relative to its largest entry
    (test_rlwe_decomp.cu:184-196 is the reference's own check of this kind)."""
    N, N1, k, feats, toks = 1 << 16, 128, 512, 768, 128
    q = params.ntt_primes(50, 2 * N, 3)
    rng = np.random.default_rng(4)
    W = rng.normal(0, 0.02, (feats, feats)).astype(np.float32)
    Xf = np.clip(rng.normal(0, 1, (feats, toks)), -8, 8)
    delta = float(1 << 40)
    s = H.sparse_ternary(rng, N, 192)
    parts = []
    for f0, num in ((0, 512), (512, 256)):
        msg = H.encode_coeffs(_pack_features(Xf[f0:f0 + num], k, k // num), delta, q)
        a, b = H.rlwe_encrypt(oracle, rng, msg, s, q)
        parts.append(oracle.rlwe_decompose(a, b, N1, k, num, q).reshape(num, len(q), (k + 1) * N1))
    X = np.concatenate(parts)
    pc = PCMM_Context(N1, k, [], q)
    out = PCMM_Scheme(pc, algo=capi.PCMM_TENSOR).PPMM_host(W, X, feats, feats, N1, feats, delta)
    for m in (0, 400, 767):
        assert np.array_equal(out[m], oracle.ppmm(W, X, q, delta, m0=m, m1=m + 1)[m])
    s_mlwe = oracle.ring_down(s, N1, k)
    expect = W.astype(np.float64) @ Xf
    scale_out = delta * delta / q[-1]
    worst = 0.0
    for m in range(0, feats, 16):
        dec = oracle.mlwe_decrypt(out[m, 0].reshape(k + 1, N1), s_mlwe, q[0])
        worst = max(worst, np.abs(H.centered(dec, q[0]) / scale_out - expect[m]).max())
    assert worst / np.abs(expect).max() < 2.0 ** -20
    pc.close()
