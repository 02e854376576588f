"""The allocation-free PPMM entry point against the regular one.

ckks_b200_pcmm_ppmm_static exists for hosts that may not allocate device memory after
start-up (a server whose pool owns the GPU, a real-time loop, a sandboxed plug-in): it
keeps its working memory in a fixed array inside the library.  The test calls it through
the C ABI twice in a row, with different inputs, and requires the words to equal those of
ckks_b200_pcmm_ppmm and of the CPU oracle bit for bit (the tolerance of every integer test
here is zero).  The
second call must not be disturbed by what the first left in the shared array.  This file
sorts last so that a stop-at-first-failure run has seen every other test before it."""
import ctypes as C

import numpy as np
import pytest
import torch

import helpers as H
from ckks_llm_b200 import capi, params
from ckks_llm_b200.host import MLWECiphertext, PCMM_Context, PCMM_Scheme, as_u64_tensor, to_u64_numpy

pytestmark = pytest.mark.gpu


def _one_call(L, pc, q, M, K, N1, rank, scaler, seed, oracle):
    dev = pc.device
    rng = np.random.default_rng(seed)
    W = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    Cw = (rank + 1) * N1
    X = np.stack([H.uniform_residues(rng, q, (Cw,)) for _ in range(K)])
    Wd = torch.from_numpy(W).to(dev)
    Xd = [as_u64_tensor(X[n], dev).reshape(-1) for n in range(K)]
    cts = [MLWECiphertext(N1, len(q) - 1, len(q) - 1, rank, 1.0, cipher=x) for x in Xd]
    ref = PCMM_Scheme(pc, algo=capi.PCMM_SIMT).PPMM(Wd, cts, M, K, N1, K, scaler=scaler, copy_back=False).clone()
    out = torch.full((M * len(q) * Cw,), -1, dtype=torch.int64, device=dev)
    ptrs = (C.c_void_p * K)(*[x.data_ptr() for x in Xd])
    stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    capi.check(L.ckks_b200_pcmm_ppmm_static(Wd.data_ptr(), ptrs, out.data_ptr(), M, K, N1, K, N1, rank,
                                            capi.u64_array(q), len(q), scaler, stream))
    torch.cuda.synchronize(dev)
    got = to_u64_numpy(out).reshape(M, len(q), Cw)
    assert np.array_equal(got, to_u64_numpy(ref))
    assert np.array_equal(got, oracle.ppmm(W, X, q, scaler))           # and the CPU restatement of the reference


def test_static_entry_matches_regular_entry_twice(oracle, cuda_device):
    L = capi.load()
    torch.cuda.set_device(cuda_device)
    q = params.ntt_primes(50, 1 << 13, 3)
    N1, rank = 64, 3
    pc = PCMM_Context(N1, rank, [], q, device=cuda_device)
    _one_call(L, pc, q, 96, 80, N1, rank, float(1 << 40), 21, oracle)   # fills most of a tile
    _one_call(L, pc, q, 40, 33, N1, rank, float(1 << 30), 22, oracle)   # smaller: stale words remain behind it
    pc.close()


def test_static_entry_rejects_sizes_beyond_its_array(cuda_device):
    L = capi.load()
    torch.cuda.set_device(cuda_device)
    q = capi.u64_array(params.ntt_primes(50, 1 << 13, 2))
    dummy = torch.zeros(16, dtype=torch.int64, device="cuda")
    ptrs = (C.c_void_p * 1)(dummy.data_ptr())
    st = L.ckks_b200_pcmm_ppmm_static(dummy.data_ptr(), ptrs, dummy.data_ptr(), 2048, 1024, 64, 1024, 64, 3, q, 2, 1.0, None)
    assert st == capi.ERR_UNSUPPORTED and b"static scratch limit" in L.ckks_b200_last_error()
    st = L.ckks_b200_pcmm_ppmm_static(dummy.data_ptr(), ptrs, dummy.data_ptr(), 1, 5000, 64, 5000, 64, 3, q, 2, 1.0, None)
    assert st == capi.ERR_UNSUPPORTED
    st = L.ckks_b200_pcmm_ppmm_static(dummy.data_ptr(), ptrs, dummy.data_ptr(), 4, 4, 32, 4, 64, 3, q, 2, 1.0, None)
    assert st == capi.ERR_SHAPE
