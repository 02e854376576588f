"""The source-level boundary: include/ckks_llm_compat/ mirrors the reference's include paths and class names, and a
driver made of the reference's own driver lines (tests/compat_tree_driver.cu) compiles against it with one -I, links
the library, and on a GPU reproduces the CPU oracle at every step of decompose -> PPMM -> packing."""
import os
import subprocess

import numpy as np
import pytest

from ckks_llm_b200 import _build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "tests", "compat_tree_driver")
TREE = os.path.join(ROOT, "include", "ckks_llm_compat")


def _compile():
    _build.build()
    src = os.path.join(ROOT, "tests", "compat_tree_driver.cu")
    deps = [src, os.path.join(TREE, "ckks_llm_compat.hpp"), os.path.join(TREE, "NTL", "RR.h"), _build.LIB]
    if os.path.exists(BIN) and os.path.getmtime(BIN) >= max(os.path.getmtime(d) for d in deps):
        return
    cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-I", TREE, src, "-L", os.path.dirname(_build.LIB),
           "-lckks_b200", "-Xlinker", "-rpath", "-Xlinker", os.path.dirname(_build.LIB), "-o", BIN]
    subprocess.run(cmd, check=True)


def test_tree_mirrors_the_reference_include_paths():
    """Every header the reference's callers of this path include exists at the same relative path."""
    for rel in ("src/ckks/include/Context_23.cuh", "src/ckks/include/Context_23.h", "src/ckks/include/Ciphertext.cuh",
                "src/ckks/include/Scheme_23.cuh", "src/ckks/include/SecretKey.cuh", "src/ckks/include/Key.cuh",
                "src/ckks/include/TimeUtils.cuh", "src/ckks/include/precision.cuh",
                "src/ckks/include/bootstrapping/Bootstrapper.cuh",
                "src/ckks/include/pcmm/PCMM_Context.h", "src/ckks/include/pcmm/PCMM_Context.cuh",
                "src/ckks/include/pcmm/PCMM_Scheme.h", "src/ckks/include/pcmm/PCMM_Scheme.cuh",
                "src/ckks/include/pcmm/MLWECiphertext.cuh", "src/ckks/include/pcmm/PPMM_kernel.cuh"):
        assert os.path.exists(os.path.join(TREE, rel)), rel


def test_driver_of_reference_lines_compiles_and_links():
    _compile()
    assert os.path.exists(BIN)


def _run(args, timeout=600):
    env = dict(os.environ, LD_LIBRARY_PATH=os.path.dirname(_build.LIB) + ":" + os.environ.get("LD_LIBRARY_PATH", ""))
    return subprocess.run([BIN] + [str(a) for a in args], capture_output=True, text=True, env=env, timeout=timeout)


@pytest.mark.gpu
def test_reference_driver_flow_matches_oracle(oracle, cuda_device, tmp_path):
    """test_rlwe_decomp.cu's flow at N = 2^12, N1 = 64 (rank 64): every intermediate the driver dumps equals the oracle's
    (decomposition, PPMM output, packed ciphertext), and the decrypted result is within 2^-20 of the plaintext product."""
    if not os.path.exists(BIN):
        _compile()
    logN, N1 = 12, 64
    N, k = 1 << logN, (1 << logN) // N1
    Cw = (k + 1) * N1
    out = tmp_path / "dump.bin"
    r = _run(["decomp", logN, N1, out])
    assert r.returncode == 0, r.stdout + r.stderr
    assert "matrix K should be equal to N1!" in r.stdout
    assert "after-ppmm scale ratio 1.000000" in r.stdout and "result level 0" in r.stdout
    raw = np.fromfile(out, dtype=np.uint64)
    hdr, pos = raw[:8], 8
    p, q0, q1, L, M = int(hdr[2]), int(hdr[3]), int(hdr[4]), int(hdr[5]), int(hdr[6])
    assert (int(hdr[0]), int(hdr[1]), M) == (logN, N1, k)
    W = raw[pos:pos + M * M // 2].view(np.float32).reshape(M, M); pos += M * M // 2
    c1 = raw[pos:pos + 2 * (L + 1) * N].reshape(2, L + 1, N); pos += 2 * (L + 1) * N
    keys = raw[pos:pos + 4 * N * k].reshape(k, 2, 2, N); pos += 4 * N * k
    mlwe = raw[pos:pos + k * 2 * Cw].reshape(k, 2, Cw); pos += k * 2 * Cw
    ppmm = raw[pos:pos + M * 2 * Cw].reshape(M, 2, Cw); pos += M * 2 * Cw
    c2 = raw[pos:pos + 2 * (L + 1) * N].reshape(2, L + 1, N)
    q = [q0, q1]
    # decomposition: inverse transform of limbs 0..1, gather
    Tq = oracle.NttTables(N, q)
    ab = np.ascontiguousarray(c1[:, :2, :]).copy()
    oracle.ntt_batch(ab, Tq, 0, 0, 2, 2, 2, inverse=True)
    exp_mlwe = oracle.rlwe_decompose(ab[0], ab[1], N1, k, k, q).reshape(k, 2, Cw)
    assert np.array_equal(mlwe, exp_mlwe)
    # PPMM at the reference's scaler (q1 for a scale of 2^49)
    exp_ppmm = oracle.ppmm(W, exp_mlwe, q, float(q1))
    assert np.array_equal(ppmm, exp_ppmm)
    # packing of limb 0 of the result rows with the driver's own keys
    Tpq = oracle.NttTables(N, [p, q0])
    packed, _ = oracle.mlwe_packing(np.ascontiguousarray(exp_ppmm[:, 0, :]).reshape(k, k + 1, N1), keys, N1, k, p, q0, Tpq)
    assert np.array_equal(c2[:, 0], packed)


@pytest.mark.gpu
def test_bert_layer_flow_decrypts(cuda_device):
    """src/bert's call sequence at its real size (N = 2^16, N1 = 128, three ciphertexts of 256 features, 768 x 768
    weights, three packings) through the compat classes: decrypted outputs within 2^-20 of the plaintext product."""
    if not os.path.exists(BIN):
        _compile()
    r = _run(["bert"])
    assert r.returncode == 0, r.stdout + r.stderr
    assert "realData_coeffShift: not defined by the reference" in r.stdout


def test_reference_programs_build_unmodified():
    """Where the reference tree is present: its own driver programs for this path (test_rlwe_decomp.cu,
    ntt_throughput.cu) compile, unmodified, with nothing but -I into the header tree, and link against the library."""
    import build_ref_callers
    if not os.path.isdir(build_ref_callers.REF_ROOT):
        pytest.skip("the reference tree is not on this machine")
    built = build_ref_callers.build_ref_callers()
    assert set(built) == set(build_ref_callers.PROGRAMS)
