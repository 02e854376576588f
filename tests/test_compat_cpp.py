"""The C++ shim (include/ckks_b200/compat.hpp): it compiles and links against the library on
CPU, and on a GPU a reference-style C++ driver produces the oracle's words."""
import os
import subprocess

import numpy as np
import pytest

import helpers as H
from ckks_llm_b200 import _build, params

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "tests", "compat_driver")


def _compile():
    _build.build()
    src = os.path.join(ROOT, "tests", "compat_driver.cu")
    if os.path.exists(BIN) and os.path.getmtime(BIN) >= max(
            os.path.getmtime(src), os.path.getmtime(os.path.join(ROOT, "include", "ckks_b200", "compat.hpp")),
            os.path.getmtime(_build.LIB)):
        return
    cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-I", os.path.join(ROOT, "include"),
           src, "-L", os.path.dirname(_build.LIB), "-lckks_b200", "-Xlinker", "-rpath", "-Xlinker",
           os.path.dirname(_build.LIB), "-o", BIN]
    subprocess.run(cmd, check=True)


def test_compat_driver_compiles_and_links():
    _compile()
    assert os.path.exists(BIN)


@pytest.mark.gpu
def test_compat_driver_matches_oracle(oracle, cuda_device, tmp_path):
    if not os.path.exists(BIN):
        _compile()
    logN, N1, rank, M, K = 12, 64, 3, 64, 64
    N, Cw = 1 << logN, (rank + 1) * N1
    q = params.ntt_primes(50, 2 * N, 2)
    rng = np.random.default_rng(33)
    poly = H.uniform_residues(rng, q, (N,))
    X = np.stack([H.uniform_residues(rng, q, (Cw,)) for _ in range(K)])
    W = rng.uniform(-0.1, 0.1, (M, K)).astype(np.float32)
    fin, fout = tmp_path / "in.bin", tmp_path / "out.bin"
    with open(fin, "wb") as f:
        f.write(np.array([q[0], q[1], logN, N1, rank, M, K], dtype=np.uint64).tobytes())
        f.write(poly.tobytes()); f.write(X.tobytes()); f.write(W.tobytes())
    env = dict(os.environ, LD_LIBRARY_PATH=os.path.dirname(_build.LIB) + ":" + os.environ.get("LD_LIBRARY_PATH", ""))
    r = subprocess.run([BIN, str(fin), str(fout)], capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0, r.stderr
    assert "matrix K should be equal to N1!" in r.stdout
    raw = np.fromfile(fout, dtype=np.uint64)
    fwd, back = raw[:2 * N].reshape(2, N), raw[2 * N:4 * N].reshape(2, N)
    out = raw[4 * N:4 * N + M * 2 * Cw].reshape(M, 2, Cw)
    ct5 = raw[4 * N + M * 2 * Cw:4 * N + M * 2 * Cw + Cw]
    ratio = raw[-1:].view(np.float64)[0]
    T = oracle.NttTables(N, q)
    exp = poly[None].copy()
    oracle.ntt_batch(exp, T, 0, 0, 1, 2, 2)
    assert np.array_equal(fwd, exp[0]) and np.array_equal(back, poly)
    scaler = float(int(q[1] * float(1 << 49) / float(1 << 49)))
    ref = oracle.ppmm(W, X, q, scaler)
    assert np.array_equal(out, ref)
    assert np.array_equal(ct5, ref[5, 0])
    assert abs(ratio - 1.0) < 1e-12          # scale * scaler / q1 with scaler == q1


def test_mirrors_agree_on_the_scale_bookkeeping(tmp_path):
    """The C++ shim, the source-level compat classes and the Python mirror derive the PPMM scaler and the scale it leaves
    from the LAST ring-pack modulus (the one the kernel rescales by): identical at the reference's two moduli, and equal
    to one another at three."""
    from ckks_llm_b200 import host
    src = tmp_path / "scale.cu"
    src.write_text(r"""
#include <cstdio>
#include "ckks_b200/compat.hpp"
int main() {
    std::vector<ckks_b200::uint64_tt> q = {%dULL, %dULL, %dULL};
    for (int n = 2; n <= 3; n++) {
        std::vector<ckks_b200::uint64_tt> qq(q.begin(), q.begin() + n);
        long double scale = 562949953421312.0L * 3 / 2;
        long s = ckks_b200::ppmm_scaler(qq, scale);
        printf("%%ld %%.6Lf\n", s, ckks_b200::ppmm_scale_after(qq, scale, s));
    }
    return 0;
}
""" % tuple(params.ntt_primes(50, 1 << 17, 3)))
    exe = tmp_path / "scale"
    subprocess.run(["nvcc", "-std=c++17", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)], check=True)
    lines = subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split("\n")
    q = params.ntt_primes(50, 1 << 17, 3)
    scale = float(1 << 49) * 1.5
    for n, ln in zip((2, 3), lines):
        s_cpp, after_cpp = ln.split()
        s_py = host.ppmm_scaler(q[:n], scale)
        assert int(s_cpp) == int(s_py)
        assert abs(float(after_cpp) - host.ppmm_scale_after(q[:n], scale, s_py)) / float(after_cpp) < 1e-12
