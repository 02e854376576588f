"""The reference's OWN driver programs for this path, compiled unmodified against include/ckks_llm_compat and linked
with libckks_b200 (tests/build_ref_callers.py), run on the GPU.

`test_rlwe_decomp <logN> <N1>` encrypts a message, decomposes the RLWE ciphertext into MLWE ciphertexts, multiplies by
a plaintext matrix (PPMM), packs the result back into one RLWE ciphertext, decrypts and prints the precision against the
plaintext product; `ntt_throughput <logN> <polys> <limbs>` transforms a counting pattern back and forth and prints it.
The binaries are built where the reference tree is present and travel with the repository's other built files; where
they are absent the tests skip and say so."""
import os
import re
import subprocess

import pytest

from ckks_llm_b200 import _build

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
DIR = os.path.join(HERE, "_ref_callers")


def _run(name, args, timeout=300):
    binary = os.path.join(DIR, name)
    if not os.path.exists(binary):
        pytest.skip(f"{name} was not built: the reference tree was not present when the repository was built")
    env = dict(os.environ, LD_LIBRARY_PATH=os.path.dirname(_build.LIB) + ":" + os.environ.get("LD_LIBRARY_PATH", ""))
    # stdin closed: the program ends on a getchar()
    r = subprocess.run([binary] + [str(a) for a in args], stdin=subprocess.DEVNULL, capture_output=True, text=True, env=env,
                       timeout=timeout)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    return r.stdout


@pytest.mark.parametrize("logN,N1", [(12, 64), (13, 64), (15, 128), (16, 128)])
def test_reference_decompose_multiply_pack_program(cuda_device, logN, N1):
    """The last two are the sizes the reference documents for this program.  The decrypted result of decompose -> PPMM ->
    packing must agree with the program's own plaintext product to 2^-20 or better (it prints the worst coefficient)."""
    out = _run("test_rlwe_decomp", [logN, N1])
    assert f"decomp_num: {(1 << logN) // N1}" in out
    m = re.search(r"precision \(log2\): min ([-0-9.]+)\s+avg ([-0-9.]+)", out)
    assert m, out[-1500:]
    assert float(m.group(1)) >= 20.0, out[-1500:]


def test_reference_transform_benchmark_program(cuda_device):
    """INTT then NTT of the pattern i mod q0 over 8 limbs (four 51-bit p, four 50-bit q: two arithmetic back ends) of 64
    polynomials gives the pattern back; the program prints the first 16 words of 64 limbs."""
    out = _run("ntt_throughput", [16, 64, 8])
    rows = re.findall(r"\[((?:\d+, ){16})\]", out)
    assert len(rows) == 64, out[-1500:]
    want = ", ".join(str(i) for i in range(16)) + ", "
    assert all(r == want for r in rows)
    assert re.search(r"Throughput: 4step\s+ntt: [0-9.]+ OPs intt: [0-9.]+ OPs", out)
