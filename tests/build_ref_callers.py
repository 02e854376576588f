"""Build recipe for the reference's OWN driver programs of this path, compiled unmodified against this repository.

`test_rlwe_decomp.cu` (RLWE -> MLWE decomposition, PPMM, ring packing, decryption check) and `ntt_throughput.cu`
(the transform benchmark) are read from the reference tree where it lies, copied to a temporary folder OUTSIDE this
repository (their quoted includes would otherwise find the reference's own headers beside them), compiled with nothing
but `-I include/ckks_llm_compat` and linked against libckks_b200.  Only the two binaries land in tests/_ref_callers/,
which version control ignores.  Where the reference tree is absent, binaries built earlier are used as they are.
"""
import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
REF_ROOT = os.environ.get("CKKS_REFERENCE_ROOT") or os.path.join(os.path.dirname(ROOT), "reference")
TREE = os.path.join(ROOT, "include", "ckks_llm_compat")
OUT_DIR = os.path.join(HERE, "_ref_callers")
# program -> include roots inside the tree, as the program's own #include lines need them
PROGRAMS = {"test_rlwe_decomp": [TREE], "ntt_throughput": [os.path.join(TREE, "src", "ckks"), TREE]}


def build_ref_callers(force=False):
    """Returns {program: path of its binary} for the programs that exist (built now or earlier)."""
    if ROOT not in sys.path:
        sys.path.insert(0, ROOT)
    from ckks_llm_b200 import _build
    out = {}
    for name, incs in PROGRAMS.items():
        src = os.path.join(REF_ROOT, name + ".cu")
        binary = os.path.join(OUT_DIR, name)
        if os.path.exists(src):
            deps = [src, os.path.join(TREE, "ckks_llm_compat.hpp"), _build.LIB]
            fresh = os.path.exists(binary) and os.path.getmtime(binary) >= max(os.path.getmtime(d) for d in deps if os.path.exists(d))
            if force or not fresh:
                _build.build()
                os.makedirs(OUT_DIR, exist_ok=True)
                with tempfile.TemporaryDirectory() as tmp:
                    shutil.copy(src, os.path.join(tmp, name + ".cu"))
                    cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-w", "-std=c++17"]
                    for inc in incs:
                        cmd += ["-I", inc]
                    cmd += [os.path.join(tmp, name + ".cu"), "-L", os.path.dirname(_build.LIB), "-lckks_b200",
                            "-Xlinker", "-rpath", "-Xlinker", os.path.dirname(_build.LIB), "-o", binary]
                    subprocess.run(cmd, check=True)
        if os.path.exists(binary):
            out[name] = binary
    return out


if __name__ == "__main__":
    print(build_ref_callers(force=True))
