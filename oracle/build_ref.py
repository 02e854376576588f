"""Build recipe for the real-reference driver (test infrastructure).

Compiles oracle/ref_driver.cu against the reference sources WHERE THEY LIE (the
reference tree is never copied) with the NTL stand-in under oracle/ref_shim/, into
oracle/_ref/libref_driver.so.  The reference's own build system is not used: it is a
single nvcc line (run.sh:13) that needs NTL/GMP, which are absent here.  Where the
reference tree is not present the prebuilt library, if any, is used as it is.
"""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
# the reference tree: named by CKKS_REFERENCE_ROOT, else a directory `reference` beside this repository
REF_ROOT = os.environ.get("CKKS_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
REF_INC = os.path.join(REF_ROOT, "src", "ckks", "include")
OUT_DIR = os.path.join(HERE, "_ref")
LIB = os.path.join(OUT_DIR, "libref_driver.so")
SRC = os.path.join(HERE, "ref_driver.cu")


def build_ref(force=False):
    """Returns the path of the driver library, or None when it cannot be built here."""
    if not os.path.isdir(REF_INC):
        return LIB if os.path.exists(LIB) else None
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= os.path.getmtime(SRC):
        return LIB
    os.makedirs(OUT_DIR, exist_ok=True)
    cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-w", "-std=c++17",
           "-I", os.path.join(HERE, "ref_shim"), "-I", REF_INC, "-shared", "-Xcompiler", "-fPIC",
           "-o", LIB, SRC]
    subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    print(build_ref(force=True))
