"""Build recipe for the CPU oracle (test infrastructure, never on the product path).

`build_oracle()` compiles oracle/ckks_oracle.c with gcc + OpenMP into
oracle/libckks_oracle.so.  `build_ref()` (oracle/build_ref.py) compiles pieces of the
real reference from the sources where they lie, when that tree is present.
"""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "ckks_oracle.c")
LIB = os.path.join(HERE, "libckks_oracle.so")


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def build_oracle(force=False):
    if force or _stale(LIB, [SRC]):
        cmd = ["gcc", "-O3", "-march=x86-64-v2", "-fopenmp", "-fPIC", "-shared",
               "-fvisibility=hidden", "-o", LIB, SRC, "-lm"]
        subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    print(build_oracle(force=True))
