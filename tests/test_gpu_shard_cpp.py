"""A C++ host shards one PCMM over the GPUs of its process with nothing but include/ckks_b200.h
(tests/shard_driver.cu): column ranges per GPU, every output row stored into its owner's buffer by the multiply itself.
Runs with as many GPUs as the machine has, up to four; on one GPU the same calls run with a world of one."""
import os
import subprocess

import pytest

from ckks_llm_b200 import _build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "shard_driver.cu")
BIN = os.path.join(ROOT, "tests", "shard_driver")


def _compile():
    _build.build()
    if os.path.exists(BIN) and os.path.getmtime(BIN) >= max(os.path.getmtime(SRC), os.path.getmtime(_build.LIB)):
        return
    subprocess.run(["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-I", os.path.join(ROOT, "include"), SRC,
                    "-L", os.path.dirname(_build.LIB), "-lckks_b200", "-Xlinker", "-rpath", "-Xlinker", os.path.dirname(_build.LIB),
                    "-o", BIN], check=True)


def test_shard_driver_compiles_and_links():
    _compile()
    assert os.path.exists(BIN)


@pytest.mark.gpu
def test_cpp_host_shards_a_multiply_by_row_owners(cuda_device):
    import torch
    if not os.path.exists(BIN):
        _compile()
    world = min(torch.cuda.device_count(), 4)
    env = dict(os.environ, LD_LIBRARY_PATH=os.path.dirname(_build.LIB) + ":" + os.environ.get("LD_LIBRARY_PATH", ""))
    for args in ([world], [world, 200, 96, 32, 15]):            # the second: rows and contraction off the tile sizes
        r = subprocess.run([BIN] + [str(a) for a in args], capture_output=True, text=True, env=env, timeout=300)
        assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
        assert "all ranks hold their rows" in r.stdout
        assert r.stdout.count("0 wrong words, 0 words written into rows it does not own") == world
