"""CPU checks of the C-ABI boundary: the library loads, exports every symbol the header
declares, validates arguments, and refuses to compute without a CUDA device."""
import ctypes as C
import os
import re

from ckks_llm_b200 import capi, params

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "ckks_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ckks_b200_\w+)\s*\(", text)))


def test_every_declared_symbol_is_exported():
    L = capi.load()
    names = _declared_symbols()
    assert len(names) >= 20
    for n in names:
        assert hasattr(L, n), n
    assert sorted(capi.SYMBOLS) == names


def test_version_and_status_strings():
    L = capi.load()
    assert L.ckks_b200_version() >= 100
    assert L.ckks_b200_status_string(capi.OK) == b"ok"
    assert b"shape" in L.ckks_b200_status_string(capi.ERR_SHAPE)


def test_argument_validation_needs_no_device():
    L = capi.load()
    assert L.ckks_b200_context_create(None, 0, 16, None, 0, None, 0, None, 0) == capi.ERR_ARG
    h = C.c_void_p()
    q = capi.u64_array([params.REF_LOGN16_Q[0]])
    assert L.ckks_b200_context_create(C.byref(h), 0, 20, None, 0, q, 1, None, 0) == capi.ERR_UNSUPPORTED
    assert b"logN" in L.ckks_b200_last_error()
    assert L.ckks_b200_ntt_forward(None, None, 0, 0, 1, 1, 1, None) == capi.ERR_ARG
    assert L.ckks_b200_pcmm_create(C.byref(h), 0, 64, 64, None, 0) == capi.ERR_ARG
    assert L.ckks_b200_context_destroy(None) == capi.OK
    assert L.ckks_b200_pcmm_destroy(None) == capi.OK
    # entry points added around the path: a null handle is an argument error everywhere, before any CUDA call
    assert L.ckks_b200_pcmm_set_host_chunks(None, 4) == capi.ERR_ARG
    assert L.ckks_b200_pcmm_ppmm_rlwe(None, None, None, 0, None, 1, 1, 1, 1, 1.0, 0, 32, None) == capi.ERR_ARG
    assert L.ckks_b200_rescale_batch(None, None, 1, 1, 1, None) == capi.ERR_ARG
    assert L.ckks_b200_modup_q0_to_ql_batch(None, None, 1, 1, 1, 1, None) == capi.ERR_ARG
    assert L.ckks_b200_conjugate(None, None, None, None, 0, 1, None) == capi.ERR_ARG
    assert L.ckks_b200_rotate(None, None, None, None, 1, 0, 1, None) == capi.ERR_ARG
    assert L.ckks_b200_keyswitch(None, None, None, None, 0, 1, None) == capi.ERR_ARG


def test_no_cpu_fallback():
    """Without a GPU a compute handle cannot even be created: the call reports a CUDA error
    instead of silently running somewhere else."""
    import torch
    if torch.cuda.is_available():
        return
    L = capi.load()
    h = C.c_void_p()
    q = capi.u64_array([params.REF_LOGN16_Q[0]])
    assert L.ckks_b200_context_create(C.byref(h), 0, 16, None, 0, q, 1, None, 0) == capi.ERR_CUDA
    assert L.ckks_b200_pcmm_create(C.byref(h), 0, 64, 64, q, 1) == capi.ERR_CUDA


def test_product_does_not_import_oracle():
    pkg = os.path.join(ROOT, "ckks_llm_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                src = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in src.replace("test-only oracle", ""), os.path.join(dirpath, f)
