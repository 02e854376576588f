"""ctypes binding of the C ABI declared in include/ckks_b200.h.

Loading fails loudly when the CUDA library has not been built: there is no CPU path.
"""
import ctypes as C
import os

from ._build import LIB

OK = 0
ERR_ARG, ERR_SHAPE, ERR_UNSUPPORTED, ERR_CUDA, ERR_NOMEM, ERR_RANGE, ERR_TIMEOUT = range(1, 8)
PCMM_AUTO, PCMM_TENSOR, PCMM_SIMT = 0, 1, 2

# every symbol include/ckks_b200.h declares
SYMBOLS = [
    "ckks_b200_version", "ckks_b200_status_string", "ckks_b200_last_error",
    "ckks_b200_context_create", "ckks_b200_context_destroy", "ckks_b200_context_psi",
    "ckks_b200_context_table",
    "ckks_b200_ntt_forward", "ckks_b200_ntt_inverse",
    "ckks_b200_ntt_forward_host", "ckks_b200_ntt_inverse_host",
    "ckks_b200_modup_qj_to_t", "ckks_b200_modup_qj_to_t_host", "ckks_b200_modup_set_algo", "ckks_b200_context_check",
    "ckks_b200_context_set_wait_budget", "ckks_b200_context_test_withhold_commit", "ckks_b200_context_test_exact_count",
    "ckks_b200_rescale", "ckks_b200_modup_q0_to_ql", "ckks_b200_rescale_batch", "ckks_b200_modup_q0_to_ql_batch",
    "ckks_b200_external_product_t", "ckks_b200_ntt_inverse_ext", "ckks_b200_modup_t_to_pql",
    "ckks_b200_moddown_pql_to_ql", "ckks_b200_keyswitch", "ckks_b200_mult", "ckks_b200_conjugate", "ckks_b200_rotate",
    "ckks_b200_rlwe_decompose", "ckks_b200_mlwe_packing",
    "ckks_b200_pcmm_create", "ckks_b200_pcmm_destroy", "ckks_b200_pcmm_ppmm",
    "ckks_b200_pcmm_ppmm_host", "ckks_b200_pcmm_ppmm_rlwe", "ckks_b200_pcmm_copy_back", "ckks_b200_pcmm_check", "ckks_b200_pcmm_set_peer_outputs", "ckks_b200_pcmm_set_host_chunks", "ckks_b200_ipc_open", "ckks_b200_ipc_close", "ckks_b200_pcmm_last_timing", "ckks_b200_pcmm_ppmm_static",
    "ckks_b200_pcmm_prepare_weights", "ckks_b200_pcmm_ppmm_rlwe_host", "ckks_b200_pcmm_set_wait_budget",
    "ckks_b200_pcmm_test_withhold_stage", "ckks_b200_pcmm_set_row_owners", "ckks_b200_pcmm_row_owner_range",
    "ckks_b200_kernel_launches",
]


class RlweSource(C.Structure):
    """ckks_b200_rlwe_source of include/ckks_b200.h."""
    _fields_ = [("d_rlwe", C.c_void_p), ("L", C.c_int), ("mlwe_num", C.c_int), ("offset", C.c_int)]


class CkksB200Error(RuntimeError):
    def __init__(self, status, message):
        super().__init__(f"ckks_b200 status {status}: {message}")
        self.status = status
        self.message = message


_lib = None


def load():
    """Load libckks_b200.so (built in-tree by ckks_llm_b200._build.build)."""
    global _lib
    if _lib is not None:
        return _lib
    lib_path = LIB
    if not os.path.exists(lib_path):
        raise ImportError(
            f"{LIB} is missing: build it with `python -m ckks_llm_b200._build` "
            "(nvcc, sm_100a).  This package has no CPU implementation.")
    L = C.CDLL(lib_path)
    vp, i, u64p, dbl, lng = C.c_void_p, C.c_int, C.POINTER(C.c_uint64), C.c_double, C.c_long
    L.ckks_b200_version.restype = i
    L.ckks_b200_status_string.restype = C.c_char_p
    L.ckks_b200_status_string.argtypes = [i]
    L.ckks_b200_last_error.restype = C.c_char_p
    L.ckks_b200_context_create.argtypes = [C.POINTER(vp), i, i, u64p, i, u64p, i, u64p, i]
    L.ckks_b200_context_destroy.argtypes = [vp]
    L.ckks_b200_context_psi.argtypes = [vp, i, u64p]
    L.ckks_b200_context_table.argtypes = [vp, i, i, vp]
    for name in ("ckks_b200_ntt_forward", "ckks_b200_ntt_inverse"):
        getattr(L, name).argtypes = [vp, vp, i, i, i, i, i, vp]
    for name in ("ckks_b200_ntt_forward_host", "ckks_b200_ntt_inverse_host"):
        getattr(L, name).argtypes = [vp, vp, i, i, i, i, i]
    L.ckks_b200_modup_qj_to_t.argtypes = [vp, vp, vp, i, i, vp]
    L.ckks_b200_modup_qj_to_t_host.argtypes = [vp, vp, vp, i, i]
    L.ckks_b200_modup_set_algo.argtypes = [vp, i]
    L.ckks_b200_context_check.argtypes = [vp, vp]
    L.ckks_b200_rescale.argtypes = [vp, vp, i, i, vp]
    L.ckks_b200_rescale_batch.argtypes = [vp, vp, i, i, i, vp]
    L.ckks_b200_modup_q0_to_ql_batch.argtypes = [vp, vp, i, i, i, C.c_longlong, vp]
    L.ckks_b200_external_product_t.argtypes = [vp, vp, vp, vp, i, i, vp]
    L.ckks_b200_ntt_inverse_ext.argtypes = [vp, vp, i, i, vp]
    L.ckks_b200_modup_t_to_pql.argtypes = [vp, vp, vp, i, i, i, vp]
    L.ckks_b200_moddown_pql_to_ql.argtypes = [vp, vp, vp, i, i, i, vp]
    L.ckks_b200_pcmm_set_peer_outputs.argtypes = [vp, vp, i]
    L.ckks_b200_pcmm_set_host_chunks.argtypes = [vp, i]
    L.ckks_b200_ipc_open.argtypes = [i, C.c_char_p, C.POINTER(C.c_void_p)]
    L.ckks_b200_ipc_close.argtypes = [i, vp]
    L.ckks_b200_keyswitch.argtypes = [vp, vp, vp, vp, i, i, vp]
    L.ckks_b200_mult.argtypes = [vp, vp, vp, vp, vp, i, i, vp]
    L.ckks_b200_conjugate.argtypes = [vp, vp, vp, vp, i, i, vp]
    L.ckks_b200_rotate.argtypes = [vp, vp, vp, vp, lng, i, i, vp]
    L.ckks_b200_modup_q0_to_ql.argtypes = [vp, vp, i, i, C.c_longlong, vp]
    L.ckks_b200_rlwe_decompose.argtypes = [vp, vp, i, i, C.POINTER(vp), i, i, i, i, vp]
    L.ckks_b200_mlwe_packing.argtypes = [vp, vp, i, C.POINTER(vp), i, i, i, vp, vp]
    L.ckks_b200_pcmm_create.argtypes = [C.POINTER(vp), i, i, i, u64p, i]
    L.ckks_b200_pcmm_destroy.argtypes = [vp]
    L.ckks_b200_pcmm_ppmm.argtypes = [vp, vp, C.POINTER(vp), vp, i, i, i, i, dbl, lng, lng, i, vp]
    L.ckks_b200_pcmm_ppmm_rlwe.argtypes = [vp, vp, C.POINTER(RlweSource), i, vp, i, i, i, i, dbl, lng, lng, vp]
    L.ckks_b200_pcmm_ppmm_host.argtypes = [vp, vp, vp, vp, i, i, i, i, dbl, i]
    L.ckks_b200_pcmm_copy_back.argtypes = [vp, vp, C.POINTER(vp), i, i, vp]
    L.ckks_b200_pcmm_check.argtypes = [vp, vp]
    L.ckks_b200_pcmm_last_timing.argtypes = [vp, C.POINTER(C.c_float), C.POINTER(C.c_float)]
    L.ckks_b200_pcmm_ppmm_static.argtypes = [vp, C.POINTER(vp), vp, i, i, i, i, i, i, u64p, i, dbl, vp]
    L.ckks_b200_context_set_wait_budget.argtypes = [vp, C.c_longlong]
    L.ckks_b200_context_test_withhold_commit.argtypes = [vp, i]
    L.ckks_b200_context_test_exact_count.argtypes = [vp, i]
    L.ckks_b200_pcmm_prepare_weights.argtypes = [vp, vp, i, i, dbl, vp]
    L.ckks_b200_pcmm_ppmm_rlwe_host.argtypes = [vp, vp, C.POINTER(RlweSource), i, vp, i, i, i, i, dbl]
    L.ckks_b200_pcmm_set_wait_budget.argtypes = [vp, C.c_longlong]
    L.ckks_b200_pcmm_test_withhold_stage.argtypes = [vp, i]
    L.ckks_b200_pcmm_set_row_owners.argtypes = [vp, vp, i, i]
    L.ckks_b200_pcmm_row_owner_range.argtypes = [i, i, i, C.POINTER(i), C.POINTER(i)]
    L.ckks_b200_kernel_launches.restype = lng
    for name in SYMBOLS:
        f = getattr(L, name)
        if f.restype is C.c_int and name not in ("ckks_b200_version",):
            f.restype = i
    _lib = L
    return L


def check(status):
    if status != OK:
        raise CkksB200Error(status, load().ckks_b200_last_error().decode())


def u64_array(values):
    arr = (C.c_uint64 * len(values))(*[int(v) for v in values])
    return arr
