"""B200-native hot path of CKKS private inference: batched negacyclic RNS NTT/INTT,
Q-digit -> T basis conversion and the ring-packed plaintext x ciphertext matrix multiply,
as hand-written sm_100a CUDA behind a C ABI (include/ckks_b200.h)."""
from . import capi, params  # noqa: F401

__all__ = ["capi", "params", "host"]


def __getattr__(name):
    if name == "host":          # needs torch; imported on first use
        import importlib
        return importlib.import_module(".host", __name__)
    raise AttributeError(name)
