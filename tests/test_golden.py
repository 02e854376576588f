"""The oracle against the committed golden fixtures, which were produced by the REAL reference:
tests/golden/ref_host.json by its host table builders, tests/golden/ref_kernels_b200.json by
its CUDA kernels on a B200 (tests/golden/gen_golden.py).  Runs anywhere, without the reference."""
import hashlib
import importlib.util
import json
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
spec = importlib.util.spec_from_file_location("gen_golden", os.path.join(HERE, "golden", "gen_golden.py"))


def _load(name):
    return json.load(open(os.path.join(HERE, "golden", name)))


def _digest(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def _cases():
    # the generator module imports oracle.ref lazily enough to load without the driver library
    gg = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gg)
    return gg


def test_roots_and_tables_match_reference_host(oracle):
    g = _load("ref_host.json")
    for q, v in g["roots"].items():
        assert oracle.find_psi(v["two_n"], int(q)) == v["psi"], q
    for key, v in g["tables"].items():
        n, q = (int(x) for x in key.split(":"))
        T = oracle.NttTables(n, [q])
        tabs = [T.psi[0], T.psiinv[0], T.psi_shoup[0], T.psiinv_shoup[0]]
        assert [_digest(t) for t in tabs] == v["sha256"]
        assert [[int(x) for x in t[:4]] for t in tabs] == v["head"]


def test_ntt_matches_reference_kernels(oracle):
    g, gg = _load("ref_kernels_b200.json"), _cases()
    for logN in (14, 16):
        pqt, data = gg.ntt_case(logN)
        T = oracle.NttTables(1 << logN, pqt)
        fwd = data.copy()
        oracle.ntt_batch(fwd, T, 0, 0, 2, len(pqt), len(pqt))
        inv = data.copy()
        oracle.ntt_batch(inv, T, 0, 0, 2, len(pqt), len(pqt), inverse=True)
        assert [int(v) for v in fwd[0, 0, :4]] == g[f"ntt{logN}"]["fwd_head"]
        assert _digest(fwd) == g[f"ntt{logN}"]["fwd"] and _digest(inv) == g[f"ntt{logN}"]["inv"]


def test_modup_matches_reference_kernel(oracle):
    g, gg = _load("ref_kernels_b200.json"), _cases()
    logN, p, q, t, l, inp = gg.modup_case()
    out = oracle.modup(inp, 1 << logN, q, t, len(p), l, 1)
    assert [int(v) for v in out[0, 0, 0, :4]] == g["modup"]["head"]
    assert _digest(out) == g["modup"]["out"]


def test_ppmm_matches_reference_kernel(oracle):
    g, gg = _load("ref_kernels_b200.json"), _cases()
    q, N1, rank, W, X, scaler = gg.ppmm_case()
    out = oracle.ppmm(W, X, q, scaler)
    assert [int(v) for v in out[0, 0, :4]] == g["ppmm"]["head"]
    assert _digest(out) == g["ppmm"]["out"]


def test_level_changes_match_reference_kernels(oracle):
    g, gg = _load("ref_kernels_b200.json"), _cases()
    logN, p, q, l, cipher = gg.rescale_case()
    T = oracle.NttTables(1 << logN, p + q)
    out = oracle.rescale(cipher.copy(), T, len(p), len(q) - 1, l)
    assert [int(v) for v in out[0, 0, :4]] == g["rescale"]["head"]
    assert _digest(out) == g["rescale"]["out"]
    logN, p, q, target, scale_up, cipher = gg.modup_q0_case()
    T = oracle.NttTables(1 << logN, p + q)
    out = oracle.modup_q0_to_ql(cipher.copy(), T, len(p), len(q) - 1, target, scale_up)
    assert [int(v) for v in out[0, 1, :4]] == g["modup_q0_to_ql"]["head"]
    assert _digest(out) == g["modup_q0_to_ql"]["out"]
