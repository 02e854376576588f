"""Benchmark of the hot path on B200: PCMM ct-rows/s (headline) with NTT / INTT
limb-transforms/s and ModUp polynomials/s measured in the same run.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload pcmm|ntt|modup]
                    [--impl b200|reference]

A step is one pass of the named kernel family over one batch of seeded synthetic input
resident in HBM.  Default workload: the BERT-base-shaped PCMM (768x768 weights ~N(0,0.02)
at scale 2^40, 768 feature ciphertexts, N=2^16, N1=128, rank 512, 20 limbs of 50-bit
primes, ciphertext words uniform in [0,q_i)).  With N>1 ranks (torchrun) every rank
multiplies its own block of 128 tokens: no data-path collective, weak scaling.  After
that headline the default run also does, at every N, the LLaMA-7B-shaped multiply
(4096x4096, 24 limbs) as ONE job split by column range over the N ranks, with the two
ways of bringing the output together (config.llama_job), and the batched NTT on every
rank (config.ntt_ranks).  Prints one JSON line (rank 0).
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

PCMM_CFG = dict(logN=16, N1=128, rank=512, M=768, K=768, limbs=20, q_bits=50, w_std=0.02, scaler=float(1 << 40))
PCMM_WORKLOAD = ("bert-base PCMM 768x768 (W~N(0,0.02) at 2^40), 768 ciphertexts x 20 limbs x 65664 words, "
                 "N=2^16, N1=128, rank 512, 50-bit limbs")
NTT_CFG = dict(logN=16, limbs=40, q_bits=50, polys=32)
MODUP_CFG = dict(logN=16, q_num=24, q_bits=50, t_num=12, t_bits=60, alpha=8, batch=32)
SW, SC = 5, 7          # byte planes the PCMM workload needs: 40-bit signed weights, 50-bit residues
# DRAM traffic (bytes) from ncu captures of the --small cases, per unit of work
PCMM_TRAFFIC_PER_LIMB = (709.12e6 + 766.83e6) / 2                    # pcmm_umma_kernel<5,7,false>, 768x768, per limb
NTT_TRAFFIC_PER_XFORM = {"forward": (167.93e6 + 110.85e6 + 188.73e6 + 108.05e6) / 320,
                         "inverse": (188.73e6 + 108.17e6 + 167.94e6 + 108.42e6) / 320}
MODUP_TRAFFIC_PER_POLY = (100.73e6 + 94.82e6) / 8
# FP64 instructions per 16 values of a whole transform of 16 stages on the FP64 back end (8 per forward butterfly:
# six for the exact product, an add and a subtract; a three-operation range reduction on five of the stages; one
# conversion in, one out; the inverse reduces its sums on ten of fifteen stages and pays two products per
# butterfly in the last one), and the rate one SM sub-partition issues them at (measured with eight independent
# fma chains per warp: 0.46 warp instructions per clock, 59 lanes per clock per SM).
NTT_FP64_PER_16 = {"forward": 1176, "inverse": 1344}
FP64_WARP_INSTR_PER_CLK_PER_SMSP = 0.46


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"],
                    bf16_tflops_sustained=d.get("bf16_tflops_sustained", d["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


def bind_to_gpu_cpus(gpu_index):
    """With several ranks on one host, keep this rank's threads, and with them the pinned staging buffers it is about to
    allocate, on the CPUs NVML lists as close to its GPU, so that host copies do not cross sockets.  Reads only; returns
    the number of CPUs bound to, or None when the affinity is unknown."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(gpu_index)
        words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(h, words)
        cpus = {64 * w + b for w, m in enumerate(mask) for b in range(64) if (m >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
            return len(cpus)
    except Exception:
        pass
    return None


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        sm, smax, reasons = [], None, set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax = float(f[2])
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": smax,
                "reasons": sorted(reasons), "samples": len(sm)}


def pcmm_inputs(torch, device, seed):
    from ckks_llm_b200 import params
    c = PCMM_CFG
    q = params.ntt_primes(c["q_bits"], 2 << c["logN"], c["limbs"])
    Cw = (c["rank"] + 1) * c["N1"]
    g = torch.Generator(device=device).manual_seed(seed)
    X = torch.empty((c["K"], c["limbs"], Cw), dtype=torch.int64, device=device)
    for i, qi in enumerate(q):
        X[:, i, :] = torch.randint(0, qi, (c["K"], Cw), generator=g, device=device, dtype=torch.int64)
    W = (torch.randn((c["M"], c["K"]), generator=g, device=device, dtype=torch.float32) * c["w_std"])
    return q, X, W, Cw


def cpu_pcmm_sample(q, X, W, Cw, rows=128, cols=16384):
    """Oracle PPMM on `rows` output rows x `cols` columns x all limbs of the same workload."""
    from oracle import oracle as O
    O.set_threads(os.cpu_count() or 1)
    c = PCMM_CFG
    Xs = np.ascontiguousarray(X[:, :, :cols].cpu().numpy().view(np.uint64))
    Wh = W.cpu().numpy()
    t0 = time.perf_counter()
    res = O.ppmm(Wh, Xs, q, c["scaler"], m0=0, m1=rows)
    dt = time.perf_counter() - t0
    frac_rows = rows * (cols / Cw)           # ct-rows worth of work
    return (frac_rows / dt, dt, O.num_threads(), f"{rows} rows x {cols} of {Cw} columns x {c['limbs']} limbs, K={c['K']}",
            res[:rows])


def ccmm_side(path):
    """python/ccmm.py of the reference, run as it is and timed by wall clock.  It simulates a rotation-based
    ciphertext-ciphertext matrix multiply on plaintext integers (python/ccmm.py:144-336): a different algorithm from the
    PCMM benched here, reported as a labelled side number only.  The file is not part of this repository; without a path
    to it the entry says so."""
    label = "plaintext CCMM simulation, not PCMM"
    if not path or not os.path.exists(path):
        return {"label": label, "unavailable": "python/ccmm.py of the reference is not on this box (pass --ccmm PATH where it is)"}
    t0 = time.perf_counter()
    r = subprocess.run([sys.executable, path], capture_output=True, text=True, cwd=os.path.dirname(path) or ".")
    return {"label": label, "seconds": time.perf_counter() - t0, "exit": r.returncode, "cores": 1,
            "what": "python ccmm.py as shipped (NumPy, one process)"}


def run_reference(args):
    """The reference has no CPU implementation of this path and its CUDA build needs NTL;
    the CPU restatement (oracle/) is timed instead, on all host threads, on a bounded
    sample of the same workload per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from ckks_llm_b200 import params
    from oracle import oracle as O
    O.set_threads(os.cpu_count() or 1)       # torchrun exports OMP_NUM_THREADS=1 to its workers
    c = PCMM_CFG
    if args.workload == "pcmm":
        q = params.ntt_primes(c["q_bits"], 2 << c["logN"], c["limbs"])
        Cw = (c["rank"] + 1) * c["N1"]
        rows, cols = 128, 16384
        rng = np.random.default_rng(0)
        Xs = np.stack([np.stack([rng.integers(0, qi, cols, dtype=np.uint64) for qi in q]) for _ in range(c["K"])])
        Wh = (rng.standard_normal((c["M"], c["K"])) * c["w_std"]).astype(np.float32)
        times = []
        for it in range(args.warmup + args.steps):
            t0 = time.perf_counter()
            O.ppmm(Wh, Xs, q, c["scaler"], m0=0, m1=rows)
            if it >= args.warmup:
                times.append(time.perf_counter() - t0)
        dt = float(np.mean(times))
        value = rows * (cols / Cw) / dt
        metric, unit = "pcmm_ct_rows_per_sec", "ct-rows/s"
        sample = f"{rows} rows x {cols} of {Cw} columns x {c['limbs']} limbs, K={c['K']} per step"
        workload = PCMM_WORKLOAD
    else:
        n = NTT_CFG
        N = 1 << n["logN"]
        q = params.ntt_primes(n["q_bits"], 2 * N, n["limbs"])
        T = O.NttTables(N, q)
        rng = np.random.default_rng(0)
        polys = 2
        data = np.stack([np.stack([rng.integers(0, qi, N, dtype=np.uint64) for qi in q]) for _ in range(polys)])
        times = []
        for it in range(args.warmup + args.steps):
            t0 = time.perf_counter()
            O.ntt_batch(data, T, 0, 0, polys, n["limbs"], n["limbs"], inverse=(it % 2 == 1))
            if it >= args.warmup:
                times.append(time.perf_counter() - t0)
        dt = float(np.mean(times))
        value = polys * n["limbs"] / dt
        metric, unit = "ntt_limb_xforms_per_sec", "limb-xforms/s"
        sample = f"{polys} polys x {n['limbs']} limbs per step"
        workload = "batched NTT N=2^16, 40x50-bit limbs"
    line = {
        "impl": "reference", "metric": metric, "value": value, "unit": unit, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "u64", "data": "synthetic",
        "config": {"workload": workload},
        "cpu_baseline": {"value": value, "unit": unit, "cores": O.num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "reference CUDA build needs NTL (absent) and the reference has no CPU path; the CPU restatement is timed",
    }
    print(json.dumps(line))


def bench_ntt(torch, device, steps, warmup, peaks):
    from ckks_llm_b200 import params
    from ckks_llm_b200.host import Context_23
    n = NTT_CFG
    N = 1 << n["logN"]
    q = params.ntt_primes(n["q_bits"], 2 * N, n["limbs"])
    ctx = Context_23(n["logN"], [], q, [], device=device.index)
    g = torch.Generator(device=device).manual_seed(1)
    data = torch.empty((n["polys"], n["limbs"], N), dtype=torch.int64, device=device)
    for i, qi in enumerate(q):
        data[:, i, :] = torch.randint(0, qi, (n["polys"], N), generator=g, device=device, dtype=torch.int64)
    xforms = n["polys"] * n["limbs"]
    res = {}
    for name, fn in (("forward", ctx.ToNTTInplace), ("inverse", ctx.FromNTTInplace)):
        for _ in range(warmup):
            fn(data, 0, 0, n["polys"], n["limbs"], n["limbs"])
        torch.cuda.synchronize(device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn(data, 0, 0, n["polys"], n["limbs"], n["limbs"])
        e1.record()
        torch.cuda.synchronize(device)
        ms = e0.elapsed_time(e1) / steps
        gbs = xforms * 16 * N / (ms * 1e-3) / 1e9
        # what the FP64 pipe alone allows at the maximum SM clock, as a fraction of the same HBM peak
        sm_clk = 1.965e9
        fp64_s = NTT_FP64_PER_16[name] / 16.0 * N / 32.0 * xforms / (FP64_WARP_INSTR_PER_CLK_PER_SMSP * 4 * 148 * sm_clk)
        res[name] = {"limb_xforms_per_sec": xforms / (ms * 1e-3), "ms_per_step": ms,
                     "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                  "frac": gbs / peaks["hbm_gbs"],
                                  "attainable_frac": min(0.5, xforms * 16 * N / fp64_s / 1e9 / peaks["hbm_gbs"]),
                                  "attainable_note": "the lower of 0.5 (two kernels: the data crosses HBM twice) and what the FP64 "
                                                     "pipe allows at %d FP64 instructions per 16 values and 0.46 warp instructions "
                                                     "per clock per scheduler at 1965 MHz (%.3f ms)" % (NTT_FP64_PER_16[name], fp64_s * 1e3),
                                  "traffic": NTT_TRAFFIC_PER_XFORM[name] * xforms,
                                  "traffic_note": "dram read+write of the two kernels in the ncu capture of 320 limb-transforms, scaled by units",
                                  "note": "two kernels per transform; achieved = 16*N bytes per limb-xform / time"}}
    ctx.close()
    res["config"] = {"workload": "batched NTT N=2^16, 40x50-bit limbs, 16 ciphertexts x 2 polys",
                     "bytes_resident": int(data.numel() * 8), "l2_policy": "inputs (671 MB) larger than L2"}
    return res


def bench_ntt_limb_sharded(torch, device, rank, world, dist, steps, warmup):
    """The same batch (32 polynomials x 40 limbs, one copy per rank, limb-major) with the LIMBS dealt to the ranks: every
    rank transforms its limbs of all polynomials, then the limbs are all-gathered over NCCL so that every rank holds the
    whole transformed batch (strong scaling; the exchange is what it costs)."""
    from ckks_llm_b200 import params, shard
    from ckks_llm_b200.host import Context_23
    n = NTT_CFG
    N = 1 << n["logN"]
    q = params.ntt_primes(n["q_bits"], 2 * N, n["limbs"])
    ctx = Context_23(n["logN"], [], q, [], device=device.index)
    g = torch.Generator(device=device).manual_seed(1)
    data = torch.empty((n["limbs"], n["polys"], N), dtype=torch.int64, device=device)     # [limb][poly][N]
    for i, qi in enumerate(q):
        data[i] = torch.randint(0, qi, (n["polys"], N), generator=g, device=device, dtype=torch.int64)
    ranges = shard.unit_ranges(n["limbs"], world)
    a, b = ranges[rank]

    def transform():
        for i in range(a, b):
            ctx.ToNTTInplace(data[i], 0, i, n["polys"], 1, 1)        # limb i of every polynomial: 32 limb-transforms

    def timed(fn):
        for _ in range(warmup):
            fn()
        dist.barrier()
        torch.cuda.synchronize(device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize(device)
        tt = torch.tensor([e0.elapsed_time(e1) / steps], device=device)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        return float(tt.item())

    ms_t = timed(transform)
    ms_g = timed(lambda: (transform(), shard.gather_limbs(data, ranges)))
    ctx.close()
    xf = n["polys"] * n["limbs"]
    return {"sharding": "limbs dealt to ranks, all polynomials on every rank; NCCL all-gather of the limbs afterwards",
            "transform_ms": ms_t, "with_gather_ms": ms_g, "limb_xforms_per_sec": xf / (ms_t * 1e-3),
            "limb_xforms_per_sec_with_gather": xf / (ms_g * 1e-3),
            "gather_bytes_received_per_rank": int(xf * N * 8 * (world - 1) / world)}


def bench_modup(torch, device, steps, warmup, peaks):
    from ckks_llm_b200 import params
    from ckks_llm_b200.host import Context_23
    m = MODUP_CFG
    N = 1 << m["logN"]
    p = params.ntt_primes(m["q_bits"] + 1, 2 * N, m["alpha"])
    q = params.ntt_primes(m["q_bits"], 2 * N, m["q_num"])
    t = params.ntt_primes(m["t_bits"], 2 * N, m["t_num"])
    ctx = Context_23(m["logN"], p, q, t, device=device.index)
    g = torch.Generator(device=device).manual_seed(2)
    inp = torch.empty((m["batch"], m["q_num"], N), dtype=torch.int64, device=device)
    for i, qi in enumerate(q):
        inp[:, i, :] = torch.randint(0, qi, (m["batch"], N), generator=g, device=device, dtype=torch.int64)
    blocks = m["q_num"] // m["alpha"]
    out = torch.empty((m["batch"], blocks, m["t_num"], N), dtype=torch.int64, device=device)
    for _ in range(warmup):
        ctx.modUpQjtoT_23(out, inp, m["q_num"] - 1, m["batch"])
    torch.cuda.synchronize(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        ctx.modUpQjtoT_23(out, inp, m["q_num"] - 1, m["batch"])
    e1.record()
    torch.cuda.synchronize(device)
    ms = e0.elapsed_time(e1) / steps
    bytes_per_poly = (m["q_num"] + blocks * m["t_num"]) * 8 * N
    gbs = m["batch"] * bytes_per_poly / (ms * 1e-3) / 1e9
    ctx.close()
    return {"polys_per_sec": m["batch"] / (ms * 1e-3), "ms_per_step": ms,
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": gbs / peaks["hbm_gbs"], "traffic": MODUP_TRAFFIC_PER_POLY * m["batch"],
                         "traffic_note": "dram read+write in the ncu capture of batch 8, scaled by units (part of the output was still dirty in L2)"},
            "config": {"workload": "ModUp N=2^16, 24x50-bit Q limbs in 3 digits -> 12x60-bit T limbs, batch 32",
                       "l2_policy": "input+output (1 GB) larger than L2"}}


def bench_levels(torch, device, steps, warmup, peaks):
    """Scheme_23::rescaleAndEqual and Bootstrapper::modUpQ0toQL on 16 ciphertexts of the BERT chain
    (N=2^16, 20 x 50-bit limbs): device time per ciphertext, with the bytes each must move."""
    from ckks_llm_b200 import capi, params
    from ckks_llm_b200.host import Context_23, _stream_ptr
    logN, limbs, cts = 16, 20, 16
    N = 1 << logN
    p = params.ntt_primes(51, 2 * N, 1)
    q = params.ntt_primes(50, 2 * N, limbs)
    ctx = Context_23(logN, p, q, [], device=device.index)
    g = torch.Generator(device=device).manual_seed(3)
    data = torch.empty((cts, 2, limbs, N), dtype=torch.int64, device=device)
    for i, qi in enumerate(q):
        data[:, :, i, :] = torch.randint(0, qi, (cts, 2, N), generator=g, device=device, dtype=torch.int64)
    L, st = limbs - 1, _stream_ptr(device)
    calls = {
        "rescale": (lambda c, s: capi.check(ctx.lib.ckks_b200_rescale(ctx._h, data[c].data_ptr(), L, L, s)),
                    (1 + 1 + 3 * L) * 2 * 8 * N, "INTT of the last limb, 19 reductions, 19 NTTs, combine"),
        "modup_q0_to_ql": (lambda c, s: capi.check(ctx.lib.ckks_b200_modup_q0_to_ql(ctx._h, data[c].data_ptr(), L, L, 1 << 10, s)),
                           (1 + 1 + L + 2 * (L + 1)) * 2 * 8 * N, "INTT of limb 0, 19 lifts, 20 NTTs"),
    }
    res = {}
    for name, (fn, bytes_per_ct, what) in calls.items():
        for _ in range(warmup):
            for c in range(cts):
                fn(c, st)
        torch.cuda.synchronize(device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            for c in range(cts):
                fn(c, st)
        e1.record()
        torch.cuda.synchronize(device)
        ms = e0.elapsed_time(e1) / (steps * cts)
        gbs = bytes_per_ct / (ms * 1e-3) / 1e9
        res[name] = {"ciphertexts_per_sec": 1e3 / ms, "ms_per_ciphertext": ms, "steps": what,
                     "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                  "frac": gbs / peaks["hbm_gbs"], "traffic": None,
                                  "note": "algorithmic bytes: every limb touched is read once and written once per step of the sandwich"}}
        # The calls are asynchronous and allocate nothing once warm, so a caller can record them in a CUDA graph:
        # the same 16 calls replayed as one graph take the host's launch cost out of the per-ciphertext time.
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                s_cap = _stream_ptr(device)
                for c in range(cts):
                    fn(c, s_cap)
            graph.replay()
            torch.cuda.synchronize(device)
            e0.record()
            for _ in range(steps):
                graph.replay()
            e1.record()
            torch.cuda.synchronize(device)
            gms = e0.elapsed_time(e1) / (steps * cts)
            res[name]["cuda_graph"] = {"ms_per_ciphertext": gms, "frac": bytes_per_ct / (gms * 1e-3) / 1e9 / peaks["hbm_gbs"]}
            del graph
        except Exception as ex:
            res[name]["cuda_graph"] = {"error": repr(ex)[:200]}
    # all 16 ciphertexts (one contiguous pool) through the batched entry points
    batched = {
        "rescale": lambda: capi.check(ctx.lib.ckks_b200_rescale_batch(ctx._h, data.data_ptr(), cts, L, L, st)),
        "modup_q0_to_ql": lambda: capi.check(ctx.lib.ckks_b200_modup_q0_to_ql_batch(ctx._h, data.data_ptr(), cts, L, L, 1 << 10, st)),
    }
    for name, fn in batched.items():
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize(device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize(device)
        bms = e0.elapsed_time(e1) / (steps * cts)
        bytes_per_ct = calls[name][1]
        res[name]["batched"] = {"ms_per_ciphertext": bms, "ciphertexts_per_sec": 1e3 / bms, "batch": cts,
                                "frac": bytes_per_ct / (bms * 1e-3) / 1e9 / peaks["hbm_gbs"]}
    ctx.close()
    res["config"] = {"workload": "level changes on 16 ciphertexts, N=2^16, 20x50-bit limbs, level 19",
                     "l2_policy": "16 ciphertexts (336 MB) larger than L2, visited round-robin"}
    return res


PCMM_SHAPES = {
    # BASELINE.json configs[3], second weight: 768 features in, 3072 out, same ciphertext set as the headline
    "pcmm-bert3072": dict(logN=16, N1=128, rank=512, M=3072, K=768, limbs=20, shard=1,
                          what="bert-base PCMM 3072x768 (W~N(0,0.02) at 2^40), 768 ciphertexts x 20 limbs x 65664 words"),
    # BASELINE.json configs[4]: one GPU's share (an eighth of the columns, all limbs) of the LLaMA-7B-shaped PCMM
    "pcmm-llama-shard": dict(logN=16, N1=2048, rank=32, M=4096, K=4096, limbs=24, shard=8,
                             what="LLaMA-7B PCMM 4096x4096 (W~N(0,0.02) at 2^40), 4096 ciphertexts x 24 limbs x 67584 words, "
                                  "columns [0, C/8) of every ciphertext: the share of one of 8 GPUs"),
    # the same column-sharded layout at a size that runs in seconds (512 x 512, four limbs): checks of the N > 1 path
    "pcmm-shard-mini": dict(logN=16, N1=2048, rank=32, M=512, K=512, limbs=4, shard=8,
                            what="column-sharded PCMM 512x512, 512 ciphertexts x 4 limbs x 67584 words"),
}


def bench_pcmm_shape(torch, device, steps, warmup, peaks, name, rank=0, world=1, dist=None):
    """Other PCMM shapes of the named configurations, through the same entry point as the headline.  A shape with
    shard > 1 is one PCMM split by column range: on one GPU it runs the share of one of `shard` GPUs, on N > 1 GPUs
    every rank runs its own range (strong scaling) and the NCCL gather of the output is timed beside it."""
    from ckks_llm_b200 import capi, params
    from ckks_llm_b200.host import MLWECiphertext, PCMM_Context, PCMM_Scheme
    c = PCMM_SHAPES[name]
    N = 1 << c["logN"]
    q = params.ntt_primes(50, 2 * N, c["limbs"])
    Cw = (c["rank"] + 1) * c["N1"]
    g = torch.Generator(device=device).manual_seed(6)
    X = torch.empty((c["K"], c["limbs"], Cw), dtype=torch.int64, device=device)
    for i, qi in enumerate(q):
        X[:, i, :] = torch.randint(0, qi, (c["K"], Cw), generator=g, device=device, dtype=torch.int64)
    W = torch.randn((c["M"], c["K"]), generator=g, device=device, dtype=torch.float32) * 0.02
    pc = PCMM_Context(c["N1"], c["rank"], [], q, device=device.index)
    sch = PCMM_Scheme(pc, algo=capi.PCMM_TENSOR)
    cts = [MLWECiphertext(c["N1"], c["limbs"] - 1, c["limbs"] - 1, c["rank"], 1.0, cipher=X[n].reshape(-1))
           for n in range(c["K"])]
    from ckks_llm_b200 import shard as sharding
    split = world if (world > 1 and c["shard"] > 1) else c["shard"]
    ranges = sharding.column_ranges(Cw, split)
    col_begin, col_end = ranges[rank if world > 1 and c["shard"] > 1 else 0]

    def step():
        return sch.PPMM(W, cts, c["M"], c["K"], c["N1"], c["K"], scaler=float(1 << 40), col_begin=col_begin, col_end=col_end,
                        copy_back=False)

    for _ in range(warmup):
        step()
    sch.check()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    mains, pres = [], []
    e0.record()
    for _ in range(steps):
        step()
        p_ms, m_ms = sch.last_timing()
        pres.append(p_ms)
        mains.append(m_ms)
    e1.record()
    torch.cuda.synchronize(device)
    sch.check()
    ms = e0.elapsed_time(e1) / steps
    gather_ms = None
    if world > 1 and c["shard"] > 1:
        tt = torch.tensor([ms], device=device)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms = float(tt.item())
        out_full = sch.ppmm_output[:c["M"] * c["limbs"] * Cw].view(c["M"], c["limbs"], Cw)
        sharding.gather_output(out_full, ranges, rows_per_step=256)            # warm-up of the collective
        torch.cuda.synchronize(device)
        dist.barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        sharding.gather_output(out_full, ranges, rows_per_step=256)
        g1.record()
        torch.cuda.synchronize(device)
        tt = torch.tensor([g0.elapsed_time(g1)], device=device)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        gather_ms = float(tt.item())
    fused = None
    if world > 1 and c["shard"] > 1:
        # Fused form: the multiply's epilogue stores every output word into the peers' buffers as well (plain peer
        # stores over NVLink), so after one launch per rank and a host barrier every rank holds the whole output.
        def checksums(t):
            flat = t.view(-1)
            return int(flat.sum().item()), int(flat[::4099].sum().item())
        want = checksums(out_full)                       # the NCCL-gathered output
        peers, bases = sharding.open_peer_buffers(sch.ppmm_output)
        pc.set_peer_outputs([peers[r] for r in sorted(peers)])
        out_full.zero_()
        torch.cuda.synchronize(device)
        dist.barrier()
        for _ in range(2):
            step()
        sch.check()
        dist.barrier()
        got = checksums(out_full)
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record()
        for _ in range(steps):
            step()
        f1.record()
        torch.cuda.synchronize(device)
        sch.check()
        tt = torch.tensor([f0.elapsed_time(f1) / steps], device=device)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        okt = torch.tensor([1 if got == want else 0], device=device)
        dist.all_reduce(okt, op=dist.ReduceOp.MIN)
        fused = {"ms": float(tt.item()), "ct_rows_per_sec": c["M"] / (float(tt.item()) * 1e-3),
                 "matches_nccl_gather": bool(okt.item()),
                 "note": "one launch per rank: every output word is stored locally and into every peer's buffer by the epilogue (whole rows as bulk copies)"}
        pc.set_peer_outputs([])
        dist.barrier()
        sharding.close_peer_buffers(device.index, bases)
    ops = 2.0 * SW * SC * c["M"] * c["K"] * (col_end - col_begin) * c["limbs"]
    main = float(np.mean(mains))
    achieved = ops / (main * 1e-3) / 1e12
    peak = 2.0 * peaks["bf16_tflops"]
    pc.close()
    res = {"ct_rows_per_sec": c["M"] / (ms * 1e-3), "ms_per_step": ms, "sharded": c["shard"] > 1,
           "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TOP/s (int8)", "frac": achieved / peak,
                        "traffic": None, "kernel": "pcmm_umma_kernel<5,7>", "kernel_ms": main, "prepass_ms": float(np.mean(pres))},
           "config": {"workload": c["what"], "columns": [int(col_begin), int(col_end)], "column_split": split,
                      "l2_policy": "ciphertext and output sets of tens of GB, far larger than L2"}}
    if gather_ms is not None:
        res["gather"] = {"ms": gather_ms, "bytes_received_per_rank": int(c["M"] * c["limbs"] * (Cw - (col_end - col_begin)) * 8),
                         "ct_rows_per_sec_with_gather": c["M"] / ((ms + gather_ms) * 1e-3),
                         "note": "NCCL all-gather of the output column ranges, after the multiply, not overlapped"}
        res["gather"]["fused_peer_stores"] = fused
    return res



LLAMA_JOB = dict(N1=2048, rank=32, M=4096, K=4096, limbs=24, split_one_gpu=8,
                 what="LLaMA-7B PCMM 4096x4096 (W~N(0,0.02) at 2^40), 4096 ciphertexts x 24 limbs x 67584 words, N=2^16, N1=2048, rank 32")


def bench_llama_job(torch, device, rank, world, dist, steps, small=False):
    """BASELINE configs[4] as one job: every rank holds the ciphertexts and multiplies its column range of all 4096 rows
    (all 24 limbs of a column stay on one GPU, so the fused rescale needs no exchange).  Timed: the whole job on one GPU
    (its columns in eight chunks), the sharded multiply alone, the multiply followed by an NCCL all-gather of the output
    (every rank ends with everything), and the multiply whose epilogue stores each output row straight into the buffer of
    the row's owner (every rank ends with all columns of its 1/N of the rows, the unit the packing step consumes).  The
    two ways of bringing the output together are compared word for word on every rank's own rows."""
    from ckks_llm_b200 import capi, params, shard as sharding
    from ckks_llm_b200.host import MLWECiphertext, PCMM_Context, PCMM_Scheme
    c = dict(LLAMA_JOB)
    if small:
        c.update(M=512, K=512, limbs=4)
    N = 1 << 16
    q = params.ntt_primes(50, 2 * N, c["limbs"])
    Cw = (c["rank"] + 1) * c["N1"]
    M, K, limbs = c["M"], c["K"], c["limbs"]
    torch.cuda.empty_cache()
    # ciphertexts + output + byte planes of one column chunk; every rank must have the room or all skip together
    need = 8 * limbs * Cw * (K + M) + limbs * (Cw // c["split_one_gpu"] + 64) * ((K + 63) // 64 * 64) * 8 + (1 << 30)
    roomy = torch.tensor([1 if torch.cuda.mem_get_info(device)[0] > need else 0], device=device)
    if world > 1:
        dist.all_reduce(roomy, op=dist.ReduceOp.MIN)
    if not bool(roomy.item()):
        return {"skipped": "a rank has less than %.0f GB of free device memory" % (need / 1e9)}
    g = torch.Generator(device=device).manual_seed(6)             # the same ciphertexts on every rank
    X = torch.empty((K, limbs, Cw), dtype=torch.int64, device=device)
    for i, qi in enumerate(q):
        X[:, i, :] = torch.randint(0, qi, (K, Cw), generator=g, device=device, dtype=torch.int64)
    W = torch.randn((M, K), generator=g, device=device, dtype=torch.float32) * 0.02
    pc = PCMM_Context(c["N1"], c["rank"], [], q, device=device.index)
    sch = PCMM_Scheme(pc, algo=capi.PCMM_TENSOR)
    sch.ppmm_output = torch.empty(M * limbs * Cw, dtype=torch.int64, device=device)
    out_full = sch.ppmm_output.view(M, limbs, Cw)
    cts = [MLWECiphertext(c["N1"], limbs - 1, limbs - 1, c["rank"], 1.0, cipher=X[n].reshape(-1)) for n in range(K)]
    scaler = float(1 << 40)
    sch.prepare_weights(W, M, K, scaler)                           # the weights of a layer are prepared once

    def multiply(c0, c1):
        sch.PPMM(None, cts, M, K, c["N1"], K, scaler=scaler, col_begin=c0, col_end=c1, copy_back=False)

    def timed(fn, n):
        fn()
        torch.cuda.synchronize(device)
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize(device)
        ms = e0.elapsed_time(e1) / n
        if world > 1:
            tt = torch.tensor([ms], device=device)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            ms = float(tt.item())
        return ms

    n = max(1, min(steps, 3))
    one_ranges = sharding.column_ranges(Cw, c["split_one_gpu"])
    one_gpu_ms = timed(lambda: [multiply(a, b) for a, b in one_ranges], 1 if world > 1 else n)
    res = {"job": c["what"] if not small else "column-sharded PCMM 512x512, 4 limbs (small case)", "ranks": world,
           "one_gpu_ms": one_gpu_ms, "one_gpu_ct_rows_per_sec": M / (one_gpu_ms * 1e-3),
           "one_gpu_note": "all columns on one GPU in eight chunks (on N > 1 ranks every rank runs it at the same time; the slowest counts)"}
    int8_ops = 2.0 * SW * SC * M * K * Cw * limbs
    res["one_gpu_frac_of_int8_peak"] = int8_ops / (one_gpu_ms * 1e-3) / 1e12 / (2.0 * measured_peaks()["bf16_tflops"])
    sch.check()
    if world > 1:
        ranges = sharding.column_ranges(Cw, world)
        c0, c1 = ranges[rank]
        res["multiply_ms"] = timed(lambda: multiply(c0, c1), n)
        # (1) multiply, then NCCL all-gather of the column ranges: every rank ends with the whole output
        def mult_gather():
            multiply(c0, c1)
            sharding.gather_output(out_full, ranges, rows_per_step=256)
        res["with_gather_ms"] = timed(mult_gather, 1)
        r0, r1 = pc.row_owner_range(M, world, rank)

        def checksums():
            mine = out_full[r0:r1].reshape(-1)
            return [int(mine.sum().item()), int(mine[::4099].sum().item()), int(mine[::65537].sum().item())]
        want = checksums()
        # (2) the epilogue stores every row into its owner's buffer only (plain peer stores over NVLink)
        peers, bases = sharding.open_peer_buffers(sch.ppmm_output)
        out_full[r0:r1].zero_()
        torch.cuda.synchronize(device)
        dist.barrier()
        pc.set_row_owners([peers.get(r, 0) for r in range(world)], rank)
        res["with_row_scatter_ms"] = timed(lambda: multiply(c0, c1), n)
        sch.check()
        dist.barrier()
        got = checksums()
        ok = torch.tensor([1 if got == want else 0], device=device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        res["outputs_match"] = bool(ok.item())
        pc.set_row_owners([], 0)
        dist.barrier()
        sharding.close_peer_buffers(device.index, bases)
        res["speedup_vs_one_gpu"] = one_gpu_ms / res["with_row_scatter_ms"]
        res["speedup_multiply_only"] = one_gpu_ms / res["multiply_ms"]
        res["speedup_with_gather"] = one_gpu_ms / res["with_gather_ms"]
        res["ct_rows_per_sec"] = M / (res["with_row_scatter_ms"] * 1e-3)
        res["bytes_sent_per_rank"] = {"row_scatter": int((M - (r1 - r0)) * limbs * (c1 - c0) * 8),
                                      "all_gather_received": int(M * limbs * (Cw - (c1 - c0)) * 8)}
        res["note"] = ("speedup_vs_one_gpu counts the multiply with the row scatter fused into it: afterwards every rank holds "
                       "all columns of its rows; with_gather_ms is the multiply plus NCCL's all-gather (every rank holds everything)")
    else:
        res["multiply_ms"] = one_gpu_ms
        res["speedup_vs_one_gpu"] = 1.0
    pc.close()
    del cts, X, out_full
    sch.ppmm_output = None
    torch.cuda.empty_cache()
    return res

def bench_pcmm_from_rlwe(torch, device, steps, warmup, sch, pc, cts, W, q, ppmm_ms):
    """The pipeline's pair of calls (Bert.cuh:249-254: rlweCipherDecompose of two ciphertexts into 512 + 256 MLWE
    ciphertexts, then PPMM) at the headline shape, as two steps and as the one call whose slicing pre-pass reads the
    RLWE ciphertexts through the decomposition's index map.  Coefficient-domain sources (the transforms around the
    decomposition are the same in both forms and are left out).  The two outputs are compared word for word."""
    from ckks_llm_b200.host import Ciphertext, Context_23
    from ckks_llm_b200 import params
    c = PCMM_CFG
    N, L = 1 << c["logN"], c["limbs"] - 1
    ctx = Context_23(c["logN"], [params.ntt_primes(51, 2 * N, 1)[0]], list(q), [], device=device.index)
    sch.context = ctx
    g = torch.Generator(device=device).manual_seed(11)
    srcs = []
    for _ in range(2):
        rl = torch.empty((2, L + 1, N), dtype=torch.int64, device=device)
        for i, qi in enumerate(q):
            rl[:, i, :] = torch.randint(0, qi, (2, N), generator=g, device=device, dtype=torch.int64)
        srcs.append(Ciphertext(N, L, L, N // 2, 1.0, device=device.index, cipher=rl.reshape(-1)))
    sources = [(srcs[0], 512, 0), (srcs[1], 256, 512)]

    def timed(fn):
        for _ in range(max(warmup, 1)):
            fn()
        torch.cuda.synchronize(device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize(device)
        return e0.elapsed_time(e1) / steps

    def one_call():
        return sch.decomposeAndPPMM(W, sources, cts, c["M"], c["K"], c["N1"], c["K"], scaler=c["scaler"], ntt_domain=False,
                                    copy_back=False)

    def decompose():
        for ct, num, off in sources:
            sch.rlweCipherDecompose(ct, cts, num, off, ntt_domain=False)

    one_ms = timed(one_call)
    pre_ms, main_ms = sch.last_timing()
    got = one_call().clone()
    dec_ms = timed(decompose)
    two = sch.PPMM(W, cts, c["M"], c["K"], c["N1"], c["K"], scaler=c["scaler"], copy_back=False)
    sch.check()
    same = bool(torch.equal(got, two))
    del got
    ctx.close()
    sch.context = None
    return {"one_call_ms": one_ms, "one_call_ct_rows_per_sec": c["M"] / (one_ms * 1e-3), "one_call_prepass_ms": pre_ms,
            "one_call_main_ms": main_ms, "decompose_ms": dec_ms, "ppmm_ms": ppmm_ms, "two_calls_ms": dec_ms + ppmm_ms,
            "outputs_identical": same,
            "note": "decompose writes and PPMM re-reads 8.07 GB of MLWE ciphertexts made from 42 MB; the one call does neither"}


def bench_ringpack(torch, device, steps, warmup, peaks):
    """rlweCipherDecompose and mlweCipherPacking at the BERT geometry the reference runs (N=2^16, N1=128, rank 512,
    two ring-pack limbs, one special prime): device time per call with the bytes each must move."""
    from ckks_llm_b200 import params
    from ckks_llm_b200.host import Ciphertext, Context_23, MLWECiphertext, PCMM_Context, PCMM_Scheme
    logN, N1, L = 16, 128, 1
    N, k = 1 << logN, (1 << logN) // N1
    q = params.ntt_primes(50, 2 * N, L + 1)
    p = [params.ntt_primes(51, 2 * N, 1)[0]]
    ctx = Context_23(logN, p, q, [], device=device.index)
    pc = PCMM_Context(N1, k, p, q, device=device.index)
    sch = PCMM_Scheme(pc, context=ctx)
    g = torch.Generator(device=device).manual_seed(5)
    rl = torch.empty((2, L + 1, N), dtype=torch.int64, device=device)
    for i, qi in enumerate(q):
        rl[:, i, :] = torch.randint(0, qi, (2, N), generator=g, device=device, dtype=torch.int64)
    ct = Ciphertext(N, L, L, N // 2, 1.0, device=device.index, cipher=rl.reshape(-1))
    mlwe = [MLWECiphertext(N1, L, L, k, 1.0, device=device.index) for _ in range(k)]
    keys = torch.empty((k, 2, 2, N), dtype=torch.int64, device=device)           # [k][a,b][p,q0][N]
    for i, m in enumerate([p[0], q[0]]):
        keys[:, :, i, :] = torch.randint(0, m, (k, 2, N), generator=g, device=device, dtype=torch.int64)
    sch.addRepakcingKey(keys.reshape(-1))
    out_ct = Ciphertext(N, L, 0, N // 2, 1.0, device=device.index)
    C = (k + 1) * N1
    calls = {
        # INTT and NTT of 2(L+1) limb-polynomials around the gather, k MLWE ciphertexts of (L+1)*C words written
        "rlwe_decompose": (lambda: sch.rlweCipherDecompose(ct, mlwe, k, 0),
                           (4 * 2 * (L + 1) * N + 2 * (L + 1) * N + k * (L + 1) * C) * 8),
        # embed k+1 polynomials over (p, q0); 2k forward transforms; keys 4kN words; 4 inverse; ModDown; 2 forward
        "mlwe_packing": (lambda: sch.mlweCipherPacking(out_ct, mlwe, k, 0),
                         (k * C + 2 * (k + 1) * N + 2 * 2 * k * N + 2 * k * N + 4 * k * N + 4 * 2 * N + 4 * N + 2 * 2 * N) * 8),
    }
    res = {}
    for name, (fn, nbytes) in calls.items():
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize(device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize(device)
        ms = e0.elapsed_time(e1) / steps
        gbs = nbytes / (ms * 1e-3) / 1e9
        res[name] = {"calls_per_sec": 1e3 / ms, "ms_per_call": ms,
                     "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                  "frac": gbs / peaks["hbm_gbs"], "traffic": None,
                                  "note": "algorithmic bytes: every stage reads its inputs and writes its outputs once"}}
    pc.close()
    ctx.close()
    res["config"] = {"workload": "ring packing N=2^16, N1=128, rank 512, 2 limbs + 1 special prime, 512 MLWE ciphertexts",
                     "l2_policy": "MLWE set 538 MB and keys 1.07 GB, larger than L2"}
    return res


def bench_keyswitch(torch, device, steps, warmup, peaks):
    """The key-switch chain (ckks_b200_keyswitch) on the ModUp configuration's moduli: N=2^16, 24 x 50-bit q,
    8 special primes (dnum 3), 12 x 60-bit t, gamma 6, top level: device time per switched polynomial."""
    from ckks_llm_b200 import params
    from ckks_llm_b200.host import Context_23
    logN, K, qn, T, gamma = 16, 8, 24, 12, 6
    N, l = 1 << logN, qn - 1
    p = params.ntt_primes(51, 2 * N, K)
    q = params.ntt_primes(50, 2 * N, qn)
    t = params.ntt_primes(60, 2 * N, T)
    ctx = Context_23(logN, p, q, t, device=device.index, gamma=gamma)
    R = (K + qn + gamma - 1) // gamma
    cb, blocks, dnum = (l + 1 + K - 1) // K, (K + l + 1 + gamma - 1) // gamma, qn // K
    g = torch.Generator(device=device).manual_seed(4)
    inp = torch.empty((qn, N), dtype=torch.int64, device=device)
    for i, qi in enumerate(q):
        inp[i] = torch.randint(0, qi, (N,), generator=g, device=device, dtype=torch.int64)
    swk = torch.empty((2 * dnum * R, T, N), dtype=torch.int64, device=device)
    for k, tk in enumerate(t):
        swk[:, k, :] = torch.randint(0, tk, (2 * dnum * R, N), generator=g, device=device, dtype=torch.int64)
    out = torch.empty((2, qn, N), dtype=torch.int64, device=device)
    for _ in range(warmup):
        ctx.keyswitch(out, inp, swk, l)
    torch.cuda.synchronize(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        ctx.keyswitch(out, inp, swk, l)
    e1.record()
    torch.cuda.synchronize(device)
    ms = e0.elapsed_time(e1) / steps
    graph_info = None
    try:                                                        # the same chain recorded once and replayed as a CUDA graph
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            ctx.keyswitch(out, inp, swk, l)
        graph.replay()
        torch.cuda.synchronize(device)
        e0.record()
        for _ in range(steps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize(device)
        graph_info = {"ms_per_switch": e0.elapsed_time(e1) / steps}
        del graph
    except Exception as ex:
        graph_info = {"error": repr(ex)[:200]}
    limb_polys = (2 * (l + 1)                                   # copy of the input
                  + 2 * (l + 1) + (l + 1) + cb * T + 2 * cb * T  # INTT, ModUp to T, NTT over T
                  + cb * T + 2 * cb * blocks * T + 2 * blocks * T  # external product: digits, key, output
                  + 4 * blocks * T                               # INTT over T
                  + 2 * blocks * T + 2 * (K + l + 1)             # T -> [p | q]
                  + 2 * (K + l + 1) + 2 * (l + 1)                # ModDown
                  + 4 * (l + 1))                                 # NTT
    gbs = limb_polys * 8 * N / (ms * 1e-3) / 1e9
    ctx.close()
    return {"switches_per_sec": 1e3 / ms, "ms_per_switch": ms, "cuda_graph": graph_info,
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": gbs / peaks["hbm_gbs"], "traffic": None,
                         "note": "algorithmic bytes: every stage reads its inputs and writes its outputs once; the key is %d MB"
                                 % (2 * dnum * R * T * N * 8 // 2**20)},
            "config": {"workload": "key-switch chain N=2^16, 24x50-bit q, 8 p, 12x60-bit t, gamma 6, level 23",
                       "l2_policy": "the key alone (216 MB) is larger than L2"}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", choices=["pcmm", "ntt", "modup", "keyswitch", "ringpack", "pcmm-bert3072", "pcmm-llama-shard", "pcmm-shard-mini"], default="pcmm")
    ap.add_argument("--impl", choices=["b200", "reference"], default="b200")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--ccmm", default=None, help="path of the reference's python/ccmm.py, timed as a labelled side number")
    ap.add_argument("--host-chunks", type=int, default=0, help="column chunks of the host-buffer call (0 = the library's choice)")
    ap.add_argument("--no-side", action="store_true", help="skip the side measurements (NTT, ModUp, ..., the sharded LLaMA-shaped job)")
    ap.add_argument("--only-rlwe-side", action="store_true",
                    help="of the side measurements run only the decompose-and-multiply comparison (profiling)")
    ap.add_argument("--small", action="store_true",
                    help="profiling-sized case: PCMM with 2 limbs, NTT with 8 polys, ModUp batch 8 (not a bench value)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    if args.small:
        PCMM_CFG["limbs"] = 2
        NTT_CFG["polys"] = 8
        MODUP_CFG["batch"] = 8

    if args.impl == "reference":
        run_reference(args)
        return

    import torch
    import torch.distributed as dist
    from ckks_llm_b200 import capi
    from ckks_llm_b200.host import MLWECiphertext, PCMM_Context, PCMM_Scheme

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: this library has no CPU path")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    numa = bind_to_gpu_cpus(local_rank) if world > 1 else None
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    capi.load()
    peaks = measured_peaks()
    launches0 = capi.load().ckks_b200_kernel_launches()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    c = PCMM_CFG
    extra = {}
    if args.workload == "pcmm":
        q, X, W, Cw = pcmm_inputs(torch, device, seed=rank)
        pc = PCMM_Context(c["N1"], c["rank"], [], q, device=local_rank)
        sch = PCMM_Scheme(pc, algo=capi.PCMM_TENSOR)
        cts = [MLWECiphertext(c["N1"], c["limbs"] - 1, c["limbs"] - 1, c["rank"], 1.0, cipher=X[n].reshape(-1))
               for n in range(c["K"])]

        def step():
            return sch.PPMM(W, cts, c["M"], c["K"], c["N1"], c["K"], scaler=c["scaler"], copy_back=False)

        for _ in range(args.warmup):
            step()
        sch.check()
        sampler = ClockSampler(local_rank)
        barrier()
        if rank == 0:
            sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        main_ms, pre_ms = [], []
        l_before = capi.load().ckks_b200_kernel_launches()
        e0.record()
        for _ in range(args.steps):
            step()
            p_ms, m_ms = sch.last_timing()
            pre_ms.append(p_ms)
            main_ms.append(m_ms)
        e1.record()
        l_after = capi.load().ckks_b200_kernel_launches()
        barrier()
        clocks = sampler.stop() if rank == 0 else None
        sch.check()
        ms = e0.elapsed_time(e1) / args.steps
        if world > 1:
            tt = torch.tensor([ms], device=device)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            ms = float(tt.item())
        launches_timed = int(l_after - l_before)
        value = world * c["M"] / (ms * 1e-3)
        macs = c["M"] * c["K"] * Cw * c["limbs"]
        int8_ops = 2.0 * SW * SC * macs
        main = float(np.mean(main_ms))
        achieved = int8_ops / (main * 1e-3) / 1e12
        peak = 2.0 * peaks["bf16_tflops"]
        roof = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TOP/s (int8)", "frac": achieved / peak,
                "traffic": PCMM_TRAFFIC_PER_LIMB * c["limbs"],
                "traffic_note": "dram read+write of the ncu capture of the 2-limb case, scaled by the limb count",
                "kernel": "pcmm_umma_kernel<5,7>", "kernel_ms": main, "prepass_ms": float(np.mean(pre_ms)),
                "peak_source": f"2 x bf16 dense {peaks['bf16_tflops']} TFLOP/s ({peaks['source']}); int8 dense is nominally 2x bf16",
                "algorithmic_ops": "2*5*7 int8 ops per modular MAC x M*K*(N+N1)*limbs",
                "frac_of_sustained_peak": achieved / (2.0 * peaks["bf16_tflops_sustained"]),
                "peak_note": "frac is against the burst figure, the stricter of the two; the kernel runs under sw_power_cap "
                             "for most of its 17 ms, where the sustained figure is the like-for-like one"}
        if rank == 0 and world == 1 and not args.no_side:
            extra["pcmm_from_rlwe"] = bench_pcmm_from_rlwe(torch, device, args.steps, args.warmup, sch, pc, cts, W, q, ms)
        metric, unit = "pcmm_ct_rows_per_sec", "ct-rows/s"
        workload = PCMM_WORKLOAD
        cfg = {"workload": workload, "tokens_per_gpu": c["N1"], "sharding": "one 128-token block per GPU, no collective",
               "l2_policy": "inputs (8.07 GB ciphertext + 8.07 GB output) larger than L2"}

        e2e, cpu = None, None
        do_e2e = not args.no_e2e
        out_bytes = c["M"] * c["limbs"] * Cw * 8
        if do_e2e:
            # every rank needs pinned host memory for its result (and, on one GPU, for the MLWE form of the inputs too);
            # skip (and say so) if the host cannot give it
            try:
                import psutil
                need = (out_bytes + (X.numel() * 8 if world == 1 else 0)) * world * 1.25
                if psutil.virtual_memory().available < need:
                    do_e2e = False
            except ImportError:
                pass
            if world > 1:
                flag = torch.tensor([1 if do_e2e else 0], device=device)
                dist.all_reduce(flag, op=dist.ReduceOp.MIN)
                do_e2e = bool(flag.item())
        if do_e2e:
            L = capi.load()
            n_e2e = max(1, min(args.steps, 3))
            Wh = W.cpu().pin_memory()
            outh = torch.empty((c["M"], c["limbs"], Cw), dtype=torch.int64).pin_memory()
            if args.host_chunks:
                pc.set_host_chunks(args.host_chunks)

            def timed_host(fn):
                fn()
                barrier()
                t0 = time.perf_counter()
                for _ in range(n_e2e):
                    fn()
                barrier()
                dt = (time.perf_counter() - t0) / n_e2e
                if world > 1:
                    tt = torch.tensor([dt], device=device, dtype=torch.float64)
                    dist.all_reduce(tt, op=dist.ReduceOp.MAX)
                    dt = float(tt.item())
                return dt

            e2e_mlwe = None
            if world == 1:
                # (a) the multiply's own entry point with HOST buffers: the 768 MLWE ciphertexts (8.07 GB) go in
                Xh = torch.empty(X.shape, dtype=torch.int64).pin_memory()
                Xh.copy_(X)
                del cts, X
                sch.ppmm_output = None
                torch.cuda.empty_cache()
                dt = timed_host(lambda: capi.check(L.ckks_b200_pcmm_ppmm_host(
                    pc._h, Wh.data_ptr(), Xh.data_ptr(), outh.data_ptr(), c["M"], c["K"], c["N1"], c["K"], c["scaler"], capi.PCMM_TENSOR)))
                e2e_mlwe = {"value": c["M"] / dt, "unit": unit, "h2d_bytes_per_step": int(Xh.numel() * 8 + Wh.numel() * 4),
                            "d2h_bytes_per_step": int(outh.numel() * 8), "ms_per_step": dt * 1e3, "steps": n_e2e,
                            "call": "ckks_b200_pcmm_ppmm_host (MLWE ciphertexts in pinned host buffers)"}
                if rank == 0 and not args.no_cpu:
                    rows_s, cols_s = 128, 16384
                    Xd = Xh[:, :, :cols_s].contiguous()
                    v, dt_cpu, cores, sample, ref_words = cpu_pcmm_sample(q, Xd, Wh, Cw, rows_s, cols_s)
                    cpu = {"value": v, "unit": unit, "cores": cores, "kind": "port", "sample": sample, "seconds": dt_cpu,
                           "ccmm_side": ccmm_side(args.ccmm)}
                    # the same sample doubles as the parity check of the benched configuration at its full limb count:
                    # the words the timed host-buffer call just produced against the CPU restatement, every one of them
                    gpu_words = outh[:rows_s, :, :cols_s].numpy().view(np.uint64)
                    equal = bool(np.array_equal(gpu_words, ref_words))
                    cfg["parity"] = {"rows": rows_s, "cols": cols_s, "limbs": c["limbs"], "equal": equal,
                                     "against": "CPU restatement of the reference kernel (oracle/), same inputs"}
                    if not equal:
                        bad = int((gpu_words != ref_words).sum())
                        raise SystemExit(f"parity failure: {bad} of {ref_words.size} words of the benched multiply differ from the oracle")
                del Xh
            else:
                del cts, X
                sch.ppmm_output = None
                torch.cuda.empty_cache()
            # (b) the reference's pair of calls, rlweCipherDecompose x2 + PPMM (Bert.cuh:249-254), as one call with HOST
            # buffers: the two RLWE ciphertexts (42 MB) go in, the same 768 x 20-limb product comes out.  This is the
            # end-to-end figure: what a caller of the pipeline step pays.
            N_, L_ = 1 << c["logN"], c["limbs"] - 1
            gsrc = torch.Generator().manual_seed(1000 + rank)
            srcs = []
            for _ in range(2):
                rl = torch.empty((2, L_ + 1, N_), dtype=torch.int64)
                for i, qi in enumerate(q):
                    rl[:, i, :] = torch.randint(0, qi, (2, N_), generator=gsrc, dtype=torch.int64)
                srcs.append(rl.pin_memory())
            arr = (capi.RlweSource * 2)()
            for kx, (rl, num, off) in enumerate(((srcs[0], 512, 0), (srcs[1], 256, 512))):
                arr[kx].d_rlwe, arr[kx].L, arr[kx].mlwe_num, arr[kx].offset = rl.data_ptr(), L_, num, off
            dt = timed_host(lambda: capi.check(L.ckks_b200_pcmm_ppmm_rlwe_host(
                pc._h, Wh.data_ptr(), arr, 2, outh.data_ptr(), c["M"], c["K"], c["N1"], c["K"], c["scaler"])))
            e2e = {"value": world * c["M"] / dt, "unit": unit,
                   "h2d_bytes_per_step": int(sum(r.numel() for r in srcs) * 8 + Wh.numel() * 4),
                   "d2h_bytes_per_step": int(outh.numel() * 8), "ms_per_step": dt * 1e3, "steps": n_e2e,
                   "call": "ckks_b200_pcmm_ppmm_rlwe_host (RLWE ciphertexts and weights in, product out, pinned host buffers, per rank)",
                   "cpus_bound_per_rank": numa, "mlwe_inputs": e2e_mlwe}
            # its words against the device-side call on the same sources (which the tests pin to the oracle)
            dsrc = [r.to(device) for r in srcs]
            for kx in range(2):
                arr[kx].d_rlwe = dsrc[kx].data_ptr()
            out_dev = torch.empty(c["M"] * c["limbs"] * Cw, dtype=torch.int64, device=device)
            capi.check(L.ckks_b200_pcmm_ppmm_rlwe(pc._h, W.data_ptr(), arr, 2, out_dev.data_ptr(), c["M"], c["K"], c["N1"], c["K"],
                                                  c["scaler"], 0, Cw, None))
            sch.check()
            same = bool(torch.equal(out_dev.view(c["M"], c["limbs"], Cw), outh.to(device)))
            e2e["equals_device_call"] = same
            # what the bus alone takes for the result, on this host and into this buffer: the floor under ms_per_step
            flat = outh.view(-1)
            best = None
            for _ in range(3):
                torch.cuda.synchronize(device)
                t0 = time.perf_counter()
                flat.copy_(out_dev, non_blocking=True)
                torch.cuda.synchronize(device)
                dt_copy = time.perf_counter() - t0
                best = dt_copy if best is None or dt_copy < best else best
            e2e["copy_out_alone_ms"] = best * 1e3
            e2e["copy_out_alone_gbs"] = out_bytes / best / 1e9
            if not same:
                raise SystemExit("the host-buffer decompose-and-multiply call and the device call differ")
            del out_dev, dsrc, outh
        pc.close()
        torch.cuda.empty_cache()
        if rank == 0 and world == 1 and not args.no_side and not args.only_rlwe_side:
            try:
                extra["ntt"] = bench_ntt(torch, device, max(args.steps, 10), args.warmup, peaks)
                extra["modup"] = bench_modup(torch, device, max(args.steps, 10), args.warmup, peaks)
                extra["levels"] = bench_levels(torch, device, max(args.steps, 10), args.warmup, peaks)
                extra["keyswitch"] = bench_keyswitch(torch, device, max(args.steps, 10), args.warmup, peaks)
                extra["ringpack"] = bench_ringpack(torch, device, max(args.steps, 10), args.warmup, peaks)
                # the second metric and the ModUp figure inside the roofline object as well
                for key, src_ in (("ntt_fwd", extra["ntt"]["forward"]), ("ntt_inv", extra["ntt"]["inverse"])):
                    roof[key] = {"value": src_["limb_xforms_per_sec"], "unit": "limb-xforms/s", "ms": src_["ms_per_step"],
                                 "frac": src_["roofline"]["frac"], "attainable_frac": src_["roofline"]["attainable_frac"], "bound": "hbm"}
                roof["modup"] = {"value": extra["modup"]["polys_per_sec"], "unit": "polys/s", "ms": extra["modup"]["ms_per_step"],
                                 "frac": extra["modup"]["roofline"]["frac"], "bound": "hbm"}
            except Exception as ex:           # the headline stays valid without the side measurements
                extra["side_error"] = repr(ex)
        if not args.no_side and not args.only_rlwe_side:
            if world > 1:
                # the second metric at N ranks: every rank transforms its own 32 polynomials x 40 limbs (no exchange)
                r = bench_ntt(torch, device, max(args.steps, 10), args.warmup, peaks)
                nt = {}
                for name in ("forward", "inverse"):
                    tt = torch.tensor([r[name]["ms_per_step"]], device=device)
                    dist.all_reduce(tt, op=dist.ReduceOp.MAX)
                    ms_n = float(tt.item())
                    xf = NTT_CFG["polys"] * NTT_CFG["limbs"]
                    nt[name] = {"limb_xforms_per_sec": world * xf / (ms_n * 1e-3), "ms_per_step": ms_n,
                                "frac_per_gpu": xf * 16 * (1 << NTT_CFG["logN"]) / (ms_n * 1e-3) / 1e9 / peaks["hbm_gbs"]}
                nt["sharding"] = "each rank its own polynomials, no collective (weak scaling)"
                nt["limb_sharded"] = bench_ntt_limb_sharded(torch, device, rank, world, dist, max(args.steps, 10), args.warmup)
                cfg["ntt_ranks"] = nt
                roof["ntt_fwd"] = {"value": nt["forward"]["limb_xforms_per_sec"], "unit": "limb-xforms/s, all ranks", "ms": nt["forward"]["ms_per_step"],
                                   "frac": nt["forward"]["frac_per_gpu"], "bound": "hbm"}
                roof["ntt_inv"] = {"value": nt["inverse"]["limb_xforms_per_sec"], "unit": "limb-xforms/s, all ranks", "ms": nt["inverse"]["ms_per_step"],
                                   "frac": nt["inverse"]["frac_per_gpu"], "bound": "hbm"}
            cfg["llama_job"] = bench_llama_job(torch, device, rank, world, dist if world > 1 else None, args.steps, small=args.small)
    else:
        sampler = ClockSampler(local_rank)
        barrier()
        if rank == 0:
            sampler.start()
        if args.workload == "ntt":
            r = bench_ntt(torch, device, args.steps, args.warmup, peaks)
            ms = r["forward"]["ms_per_step"]
            value = world * r["forward"]["limb_xforms_per_sec"]
            roof = r["forward"]["roofline"]
            extra["ntt"] = r
            metric, unit, cfg = "ntt_limb_xforms_per_sec", "limb-xforms/s", r["config"]
        elif args.workload in PCMM_SHAPES:
            r = bench_pcmm_shape(torch, device, args.steps, args.warmup, peaks, args.workload, rank, world,
                                 dist if world > 1 else None)
            ms = r["ms_per_step"]
            # a column-sharded multiply is one job split over the ranks; independent replicas otherwise
            value = r["ct_rows_per_sec"] if r["sharded"] else world * r["ct_rows_per_sec"]
            roof = r["roofline"]
            if "gather" in r:
                extra["gather"] = r["gather"]
            metric, unit, cfg = "pcmm_ct_rows_per_sec", "ct-rows/s", r["config"]
        elif args.workload == "ringpack":
            r = bench_ringpack(torch, device, args.steps, args.warmup, peaks)
            ms = r["mlwe_packing"]["ms_per_call"]
            value = world * r["mlwe_packing"]["calls_per_sec"]
            roof = r["mlwe_packing"]["roofline"]
            extra["ringpack"] = r
            metric, unit, cfg = "mlwe_packings_per_sec", "packings/s", r["config"]
        elif args.workload == "keyswitch":
            r = bench_keyswitch(torch, device, args.steps, args.warmup, peaks)
            ms = r["ms_per_switch"]
            value = world * r["switches_per_sec"]
            roof = r["roofline"]
            metric, unit, cfg = "keyswitch_per_sec", "switches/s", r["config"]
        else:
            r = bench_modup(torch, device, args.steps, args.warmup, peaks)
            ms = r["ms_per_step"]
            value = world * r["polys_per_sec"]
            roof = r["roofline"]
            metric, unit, cfg = "modup_polys_per_sec", "polys/s", r["config"]
        barrier()
        clocks = sampler.stop() if rank == 0 else None
        launches_timed = None
        e2e, cpu = None, None

    if rank == 0:
        line = {"metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
                "scaling": "strong" if (args.workload in PCMM_SHAPES and PCMM_SHAPES[args.workload]["shard"] > 1 and world > 1) else "weak",
                "vs_baseline": None, "dtype": "u64 (int8 planes on tensor cores, s32 accumulate)" if args.workload == "pcmm" else "u64",
                "data": "synthetic", "config": dict(cfg, small=True) if args.small else cfg, "roofline": roof, "clocks": clocks,
                "gpu_launches": launches_timed if launches_timed is not None else int(capi.load().ckks_b200_kernel_launches() - launches0),
                "e2e": e2e, "cpu_baseline": cpu}
        line.update(extra)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
