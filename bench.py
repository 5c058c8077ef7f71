#!/usr/bin/env python
"""Benchmark of the accelerated path on N GPUs of one node.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload spmv|spmv1|spmm|pcg|bgemm|gemm]
                    [--impl ours|reference]

Default workload: CSR SpMV fp64 on the large skewed matrix (2^23 rows, power-law row
lengths with mean 16 capped at 4096, int64 offsets/indices, about 1.34e8 entries), rows
partitioned by nnz over the GPUs, x replicated.  A step is one y = A x pass.  The inputs
of a pass (2.35 GB; 0.29 GB per GPU at N = 8) are larger than the 126 MB L2, so no flush
is needed between timed iterations.

Prints ONE JSON line on rank 0.  `value` is the whole-job throughput with operands
resident in HBM (CUDA events around exactly K steps, barrier + synchronize on both
sides, max over ranks); `e2e` is the same metric through the package's public call with
pinned HOST buffers (host-to-device copies and the device-to-host copy of the result inside
the timed region); `roofline` relates the dominant kernel to the measured HBM copy
bandwidth; `cpu_baseline` is the CPU restatement of the reference's emitted loop timed on
this box's cores (rank 0, N = 1 only, before any CUDA context exists in the process);
`verified` says whether a sample of the last timed result matched the CPU oracle (checked
outside the timed region).  The default run also carries `secondary`: the other two thirds
of the headline metric -- PCG iterations/s on the 4096^2 Laplacian (row-partitioned over
the N GPUs, exchanges by stores into peer memory), the 8192^3 fp32 GEMM and the
4096 x 128^3 batched GEMM (split by batch) -- each a few hundred milliseconds.

`--impl reference` times the CPU restatement alone, with all host threads, on the same
configuration (the reference's own Kokkos build cannot be produced without LLVM/MLIR and
Kokkos, which are not available offline).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

# CPUs this process may use, read before any OpenMP runtime is loaded: with OMP_PROC_BIND set the runtime pins
# the initial thread to the first place, after which the process's own affinity mask shows one CPU only
try:
    _CPU_MASK = os.sched_getaffinity(0)
except Exception:
    _CPU_MASK = None
_CPUS_ALLOWED = len(_CPU_MASK) if _CPU_MASK else (os.cpu_count() or 1)
# The CPU restatement's OpenMP threads stay on their cores (read by the OpenMP runtime when it is loaded).  Only in
# a process that times the CPU restatement (one rank, or the reference arm): in a multi-rank job every rank's main
# thread would be pinned to the same first core.
if int(os.environ.get("WORLD_SIZE", "1")) == 1 or "reference" in sys.argv:
    os.environ.setdefault("OMP_PROC_BIND", "close")
    os.environ.setdefault("OMP_PLACES", "cores")


def release_main_thread():
    """Gives the main thread its original CPU mask back after the CPU timing (the OpenMP runtime pinned it)."""
    if _CPU_MASK:
        try:
            os.sched_setaffinity(0, _CPU_MASK)
        except Exception:
            pass


import numpy as np  # noqa: E402

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

FALLBACK_HBM_GBS = 6650.0
L2_NOTE = "inputs larger than L2, no flush between iterations"


# ---------------------------------------------------------------------------
# helpers
# ---------------------------------------------------------------------------
def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": FALLBACK_HBM_GBS, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """Samples SM clock, power draw and throttle reasons of one GPU while the timed region runs (read-only NVML)."""

    def __init__(self, index: int, period_s: float = 0.005):
        self.index, self.period = index, period_s
        self.samples, self.watts, self.reasons, self.max_mhz, self.limit_w = [], [], set(), None, None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nvml = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nvml = None
            return
        try:
            self.limit_w = pynvml.nvmlDeviceGetEnforcedPowerLimit(self._h) / 1000.0
        except Exception:
            pass

    def _loop(self):
        nv = self._nvml
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
            "hw_power_brake": getattr(nv, "nvmlClocksThrottleReasonHwPowerBrakeSlowdown", 0x80),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                self.watts.append(nv.nvmlDeviceGetPowerUsage(self._h) / 1000.0)
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            self._stop.wait(self.period)

    def start(self):
        if self._nvml is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples),
                "power_w": statistics.median(self.watts) if self.watts else None, "power_limit_w": self.limit_w}


def physical_cores() -> int:
    try:
        import psutil
        return psutil.cpu_count(logical=False) or os.cpu_count() or 1
    except Exception:
        return os.cpu_count() or 1


def host_threads() -> int:
    return max(1, min(_CPUS_ALLOWED, physical_cores()))


def oracle_native():
    """The CPU restatement built for this box's cores (falls back to the portable build)."""
    from oracle import oracle
    try:
        oracle.build(native=True)
        oracle.lib(native=True)
        return oracle, True
    except Exception:
        return oracle, False


# ---------------------------------------------------------------------------
# workloads: each returns host data + byte/flop accounting
# ---------------------------------------------------------------------------
def make_workload(name: str, small: bool, shrink: int = 0):
    from lapis_b200 import workloads as w
    if name == "spmv":
        d = w.spmv_power_law(1 << 16 if small else (1 << 23) >> shrink)
        n, nnz = d["shape"][0], int(d["crd"].size)
        d.update(unit="GB/s", metric="csr_spmv_hbm_gbs", dtype="f64", unit_scale=1e-9,
                 work=w.spmv_bytes(n, n, nnz, 8), label=f"CSR SpMV fp64 power-law rows (config 2): {n} rows, {nnz} nnz, int64 indices")
    elif name == "spmv1":
        d = w.spmv_uniform(10_000, 10, np.int64)
        n, nnz = d["shape"][0], int(d["crd"].size)
        d.update(unit="GB/s", metric="csr_spmv_hbm_gbs", dtype="f64", unit_scale=1e-9, work=w.spmv_bytes(n, n, nnz, 8),
                 label=f"CSR SpMV fp64 (config 1): {n} rows, 10 nnz/row, int64 indices; 1.84 MB, launch-latency bound")
    elif name == "spmm":
        d = w.spmm_uniform(1 << 13 if small else (1 << 21) >> shrink)
        n, nnz = d["shape"][0], int(d["crd"].size)
        d.update(unit="GB/s", metric="csr_spmm_hbm_gbs", dtype="f64", unit_scale=1e-9,
                 work=w.spmm_bytes(n, n, nnz, 64, 8), label=f"CSR SpMM fp64 (config 3): {n} rows, 32 nnz/row, k=64, int64 indices")
    elif name == "pcg":
        g = 256 if small else 4096 >> shrink
        d = w.pcg_laplacian(g)
        n, nnz = d["shape"][0], int(d["crd"].size)
        d.update(unit="it/s", metric="pcg_iterations_per_s", dtype="f64", unit_scale=1.0, work=1, grid=g,
                 bytes_per_step=w.pcg_bytes_per_iteration(n, nnz, 4),
                 label=f"PCG fp64, 5-point Laplacian {g}x{g} (config 5), Jacobi, int32 indices")
    elif name == "bgemm":
        b, m = (64, 128) if small else (4096, 128)
        d = w.batched_gemm(b, m)
        d.update(unit="TFLOP/s", metric="batched_gemm_fp32_tflops", dtype="f32 (3xTF32)", unit_scale=1e-12,
                 work=w.gemm_flops(b, m, m, m), bytes_per_step=w.gemm_bytes(b, m, m, m),
                 label=f"batched GEMM fp32 (config 4a): {b} x {m}^3")
    elif name == "gemm":
        m = 1024 if small else 8192
        d = w.dense_gemm(m)
        d.update(unit="TFLOP/s", metric="gemm_fp32_tflops", dtype="f32 (3xTF32)", unit_scale=1e-12,
                 work=w.gemm_flops(1, m, m, m), bytes_per_step=w.gemm_bytes(1, m, m, m),
                 label=f"GEMM fp32 (config 4b): {m}^3")
    else:
        raise SystemExit(f"unknown workload {name}")
    d["name"] = name
    return d


def config_for(d, world: int) -> dict:
    """The `config` object of the JSON line: identical in both arms for the same workload and N."""
    name = d["name"]
    cfg = {"workload": d["label"], "l2": L2_NOTE}
    if name in ("spmv", "spmv1"):
        cfg.update(partition="contiguous row blocks, equal nnz", replicated="x")
    elif name == "spmm":
        cfg.update(partition="contiguous row blocks, equal nnz", replicated="B")
    elif name == "pcg":
        cfg.update(partition="contiguous row blocks, equal nnz; halo of p and two scalar sums exchanged per iteration")
    elif name == "bgemm":
        cfg.update(partition="by batch")
    else:
        cfg.update(partition="replicas only (one problem per GPU)")
    cfg["ranks"] = world
    return cfg


# ---------------------------------------------------------------------------
# the CPU restatement on the host cores: shared by `cpu_baseline` of our arm and by the reference arm
# ---------------------------------------------------------------------------
def time_cpu(d, warmup: int, steps, min_seconds: float, budget_s: float):
    """Times the CPU restatement (OpenMP over rows / problems, threads pinned to cores) on a bounded sample of
    the workload.  steps = None: repeat until `min_seconds` have passed (at least three repetitions).  Returns
    value (median step, scaled to the metric's unit), median and mean milliseconds per step, and what the
    sample was."""
    oracle, native = oracle_native()
    threads = host_threads()
    name = d["name"]
    scale_note = ""
    if name in ("spmv", "spmv1", "spmm"):
        pos, crd, val = d["pos"], d["crd"], d["val"]
        n = len(pos) - 1

        def make_step(rows):
            p = np.ascontiguousarray(pos[:rows + 1])
            if name != "spmm":
                y = np.zeros(rows)
                return lambda: oracle.spmv_inplace(p, crd, val, d["x"], y, threads, native)
            C = np.zeros((rows, 64))
            return lambda: oracle.spmm_inplace(p, crd, val, d["B"], C, threads, native)

        rows = n
        step = make_step(rows)
        t0 = time.perf_counter()
        step()
        t1 = time.perf_counter() - t0
        est = t1 * ((steps or 3) + warmup)
        if est > budget_s:
            rows = max(1, int(n * budget_s / est))
            step = make_step(rows)
        frac = float(pos[rows]) / float(pos[n]) if pos[n] else 1.0
        work = d["work"] * frac
        sample = f"rows [0, {rows}) of {n} ({100 * frac:.1f}% of the entries) per step, x/B whole"
    elif name == "pcg":
        from lapis_b200 import workloads as w
        g_full = int(round(len(d["b"]) ** 0.5))
        g = g_full
        its = 5
        while True:
            dd = w.pcg_laplacian(g) if g != g_full else d
            t0 = time.perf_counter()
            oracle.pcg(dd["pos"], dd["crd"], dd["val"], dd["b"], dd["dinv"], 0.0, 2, threads, native=native)
            t1 = (time.perf_counter() - t0) / 2 * its
            if t1 * ((steps or 3) + warmup) <= budget_s or g <= 256:
                break
            g //= 2
        step = lambda: oracle.pcg(dd["pos"], dd["crd"], dd["val"], dd["b"], dd["dinv"], 0.0, its, threads, native=native)
        work = its * (g * g) / float(g_full * g_full)   # iterations rescaled by rows (bandwidth-bound)
        sample = f"{its} iterations per step on a {g}x{g} grid"
        if g != g_full:
            scale_note = f"; it/s scaled by rows to the {g_full}^2 grid"
    else:
        A, B = d["A"], d["B"]
        rate = 0.3e9 * max(1, threads)  # flop/s guess of the naive loop, only used to size the sample
        if A.ndim == 2:
            mm_ = A.shape[0]
            while 2.0 * mm_ ** 3 / rate * ((steps or 3) + warmup) > budget_s and mm_ > 256:
                mm_ //= 2
            A, B = np.ascontiguousarray(A[:mm_, :mm_]), np.ascontiguousarray(B[:mm_, :mm_])
            work = 2.0 * mm_ ** 3
            sample = f"{mm_}^3 sub-problem per step (naive loop order as emitted)"
        else:
            nb = A.shape[0]
            bb = nb
            while 2.0 * bb * A.shape[1] ** 3 / rate * ((steps or 3) + warmup) > budget_s and bb > 8:
                bb //= 2
            A, B = A[:bb], B[:bb]
            work = 2.0 * bb * A.shape[1] ** 3
            sample = f"{bb} of {nb} problems per step"
        C = np.zeros(A.shape[:-1] + (B.shape[-1],), dtype=np.float32)
        step = lambda: oracle.bgemm(A, B, C, threads, native)
    for _ in range(max(1, warmup)):
        step()
    times = []
    t_start = time.perf_counter()
    while True:
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
        if steps is not None:
            if len(times) >= steps:
                break
        elif len(times) >= 3 and (time.perf_counter() - t_start >= min_seconds or len(times) >= 200):
            break
    med = statistics.median(times)
    return {"value": work / med * d["unit_scale"], "unit": d["unit"], "cores": threads, "kind": "port",
            "sample": f"{sample}; {len(times)} timed steps, median{scale_note}; threads pinned (OMP_PROC_BIND=close, "
                      f"OMP_PLACES=cores); " + ("-march=native build" if native else "portable build"),
            "ms_per_step": med * 1e3, "ms_per_step_mean": statistics.fmean(times) * 1e3}


def run_reference(args, d):
    r = time_cpu(d, args.warmup, args.steps, 0.0, 120.0)
    line = {
        "impl": "reference", "metric": d["metric"], "value": r["value"], "unit": d["unit"], "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": d["dtype"].split(" ")[0], "data": "synthetic",
        "config": config_for(d, args.gpus),
        "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": r["value"], "unit": d["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "CPU restatement of the emitted Kokkos loops (OpenMP); the reference's own Kokkos build needs "
                "LLVM/MLIR and Kokkos, which are not available offline",
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------
# DRAM bytes per launch of the dominant kernel from the committed ncu captures under profiles/
# (dram__bytes_read.sum + dram__bytes_write.sum, scaled to a full launch by entries processed).
NCU_TRAFFIC = {
    "spmv_walk_kernel": 3.428e9,    # profiles/spmv_walk_kernel_config2.md
    "spmv_chunk_kernel": 3.325e9,   # profiles/spmv_chunk_kernel_config2.md
    "spmv_scan_kernel": 3.290e9,    # profiles/spmv_walk_kernel_config2.md (launch list of the tuner's candidates)
    "spmv_pipe_kernel": 3.160e9,    # same list
    "spmm": 3.387e10,               # profiles/spmm_row_kernel_config3.md
    "bgemm": 1.036e9,               # profiles/bgemm_tcgen05_kernel.md (4096 x 128^3)
    "gemm": 8.15e9,                 # profiles/bgemm_tcgen05_kernel.md (8192^3, K in segments of 1024)
    "pcg": 2.715e9,                 # profiles/pcg_iteration_config5.md (the three kernels of one iteration)
    "pcg_two_pass": 2.565e9,        # same file (the two kernels of one iteration)
}


class Harness:
    """Timing helpers bound to this rank's device and process group."""

    def __init__(self, rank, world, local_rank):
        import torch
        import torch.distributed as dist
        self.torch, self.dist = torch, dist
        self.rank, self.world, self.local_rank = rank, world, local_rank
        self.dev = torch.device(f"cuda:{local_rank}")
        torch.cuda.set_device(self.dev)
        self.peaks, self.peak_kind = measured_peaks()

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, v: float) -> float:
        if self.world == 1:
            return v
        t = self.torch.tensor([v], dtype=self.torch.float64, device=self.dev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def all_true(self, ok: bool) -> bool:
        if self.world == 1:
            return bool(ok)
        t = self.torch.tensor([1.0 if ok else 0.0], dtype=self.torch.float64, device=self.dev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MIN)
        return bool(t.item() > 0.5)

    def timed(self, step, steps, warmup):
        """CUDA events on the current stream around exactly `steps` steps; max over ranks; clocks sampled."""
        torch = self.torch
        for _ in range(warmup):
            step()
        self.barrier()
        sampler = ClockSampler(self.local_rank)
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        self.barrier()
        clocks = sampler.stop()
        return self.max_over_ranks(e0.elapsed_time(e1)), clocks

    def wall(self, step, steps):
        """Host clock around `steps` calls that each return with their result on the host; max over ranks."""
        if self.world > 1:
            self.dist.barrier()
        t0 = time.perf_counter()
        for _ in range(steps):
            step()
        return self.max_over_ranks(time.perf_counter() - t0)

    def hbm_roofline(self, algo_bytes_rank, kernel_ms, kernel, traffic):
        achieved = algo_bytes_rank / (kernel_ms * 1e-3) * 1e-9
        peak = float(self.peaks["hbm_gbs"])
        return {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": traffic, "kernel": kernel, "peak_source": f"{self.peak_kind} copy bandwidth",
                "algorithmic_bytes_per_launch": algo_bytes_rank, "frac_of_8TBs": achieved / 8000.0}

    def tensor_roofline(self, flops_rank, kernel_ms, kernel, traffic):
        # 3xTF32: three tensor-core products per fp32 product; dense TF32 peak taken as half the measured bf16 peak;
        # the kernel is timed alone over a few tens of milliseconds: the burst figure applies
        tf32_peak = float(self.peaks["bf16_tflops"]) / 2.0
        achieved = 3.0 * flops_rank / (kernel_ms * 1e-3) * 1e-12
        return {"bound": "tensor", "achieved": achieved, "peak": tf32_peak, "unit": "TFLOP/s", "frac": achieved / tf32_peak,
                "traffic": traffic, "kernel": kernel,
                "peak_source": f"{self.peak_kind} bf16 burst / 2 (TF32); achieved counts the 3 TF32 products per fp32 product"}


def spmv_kernel_name(tuned):
    t = tuned[0]
    return {4: "spmv_walk_kernel", 2: "spmv_scan_kernel", 3: "spmv_scan_kernel", 1: "spmv_rowthread_kernel"}.get(
        t, "spmv_pipe_kernel" if t < 0 else "spmv_chunk_kernel")


def sample_rows_csr(pos, crd, val, rows):
    """The sub-matrix made of the given rows (same column space), for a check against the oracle."""
    lens = (pos[rows + 1] - pos[rows]).astype(np.int64)
    spos = np.zeros(len(rows) + 1, dtype=pos.dtype)
    np.cumsum(lens, out=spos[1:])
    idx = np.concatenate([np.arange(int(pos[r]), int(pos[r + 1])) for r in rows]) if len(rows) else np.zeros(0, np.int64)
    return spos, np.ascontiguousarray(crd[idx]), np.ascontiguousarray(val[idx])


def run_sparse(args, d, hx: Harness):
    """SpMV (configs 1, 2) and SpMM (config 3): rows split by nnz over the ranks, x / B replicated."""
    import torch
    from oracle import oracle
    from lapis_b200 import KokkosBackend as KB
    from lapis_b200 import modules as mm
    from lapis_b200.dist import ShardedSpmv
    name, dev, world, rank = d["name"], hx.dev, hx.world, hx.rank
    pos, crd, val = d["pos"], d["crd"], d["val"]
    n = len(pos) - 1
    k = 64 if name == "spmm" else 1
    # per-matrix choice of the SpMV kernel; relaxed: the kernels that sum a row in scan order (within 1e-12 of the
    # others, the parity bar of this metric, but not their bits) are candidates
    sh = ShardedSpmv(pos, crd, val, (n, n), rank, world, dev, tune="relaxed" if name != "spmm" else "none")
    A, r0, r1 = sh.matrix, sh.r0, sh.r1
    tuned = A.tuned_kernel() if name != "spmm" else (0, 0)
    lnnz = int(pos[r1] - pos[r0])
    detail = {"rows_rank0": int(sh.bounds[1] - sh.bounds[0]), "spmv_kernel_tuned": list(tuned)}
    if name != "spmm":
        xd = torch.as_tensor(d["x"]).to(dev)
        yd = torch.zeros(r1 - r0, dtype=torch.float64, device=dev)
        step = lambda: A.spmv(xd, yd, accumulate=False)
        kernel = spmv_kernel_name(tuned)
        launches_per_step = 1 if tuned[0] == 1 else 2  # SpMV kernel + carry fix-up
        traffic = NCU_TRAFFIC.get(kernel) if name == "spmv" else None
    else:
        xd = torch.as_tensor(d["B"]).to(dev)
        yd = torch.zeros((r1 - r0, 64), dtype=torch.float64, device=dev)
        step = lambda: A.spmm(xd, yd, accumulate=False)
        kernel, launches_per_step, traffic = "spmm_row_direct_kernel", 1, NCU_TRAFFIC["spmm"]
    ms, clocks = hx.timed(step, args.steps, args.warmup)
    ms_step = ms / args.steps
    value = d["work"] / (ms_step * 1e-3) * d["unit_scale"]
    algo_bytes_rank = lnnz * 16 + (r1 - r0 + 1) * 8 + (8 * n + 8 * (r1 - r0)) * k
    roof = hx.hbm_roofline(algo_bytes_rank, ms_step, kernel, traffic * (lnnz / float(pos[n])) if traffic else None)

    # ---- a sample of the last timed result against the CPU oracle (outside the timed region) ----------------
    rows = np.sort(np.random.default_rng(11 + rank).integers(r0, r1, min(1000, r1 - r0))) if r1 > r0 else np.zeros(0, np.int64)
    spos, scrd, sval = sample_rows_csr(pos, crd, val, rows)
    got = yd[torch.as_tensor(rows - r0, device=dev)].cpu().numpy() if len(rows) else np.zeros(0)
    if name != "spmm":
        ref = oracle.spmv(spos, scrd, sval, d["x"], np.zeros(len(rows)))
        scale = oracle.spmv(spos, scrd, np.abs(sval) * np.abs(d["x"][scrd]), np.ones(n), np.zeros(len(rows)))
        ok = bool(np.all(np.abs(got - ref) <= 1e-12 * np.maximum(scale, np.finfo(np.float64).tiny)))
    else:
        ok = bool(np.array_equal(got, oracle.spmm(spos, scrd, sval, d["B"], np.zeros((len(rows), 64)))))
    verified = hx.all_true(ok)

    # ---- e2e: host buffers in, host result out, through the package's public call ---------------------------
    e2e = None
    if not args.no_e2e:
        pin = lambda a: torch.as_tensor(np.ascontiguousarray(a)).pin_memory()
        x_pin = pin(d["B"] if name == "spmm" else d["x"])
        out_pin = torch.zeros(tuple(yd.shape), dtype=torch.float64).pin_memory()
        d2h = int(out_pin.numel() * 8)
        if world == 1:
            from lapis_b200.dualview import DualView
            lpos, lcrd, lval = pos, crd, val
            module = KB.KokkosBackend(decompose_tensors=True).compile(mm.spmm(mm.CSR64) if name == "spmm" else mm.spmv(mm.CSR64))
            fn = module.spmm if name == "spmm" else module.spmv
            spec = ((n, n), (len(lpos), len(lcrd), len(lval)))
            pnp = [pin(a).numpy() for a in (lpos, lcrd, lval)] + [x_pin.numpy()]
            # (i) every operand uploaded on every call: the generated module's own calling convention
            all_steps = max(1, min(args.steps, 3))
            plain = lambda: fn(pnp[0], pnp[1], pnp[2], spec, pnp[3], out_pin.numpy())
            plain()
            t_all = hx.wall(plain, all_steps)
            h2d_all = sum(int(a.nbytes) for a in pnp) + d2h
            per_call = {"value": d["work"] * all_steps / t_all * d["unit_scale"], "unit": d["unit"],
                        "h2d_bytes_per_step": h2d_all, "d2h_bytes_per_step": d2h, "steps": all_steps,
                        "api": f"KokkosBackend.compile(...).{fn.__name__} -> py_{fn.__name__}, pinned host buffers"}
            # (ii) headline: the matrix stays resident (DualView arguments), the dense operand is re-uploaded and
            # the result downloaded on every step -- what benchmarks/spmv/main.cpp:42-62 does with its DualViews
            dvs = [DualView(a, device=dev) for a in pnp]
            out_dv = DualView(out_pin.numpy(), device=dev)

            def resident():
                dvs[3].modifyHost()
                fn(dvs[0], dvs[1], dvs[2], spec, dvs[3], out_dv, sync_host=True)

            resident()
            torch.cuda.synchronize()
            res_steps = max(3, min(args.steps, 20))
            t_res = hx.wall(resident, res_steps)
            e2e = {"value": d["work"] * res_steps / t_res * d["unit_scale"], "unit": d["unit"],
                   "h2d_bytes_per_step": int(x_pin.numel() * 8), "d2h_bytes_per_step": d2h, "steps": res_steps,
                   "api": f"KokkosBackend.compile(...).{fn.__name__} with lapis_b200.dualview.DualView arguments over pinned "
                          "host buffers: matrix uploaded once before the timed region, dense operand re-uploaded "
                          "(modifyHost) every step, result downloaded every step (sync_host=True)",
                   "all_operands_uploaded_per_call": per_call}
            del dvs, out_dv
        elif name != "spmm":
            # several ranks: every rank uploads its 1/N slice of x, the slices are gathered over NVLink, the
            # kernel runs, every rank downloads its block of y
            e2e_step = lambda: sh.spmv_from_host(x_pin, out_pin)
            e2e_step()
            res_steps = max(3, min(args.steps, 20))
            t_res = hx.wall(e2e_step, res_steps)
            e2e = {"value": d["work"] * res_steps / t_res * d["unit_scale"], "unit": d["unit"],
                   "h2d_bytes_per_step": int(x_pin.numel() * 8) // world if n % world == 0 else int(x_pin.numel() * 8),
                   "d2h_bytes_per_step": d2h, "steps": res_steps,
                   "api": "lapis_b200.dist.ShardedSpmv.spmv_from_host: matrix resident, each rank uploads 1/N of x from "
                          "pinned host memory, NCCL all-gather of x over NVLink, kernel, download of this rank's block of y; "
                          "bytes are per rank"}
    # with x arriving split over the ranks and gathered on the device first (reported beside the headline)
    if world > 1 and name == "spmv" and n % world == 0:
        x_part = xd[rank * (n // world):(rank + 1) * (n // world)].clone()

        def step_gather():
            hx.dist.all_gather_into_tensor(xd, x_part)
            A.spmv(xd, yd, accumulate=False)

        try:
            ms_g, _ = hx.timed(step_gather, args.steps, 3)
            detail["with_x_allgather"] = {"ms_per_step": ms_g / args.steps, "unit": d["unit"],
                                          "value": d["work"] / (ms_g / args.steps * 1e-3) * d["unit_scale"]}
        except RuntimeError as exc:  # a side measurement: its failure must not take the headline line with it
            detail["with_x_allgather"] = {"error": str(exc)[:200]}
    return {"value": value, "ms_per_step": ms_step, "clocks": clocks, "e2e": e2e,
            "gpu_launches": launches_per_step * args.steps * world, "roofline": roof, "verified": verified, "detail": detail}


def run_pcg(args, d, hx: Harness, iterations: int, with_e2e: bool):
    """Config 5: fixed number of Jacobi-PCG iterations on the 5-point Laplacian, rows split over the ranks."""
    import torch
    from oracle import oracle
    from lapis_b200 import KokkosBackend as KB
    from lapis_b200 import modules as mm
    from lapis_b200.dist import DistPcg
    dev, world = hx.dev, hx.world
    n = d["shape"][0]
    solver = DistPcg(d["pos"], d["crd"], d["val"], (n, n), d["b"], d["dinv"], dev, use_graph=True, comm=args.comm)
    state = {}

    def solve(k):
        state["out"] = solver.solve(0.0, k, check_every=50)

    # Warm-up is a whole untimed solve with the same solver (it also captures the CUDA graph of one iteration that
    # the timed solve replays); the timed region is one solve of `iterations` iterations.
    solve(iterations)
    ms, clocks = hx.timed(lambda: solve(iterations), 1, 0)
    it = state["out"][1]
    tuned = solver.matrix.tuned_kernel()
    if solver.comm == "nccl":
        launches_per_it = 8 - (1 if tuned[0] == 1 else 0)
    elif solver.fused and solver._two_pass():
        launches_per_it = 2
    elif solver.fused:
        launches_per_it = 3 if tuned[0] == 1 else (5 if tuned[0] in (-256, -512) else 6)
    else:
        launches_per_it = (6 if world == 1 and solver.comm == "none" else 12) - (1 if tuned[0] == 1 else 0)
    ms_it = ms / max(1, it)
    roof = hx.hbm_roofline(d["bytes_per_step"] / world, ms_it,
                           "pcg_spmv_direction_kernel + pcg_update_fused_kernel" if solver.fused and solver._two_pass() else
                           "spmv_rowthread_kernel (pass A) + pcg_update_fused_kernel + pcg_direction(_fused)_kernel",
                           NCU_TRAFFIC["pcg_two_pass" if solver.fused and solver._two_pass() else "pcg"] / world)
    # check: the relative residual after three iterations against the CPU oracle's (same recurrences, full grid)
    _, it3, rel3 = solver.solve(0.0, 3, check_every=3)
    ok = True
    if hx.rank == 0:
        _, io, ro = oracle.pcg(d["pos"], d["crd"], d["val"], d["b"], d["dinv"], 0.0, 3, host_threads())
        ok = it3 == io == 3 and abs(rel3 - ro) <= 1e-9 * abs(ro)
    verified = hx.all_true(ok)
    e2e = None
    if with_e2e and world == 1:
        module = KB.KokkosBackend(decompose_tensors=True).compile(mm.pcg(mm.CSR32))
        pinned = [torch.as_tensor(np.ascontiguousarray(a)).pin_memory().numpy()
                  for a in (d["pos"], d["crd"], d["val"], d["b"], d["dinv"])]
        spec = ((n, n), (n + 1, len(d["crd"]), len(d["val"])))
        t0 = time.perf_counter()
        _, it2, _ = module.pcg(pinned[0], pinned[1], pinned[2], spec, pinned[3], pinned[4], 0.0, iterations)
        t_e2e = time.perf_counter() - t0
        e2e = {"value": it2 / t_e2e, "unit": "it/s", "h2d_bytes_per_step": sum(a.nbytes for a in pinned) / it2,
               "d2h_bytes_per_step": 8 * n / it2, "steps": it2,
               "api": "KokkosBackend.compile(...).pcg -> py_pcg, pinned host buffers, copies amortised over the solve"}
    detail = {"spmv_kernel_tuned": list(tuned), "iterations": int(it), "launches_per_iteration": launches_per_it,
              "exchange": {"p2p": "stores into peer memory + flags inside the passes (own kernels)"
                                  if solver.fused else "stores into peer memory + flags (own kernels between the passes)",
                           "nccl": "NCCL send/recv + allreduce", "none": "none (one rank)"}[solver.comm]}
    return {"value": it / (ms * 1e-3), "ms_per_step": ms_it, "clocks": clocks, "e2e": e2e,
            "gpu_launches": launches_per_it * it * world, "roofline": roof, "verified": verified, "detail": detail}


def run_gemm(args, d, hx: Harness, steps: int, warmup: int, with_e2e: bool):
    """Configs 4a (batch of 128^3, split by batch) and 4b (one 8192^3 problem per GPU: replicas only)."""
    import torch
    from oracle import oracle
    from lapis_b200 import KokkosBackend as KB
    from lapis_b200 import device as D
    from lapis_b200 import modules as mm
    dev, world, rank = hx.dev, hx.world, hx.rank
    A_h, B_h = d["A"], d["B"]
    batched = A_h.ndim == 3
    if batched:
        nb = A_h.shape[0]
        per = nb // world
        sl = slice(rank * per, (rank + 1) * per if rank < world - 1 else nb)
        A_h, B_h = A_h[sl], B_h[sl]
    Ad, Bd = torch.as_tensor(A_h).to(dev), torch.as_tensor(B_h).to(dev)
    Cd = torch.zeros(A_h.shape[:-1] + (B_h.shape[-1],), dtype=torch.float32, device=dev)
    step = lambda: D.bgemm(Ad, Bd, Cd)
    ms, clocks = hx.timed(step, steps, warmup)
    D.bgemm_status()
    ms_step = ms / steps
    if batched:
        total_work = d["work"]                      # the batch is split: the job is the whole batch
        roof = hx.hbm_roofline(d["bytes_per_step"] / world, ms_step, "bgemm_tcgen05_kernel", NCU_TRAFFIC["bgemm"] / world)
    else:
        total_work = d["work"] * world              # one full problem per GPU
        roof = hx.tensor_roofline(d["work"], ms_step, "bgemm_tcgen05_kernel", NCU_TRAFFIC["gemm"])
    value = total_work / (ms_step * 1e-3) * d["unit_scale"]
    # check of the last result (C accumulated steps + warmup products): sampled rows against fp64 dot products
    reps = steps + warmup
    Ch = None
    if batched:
        pick = np.unique(np.linspace(0, A_h.shape[0] - 1, 6).astype(int))
        Ch = Cd[torch.as_tensor(pick, device=dev)].cpu().numpy().astype(np.float64)
        exact = reps * oracle.bgemm_acc64(np.ascontiguousarray(A_h[pick]), np.ascontiguousarray(B_h[pick]),
                                          np.zeros((len(pick),) + A_h.shape[1:2] + B_h.shape[2:3], np.float32)).astype(np.float64)
    else:
        pick = np.unique(np.linspace(0, A_h.shape[0] - 1, 48).astype(int))
        Ch = Cd[torch.as_tensor(pick, device=dev)].cpu().numpy().astype(np.float64)
        exact = reps * (A_h[pick].astype(np.float64) @ B_h.astype(np.float64))
    # norm-wise bar of the tensor-core tests: 1e-5 of the result's magnitude (fp32 accumulation over the repetitions
    # adds at most reps roundings of the same size)
    err = float(np.max(np.abs(Ch - exact)) / np.max(np.abs(exact)))
    ok = bool(err <= 1e-5 * max(1.0, reps ** 0.5))
    verified = hx.all_true(ok)
    e2e = None
    if with_e2e:
        module = KB.KokkosBackend().compile(mm.MATMUL if not batched else mm.BATCH_MATMUL)
        pa, pb = torch.as_tensor(A_h).pin_memory(), torch.as_tensor(B_h).pin_memory()
        pc = torch.zeros(tuple(Cd.shape), dtype=torch.float32).pin_memory()
        module.forward(pa.numpy(), pb.numpy(), pc.numpy())
        t_e2e = hx.wall(lambda: module.forward(pa.numpy(), pb.numpy(), pc.numpy()), 1)
        e2e = {"value": total_work / t_e2e * d["unit_scale"], "unit": d["unit"],
               "h2d_bytes_per_step": int(pa.numel() + pb.numel() + pc.numel()) * 4, "d2h_bytes_per_step": int(pc.numel()) * 4,
               "steps": 1, "api": "KokkosBackend.compile(...).forward -> py_forward, pinned host buffers"}
    return {"value": value, "ms_per_step": ms_step, "clocks": clocks, "e2e": e2e, "gpu_launches": steps * world,
            "roofline": roof, "verified": verified,
            "detail": {"tflops_per_gpu": value / world if not batched else None, "sample_max_err_over_max_abs": err,
                       "accumulated_products": reps}}


def cpu_baseline(d):
    """The CPU restatement timed on this box's cores on a bounded sample (at least 2 s of repetitions, median),
    before this process has created a CUDA context."""
    return time_cpu(d, 1, None, 2.0, 20.0)


def run_secondary(args, hx: Harness):
    """PCG iterations/s, GEMM and batched-GEMM TFLOP/s on the same N GPUs: the rest of the headline metric."""
    out = {}
    plan = (("pcg", lambda dd: run_pcg(args, dd, hx, 200 if not args.small else 50, False)),
            ("gemm", lambda dd: run_gemm(args, dd, hx, 10, 3, False)),
            ("bgemm", lambda dd: run_gemm(args, dd, hx, 50, 5, False)))
    for name, fn in plan:
        try:
            dd = make_workload(name, args.small)
            r = fn(dd)
            entry = {"metric": dd["metric"], "value": r["value"], "unit": dd["unit"], "ms_per_step": r["ms_per_step"],
                     "dtype": dd["dtype"], "config": config_for(dd, hx.world), "roofline": r["roofline"],
                     "verified": r["verified"], "clocks": r["clocks"], "gpu_launches": r["gpu_launches"]}
            entry.update({k: v for k, v in r["detail"].items() if v is not None})
            out[name] = entry
            del dd, r
        except Exception as exc:  # a secondary figure must not take the headline line with it
            out[name] = {"error": f"{type(exc).__name__}: {str(exc)[:300]}"}
        import torch
        torch.cuda.empty_cache()
    return out


def run_ours(args, d, hx: Harness, cpu_base):
    name = d["name"]
    if name in ("spmv", "spmv1", "spmm"):
        r = run_sparse(args, d, hx)
    elif name == "pcg":
        r = run_pcg(args, d, hx, args.steps, not args.no_e2e)
    else:
        r = run_gemm(args, d, hx, args.steps, args.warmup, not args.no_e2e)
    secondary = None
    if name == "spmv" and not args.no_secondary:
        import torch
        del d["pos"], d["crd"], d["val"]
        torch.cuda.empty_cache()
        secondary = run_secondary(args, hx)
    if hx.rank != 0:
        return
    line = {
        "metric": d["metric"], "value": r["value"], "unit": d["unit"], "n_gpus": hx.world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True,
        "scaling": "weak" if name == "gemm" else "strong", "vs_baseline": None, "dtype": d["dtype"], "data": "synthetic",
        "config": config_for(d, hx.world), "clocks": r["clocks"], "e2e": r["e2e"], "gpu_launches": r["gpu_launches"],
        "roofline": r["roofline"], "verified": r["verified"], "detail": r["detail"],
    }
    if cpu_base is not None:
        line["cpu_baseline"] = cpu_base
    if secondary is not None:
        line["secondary"] = secondary
    print(json.dumps(line), flush=True)


def run_formats(args):
    """The neighbouring kernels of the path (CSRV batched SpMM, DCSR SpMM, hitting-time moments) on one GPU: device
    time with operands resident, algorithmic GB/s against the measured copy bandwidth, and the CPU restatement on
    a sample of the same inputs.  One JSON line per kernel; these are not the headline metric."""
    import torch
    from lapis_b200 import device as D
    from lapis_b200 import workloads as w
    from oracle import oracle
    dev = torch.device("cuda:0")
    peaks, peak_kind = measured_peaks()
    t = lambda a: torch.as_tensor(np.ascontiguousarray(a)).to(dev)
    steps = max(3, min(args.steps, 20))

    def gpu_ms(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    def line(kernel, workload, ms, nbytes, cpu_ms, extra):
        gbs = nbytes / (ms * 1e-3) * 1e-9
        out = {"workload": "formats", "kernel": kernel, "case": workload, "ms": ms, "algorithmic_bytes": int(nbytes),
               "gbs": gbs, "frac_of_copy_peak": gbs / peaks["hbm_gbs"], "peak_source": peak_kind,
               "cpu_ms_1_thread": cpu_ms, "steps": steps}
        out.update(extra)
        print(json.dumps(out), flush=True)

    # CSRV batched SpMM: 32 stored fibers per row, fibers of 8, dh = 64 (2 KiB rows of B and C)
    n = 1 << (14 if args.small else 17)
    sp = w.spmm_uniform(n, per_row=32, k=1, idx_dtype=np.int32)
    nh, dh = 8, 64
    rng = np.random.default_rng(12)
    nnz = len(sp["crd"])
    val = rng.standard_normal(nnz * nh).astype(np.float32)
    B = rng.standard_normal((n, dh, nh)).astype(np.float32)
    dpos, dcrd, dval, dB = t(sp["pos"]), t(sp["crd"]), t(val), t(B)
    C = torch.zeros((n, dh, nh), dtype=torch.float32, device=dev)
    ms = gpu_ms(lambda: D.bspmm_csrv(dpos, dcrd, dval, dB, n, C))
    rows_cpu = min(n, 1 << 12)
    end = int(sp["pos"][rows_cpu])
    t0 = time.perf_counter()
    oracle.bspmm(sp["pos"][:rows_cpu + 1], sp["crd"][:end], val[:end * nh], B)
    cpu_ms = (time.perf_counter() - t0) * 1e3 * n / rows_cpu
    line("bspmm_csrv_kernel", f"CSRV {n} x {n}, 32 per row, nh 8, dh 64, fp32, int32 indices", ms,
         nnz * (4 + 4 * nh) + 4 * (n + 1) + 3 * 4 * n * dh * nh, cpu_ms,
         {"gathered_B_bytes": nnz * dh * nh * 4, "cpu_sample": f"first {rows_cpu} rows, scaled by rows"})
    del dB, C, dval

    # DCSR SpMM: every other row stored, 32 per stored row, k = 64
    n = 1 << (15 if args.small else 19)
    sp = w.spmm_uniform(n, per_row=32, k=64, idx_dtype=np.int64)
    nnz = len(sp["crd"])
    i1 = np.arange(0, 2 * n, 2, dtype=np.int64)
    dB = t(sp["B"])
    Cd = torch.zeros((2 * n, 64), dtype=torch.float64, device=dev)
    di1, dp2, di2, dv = t(i1), t(sp["pos"]), t(sp["crd"]), t(sp["val"])
    ms = gpu_ms(lambda: D.spmm_dcsr(di1, dp2, di2, dv, dB, Cd, n))
    rows_cpu = min(n, 1 << 13)
    t0 = time.perf_counter()
    oracle.spmm_dcsr(i1[:rows_cpu], sp["pos"][:rows_cpu + 1], sp["crd"], sp["val"], sp["B"], np.zeros((2 * rows_cpu, 64)))
    cpu_ms = (time.perf_counter() - t0) * 1e3 * n / rows_cpu
    line("spmm_dcsr_kernel", f"DCSR {2 * n} x {n}, {n} stored rows, 32 per row, k 64, fp64, int64 indices", ms,
         nnz * 16 + 8 * (2 * n + 1) + 3 * 8 * n * 64, cpu_ms,
         {"gathered_B_bytes": nnz * 64 * 8, "cpu_sample": f"first {rows_cpu} stored rows, scaled by rows"})
    del dB, Cd

    # hitting-time moments on a grid graph: adjacency of the 5-point stencil (unit weights), d = degree
    def grid_graph(gg):
        pos, crd, _ = w.laplacian_2d(gg, idx_dtype=np.int32)
        rows = np.repeat(np.arange(gg * gg), np.diff(pos))
        off = crd != rows
        apos_ = np.concatenate([[0], np.cumsum(np.bincount(rows[off], minlength=gg * gg))]).astype(np.int32)
        mask_ = np.ones(gg * gg)
        mask_[:: gg * 7 + 3] = 0.0
        return apos_, crd[off].astype(np.int32), np.diff(apos_).astype(np.float64), mask_

    g = 512 if args.small else 2048
    apos, acrd, dvec, mask = grid_graph(g)
    A = D.CsrMatrix.from_host(apos, acrd, np.ones(len(acrd)), (g * g, g * g), dev, tune=True)
    dm, dd = t(mask), t(dvec)
    A.mht(dm, dd, 0.95, 0.0, 100)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    _, _, iters, _ = A.mht(dm, dd, 0.95, 0.0, 100, info=True)
    torch.cuda.synchronize()
    ms = (time.perf_counter() - t0) * 1e3 / sum(iters)
    gc = min(g, 512)
    cpos, ccrd, cd, cmask = (apos, acrd, dvec, mask) if gc == g else grid_graph(gc)
    t0 = time.perf_counter()
    oracle.mht(cpos, ccrd, np.ones(len(ccrd)), cmask, cd, 0.95, 0.0, 8)
    cpu_ms = (time.perf_counter() - t0) * 1e3 / 16 * (g * g) / (gc * gc)
    nn, nnz = g * g, len(acrd)
    line("mht passes (spmv + mht_update + mht_direction)", f"hitting-time moments, {g} x {g} grid graph, int32 indices, "
         f"{sum(iters)} iterations over the two solves (host-timed, whole solve)", ms,
         nnz * 12 + 4 * (nn + 1) + 19 * 8 * nn, cpu_ms, {"cpu_sample": f"{gc} x {gc} grid, 16 iterations, scaled by rows"})


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--workload", default="spmv", choices=["spmv", "spmv1", "spmm", "pcg", "bgemm", "gemm", "formats"],
                    help="'formats' times the CSRV, DCSR and hitting-time kernels on one GPU (one line per kernel)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--comm", default="p2p", choices=["p2p", "nccl"],
                    help="exchange of the row-partitioned PCG on several GPUs: own peer-memory kernels or NCCL")
    ap.add_argument("--small", action="store_true", help="reduced sizes (for profiler captures and quick checks)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiler captures)")
    ap.add_argument("--no-secondary", action="store_true", help="skip the PCG / GEMM figures of the default run")
    ap.add_argument("--shrink", type=int, default=0, help="divide the SpMV/SpMM row count by 2^SHRINK (profiler captures)")
    args = ap.parse_args()
    defaults = {"spmv": (500, 10), "spmv1": (1000, 10), "spmm": (50, 5), "pcg": (200, 5), "bgemm": (200, 10), "gemm": (20, 3),
                "formats": (20, 3)}
    if args.steps is None:
        args.steps = defaults[args.workload][0] if args.impl == "ours" else 10
    if args.warmup is None:
        args.warmup = defaults[args.workload][1] if args.impl == "ours" else 3

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.workload == "formats":
        if rank == 0 and args.impl == "ours":
            release_main_thread()
            run_formats(args)
        elif rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": "the formats lines time the CPU restatement beside each kernel"}))
        return 0
    if args.impl == "reference":
        if rank != 0:
            return 0
        run_reference(args, make_workload(args.workload, args.small, args.shrink))
        return 0

    d = make_workload(args.workload, args.small, args.shrink)
    # the CPU baseline first, while this process holds no CUDA context, pinned buffers or helper threads
    cpu_base = cpu_baseline(d) if (world == 1 and not args.no_cpu_baseline) else None
    release_main_thread()

    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: lapis_b200 has no CPU path")
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local_rank}"))
    run_ours(args, d, Harness(rank, world, local_rank), cpu_base)
    if world > 1:
        # All ranks have reported; leave without communicator teardown (destroy_process_group() has
        # been seen to block when captured graphs still hold NCCL work).
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        os._exit(0)
    return 0


if __name__ == "__main__":
    sys.exit(main())
