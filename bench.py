#!/usr/bin/env python
"""Benchmark of the accelerated path on N GPUs of one node.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload spmv|spmm|pcg|bgemm|gemm]
                    [--impl ours|reference]

Default workload: CSR SpMV fp64 on the large skewed matrix (2^23 rows, power-law row
lengths with mean 16 capped at 4096, int64 offsets/indices, about 1.34e8 entries), rows
partitioned by nnz over the GPUs, x replicated.  A step is one y = A x pass.  The inputs
of a pass (2.35 GB; 0.29 GB per GPU at N = 8) are larger than the 126 MB L2, so no flush
is needed between timed iterations.

Prints ONE JSON line on rank 0.  `value` is the whole-job throughput with operands
resident in HBM (CUDA events around exactly K steps, barrier + synchronize on both
sides, max over ranks); `e2e` is the same metric through the emitted-module ABI
(py_spmv with pinned host buffers: host-to-device copies of every operand and the
device-to-host copy of y inside the timed region); `roofline` relates the dominant
kernel to the measured HBM copy bandwidth; `cpu_baseline` is the CPU restatement of the
reference's emitted loop timed on this box's cores (rank 0, N = 1 only).

`--impl reference` times that CPU restatement alone, with all host threads, on the same
configuration (the reference's own Kokkos build cannot be produced without LLVM/MLIR and
Kokkos, which are not available offline).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

FALLBACK_HBM_GBS = 6650.0


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
    """Samples SM clocks and throttle reasons of one GPU while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.02):
        self.index, self.period = index, period_s
        self.samples, self.reasons, self.max_mhz = [], set(), None
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
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


def physical_cores() -> int:
    try:
        import psutil
        return psutil.cpu_count(logical=False) or os.cpu_count() or 1
    except Exception:
        return os.cpu_count() or 1


def host_threads() -> int:
    try:
        avail = len(os.sched_getaffinity(0))
    except Exception:
        avail = os.cpu_count() or 1
    return max(1, min(avail, physical_cores()))


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
        d.update(unit="it/s", metric="pcg_iterations_per_s", dtype="f64", unit_scale=1.0, work=1,
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


# ---------------------------------------------------------------------------
# reference arm: the CPU restatement on the host cores
# ---------------------------------------------------------------------------
def run_reference(args, d):
    oracle, native = oracle_native()
    threads = host_threads()
    name = d["name"]
    budget_s = 120.0
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
        t0 = time.perf_counter(); step(); t1 = time.perf_counter() - t0
        est = t1 * (args.steps + args.warmup)
        if est > budget_s:
            rows = max(1, int(n * budget_s / est))
            step = make_step(rows)
        frac_nnz = float(pos[rows]) / float(pos[n])
        work = d["work"] * frac_nnz
        sample = (f"rows [0, {rows}) of {n} ({100 * frac_nnz:.1f}% of the entries) per step, x/B whole; "
                  f"throughput scaled by the entries processed")
    elif name == "pcg":
        # a solve of `steps` iterations on a grid small enough for the budget
        g = int(round(len(d["b"]) ** 0.5))
        from lapis_b200 import workloads as w
        while True:
            dd = w.pcg_laplacian(g)
            t0 = time.perf_counter()
            oracle.pcg(dd["pos"], dd["crd"], dd["val"], dd["b"], dd["dinv"], 0.0, 2, threads, native=native)
            t1 = (time.perf_counter() - t0) / 2
            if t1 * (args.steps + args.warmup) <= budget_s or g <= 256:
                break
            g //= 2
        its = args.steps
        step = None
        sample = f"{g}x{g} grid, {its} iterations"
        for _ in range(1):
            oracle.pcg(dd["pos"], dd["crd"], dd["val"], dd["b"], dd["dinv"], 0.0, max(1, args.warmup), threads, native=native)
        t0 = time.perf_counter()
        oracle.pcg(dd["pos"], dd["crd"], dd["val"], dd["b"], dd["dinv"], 0.0, its, threads, native=native)
        total = time.perf_counter() - t0
        scale = (g * g) / float(len(d["b"]))
        value = its / total * scale  # iterations/s rescaled to the full grid by rows (bandwidth-bound)
        sample += f"; it/s scaled by rows to the {int(round(len(d['b']) ** 0.5))}^2 grid"
        return finish_reference(args, d, value, total / its * 1e3, threads, native, sample)
    else:
        A, B = d["A"], d["B"]
        if A.ndim == 2:
            m = A.shape[0]
            mm = m
            while 2.0 * mm ** 3 / 0.3e9 / max(1, threads) * (args.steps + args.warmup) > budget_s and mm > 256:
                mm //= 2
            A, B = np.ascontiguousarray(A[:mm, :mm]), np.ascontiguousarray(B[:mm, :mm])
            C = np.zeros((mm, mm), dtype=np.float32)
            work = 2.0 * mm ** 3
            sample = f"{mm}^3 sub-problem per step (naive loop order as emitted)"
        else:
            nb = A.shape[0]
            bb = nb
            while 2.0 * bb * A.shape[1] ** 3 / 1e9 / max(1, threads) * (args.steps + args.warmup) > budget_s and bb > 8:
                bb //= 2
            A, B = A[:bb], B[:bb]
            C = np.zeros(A.shape, dtype=np.float32)
            work = 2.0 * bb * A.shape[1] ** 3
            sample = f"{bb} of {nb} problems per step"
        lib = oracle.lib(native)
        import ctypes
        bt, M, K = (1, *A.shape) if A.ndim == 2 else A.shape
        N = B.shape[-1]

        def step():
            lib.oracle_bgemm_f32(ctypes.c_int64(bt), ctypes.c_int64(M), ctypes.c_int64(N), ctypes.c_int64(K),
                                 A.ctypes.data_as(ctypes.c_void_p), B.ctypes.data_as(ctypes.c_void_p),
                                 C.ctypes.data_as(ctypes.c_void_p), ctypes.c_int(threads))
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    total = time.perf_counter() - t0
    value = work * args.steps / total * d["unit_scale"]
    return finish_reference(args, d, value, total / args.steps * 1e3, threads, native, sample)


def finish_reference(args, d, value, ms, threads, native, sample):
    line = {
        "impl": "reference", "metric": d["metric"], "value": value, "unit": d["unit"], "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": d["dtype"].split(" ")[0], "data": "synthetic",
        "config": {"workload": d["label"]},
        "cpu_baseline": {"value": value, "unit": d["unit"], "cores": threads, "kind": "port",
                         "sample": sample + ("; -march=native build" if native else "; portable build"),
                         "note": "CPU restatement of the emitted Kokkos loops (OpenMP); the reference's own Kokkos "
                                 "build needs LLVM/MLIR and Kokkos, which are not available offline"},
        "e2e": {"value": value, "unit": d["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------
def run_ours(args, d, rank, world, local_rank):
    import torch
    import torch.distributed as dist

    from lapis_b200 import KokkosBackend as KB
    from lapis_b200 import device as D
    from lapis_b200 import partition as part
    from lapis_b200 import modules as mm

    dev = torch.device(f"cuda:{local_rank}")
    torch.cuda.set_device(dev)
    name = d["name"]
    peaks, peak_kind = measured_peaks()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(step, steps, warmup):
        for _ in range(warmup):
            step()
        barrier()
        sampler = ClockSampler(local_rank)
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        barrier()
        clocks = sampler.stop()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, clocks

    launches_per_step = 2 if args.workload in ("spmv", "spmv1") else 1  # SpMV: chunk kernel + carry fix-up
    e2e = None
    kernel_name = ""
    extra_cfg = {}
    if name in ("spmv", "spmv1", "spmm"):
        pos, crd, val = d["pos"], d["crd"], d["val"]
        n = len(pos) - 1
        bounds = part.partition_rows(pos, world)
        r0, r1 = int(bounds[rank]), int(bounds[rank + 1])
        lpos, lcrd, lval = part.row_block(pos, crd, val, r0, r1)
        A = D.CsrMatrix.from_host(lpos, lcrd, lval, (r1 - r0, n), dev)
        # per-matrix choice of the SpMV kernel; relaxed: the segmented-scan kernel (within 1e-12 of the others,
        # the parity bar of this metric, but not their bits) is a candidate
        extra_cfg_kernel = A.tune(relaxed=True) if name != "spmm" else (0, 0)
        extra_cfg = {"partition": "contiguous row blocks, equal nnz", "rows_rank0": int(bounds[1] - bounds[0]),
                     "replicated": "B" if name == "spmm" else "x", "spmv_kernel_tuned": list(extra_cfg_kernel)}
        if name != "spmm":
            xd = torch.as_tensor(d["x"]).to(dev)
            yd = torch.zeros(r1 - r0, dtype=torch.float64, device=dev)
            step = lambda: A.spmv(xd, yd, accumulate=False)
            kernel_name = {2: "spmv_scan_kernel", 3: "spmv_scan_kernel", 1: "spmv_rowthread_kernel"}.get(
                extra_cfg_kernel[0], "spmv_pipe_kernel" if extra_cfg_kernel[0] < 0 else "spmv_chunk_kernel")
            host_in = [lpos, lcrd, lval, d["x"]]
            module = KB.KokkosBackend(decompose_tensors=True).compile(mm.spmv(mm.CSR64))
        else:
            Bd = torch.as_tensor(d["B"]).to(dev)
            Cd = torch.zeros((r1 - r0, 64), dtype=torch.float64, device=dev)
            step = lambda: A.spmm(Bd, Cd, accumulate=False)
            kernel_name = "spmm_row_direct_kernel"
            host_in = [lpos, lcrd, lval, d["B"]]
            module = KB.KokkosBackend(decompose_tensors=True).compile(mm.spmm(mm.CSR64))
        # ---- e2e through the emitted-module ABI with pinned host buffers -------------
        pinned = [torch.as_tensor(np.ascontiguousarray(a)).pin_memory() for a in host_in]
        out_shape = (r1 - r0, 64) if name == "spmm" else (r1 - r0,)
        out = torch.zeros(out_shape, dtype=torch.float64).pin_memory()
        pnp = [t.numpy() for t in pinned]
        spec = ((r1 - r0, n), (len(lpos), len(lcrd), len(lval)))
        fn = module.spmm if name == "spmm" else module.spmv

        def e2e_step():
            fn(pnp[0], pnp[1], pnp[2], spec, pnp[3], out.numpy())

        h2d = sum(int(t.numel() * t.element_size()) for t in pinned) + int(out.numel() * 8)
        d2h = int(out.numel() * 8)
        e2e_steps = 0 if args.no_e2e else max(1, min(args.steps, 3))
        if e2e_steps:
            e2e_step()
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        t_e2e = time.perf_counter() - t0
        if world > 1:
            t = torch.tensor([t_e2e], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            t_e2e = float(t.item())
        if e2e_steps:
            e2e = {"value": d["work"] * e2e_steps / t_e2e * d["unit_scale"], "unit": d["unit"],
                   "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                   "api": f"KokkosBackend.compile(...).{fn.__name__} -> py_{fn.__name__}_f64_i64, pinned host buffers"}
            # The same call with resident operands (DualView arguments): the matrix is uploaded once before
            # the timed region; every step the dense operand is declared modified on the host (re-uploaded)
            # and the result is brought back.
            from lapis_b200.dualview import DualView
            dvs = [DualView(a, device=dev) for a in pnp]
            out_dv = DualView(out.numpy(), device=dev)
            def resident_step():
                fn(dvs[0], dvs[1], dvs[2], spec, dvs[3], out_dv, sync_host=True)

            resident_step()
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            res_steps = max(e2e_steps, min(args.steps, 20))
            t0 = time.perf_counter()
            for _ in range(res_steps):
                dvs[3].modifyHost()
                resident_step()
            t_res = time.perf_counter() - t0
            if world > 1:
                t = torch.tensor([t_res], dtype=torch.float64, device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                t_res = float(t.item())
            # Headline e2e: the call as a caller who keeps the matrix between calls makes it (the reference's
            # driver, benchmarks/spmv/main.cpp:42-62, also uploads once and loops on the device).  The figure
            # with every operand uploaded on every call stays beside it.
            e2e = {"value": d["work"] * res_steps / t_res * d["unit_scale"], "unit": d["unit"],
                   "h2d_bytes_per_step": int(pnp[3].nbytes), "d2h_bytes_per_step": d2h, "steps": res_steps,
                   "api": f"KokkosBackend.compile(...).{fn.__name__} with lapis_b200.dualview.DualView arguments over pinned "
                          "host buffers: matrix uploaded once before the timed region, dense operand re-uploaded "
                          "(modifyHost) every step, result downloaded every step row block by row block while the "
                          "next block computes (sync_host=True)",
                   "all_operands_uploaded_per_call": e2e}
            del dvs, out_dv
        del pinned, out
        algo_bytes_rank = (len(lcrd) * 16 + len(lpos) * 8 + (8 * n + 8 * (r1 - r0)) * (64 if name == "spmm" else 1))
    elif name == "pcg":
        from lapis_b200.dist import DistPcg
        n = d["shape"][0]
        solver = DistPcg(d["pos"], d["crd"], d["val"], (n, n), d["b"], d["dinv"], dev, use_graph=True, comm=args.comm)
        if world > 1:
            extra_cfg = dict(extra_cfg or {}, exchange={"p2p": "stores into peer memory + flags (own kernels)",
                                                        "nccl": "NCCL send/recv + allreduce"}[solver.comm])
        state = {}

        def solve(k):
            state["out"] = solver.solve(0.0, k, check_every=50)

        # The timed region is one solve of K iterations.  Warm-up is a whole untimed solve with the same
        # solver (it also captures the CUDA graph of one iteration that the timed solve replays).
        solver.solve(0.0, args.steps)
        kernel_name = "spmv_rowthread_kernel|spmv_pipe_kernel|spmv_chunk_kernel (pass A) + pcg_update_kernel + pcg_direction_kernel"
        # ours per iteration: SpMV + its fix-up, three vector passes... 6 on one rank; the NCCL transport adds
        # two scalar-step kernels, the peer-to-peer one six exchange kernels
        launches_per_step = 6 if world == 1 else (8 if solver.comm == "nccl" else 12)
        if solver.matrix.tuned_kernel()[0] == 1:
            launches_per_step -= 1  # the one-thread-per-row SpMV kernel has no carry fix-up launch
        extra_cfg = dict(extra_cfg or {}, spmv_kernel_tuned=list(solver.matrix.tuned_kernel()))
        steps_holder = {"k": args.steps}
        ms, clocks = timed(lambda: solve(steps_holder["k"]), 1, 0)
        it = state["out"][1]
        value = it / (ms * 1e-3)
        algo_bytes_rank = d["bytes_per_step"] / world
        # e2e: py_pcg with pinned host buffers (single process path only)
        if world == 1:
            module = KB.KokkosBackend(decompose_tensors=True).compile(mm.pcg(mm.CSR32))
            pinned = [torch.as_tensor(np.ascontiguousarray(a)).pin_memory().numpy()
                      for a in (d["pos"], d["crd"], d["val"], d["b"], d["dinv"])]
            spec = ((n, n), (n + 1, len(d["crd"]), len(d["val"])))
            t0 = time.perf_counter()
            _, it2, _ = module.pcg(pinned[0], pinned[1], pinned[2], spec, pinned[3], pinned[4], 0.0, args.steps)
            t_e2e = time.perf_counter() - t0
            e2e = {"value": it2 / t_e2e, "unit": "it/s", "h2d_bytes_per_step": sum(a.nbytes for a in pinned) / it2,
                   "d2h_bytes_per_step": 8 * n / it2, "steps": it2,
                   "api": "KokkosBackend.compile(...).pcg -> py_pcg_f64_i32, pinned host buffers, copies amortised over the solve"}
        return emit(args, d, value, ms / max(1, it), clocks, e2e, launches_per_step * it * world, kernel_name,
                    algo_bytes_rank, ms / max(1, it), peaks, peak_kind, world, rank, extra_cfg, bound="hbm")
    else:
        A_h, B_h = d["A"], d["B"]
        if A_h.ndim == 3:
            nb = A_h.shape[0]
            per = nb // world
            sl = slice(rank * per, (rank + 1) * per if rank < world - 1 else nb)
            A_h, B_h = A_h[sl], B_h[sl]
            extra_cfg = {"partition": "by batch"}
        Ad, Bd = torch.as_tensor(A_h).to(dev), torch.as_tensor(B_h).to(dev)
        Cd = torch.zeros(A_h.shape[:-1] + (B_h.shape[-1],), dtype=torch.float32, device=dev)
        step = lambda: D.bgemm(Ad, Bd, Cd)
        kernel_name = "bgemm_tcgen05_kernel"
        module = KB.KokkosBackend().compile(mm.MATMUL if A_h.ndim == 2 else mm.BATCH_MATMUL)
        pa, pb = torch.as_tensor(A_h).pin_memory(), torch.as_tensor(B_h).pin_memory()
        pc = torch.zeros(Cd.shape, dtype=torch.float32).pin_memory()
        module.forward(pa.numpy(), pb.numpy(), pc.numpy())
        t0 = time.perf_counter()
        module.forward(pa.numpy(), pb.numpy(), pc.numpy())
        t_e2e = time.perf_counter() - t0
        if world > 1:
            t = torch.tensor([t_e2e], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            t_e2e = float(t.item())
        e2e = {"value": d["work"] / t_e2e * d["unit_scale"], "unit": d["unit"],
               "h2d_bytes_per_step": int(pa.numel() + pb.numel() + pc.numel()) * 4, "d2h_bytes_per_step": int(pc.numel()) * 4,
               "steps": 1, "api": "KokkosBackend.compile(...).forward -> py_(batch_)matmul_f32, pinned host buffers"}
        algo_bytes_rank = d["bytes_per_step"] / world

    ms, clocks = timed(step, args.steps, args.warmup)
    ms_step = ms / args.steps
    value = d["work"] / (ms_step * 1e-3) * d["unit_scale"]
    bound = "tensor" if name == "gemm" else "hbm"
    if world > 1 and name == "spmv" and len(d["x"]) % world == 0:
        # Reported beside the headline, not in it: the same step when x arrives split over the ranks and has to
        # be gathered first (for these random-column matrices every rank needs all of x).
        n_x = len(d["x"])
        x_part = xd[rank * (n_x // world):(rank + 1) * (n_x // world)].clone()

        def step_gather():
            dist.all_gather_into_tensor(xd, x_part)
            A.spmv(xd, yd, accumulate=False)

        try:
            ms_g, _ = timed(step_gather, args.steps, 3)
            extra_cfg["with_x_allgather"] = {"ms_per_step": ms_g / args.steps, "unit": d["unit"],
                                             "value": d["work"] / (ms_g / args.steps * 1e-3) * d["unit_scale"]}
        except RuntimeError as exc:  # a side measurement: its failure must not take the headline line with it
            extra_cfg["with_x_allgather"] = {"error": str(exc)[:200]}
    emit(args, d, value, ms_step, clocks, e2e, launches_per_step * args.steps * world, kernel_name, algo_bytes_rank,
         ms_step, peaks, peak_kind, world, rank, extra_cfg, bound=bound)


# DRAM bytes per launch of the dominant kernel from the committed ncu captures under profiles/
# (dram__bytes_read.sum + dram__bytes_write.sum, scaled to a full launch by entries processed).
NCU_TRAFFIC = {
    "spmv": 3.325e9,    # profiles/spmv_chunk_kernel_config2.md
    "spmm": 3.387e10,   # profiles/spmm_row_kernel_config3.md
    "bgemm": 1.036e9,   # profiles/bgemm_tcgen05_kernel.md (4096 x 128^3)
    "gemm": 3.455e9,    # profiles/bgemm_tcgen05_kernel.md (8192^3)
    "pcg": 2.69e9,      # profiles/pcg_iteration_config5.md (all kernels of one iteration)
}


def emit(args, d, value, ms_step, clocks, e2e, launches, kernel_name, algo_bytes_rank, kernel_ms, peaks, peak_kind,
         world, rank, extra_cfg, bound):
    if rank != 0:
        return
    traffic = NCU_TRAFFIC[d["name"]] / world if d["name"] in NCU_TRAFFIC else None
    if d["name"] == "spmv" and kernel_name != "spmv_chunk_kernel":
        traffic = None  # the committed capture is of the chunk kernel
    if bound == "hbm":
        achieved = algo_bytes_rank / (kernel_ms * 1e-3) * 1e-9
        peak = float(peaks["hbm_gbs"])
        roof = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": traffic, "kernel": kernel_name,
                "peak_source": f"{peak_kind} copy bandwidth",
                "algorithmic_bytes_per_launch": algo_bytes_rank, "frac_of_8TBs": achieved / 8000.0}
    else:
        # 3xTF32: three tensor-core products per fp32 product; dense TF32 peak taken as half the measured bf16 peak
        # the kernel is timed alone over a few tens of milliseconds: the burst figure applies
        tf32_peak = float(peaks["bf16_tflops"]) / 2.0
        achieved = 3.0 * d["work"] / world / (kernel_ms * 1e-3) * 1e-12
        roof = {"bound": "tensor", "achieved": achieved, "peak": tf32_peak, "unit": "TFLOP/s", "frac": achieved / tf32_peak,
                "traffic": traffic, "kernel": kernel_name,
                "peak_source": f"{peak_kind} bf16 burst / 2 (TF32); achieved counts the 3 TF32 products per fp32 product"}
    line = {
        "metric": d["metric"], "value": value, "unit": d["unit"], "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": d["dtype"], "data": "synthetic",
        "config": {"workload": d["label"], "l2": "inputs larger than L2, no flush between iterations", **extra_cfg},
        "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "roofline": roof,
    }
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(d)
    print(json.dumps(line), flush=True)


def cpu_baseline(d):
    """The CPU restatement timed on this box's cores on a bounded sample (about 10-30 s)."""
    oracle, native = oracle_native()
    threads = host_threads()
    name = d["name"]
    budget = 15.0
    if name in ("spmv", "spmv1"):
        y = np.zeros(len(d["pos"]) - 1)
        step = lambda: oracle.spmv_inplace(d["pos"], d["crd"], d["val"], d["x"], y, threads, native)
        work, sample = d["work"], "the whole matrix, repeated"
    elif name == "spmm":
        C = np.zeros((len(d["pos"]) - 1, 64))
        step = lambda: oracle.spmm_inplace(d["pos"], d["crd"], d["val"], d["B"], C, threads, native)
        work, sample = d["work"], "the whole matrix, repeated"
    elif name == "pcg":
        its = 5
        step = lambda: oracle.pcg(d["pos"], d["crd"], d["val"], d["b"], d["dinv"], 0.0, its, threads, native=native)
        work, sample = its, f"{its} iterations per repetition on the full grid"
    else:
        A, B = d["A"], d["B"]
        if A.ndim == 2:
            m = min(A.shape[0], 1024)
            A, B = np.ascontiguousarray(A[:m, :m]), np.ascontiguousarray(B[:m, :m])
            sample = f"{m}^3 sub-problem (naive loop order as emitted)"
            work = 2.0 * m ** 3
        else:
            nb = min(A.shape[0], 256)
            A, B = A[:nb], B[:nb]
            sample = f"{nb} problems of {A.shape[1]}^3"
            work = 2.0 * nb * A.shape[1] ** 3
        C = np.zeros(A.shape[:-1] + (B.shape[-1],), dtype=np.float32)
        step = lambda: oracle.bgemm(A, B, C, threads, native)
    step()
    reps, t0 = 0, time.perf_counter()
    while True:
        step()
        reps += 1
        el = time.perf_counter() - t0
        if el > budget or reps >= 50:
            break
    return {"value": work * reps / el * d["unit_scale"], "unit": d["unit"], "cores": threads, "kind": "port",
            "sample": f"{sample}; {reps} repetitions in {el:.1f} s; " + ("-march=native build" if native else "portable build"),
            "ms_per_step": el / reps * 1e3}


def probe_gather(args, d):
    """Yardstick for the SpMV: the same 8-byte index stream and the same random gathers of x, with a
    plain 8-byte store per entry instead of the row reduction (a library kernel, not part of the product)."""
    import torch
    dev = torch.device("cuda:0")
    x = torch.as_tensor(d["x"]).to(dev)
    idx = torch.as_tensor(d["crd"]).to(dev)
    out = torch.empty(idx.numel(), dtype=torch.float64, device=dev)
    for _ in range(max(3, args.warmup)):
        torch.index_select(x, 0, idx, out=out)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        torch.index_select(x, 0, idx, out=out)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    print(json.dumps({"probe": "gather", "entries": int(idx.numel()), "x_bytes": int(x.numel() * 8), "ms": ms,
                      "gathers_per_s": idx.numel() / (ms * 1e-3),
                      "stream_gbs": idx.numel() * 16 / (ms * 1e-3) * 1e-9}), flush=True)
    return 0


def probe_flatdot(args, d):
    """Floor for the SpMV: the library's flat-dot yardstick kernel over the workload's own crd / val / x (same
    streams, same gathers, four entries per thread, no row structure, no per-entry store)."""
    import ctypes
    import torch
    from lapis_b200._lib import check, load
    dev = torch.device("cuda:0")
    lib = load()
    x, crd, val = (torch.as_tensor(d[k]).to(dev) for k in ("x", "crd", "val"))
    out = torch.zeros(1, dtype=torch.float64, device=dev)
    vp = lambda t: ctypes.c_void_p(t.data_ptr())
    run = lambda: check(lib.lapis_b200_probe_flat_dot_f64(crd.element_size(), crd.numel(), vp(crd), vp(val), vp(x), vp(out),
                                                          ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
    for _ in range(max(3, args.warmup)):
        run()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        run()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    nbytes = crd.numel() * (8 + crd.element_size()) + x.numel() * 8
    print(json.dumps({"probe": "flatdot", "entries": int(crd.numel()), "ms": ms, "gathers_per_s": crd.numel() / (ms * 1e-3),
                      "stream_plus_x_gbs": nbytes / (ms * 1e-3) * 1e-9}), flush=True)
    return 0


def probe_formats(args):
    """Timings of the neighbouring kernels (hitting-time moments, CSRV batched SpMM, DCSR SpMM): device time
    with operands resident, algorithmic GB/s against the measured copy bandwidth, and the CPU restatement on
    the same inputs.  One JSON line per kernel; informational, not the headline metric."""
    import torch
    from lapis_b200 import device as D
    from lapis_b200 import workloads as w
    from oracle import oracle
    dev = torch.device("cuda:0")
    peaks, peak_kind = measured_peaks()
    t = lambda a: torch.as_tensor(np.ascontiguousarray(a)).to(dev)

    def gpu_ms(fn, steps, warmup=3):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    def line(kernel, workload, ms, nbytes, cpu_ms, extra=None):
        gbs = nbytes / (ms * 1e-3) * 1e-9
        out = {"probe": "formats", "kernel": kernel, "workload": workload, "ms": ms, "algorithmic_bytes": int(nbytes),
               "gbs": gbs, "frac_of_copy_peak": gbs / peaks["hbm_gbs"], "peak_source": peak_kind,
               "cpu_ms_1_thread": cpu_ms, "speedup_vs_1_cpu_thread": cpu_ms / ms}
        out.update(extra or {})
        print(json.dumps(out), flush=True)

    small = args.small
    # -- CSRV batched SpMM: 32 stored entries per row, fibers of 8, dh = 64 (2 KiB rows of B and C) --------
    n = 1 << (14 if small else 17)
    sp = w.spmm_uniform(n, per_row=32, k=1, idx_dtype=np.int32)
    nh, dh = 8, 64
    rng = np.random.default_rng(12)
    val = rng.standard_normal(len(sp["crd"]) * nh).astype(np.float32)
    B = rng.standard_normal((n, dh, nh)).astype(np.float32)
    dpos, dcrd, dval, dB = t(sp["pos"]), t(sp["crd"]), t(val), t(B)
    C = torch.zeros((n, dh, nh), dtype=torch.float32, device=dev)
    ms = gpu_ms(lambda: D.bspmm_csrv(dpos, dcrd, dval, dB, n, C), max(3, min(args.steps, 20)))
    rows_cpu = min(n, 1 << 12)
    t0 = time.perf_counter()
    oracle.bspmm(sp["pos"][:rows_cpu + 1], sp["crd"][:int(sp["pos"][rows_cpu])], val[:int(sp["pos"][rows_cpu]) * nh], B)
    cpu_ms = (time.perf_counter() - t0) * 1e3 * n / rows_cpu
    nnz = len(sp["crd"])
    line("bspmm_csrv_kernel", f"CSRV {n} x {n}, 32 per row, nh 8, dh 64, fp32, int32 indices", ms,
         nnz * (4 + 4 * nh) + 4 * (n + 1) + 2 * 4 * n * dh * nh + 4 * n * dh * nh, cpu_ms,
         {"gathered_B_bytes": int(nnz) * dh * nh * 4, "cpu_sample": f"first {rows_cpu} rows, scaled by rows"})
    del dB, C, dval
    # -- DCSR SpMM: every other row stored, 32 per stored row, k = 64 ------------------------------------
    n = 1 << (15 if small else 19)
    sp = w.spmm_uniform(n, per_row=32, k=64, idx_dtype=np.int64)
    i1 = np.arange(0, 2 * n, 2, dtype=np.int64)
    dB = t(sp["B"])
    Cd = torch.zeros((2 * n, 64), dtype=torch.float64, device=dev)
    di1, dp2, di2, dv = t(i1), t(sp["pos"]), t(sp["crd"]), t(sp["val"])
    ms = gpu_ms(lambda: D.spmm_dcsr(di1, dp2, di2, dv, dB, Cd, n), max(3, min(args.steps, 20)))
    rows_cpu = min(n, 1 << 13)
    t0 = time.perf_counter()
    oracle.spmm_dcsr(i1[:rows_cpu], sp["pos"][:rows_cpu + 1], sp["crd"], sp["val"], sp["B"], np.zeros((2 * rows_cpu, 64)))
    cpu_ms = (time.perf_counter() - t0) * 1e3 * n / rows_cpu
    nnz = len(sp["crd"])
    line("spmm_dcsr_kernel", f"DCSR {2 * n} x {n}, {n} stored rows, 32 per row, k 64, fp64, int64 indices", ms,
         nnz * 16 + 8 * (2 * n + 1) + 8 * n * 64 + 2 * 8 * n * 64, cpu_ms,
         {"gathered_B_bytes": int(nnz) * 64 * 8, "cpu_sample": f"first {rows_cpu} stored rows, scaled by rows"})
    del dB, Cd
    # -- hitting-time moments on a grid graph: adjacency of the 5-point stencil, d = degree --------------
    g = 512 if small else 2048
    def grid_graph(gg):
        """Adjacency (unit weights) of the gg x gg grid as int32 CSR, its degree vector and a seed mask."""
        pos, crd, _ = w.laplacian_2d(gg, idx_dtype=np.int32)
        rows = np.repeat(np.arange(gg * gg), np.diff(pos))
        off = crd != rows
        apos_ = np.concatenate([[0], np.cumsum(np.bincount(rows[off], minlength=gg * gg))]).astype(np.int32)
        mask_ = np.ones(gg * gg)
        mask_[:: gg * 7 + 3] = 0.0
        return apos_, crd[off].astype(np.int32), np.diff(apos_).astype(np.float64), mask_

    apos, acrd, dvec, mask = grid_graph(g)
    aval = np.ones(len(acrd))
    its = 100
    A = D.CsrMatrix.from_host(apos, acrd, aval, (g * g, g * g), dev, tune=True)
    dm, dd = t(mask), t(dvec)
    A.mht(dm, dd, 0.95, 0.0, its)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    _, _, iters, _ = A.mht(dm, dd, 0.95, 0.0, its, info=True)
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
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--workload", default="spmv", choices=["spmv", "spmv1", "spmm", "pcg", "bgemm", "gemm"])
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--comm", default="p2p", choices=["p2p", "nccl"],
                    help="exchange of the row-partitioned PCG on several GPUs: own peer-memory kernels or NCCL")
    ap.add_argument("--small", action="store_true", help="reduced sizes (for profiler captures and quick checks)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiler captures)")
    ap.add_argument("--probe", choices=["gather", "flatdot", "formats"], default=None,
                    help="diagnostic instead of the benchmark: 'gather' times out[j] = x[crd[j]] over the SpMV "
                         "workload's own index stream (torch.index_select: index read, gather, 8-byte store per entry); "
                         "'flatdot' times the library's store-free yardstick sum_j val[j]*x[crd[j]] over the same "
                         "arrays, the floor for an SpMV; "
                         "'formats' times the hitting-time moments, CSRV batched SpMM and DCSR SpMM kernels")
    ap.add_argument("--shrink", type=int, default=0, help="divide the SpMV/SpMM row count by 2^SHRINK (profiler captures)")
    args = ap.parse_args()
    defaults = {"spmv": (500, 10), "spmv1": (1000, 10), "spmm": (50, 5), "pcg": (200, 5), "bgemm": (200, 10), "gemm": (20, 3)}
    if args.steps is None:
        args.steps = defaults[args.workload][0] if args.impl == "ours" else 10
    if args.warmup is None:
        args.warmup = defaults[args.workload][1] if args.impl == "ours" else 3

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        if rank != 0:
            return 0
        d = make_workload(args.workload, args.small, args.shrink)
        run_reference(args, d)
        return 0

    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: lapis_b200 has no CPU path")
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local_rank}"))
    if args.probe == "formats":
        return probe_formats(args)
    d = make_workload(args.workload, args.small, args.shrink)
    if args.probe == "gather":
        return probe_gather(args, d)
    if args.probe == "flatdot":
        return probe_flatdot(args, d)
    run_ours(args, d, rank, world, local_rank)
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
