#!/usr/bin/env python
"""Benchmark of the CSR SpMV / SpMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload C5] [--impl reference]

One JSON line on stdout (rank 0). The headline workload is the 27-point stencil SpMV
(fp64, 16.8 M rows, 449 M nonzeros): the largest single-GPU configuration and one of the two
that are sharded over several GPUs, so the same matrix is measured at every N (strong
scaling: nnz-balanced row blocks, x replicated, y assembled on every GPU). At N = 1 the line
also carries the other configurations under "configs".

  value     algorithmic bytes / s with all operands resident in HBM (events on the handle's stream)
  e2e       same metric through the C ABI with x copied from pinned host memory and y copied back
            inside the timed region of every step (the matrix stays resident): throughput with
            --e2e-depth independent products in flight (HostSpmvPipeline), and serial_ms_per_step
            for one product at a time
  roofline  algorithmic bytes / mean device time of one mcsparseSpMV call (tile kernel + carry
            fix-up kernel, so slightly conservative for the tile kernel alone) against the measured
            HBM copy bandwidth in MEASURED_PEAKS.json
  --transposed       y = A^T x of the chosen workload instead (conversion timed once, then the products)
  --impl reference   the OpenMP C CSR kernels of oracle/ on the host cores (the mcSparse reference has
            no CPU implementation and builds only with the MetaX toolchain), on a bounded row block
"""

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

L2_BYTES = 126 * 1024 * 1024
# DRAM bytes (read + write) of one spmv_tile_kernel launch divided by its algorithmic bytes, from the ncu
# captures summarised under profiles/ (taken at reduced scale and scaled by the units processed).
TRAFFIC_RATIO = {"C5": 0.985, "C5_fp16_operands": 1.003, "C2": 0.99, "C3": 1.71, "C4_n64": 3.18}
FALLBACK_HBM_GBS = 6650.0


def PUSH_CHUNKS_DEFAULT(world):
    """Chunks of the pipelined row push the library chooses for `world` GPUs (0: the tile kernel pushes)."""
    return 4 if world == 2 else 0
METRIC = "csr_spmv_spmm_algorithmic_hbm_throughput"
UNIT = "GB/s"


def hbm_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


# ----------------------------------------------------------------------------- clocks

class ClockSampler:
    """Reads (never sets) SM clock and throttle reasons through NVML while the timed region runs."""

    REASONS = {
        0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
        0x80: "hw_power_brake_slowdown",
    }

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.dev = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.dev, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None
        self.thread = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        while not self._stop.is_set():
            try:
                self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.dev, self.nv.NVML_CLOCK_SM))
                mask = self.nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.dev)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.01)

    def __enter__(self):
        if self.nv:
            self.thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self.nv:
            self.thread.join()

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ----------------------------------------------------------------------------- GPU arm

def visible_device_index(local_rank):
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except Exception:
            return local_rank
    return local_rank


class SpmvJob:
    """One configuration on one rank: a row block of A resident in HBM, x replicated."""

    def __init__(self, name, device, rank, world, handle, scale=1, index_bits=32, complex_values=False,
                 half_operands=False):
        import torch

        import mcsparse_b200 as mc
        from mcsparse_b200 import workloads

        self.torch, self.mc, self.h = torch, mc, handle
        cfg = workloads.CONFIGS[name] if scale == 1 else workloads.scaled(name, scale)
        self.cfg, self.world, self.rank = cfg, world, rank
        self.vsize = 8 if cfg.dtype == torch.float64 else 4
        lengths = workloads.row_lengths(cfg, device)
        if world > 1:
            from mcsparse_b200 import sharding

            bounds, self.total_nnz = sharding.shard_bounds(lengths, world)  # nnz-balanced contiguous row blocks
        else:
            bounds, self.total_nnz = [0, cfg.rows], int(lengths.sum().item())
        del lengths
        self.bounds = bounds
        r0, r1 = bounds[rank], bounds[rank + 1]
        w = workloads.generate(cfg, device, row_range=(r0, r1))
        self.w = w
        isize = 4
        if index_bits == 64:  # variant: the same matrix with 64-bit row offsets and column indices (N = 1 only)
            w.row_ptr, w.col, isize = w.row_ptr.long(), w.col.long(), 8
        if complex_values:  # variant: the same structure with complex values, x and y of twice the bytes (N = 1 only)
            cdt = torch.complex64 if cfg.dtype == torch.float32 else torch.complex128
            w.val = torch.complex(w.val, w.val.flip(0)).to(cdt)
            w.x = torch.complex(w.x, w.x.flip(0)).to(cdt)
            if w.y0 is not None:
                w.y0 = torch.complex(w.y0, w.y0.flip(0)).to(cdt)
            self.vsize *= 2
        self.compute_dtype = None
        if half_operands:  # variant: the same matrix with A and x in fp16, sums and y in fp32 (N = 1 only)
            w.val, w.x = w.val.to(torch.float16), w.x.to(torch.float16)
            self.compute_dtype = torch.float32
        self.A = mc.CsrMatrix(w.rows, w.cols, w.row_ptr, w.col, w.val)
        if world > 1:
            from mcsparse_b200 import sharding

            # product path: the kernel pushes finished rows into every peer's y over NVLink
            self.sharded = sharding.ShardedSpmv(handle, self.A, w.x, r0, cfg.rows)
            self.y_full = self.sharded.y.tensor
            self.y = self.sharded.y_local
            self.X, self.Y, self.buf = self.sharded.X, self.sharded.Y, self.sharded.buffer
        else:
            self.sharded = None
            self.y_full = torch.zeros(cfg.rows, dtype=self.compute_dtype or w.val.dtype, device=device)
            self.y = self.y_full[r0:r1]
            self.X, self.Y = mc.DnVec(w.x), mc.DnVec(self.y)
            self.buf = torch.empty(mc.spmv_buffer_size(handle, self.A, self.X, self.Y, compute=self.compute_dtype),
                                   dtype=torch.uint8, device=device)
            mc.spmv_preprocess(handle, self.A, self.X, self.Y, self.buf, compute=self.compute_dtype)
        if cfg.beta != 0:
            self.y.copy_(w.y0)
        self.parts = [self.y_full[bounds[g]:bounds[g + 1]] for g in range(world)]
        self.bytes = workloads.algorithmic_bytes(cfg.rows, cfg.rows, self.total_nnz, self.vsize, cfg.beta, index_size=isize)
        # what this rank's kernel must move: of x only the span of columns its row block touches (a block of a
        # stencil reaches one plane beyond itself; a block of a random matrix reaches all of x)
        span = int((w.col.max() - w.col.min()).item()) + 1 if w.nnz else 0
        self.local_bytes = workloads.algorithmic_bytes(w.rows, min(w.cols, span), w.nnz, self.vsize, cfg.beta,
                                                       index_size=isize)
        if half_operands:  # 2-byte values and x, 4-byte y
            self.bytes = self.local_bytes = (w.nnz * (2 + isize) + (w.rows + 1) * isize + w.cols * 2
                                             + w.rows * 4 * (2 if cfg.beta != 0 else 1))
        self.flops = 2 * self.total_nnz
        # tile kernel + carry fix-up; sharded: per chunk a tile launch and a fix-up (pipelined push), or one of each
        # (rows pushed by the tile kernel), and the kernel that orders the GPUs
        chunks = int(os.environ.get("MCSPARSE_B200_PUSH_CHUNKS", PUSH_CHUNKS_DEFAULT(world)))
        # (one launch when the push crew of the tile launch also adds the carries)
        self.launches_per_step = 2 if world == 1 else (2 * chunks if chunks else 1) + 1

    def compute(self):
        """The local SpMV only (no assembly of y): what the roofline fraction is computed from."""
        self.mc.spmv(self.h, self.A, self.X, self.Y, self.buf, alpha=self.cfg.alpha, beta=self.cfg.beta,
                     compute=self.compute_dtype)

    def step(self):
        """One full step: at N > 1 the SpMV with the fused push of y to all GPUs, then the ordering collective."""
        if self.sharded is not None:
            self.sharded.step(self.cfg.alpha, self.cfg.beta)
        else:
            self.compute()

    def step_allgather(self):
        """Baseline assembly for comparison: local SpMV, then a ragged NCCL all-gather of y."""
        from mcsparse_b200 import sharding

        self.compute()
        sharding.all_gather_ragged(self.parts, self.y)


class TransposedSpmvJob:
    """y = A^T x through mcsparseSpMV with op(A) = A^T: conversion recorded once by the preprocess call
    (timed separately), every step re-gathers the values and runs the tile kernels on the converted matrix."""

    def __init__(self, name, device, handle, scale=1, keep_values=False):
        import torch

        import mcsparse_b200 as mc
        from mcsparse_b200 import capi, workloads

        self.torch, self.mc, self.h, self.op = torch, mc, handle, capi.MCSPARSE_OPERATION_TRANSPOSE
        cfg = workloads.CONFIGS[name] if scale == 1 else workloads.scaled(name, scale)
        self.cfg = cfg
        w = workloads.generate(cfg, device)
        self.w, self.total_nnz = w, w.nnz
        self.vsize = 8 if cfg.dtype == torch.float64 else 4
        self.A = mc.CsrMatrix(w.rows, w.cols, w.row_ptr, w.col, w.val)
        if keep_values:  # the caller's promise to announce value changes: products reuse the gathered values
            capi.check(capi.lib.mcsparseB200SpMatKeepConvertedValues(self.A.d, 1))
        self.x = workloads.dense_values(cfg, device, w.rows, 77)
        self.y = torch.zeros(w.cols, dtype=cfg.dtype, device=device)
        self.X, self.Y = mc.DnVec(self.x), mc.DnVec(self.y)
        self.buf = torch.empty(mc.spmv_buffer_size(handle, self.A, self.X, self.Y, op=self.op), dtype=torch.uint8,
                               device=device)
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        t0.record()
        mc.spmv_preprocess(handle, self.A, self.X, self.Y, self.buf, op=self.op)
        t1.record()
        torch.cuda.synchronize()
        self.preprocess_ms = t0.elapsed_time(t1)
        self.bytes = workloads.algorithmic_bytes(w.cols, w.rows, w.nnz, self.vsize, 0.0)
        self.flops = 2 * w.nnz
        self.launches_per_step = 3

    def step(self):
        self.mc.spmv(self.h, self.A, self.X, self.Y, self.buf, alpha=1.0, beta=0.0, op=self.op)

    compute = step


class SpmmJob:
    def __init__(self, name, n, device, handle, scale=1, keep_values=False):
        import torch

        import mcsparse_b200 as mc
        from mcsparse_b200 import workloads

        self.torch, self.mc, self.h = torch, mc, handle
        cfg = workloads.CONFIGS[name] if scale == 1 else workloads.scaled(name, scale)
        self.cfg, self.n, self.world = cfg, n, 1
        w = workloads.generate(cfg, device)
        self.w = w
        self.total_nnz = w.nnz
        self.C = torch.zeros(w.rows, n, dtype=cfg.dtype, device=device)
        self.A = mc.CsrMatrix(w.rows, w.cols, w.row_ptr, w.col, w.val)
        self.Bm, self.Cm = mc.DnMat(w.B[n], w.cols, n, n), mc.DnMat(self.C, w.rows, n, n)
        self.buf = torch.empty(mc.spmm_buffer_size(handle, self.A, self.Bm, self.Cm), dtype=torch.uint8, device=device)
        mc.spmm_preprocess(handle, self.A, self.Bm, self.Cm, self.buf)
        if keep_values:  # the caller's promise to announce value changes: later products skip the regrouping pass
            from mcsparse_b200 import capi

            capi.check(capi.lib.mcsparseB200SpMatKeepConvertedValues(self.A.d, 1))
        self.panel_buffer_bytes = self.buf.numel()
        self.bytes = workloads.algorithmic_bytes(w.rows, w.cols, w.nnz, 4, cfg.beta, dense_cols=n)
        self.gather_model_bytes = w.nnz * (8 + 4 * n) + (w.rows + 1) * 4 + w.rows * n * 4
        self.flops = 2 * w.nnz * n
        self.launches_per_step = 1

    def step(self):
        self.mc.spmm(self.h, self.A, self.Bm, self.Cm, self.buf, alpha=self.cfg.alpha, beta=self.cfg.beta)

    compute = step


def time_steps(torch, fn, steps, warmup, flush_buf=None, barrier=None):
    """Returns (total_ms over exactly `steps` calls, list of per-call ms). With flush_buf, a buffer larger than
    L2 is rewritten before every call (outside the per-call events) and total_ms is the sum of the calls."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if barrier:
        barrier()
        torch.cuda.synchronize()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for a, b in evs:
        if flush_buf is not None:
            flush_buf.add_(1)
        a.record()
        fn()
        b.record()
    t1.record()
    torch.cuda.synchronize()
    if barrier:
        barrier()
        torch.cuda.synchronize()
    per = [a.elapsed_time(b) for a, b in evs]
    total = sum(per) if flush_buf is not None else t0.elapsed_time(t1)
    return total, per


def gather_rate(torch, handle, device, elem_bytes=4, count=1 << 26, table_elems=1 << 24):
    """Gathers per second this GPU sustains on unrelated elements (mcsparseB200GatherProbe, timed here with
    events): the second roofline of an SpMV whose columns are scattered."""
    import ctypes as C

    from mcsparse_b200 import capi

    idx = torch.randint(0, table_elems, (count,), dtype=torch.int32, device=device)
    table = torch.zeros(table_elems, dtype=torch.float64 if elem_bytes == 8 else torch.float32, device=device)
    blocks = 148 * 8
    out = torch.empty(blocks * 256, dtype=table.dtype, device=device)

    def fn():
        capi.check(capi.lib.mcsparseB200GatherProbe(handle.h, C.c_void_p(idx.data_ptr()), count,
                                                    C.c_void_p(table.data_ptr()), elem_bytes,
                                                    C.c_void_p(out.data_ptr()), blocks))

    total, _ = time_steps(torch, fn, 5, 3)
    return count / (total / 5 * 1e-3)


def reference_kernel_ms(torch, job, steps=3):
    """Device time of the mcSparse reference's own CSR kernel on this job's operands, where the checker library
    oracle/_ref/libmcsp_refkernels.so was built from the reference tree (else None): the reference's kernel source,
    its launch shape, compiled for sm_100a; launched from here, outside the product. SpMM gets the column-major
    copy of B that the reference kernel requires (its own transpose step is not timed)."""
    import ctypes as C

    path = os.path.join(ROOT, "oracle", "_ref", "libmcsp_refkernels.so")
    if not os.path.exists(path):
        return None
    ref = C.CDLL(path)
    w = job.w
    P = lambda t: C.c_void_p(t.data_ptr())
    f64 = w.val.dtype == torch.float64
    ct = C.c_double if f64 else C.c_float
    if isinstance(job, SpmmJob):
        n = job.n
        Bt = w.B[n].t().contiguous()  # column-major B with ldb = rows of B
        Cm = torch.zeros_like(job.C)
        fn = lambda: ref.ref_csr_spmm_f32(w.rows, n, C.c_float(1.0), C.c_float(0.0), P(w.row_ptr), P(w.col), P(w.val),
                                          P(Bt), w.cols, P(Cm), n, 0, 2)
    else:
        y = torch.zeros(w.rows, dtype=w.val.dtype, device=w.val.device)
        call = ref.ref_csr_spmv_f64 if f64 else ref.ref_csr_spmv_f32
        fn = lambda: call(w.rows, ct(job.cfg.alpha), ct(job.cfg.beta), P(w.row_ptr), P(w.col), P(w.val), P(w.x), P(y), 0)
    total, per = time_steps(torch, fn, steps, 1)
    return round(min(per), 5)


def measure_job(torch, job, steps, warmup, peak, flush_buf):
    flush = flush_buf if job.bytes < 4 * L2_BYTES else None
    total, per = time_steps(torch, job.compute, steps, warmup, flush)
    ms = total / steps
    gbs = job.bytes / (ms * 1e-3) / 1e9
    out = {"ms_per_step": round(ms, 5), "best_ms": round(min(per), 5), "gbs": round(gbs, 1),
           "gflops": round(job.flops / (ms * 1e-3) / 1e9, 1), "frac_of_measured_hbm": round(gbs / peak, 4),
           "frac_of_nominal_8tbs": round(gbs / 8000.0, 4), "bytes": job.bytes, "nnz": job.total_nnz,
           "l2": "flushed between steps" if flush is not None else "inputs exceed L2"}
    if hasattr(job, "gather_model_bytes"):
        g = job.gather_model_bytes / (ms * 1e-3) / 1e9
        out["gather_model_gbs"] = round(g, 1)
        out["gather_model_frac"] = round(g / peak, 4)
    return out


def cpu_baseline(name, seconds=12.0, steps=None, step_seconds=0.3):
    """Times the OpenMP CSR kernel of oracle/ on a bounded row block of the workload, on all the host cores
    this process may use. Warm-up is by time (3 s: the OpenMP team and the caches are cold in a process that
    has done nothing else). With `steps`, a step is as many passes as fill `step_seconds`; otherwise passes
    are repeated for about `seconds`. Returns (cpu_baseline dict, seconds per pass, steps, passes per step)."""
    import numpy as np
    import torch

    from mcsparse_b200 import workloads
    from oracle import oracle

    cores = oracle.use_host_cores()
    cfg = workloads.CONFIGS[name]
    target_nnz = 40_000_000
    lengths_mean = {"C1": 5, "C2": 16, "C3": 12, "C4": 32, "C5": 27}[name]
    rows = min(cfg.rows, max(1, target_nnz // lengths_mean))
    if cfg.op == "spmm":
        rows = min(rows, 131072)
    w = workloads.generate(cfg, "cpu", row_range=(0, rows), with_dense=False)
    rp, col, val = w.row_ptr.numpy(), w.col.numpy(), w.val.numpy()
    vsize = val.dtype.itemsize
    if cfg.op == "spmv":
        x = workloads.dense_values(cfg, "cpu", cfg.rows, 41, normal=cfg.values == "normal").numpy()
        y = np.zeros(rows, val.dtype)
        fn = lambda: oracle.baseline_spmv(rp, col, val, x, cfg.alpha, cfg.beta, y)
        # x bytes: the part of x this row block can touch (a stencil block reaches one plane beyond itself)
        reach = {"stencil2d": cfg.grid + 1, "stencil3d": cfg.grid * cfg.grid + cfg.grid + 1}.get(cfg.kind, cfg.rows)
        nbytes = workloads.algorithmic_bytes(rows, min(cfg.rows, rows + reach), w.nnz, vsize, cfg.beta)
        desc = f"rows [0, {rows}) of {name} ({w.nnz} nnz), x of full length"
    else:
        n = cfg.dense_cols[0]
        B = workloads.dense_values(cfg, "cpu", cfg.rows * n, 61 + n).numpy().reshape(cfg.rows, n)
        Cm = np.zeros((rows, n), val.dtype)
        fn = lambda: oracle.baseline_spmm(rp, col, val, B, n, cfg.alpha, cfg.beta, Cm)
        nbytes = workloads.algorithmic_bytes(rows, cfg.rows, w.nnz, vsize, cfg.beta, dense_cols=n)
        desc = f"rows [0, {rows}) of {name} ({w.nnz} nnz), B {cfg.rows} x {n}"
    t_end = time.perf_counter() + 3.0
    passes = 0
    while time.perf_counter() < t_end or passes < 3:
        fn()
        passes += 1
    t = time.perf_counter()
    fn()
    one = max(time.perf_counter() - t, 1e-6)
    if steps is None:
        per_step, steps_run = 1, int(min(20000, max(3, seconds / one)))
    else:
        per_step, steps_run = max(1, int(round(step_seconds / one))), steps
    t = time.perf_counter()
    for _ in range(steps_run * per_step):
        fn()
    dt = (time.perf_counter() - t) / (steps_run * per_step)
    return {"value": round(nbytes / dt / 1e9, 2), "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"{desc}; {steps_run} steps of {per_step} passes, {dt * 1e3:.2f} ms per pass, after 3 s of warm-up",
            "gflops": round(2 * w.nnz * (1 if cfg.op == "spmv" else cfg.dense_cols[0]) / dt / 1e9, 2)}, dt, steps_run, per_step


def workload_config(name, scale, world, rows, total_nnz, alpha, beta, algorithmic_bytes, flushed):
    """The `config` object of a bench line: the same for the GPU arm and the reference arm of one workload."""
    return {"workload": workload_label(name) + ("" if scale == 1 else f" / {scale}"), "rows": rows, "nnz": total_nnz,
            "alpha": alpha, "beta": beta, "index_base": 0,
            "sharding": "replicas only (N=1)" if world == 1 else
            f"{world} nnz-balanced row blocks, x replicated, y rows moved to every GPU over NVLink while the product "
            "runs, GPUs ordered by device-side arrival flags",
            "l2": "L2 flushed between steps" if flushed else "inputs exceed L2",
            "algorithmic_bytes": algorithmic_bytes}


def run_reference(args, rank):
    if rank != 0:
        return
    import torch

    from mcsparse_b200 import workloads

    base, dt, steps, per_step = cpu_baseline(args.workload, steps=args.steps)
    cfg = workloads.CONFIGS[args.workload]
    # the full workload's figures, for the config object (the timed sample is described in cpu_baseline.sample)
    total_nnz = int(workloads.row_lengths(cfg, "cpu").sum().item())
    vsize = cfg.dtype.itemsize
    if cfg.op == "spmv":
        nbytes = workloads.algorithmic_bytes(cfg.rows, cfg.rows, total_nnz, vsize, cfg.beta)
        local = workloads.algorithmic_bytes(cfg.rows // args.gpus, cfg.rows, total_nnz // args.gpus, vsize, cfg.beta)
        config = workload_config(args.workload, 1, args.gpus, cfg.rows, total_nnz, cfg.alpha, cfg.beta, nbytes,
                                 local < 4 * L2_BYTES)
    else:
        config = {"workload": workload_label("C4"), "dense_cols": args.dense_cols}
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": args.warmup, "ms_per_step": round(dt * 1e3, 4), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f64" if vsize == 8 else "f32",
        "data": "synthetic", "config": config,
        "note": "OpenMP C CSR kernel of oracle/ on the host cores (the mcSparse reference has no CPU path and builds "
                f"only with the MetaX toolchain); a step is {per_step} passes over the sample, ms_per_step is one pass",
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_label(name):
    return {
        "C1": "C1 CSR SpMV fp32 5-point Poisson 1024x1024",
        "C2": "C2 CSR SpMV fp64 Poisson(16) rows n=4194304 beta=0.5",
        "C3": "C3 CSR SpMV fp32 power-law rows n=16777216 nnz~2e8",
        "C4": "C4 CSR SpMM fp32 Poisson(32) rows n=1048576, B row-major 64/128 columns",
        "C5": "C5 CSR SpMV fp64 27-point stencil 256^3",
    }[name]


def parity_sample(torch, job, blocks=6, block_rows=1024):
    """Checks row blocks spread over the whole (assembled) y of this rank against the CPU oracle: the rows of
    every shard are sampled, so at N > 1 rows that arrived from the peers are checked as well.
    Returns (rows checked, all within tolerance, largest error in units of tolerance * d)."""
    import numpy as np

    from mcsparse_b200 import workloads
    from oracle import oracle

    cfg = job.cfg
    x = job.w.x.cpu()
    tol = 1e-12 if job.vsize == 8 else 1e-5
    y_all = job.y_full
    checked, ok, worst = 0, True, 0.0
    for b in range(blocks):
        r0 = min(cfg.rows - 1, (cfg.rows * b) // blocks + 17 * b)
        r1 = min(cfg.rows, r0 + block_rows)
        w = workloads.generate(cfg, "cpu", row_range=(r0, r1), with_dense=False)
        y0 = workloads.dense_values(cfg, "cpu", r1 - r0, 51, first=r0) if cfg.beta != 0 else None
        ref, d = oracle.spmv(w.row_ptr, w.col, w.val, x, cfg.alpha, cfg.beta, y0)
        got = y_all[r0:r1].cpu().numpy().astype(np.float64)
        ratio = np.abs(got - ref) / (tol * d + 1e-300)
        worst = max(worst, float(ratio.max()) if ratio.size else 0.0)
        ok = ok and bool((ratio <= 1.0).all())
        checked += r1 - r0
    return checked, ok, worst


def run_gpu(args, rank, world, local_rank):
    import torch

    import mcsparse_b200 as mc

    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    barrier = None
    if world > 1:
        import torch.distributed as dist

        if os.environ.get("NCCL_DEBUG", "").upper() in ("", "VERSION"):
            os.environ["NCCL_DEBUG"] = "WARN"  # keep NCCL's version banner off stdout: one JSON line only
        dist.init_process_group("nccl", device_id=device)
        barrier = dist.barrier
    peak, peak_kind = hbm_peak()
    h = mc.Handle()
    flush_buf = torch.zeros(4 * L2_BYTES // 4, dtype=torch.float32, device=device)
    if args.workload == "C4":  # SpMM: single GPU ("replicas only"), one compact line
        if rank == 0:
            j = SpmmJob("C4", args.dense_cols, device, h, args.scale)
            r = measure_job(torch, j, args.steps, args.warmup, peak, flush_buf)
            r.update({"metric": METRIC, "value": r["gbs"], "unit": UNIT, "n_gpus": 1, "steps": args.steps,
                      "warmup": args.warmup, "higher_is_better": True, "dtype": "f32", "data": "synthetic",
                      "config": {"workload": workload_label("C4"), "dense_cols": args.dense_cols}})
            print(json.dumps(r), flush=True)
        return

    if args.transposed:  # y = A^T x through the conversion: single GPU, one compact line
        if rank == 0:
            j = TransposedSpmvJob(args.workload, device, h, args.scale)
            r = measure_job(torch, j, args.steps, args.warmup, peak, flush_buf)
            r.update({"metric": METRIC, "value": r["gbs"], "unit": UNIT, "n_gpus": 1, "steps": args.steps,
                      "warmup": args.warmup, "higher_is_better": True, "dtype": "f64" if j.vsize == 8 else "f32",
                      "data": "synthetic", "conversion_ms_once": round(j.preprocess_ms, 3),
                      "buffer_bytes": j.buf.numel(),
                      "config": {"workload": workload_label(args.workload) + " transposed (op(A) = A^T)"
                                 + ("" if args.scale == 1 else f" / {args.scale}")}})
            print(json.dumps(r), flush=True)
        return

    if args.half_operands:  # A and x in fp16, sums and y in fp32: single GPU, one compact line
        if rank == 0:
            j = SpmvJob(args.workload, device, 0, 1, h, args.scale, half_operands=True)
            r = measure_job(torch, j, args.steps, args.warmup, peak, flush_buf)
            r.update({"metric": METRIC, "value": r["gbs"], "unit": UNIT, "n_gpus": 1, "steps": args.steps,
                      "warmup": args.warmup, "higher_is_better": True, "dtype": "f16 operands, f32 sums",
                      "data": "synthetic",
                      "config": {"workload": workload_label(args.workload) + " with fp16 A and x, fp32 y"
                                 + ("" if args.scale == 1 else f" / {args.scale}")}})
            print(json.dumps(r), flush=True)
        return

    job = SpmvJob(args.workload, device, rank, world, h, args.scale)
    flush = flush_buf if job.local_bytes < 4 * L2_BYTES else None

    # kernel-only timing of the local SpMV call (roofline), then the full step (with y assembly at N > 1)
    _, per_compute = time_steps(torch, job.compute, max(10, args.steps // 4), args.warmup, flush, barrier)
    with ClockSampler(visible_device_index(local_rank)) as clocks:
        total_ms, per = time_steps(torch, job.step, args.steps, args.warmup, flush, barrier)
    ag_ms = push_ms = 0.0
    if world > 1 and not args.quick:
        k = max(10, args.steps // 4)
        ag_total, _ = time_steps(torch, job.step_allgather, k, args.warmup, flush, barrier)
        push_total, _ = time_steps(torch, lambda: job.sharded.compute(job.cfg.alpha, job.cfg.beta), k, args.warmup,
                                   flush, barrier)
        ag_ms, push_ms = ag_total / k, push_total / k
    # parity of the result the timed steps left (beta == 0 for the sharded workloads: every step gives the same y;
    # with beta != 0 one fresh step from y0 is run for the check)
    if job.cfg.beta != 0:
        job.y.copy_(job.w.y0)
        job.step()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    p_rows, p_ok, p_worst = parity_sample(torch, job)
    t = torch.tensor([total_ms, statistics.mean(per_compute), ag_ms, push_ms, 0.0 if p_ok else 1.0, p_worst],
                     dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, compute_ms, ag_ms, push_ms, p_bad, p_worst = t.tolist()
    ms_per_step = total_ms / args.steps
    value = job.bytes / (ms_per_step * 1e-3) / 1e9

    # end to end: x from pinned host memory every step, y back to pinned host memory, through
    # HostSpmvPipeline. Measured twice: one product at a time (depth 1: latency), and with several
    # independent products in flight so that one product's upload overlaps the previous download
    # (throughput; this is the e2e value, the metric being a throughput). At N > 1 every rank uploads
    # its 1/N slice of x and the GPUs all-gather the slices; every rank downloads its rows of y.
    y_device = job.y.cpu()  # result of the device-resident steps above (same x, beta == 0: same y)
    x_host = job.w.x.cpu().pin_memory()
    e2e_steps = 4 if args.quick else max(6, min(args.steps, 50))
    main = torch.cuda.current_stream()
    shard = None if world == 1 else (job.bounds[rank], job.cfg.rows, None)

    def time_pipeline(depth):
        pipe = mc.HostSpmvPipeline(h, job.w.rows, job.w.cols, job.w.row_ptr, job.w.col, job.w.val, depth=depth,
                                   shard=shard)
        xs = [x_host] + [x_host.clone().pin_memory() for _ in range(depth - 1)]
        ys = [torch.empty(job.y.numel(), dtype=job.cfg.dtype).pin_memory() for _ in range(depth)]
        if job.cfg.beta != 0:
            for y in ys:
                y.copy_(job.w.y0)

        def run(count):
            pipe.start_after(main)
            for i in range(count):
                pipe.submit(xs[i % depth], ys[i % depth], job.cfg.alpha, job.cfg.beta)
                if depth == 1:
                    pipe.wait()  # one product at a time: the host has y before it sends the next x
            pipe.join(main)

        run(max(3, depth))  # warm-up
        torch.cuda.synchronize()
        same = bool(torch.equal(ys[0], y_device)) if job.cfg.beta == 0 else None
        if barrier:
            barrier()
            torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        run(e2e_steps)
        t1.record()
        torch.cuda.synchronize()
        if barrier:
            barrier()
            torch.cuda.synchronize()
        ms = t0.elapsed_time(t1)
        pipe.close()
        return ms, same

    depth = max(2, args.e2e_depth)
    serial_total, serial_same = time_pipeline(1)
    piped_total, piped_same = time_pipeline(depth)
    pipe_ok = None if piped_same is None else (piped_same and serial_same)
    t = torch.tensor([piped_total, serial_total], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms, e2e_serial_ms = (v / e2e_steps for v in t.tolist())
    x_up = x_host.numel() + (job.cfg.rows if job.cfg.beta != 0 else 0)  # elements uploaded per step, all ranks

    # the other sharded configuration (the power-law matrix) on the same GPUs: the step with the row push, the
    # local kernels alone, and the oracle check of the assembled y
    c3 = None
    if world > 1 and args.workload == "C5" and args.scale == 1 and not args.headline_only and not args.quick:
        j3 = SpmvJob("C3", device, rank, world, h)
        k = max(10, args.steps // 4)
        _, per3 = time_steps(torch, j3.compute, k, args.warmup, None, barrier)
        tot3, _ = time_steps(torch, j3.step, k, args.warmup, None, barrier)
        torch.cuda.synchronize()
        barrier()
        rows3, ok3, worst3 = parity_sample(torch, j3)
        t3 = torch.tensor([tot3 / k, statistics.mean(per3), 0.0 if ok3 else 1.0, worst3], dtype=torch.float64,
                          device=device)
        dist.all_reduce(t3, op=dist.ReduceOp.MAX)
        step3, comp3, bad3, worst3 = t3.tolist()
        c3 = {"workload": workload_label("C3"), "n_gpus": world, "ms_per_step": round(step3, 5),
              "kernel_only_ms": round(comp3, 5), "gbs": round(j3.bytes / (step3 * 1e-3) / 1e9, 1),
              "frac_of_measured_hbm_per_gpu": round(j3.bytes / (step3 * 1e-3) / 1e9 / peak / world, 4),
              "nvlink_lower_bound_ms": round((world - 1) / world * j3.cfg.rows * j3.vsize / 770e9 * 1e3, 5),
              "bytes": j3.bytes, "nnz": j3.total_nnz,
              "parity": {"checked_rows": rows3, "ok": bad3 == 0.0, "worst_error_over_tolerance": round(worst3, 4)}}
        j3.sharded.close()
        del j3
        torch.cuda.empty_cache()

    if rank == 0:
        local_gbs = job.local_bytes / (compute_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": round(value, 1), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms_per_step, 5), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f64" if job.vsize == 8 else "f32",
            "data": "synthetic",
            "config": workload_config(args.workload, args.scale, world, job.cfg.rows, job.total_nnz, job.cfg.alpha,
                                      job.cfg.beta, job.bytes, flush is not None),
            "gflops": round(job.flops / (ms_per_step * 1e-3) / 1e9, 1),
            "roofline": {"bound": "hbm", "achieved": round(local_gbs, 1), "peak": peak, "unit": "GB/s",
                         "frac": round(local_gbs / peak, 4),
                         # DRAM bytes per launch from the ncu capture under profiles/ (N = 1 only: nothing was captured
                         # on a shard)
                         "traffic": (round(TRAFFIC_RATIO[args.workload] * job.local_bytes)
                                     if args.workload in TRAFFIC_RATIO and args.scale == 1 and world == 1 else None),
                         "accounting": ("per-rank bytes: the rank's rows of A and y, and the span of x its columns touch"
                                        + ("; a fraction above 1 would be an accounting error" if local_gbs > peak else "")),
                         "peak_kind": peak_kind,
                         "frac_of_nominal_8tbs": round(local_gbs / 8000.0, 4),
                         "kernel": "spmv_tile_kernel (+ carry fix-up) per rank", "ms": round(compute_ms, 5)},
            # e2e.value: one product at a time (what a solver whose next x depends on this y gets); the
            # pipelined figure needs independent products and is reported beside it
            "e2e": {"value": round(job.bytes / (e2e_serial_ms * 1e-3) / 1e9, 1), "unit": UNIT,
                    "h2d_bytes_per_step": x_up * job.vsize, "d2h_bytes_per_step": job.cfg.rows * job.vsize,
                    "ms_per_step": round(e2e_serial_ms, 4), "steps": e2e_steps,
                    "mode": "one product at a time through HostSpmvPipeline (depth 1): x up, product, y down, "
                            "then the next; bytes are totals over all ranks",
                    "pipelined_value": round(job.bytes / (e2e_ms * 1e-3) / 1e9, 1),
                    "pipelined_ms_per_step": round(e2e_ms, 4),
                    "pipelined_mode": f"{depth} independent products in flight: the upload of one overlaps the "
                                      "download of the previous (only for products that do not depend on each other)",
                    "equals_device_resident_result_bitwise": pipe_ok},
            "parity": {"checked_rows": p_rows, "ok": p_bad == 0.0, "worst_error_over_tolerance": round(p_worst, 4),
                       "against": "CPU oracle on row blocks spread over the whole assembled y, on every rank"},
            "gpu_launches": job.launches_per_step * args.steps,
            "multi_gpu": None if world == 1 else {
                "kernel_only_ms": round(compute_ms, 5), "push_kernels_ms": round(push_ms, 5),
                "fused_push_ms": round(ms_per_step, 5),
                "nccl_allgather_ms": round(ag_ms, 5),
                "nvlink_lower_bound_ms": round((world - 1) / world * job.cfg.rows * job.vsize / 770e9 * 1e3, 5)},
            "clocks": clocks.summary(),
        }
        if world == 1 and args.scale == 1:
            base = cpu_baseline(args.workload)[0]
            line["cpu_baseline"] = base
        if world == 1 and args.scale == 1 and not args.headline_only:
            extra = {}
            line["reference_kernel_ms"] = reference_kernel_ms(torch, job)  # the reference's kernel on the headline matrix
            del job
            torch.cuda.empty_cache()
            # second roofline of the scattered-column matrices: one L2 sector request per nonzero
            rate = gather_rate(torch, h, device)
            line["gather_rate"] = {"gathers_per_s": round(rate), "per_sm_per_clock_at_1965_mhz": round(rate / 148 / 1.965e9, 3),
                                   "probe": "mcsparseB200GatherProbe: 2^26 random fp32 gathers from a 64 MiB table"}
            for name in ("C1", "C2", "C3"):
                j = SpmvJob(name, device, 0, 1, h)
                extra[name] = measure_job(torch, j, 100, 5, peak, flush_buf)
                if name in ("C2", "C3"):  # every nonzero gathers an unrelated element of x
                    bound_ms = j.total_nnz / rate * 1e3
                    extra[name].update({"gather_bound_ms": round(bound_ms, 5),
                                        "frac_of_gather_bound": round(bound_ms / extra[name]["ms_per_step"], 4),
                                        "hbm_frac_at_gather_bound": round(j.bytes / (bound_ms * 1e-3) / 1e9 / peak, 4)})
                if name in TRAFFIC_RATIO:
                    extra[name]["traffic"] = round(TRAFFIC_RATIO[name] * j.bytes)
                if name in ("C2", "C3"):
                    extra[name]["reference_kernel_ms"] = reference_kernel_ms(torch, j)
                del j
                torch.cuda.empty_cache()
            # the headline matrix with 64-bit indices, and with complex double values (bytes counted accordingly)
            for key, kw in (("C5_index64", {"index_bits": 64}), ("C5_complex", {"complex_values": True})):
                j = SpmvJob("C5", device, 0, 1, h, **kw)
                extra[key] = measure_job(torch, j, 30, 3, peak, flush_buf)
                del j
                torch.cuda.empty_cache()
            # fp16 operands with fp32 sums and y (6 bytes per nonzero)
            for name in ("C5", "C2", "C3"):
                j = SpmvJob(name, device, 0, 1, h, half_operands=True)
                extra[f"{name}_fp16_operands"] = measure_job(torch, j, 30, 3, peak, flush_buf)
                if f"{name}_fp16_operands" in TRAFFIC_RATIO:
                    extra[f"{name}_fp16_operands"]["traffic"] = round(TRAFFIC_RATIO[f"{name}_fp16_operands"] * j.bytes)
                del j
                torch.cuda.empty_cache()
            for name in ("C2", "C5"):
                j = TransposedSpmvJob(name, device, h)
                extra[f"{name}_transposed"] = measure_job(torch, j, 30, 3, peak, flush_buf)
                extra[f"{name}_transposed"].update({"conversion_ms_once": round(j.preprocess_ms, 3),
                                                    "buffer_bytes": j.buf.numel()})
                del j
                torch.cuda.empty_cache()
                j = TransposedSpmvJob(name, device, h, keep_values=True)
                extra[f"{name}_transposed"]["ms_per_step_values_kept"] = measure_job(torch, j, 30, 3, peak, flush_buf)["ms_per_step"]
                del j
                torch.cuda.empty_cache()
            for n in (64, 128):
                j = SpmmJob("C4", n, device, h)
                extra[f"C4_n{n}"] = measure_job(torch, j, 30, 3, peak, flush_buf)
                extra[f"C4_n{n}"]["work_buffer_bytes"] = j.panel_buffer_bytes
                if n == 64:
                    extra[f"C4_n{n}"]["reference_kernel_ms"] = reference_kernel_ms(torch, j, steps=2)
                del j
                torch.cuda.empty_cache()
                j = SpmmJob("C4", n, device, h, keep_values=True)
                extra[f"C4_n{n}"]["ms_per_step_values_kept"] = measure_job(torch, j, 30, 3, peak, flush_buf)["ms_per_step"]
                if f"C4_n{n}" in TRAFFIC_RATIO:
                    extra[f"C4_n{n}"]["traffic"] = round(TRAFFIC_RATIO[f"C4_n{n}"] * j.bytes)
                del j
                torch.cuda.empty_cache()
            line["configs"] = extra
        if c3 is not None:
            line["configs"] = {"C3": c3}
        print(json.dumps(line), flush=True)
    if world > 1:
        job.sharded.close()
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", default="C5", choices=["C1", "C2", "C3", "C4", "C5"])
    ap.add_argument("--dense-cols", type=int, default=64, help="columns of B for the SpMM workload C4 (64 or 128)")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--scale", type=int, default=1, help="shrink the workload's rows by this factor (profiling)")
    ap.add_argument("--e2e-depth", type=int, default=3,
                    help="independent products kept in flight by the end-to-end (host buffer) measurement")
    ap.add_argument("--transposed", action="store_true",
                    help="time y = A^T x (conversion once, then value gather + SpMV per step) instead of y = A x")
    ap.add_argument("--half-operands", action="store_true",
                    help="the SpMV workload with A and x in fp16, sums and y in fp32 (N = 1)")
    ap.add_argument("--quick", action="store_true", help="tuning runs: skip the comparison timings")
    ap.add_argument("--headline-only", action="store_true", help="skip the per-configuration block at N=1")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    run_gpu(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
