#!/usr/bin/env python
"""Benchmark of the vectorized-pipeline hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--rows R]

One "step" = one pass of the column standardisation + aggregation pipeline (16,777,216 x 32 f64 = 4 GiB per GPU) over
a seeded synthetic N(5,2) matrix; with N > 1 every rank owns its own 4 GiB row block (weak scaling) and the column
statistics are combined across ranks.  Prints ONE JSON line (rank 0).  `value` is rows/s with the input resident in
HBM; `e2e` is the same pipeline through the host-buffer API (H2D of the input and D2H of every result inside the timed
region).  `--impl reference` times the reference's own multithreaded CPU engine on the host cores on the same rows."""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

ROWS_PER_GPU = 16_777_216
COLS = 32
SEED = 2
# algorithmic bytes per row of the whole pipeline with nothing materialised: one statistics pass and one
# normalise + aggregate pass read the row (2 x 256 B), three row results are written (24 B) = 536 B/row
PIPELINE_MIN_BYTES_PER_ROW = 2 * COLS * 8 + 24
# FP64 tensor peak used when it is not measured in the same run (cuBLAS DGEMM 8192^3 through torch.mm on a B200)
FP64_PEAK_TFLOPS = 35.4
# DRAM traffic of the dominant kernel per row, from an ncu capture of the 2,097,152-row case
# (dram__bytes_read.sum + dram__bytes_write.sum = 536.92 MB + 44.54 MB), scaled by the rows of a launch
DOMINANT_TRAFFIC_BYTES_PER_ROW = (536.92e6 + 44.54e6) / 2_097_152


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []
        self.t = None
        self.t0 = self.t1 = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "20", "-i", str(self.gpu)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.t = threading.Thread(target=self._read, daemon=True)
        self.t.start()

    def _read(self):
        for ln in self.proc.stdout:
            self.lines.append((time.perf_counter(), ln.strip()))

    def mark_start(self):
        self.t0 = time.perf_counter()

    def mark_stop(self):
        self.t1 = time.perf_counter()

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        inside = [ln for (t, ln) in self.lines if self.t0 is not None and self.t0 <= t <= (self.t1 or t)]
        window = "timed region"
        if len(inside) < 3:  # a timed region of a few ms holds fewer than three 20 ms samples: add the warm-up
            inside = [ln for (_, ln) in self.lines]
            window = "warm-up + timed region"
        for ln in inside:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "window": window}


def make_input(rows: int, cols: int, seed: int, out: np.ndarray) -> None:
    """N(5, 2) entries, seeded; filled in chunks so that no second 4 GiB temporary is needed."""
    rng = np.random.default_rng(seed)
    step = 1 << 20
    for lo in range(0, rows, step):
        hi = min(rows, lo + step)
        blk = rng.standard_normal((hi - lo, cols))
        blk *= 2.0
        blk += 5.0
        out[lo:hi] = blk


def pinned_array(lib, rows: int, cols: int):
    from daphne_b200.lib import check
    p = C.c_void_p()
    nbytes = rows * cols * 8
    check(lib.db2_malloc_host(C.byref(p), nbytes))
    buf = (C.c_double * (rows * cols)).from_address(p.value)
    return np.frombuffer(buf, dtype=np.float64).reshape(rows, cols), p


def run_ours(args) -> dict:
    import daphne_b200.kernels as K
    from daphne_b200 import pipelines
    from daphne_b200.dist import Comm
    from daphne_b200.lib import check, lib, require_device

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    require_device()
    if world > 1:
        import torch
        torch.cuda.set_device(local_rank)
    comm = Comm.from_env("nccl")
    ctx = K.Context(local_rank)
    comm.init_device(ctx)  # NCCL communicator inside the runtime: partials are combined on the device
    rows, cols = args.rows, COLS
    n_total = rows * world

    host, host_ptr = pinned_array(lib, rows, cols)
    make_input(rows, cols, SEED + rank, host)

    def ev():
        e = C.c_void_p()
        check(lib.db2_event_create(C.byref(e)))
        return e

    stream = C.c_void_p(ctx.stream)

    def sync_all():
        comm.barrier()
        check(lib.db2_device_sync())

    probe = pipelines.Probe(lib, stream) if hasattr(pipelines, "Probe") else None

    # ---- device-resident timing (`value`) ----
    Xd = K.DenseMatrix.from_numpy(ctx, host)
    Xd.device_ptr()  # H2D once, outside the timed region
    ctx.sync()
    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.3)  # nvidia-smi needs a moment before its first sample
    for _ in range(args.warmup):
        res = pipelines.standardise_aggregate_native(ctx, Xd, n_total)
    sync_all()
    sampler.mark_start()
    launches0 = lib.db2_launch_count()
    e0, e1 = ev(), ev()
    if probe:
        probe.reset()
    check(lib.db2_event_record(e0, stream))
    for _ in range(args.steps):
        # the operator calls of the pipeline, issued from native code like a JIT-compiled caller's (db2w_standardise);
        # the context's communicator combines the row shards
        res = pipelines.standardise_aggregate_native(ctx, Xd, n_total, probe=probe)
    check(lib.db2_event_record(e1, stream))
    sync_all()
    sampler.mark_stop()
    ms = C.c_float()
    check(lib.db2_event_elapsed_ms(e0, e1, C.byref(ms)))
    launches = lib.db2_launch_count() - launches0
    clocks = sampler.stop()
    ms_step = comm.max_float(ms.value / args.steps)
    s_value = res.s
    dom = probe.summary() if probe else None
    del res

    # ---- end to end through host buffers (`e2e`) ----
    # results land in pinned host buffers, like the input leaves from one
    # (two sets: a step's three row results travel to the host on the context's second stream while the next step's
    # input travels to the device -- the link carries both directions at once)
    pinned = [[pinned_array(lib, rows, 1) for _ in range(3)] for _ in range(2)]
    outs = [[a for a, _ in trio] for trio in pinned]
    Xd.free()
    e2e_steps = max(1, min(args.steps, 3))

    def e2e_step(i):
        Xh = K.DenseMatrix.from_numpy(ctx, host)  # host placement only; the first kernel triggers the H2D copy
        r = pipelines.standardise_aggregate_native(ctx, Xh, n_total)
        for m, dst in zip((r.r, r.row_max, r.row_idx_max), outs[i % 2]):
            check(lib.db2_matrix_to_host_async(m.handle, C.c_void_p(dst.ctypes.data), 1))
        mu, sd = r.mu.to_numpy(), r.sd.to_numpy()
        Xh.free()
        return r.s, mu, sd

    e2e_step(0)
    check(lib.db2_context_side_sync(ctx.handle))
    sync_all()
    t0 = time.perf_counter()
    e2, e3 = ev(), ev()
    check(lib.db2_event_record(e2, stream))
    for i in range(e2e_steps):
        e2e_step(i + 1)
    check(lib.db2_context_side_sync(ctx.handle))  # the last step's results have arrived
    check(lib.db2_event_record(e3, stream))
    sync_all()
    wall_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
    check(lib.db2_event_elapsed_ms(e2, e3, C.byref(ms)))
    e2e_ms = comm.max_float(max(ms.value / e2e_steps, wall_ms))

    extra = {}
    if not args.no_extra:
        leg_sampler = ClockSampler(local_rank)  # the side legs get their own clock record
        leg_sampler.start()
        for name, leg in (("normal_equations_shard", normal_equations_leg),
                          ("normal_equations_full", normal_equations_full_leg), ("kmeans_shard", kmeans_leg),
                          ("connected_components", components_leg), ("f32_matmul_tcgen05", f32_matmul_leg),
                          ("scheduler_group", scheduler_group_leg), ("generic_chain", generic_chain_leg),
                          ("solve_512", solve_leg)):
            try:
                extra[name] = leg(ctx, comm, lib, host, world, args)
            except Exception as e:  # a side leg must not take the headline down with it
                extra[name] = {"error": f"{type(e).__name__}: {e}"[:300]}
        extra["clocks"] = leg_sampler.stop()

    peak, peak_kind = measured_peaks()
    line = {
        "metric": "pipeline_rows_per_s", "value": n_total / (ms_step * 1e-3), "unit": "rows/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": {"workload": "cfg2 column standardisation + aggregation (mean, sd, Z=(X-mu)/sd, rowSums(Z^2), "
                               "sum, rowMaxs, idxMax) on f64 %d x %d per GPU, N(5,2) seed %d" % (rows, cols, SEED),
                   "rows_per_gpu": rows, "cols": cols, "parallelism": f"rows{world}",
                   "l2": "input (4 GiB) larger than L2, no flush needed"},
        "clocks": clocks,
        "e2e": {"value": n_total / (e2e_ms * 1e-3), "unit": "rows/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": rows * cols * 8, "d2h_bytes_per_step": rows * 24 + 2 * cols * 8 + 8,
                "steps": e2e_steps},
        "gpu_launches": int(launches),
        "pipeline_hbm_gbs": n_total / world * PIPELINE_MIN_BYTES_PER_ROW / (ms_step * 1e-3) / 1e9,
        "pipeline_hbm_frac_of_" + peak_kind: (rows * PIPELINE_MIN_BYTES_PER_ROW / (ms_step * 1e-3) / 1e9) / peak,
        "checksum_s": s_value,
        "extra": extra,
    }
    if dom:
        line["roofline"] = {"bound": "hbm", "kernel": dom["name"], "achieved": dom["gbs"], "peak": peak,
                            "unit": "GB/s", "frac": dom["gbs"] / peak,
                            "traffic": rows * DOMINANT_TRAFFIC_BYTES_PER_ROW if cols == COLS else None,
                            "peak_kind": peak_kind, "launches_timed": dom["launches"],
                            "avg_ms": dom["avg_ms"], "algorithmic_bytes_per_launch": dom["bytes"]}
    if rank == 0:
        line["cpu_baseline"] = cpu_baseline(min(rows, args.cpu_rows) if args.cpu_rows > 0 else rows, cols, steps=3,
                                            budget_s=30.0)
    for p_ in [host_ptr] + [p for trio in pinned for _, p in trio]:
        lib.db2_free_host(p_)
    return line if rank == 0 else {}


def normal_equations_leg(ctx, comm, lib, host, world, args) -> dict:
    """Second workload, reported beside the headline: the per-GPU shard of the sharded normal equations
    (8,388,608 x 512 over 8 GPUs = 1,048,576 x 512 f64 = 4 GiB per GPU, U[-1,1)): t(X)X by syrk, t(X)y by gemv, both
    combined across ranks, then solve.  FLOP convention: BLAS syrk count n*d*(d+1) for t(X)X."""
    import daphne_b200.kernels as K
    from daphne_b200 import pipelines
    from daphne_b200.lib import check
    n, d = (1_048_576, 512) if args.rows >= ROWS_PER_GPU else (max(args.rows // 16, 1024), 512)
    x = host.reshape(-1)[: n * d].reshape(n, d)  # reuse the pinned buffer
    rng = np.random.default_rng(5 + comm.rank)
    step = 1 << 14
    for lo in range(0, n, step):
        hi = min(n, lo + step)
        x[lo:hi] = rng.random((hi - lo, d)) * 2.0 - 1.0
    w = np.random.default_rng(55).standard_normal((d, 1))
    y = x @ w + 0.01 * np.random.default_rng(56 + comm.rank).standard_normal((n, 1))
    X, Y = K.DenseMatrix.from_numpy(ctx, x), K.DenseMatrix.from_numpy(ctx, y)
    X.device_ptr()
    Y.device_ptr()
    stream = C.c_void_p(ctx.stream)
    probe = pipelines.Probe(lib, stream)
    for _ in range(2):
        res = pipelines.normal_equations(ctx, X, Y, 0.001, comm)
    comm.barrier()
    check(lib.db2_device_sync())
    e0, e1 = C.c_void_p(), C.c_void_p()
    check(lib.db2_event_create(C.byref(e0)))
    check(lib.db2_event_create(C.byref(e1)))
    reps = 5
    check(lib.db2_event_record(e0, stream))
    for _ in range(reps):
        res = pipelines.normal_equations(ctx, X, Y, 0.001, comm, probe=probe)
    check(lib.db2_event_record(e1, stream))
    comm.barrier()
    check(lib.db2_device_sync())
    ms = C.c_float()
    check(lib.db2_event_elapsed_ms(e0, e1, C.byref(ms)))
    step_ms = comm.max_float(ms.value / reps)
    syrk = probe.summary()
    beta = res.beta.to_numpy()
    flop = float(n) * d * (d + 1) + 2.0 * n * d  # BLAS syrk count + t(X) y
    peak = fp64_peak_live(ctx, lib)
    return {"workload": f"t(X)X + lambda I, t(X)y, solve on f64 {n} x {d} per GPU (U[-1,1)), combined over {world} GPU(s)",
            "ms_per_step": step_ms, "rows_per_s": n * world / (step_ms * 1e-3),
            "syrk_gemv_ms": syrk["avg_ms"], "syrk_gemv_kernel": syrk["name"],
            "syrk_tflops_syrk_count": flop / (syrk["avg_ms"] * 1e-3) / 1e12,
            "syrk_frac_of_fp64_peak": flop / (syrk["avg_ms"] * 1e-3) / 1e12 / peak["tflops"],
            "fp64_peak_measured": peak, "beta_max_abs_err_vs_w": float(np.abs(beta - w).max())}


def fp64_peak_live(ctx, lib) -> dict:
    """FP64 tensor peak measured in this run: cuBLAS DGEMM 8192^3 (2 n^3 flop), called through the library's C API on
    the context's stream and timed with CUDA events, best of 5 after a warm-up.  It is the denominator of the FP64
    roofline fractions; a constant is used (and named) when cuBLAS cannot be loaded."""
    from daphne_b200.lib import check
    n = 8192
    try:
        cublas = None
        for name in ("libcublas.so.12", "libcublas.so"):
            try:
                cublas = C.CDLL(name)
                break
            except OSError:
                continue
        if cublas is None:
            import glob
            import sysconfig
            hits = glob.glob(sysconfig.get_paths()["purelib"] + "/nvidia/cublas/lib/libcublas.so.*")
            cublas = C.CDLL(hits[0])
        handle = C.c_void_p()
        assert cublas.cublasCreate_v2(C.byref(handle)) == 0
        stream = C.c_void_p(ctx.stream)
        assert cublas.cublasSetStream_v2(handle, stream) == 0
        bufs = [C.c_void_p() for _ in range(3)]
        for b in bufs:
            check(lib.db2_malloc(C.byref(b), n * n * 8))
            check(lib.db2_memset(b, 0, n * n * 8, stream))
        one, zero = C.c_double(1.0), C.c_double(0.0)
        cublas.cublasDgemm_v2.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p,
                                          C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int]

        def gemm():
            assert cublas.cublasDgemm_v2(handle, 0, 0, n, n, n, C.byref(one), bufs[0], n, bufs[1], n, C.byref(zero),
                                         bufs[2], n) == 0
        gemm()
        check(lib.db2_device_sync())
        best = None
        for _ in range(5):
            e0, e1 = C.c_void_p(), C.c_void_p()
            check(lib.db2_event_create(C.byref(e0)))
            check(lib.db2_event_create(C.byref(e1)))
            check(lib.db2_event_record(e0, stream))
            gemm()
            check(lib.db2_event_record(e1, stream))
            ms = C.c_float()
            check(lib.db2_event_elapsed_ms(e0, e1, C.byref(ms)))
            best = ms.value if best is None else min(best, ms.value)
        for b in bufs:
            check(lib.db2_free(b))
        cublas.cublasDestroy_v2(handle)
        return {"tflops": 2.0 * n ** 3 / (best * 1e-3) / 1e12, "kind": "measured in this run",
                "how": f"cuBLAS DGEMM {n}^3, best of 5, CUDA events, {best:.2f} ms"}
    except Exception as e:  # cuBLAS not loadable: the constant measured earlier on the same kind of GPU
        return {"tflops": FP64_PEAK_TFLOPS, "kind": "constant", "how": f"cuBLAS unavailable ({type(e).__name__})"}


def normal_equations_full_leg(ctx, comm, lib, host, world, args) -> dict:
    """The sharded normal equations at the size the configuration names: X f64 8,388,608 x 512 (32 GiB, U[-1,1)) in
    TOTAL, rows split over the ranks (strong scaling: one GPU holds all of it, eight hold 1,048,576 rows each);
    t(X)X by syrk and t(X)y by gemv combined over the ranks, then solve.  The data are generated in 64 blocks with one
    seed per block, so every number of ranks works on the same matrix.  FLOP convention: BLAS syrk count n d (d+1)."""
    import daphne_b200.kernels as K
    from daphne_b200 import pipelines
    from daphne_b200.lib import check
    full = args.rows >= ROWS_PER_GPU
    n_total, d, blocks = (8_388_608, 512, 64) if full else (max(args.rows // 2, 8192), 512, 8)
    per_block = n_total // blocks
    mine = [b for b in range(blocks) if b * world // blocks == comm.rank]
    n = per_block * len(mine)
    w = np.random.default_rng(55).standard_normal((d, 1))
    X = K.DenseMatrix.empty(ctx, n, d)
    Y = K.DenseMatrix.empty(ctx, n, 1)
    stage = host.reshape(-1)[: per_block * d].reshape(per_block, d)  # the pinned buffer, one block at a time
    ybuf = np.empty((per_block, 1))
    for i, b in enumerate(mine):
        rng = np.random.default_rng(5000 + b)
        step = 1 << 13
        for lo in range(0, per_block, step):
            hi = min(per_block, lo + step)
            stage[lo:hi] = rng.random((hi - lo, d)) * 2.0 - 1.0
        ybuf[:] = stage @ w + 0.01 * rng.standard_normal((per_block, 1))
        xs, ys = X.slice_rows(i * per_block, (i + 1) * per_block), Y.slice_rows(i * per_block, (i + 1) * per_block)
        check(lib.db2_memcpy_h2d(C.c_void_p(xs.device_ptr()[0]), C.c_void_p(stage.ctypes.data), stage.nbytes,
                                 C.c_void_p(ctx.stream)))
        check(lib.db2_memcpy_h2d(C.c_void_p(ys.device_ptr()[0]), C.c_void_p(ybuf.ctypes.data), ybuf.nbytes,
                                 C.c_void_p(ctx.stream)))
        ctx.sync()
    peak = fp64_peak_live(ctx, lib)
    ms, res = _timed(lib, ctx, comm, lambda: pipelines.normal_equations_native(ctx, X, Y, 0.001), 3)
    beta = res.beta.to_numpy()
    flop = float(n_total) * d * (d + 1) + 2.0 * n_total * d
    return {"workload": f"t(X)X + lambda I, t(X)y, solve on f64 {n_total} x {d} in total (U[-1,1)), rows over "
                        f"{world} GPU(s): {n} per GPU", "scaling": "strong", "rows_total": n_total, "rows_per_gpu": n,
            "ms_per_step": ms, "rows_per_s": n_total / (ms * 1e-3),
            "tflops_syrk_count": flop / (ms * 1e-3) / 1e12,
            "frac_of_fp64_peak_all_gpus": flop / (ms * 1e-3) / 1e12 / (peak["tflops"] * world),
            "fp64_peak_measured": peak, "beta_max_abs_err_vs_w": float(np.abs(beta - w).max()),
            "beta_checksum": float(beta.sum())}


def scheduler_group_leg(ctx, comm, lib, host, world, args) -> dict:
    """The scheduler that splits row blocks over the GPUs INSIDE one process (db2_vectorizedPipelineGroup: one host
    thread and one context per device, partials combined with NCCL or peer copies): the column standardisation
    workload on 16,777,216 x 32 f64 in TOTAL (strong scaling), through db2w_standardise_group with native pipeline
    bodies.  Run by rank 0 alone over as many GPUs as the launch has ranks (all visible ones without a launcher); the
    other ranks wait on the host.  `first_ms` includes every device fetching its row block from pinned host memory
    (all uploads overlap); `ms_per_step` is with the blocks resident."""
    import daphne_b200.kernels as K
    from daphne_b200.lib import check, device_count
    store = None
    if world > 1:
        import torch.distributed as dist
        store = dist.distributed_c10d._get_default_store()
        if comm.rank != 0:
            store.wait(["db2_scheduler_group_leg"])
            return {}
    rows_total, cols = (ROWS_PER_GPU, COLS) if args.rows >= ROWS_PER_GPU else (max(args.rows, 1 << 16), COLS)
    x = host.reshape(-1)[: rows_total * cols].reshape(rows_total, cols)
    make_input(rows_total, cols, SEED, x)
    ndev = world if world > 1 else device_count()
    out = {}
    try:
        grp = K.Group(list(range(ndev)))
        X = K.DistMatrix.from_numpy(grp, x)
        hs = [C.c_void_p() for _ in range(6)]

        def step():
            for h in hs:
                if h.value:
                    lib.db2_dist_decref(h)
                    h.value = None
            check(lib.db2w_standardise_group(grp.handle, X.handle, *[C.byref(h) for h in hs]))
            grp.sync()
        t0 = time.perf_counter()
        step()
        first_ms = (time.perf_counter() - t0) * 1e3
        for _ in range(3):
            step()
        reps, ts = 20, []
        for _ in range(reps):
            t0 = time.perf_counter()
            step()
            ts.append((time.perf_counter() - t0) * 1e3)
        ms = float(np.median(ts))
        s = K.DistMatrix(grp, hs[5])
        s_val = float(s.to_numpy()[0, 0])
        s._h = C.c_void_p()  # (released with the others below)
        peak, kind = measured_peaks()
        out = {"workload": f"column standardisation + aggregation on f64 {rows_total} x {cols} in total, rows split "
                           f"over {ndev} GPU(s) by the scheduler of ONE process",
               "scaling": "strong", "devices": ndev, "combine": "nccl" if grp.uses_nccl else "peer copies + fold",
               "ms_per_step": ms, "rows_per_s": rows_total / (ms * 1e-3), "first_ms": first_ms,
               "first_rows_per_s": rows_total / (first_ms * 1e-3),
               "hbm_gbs_all_devices": rows_total * PIPELINE_MIN_BYTES_PER_ROW / (ms * 1e-3) / 1e9,
               "hbm_frac_of_" + kind + "_all_devices":
                   rows_total * PIPELINE_MIN_BYTES_PER_ROW / (ms * 1e-3) / 1e9 / (peak * ndev),
               "timing": "wall clock around the call and a synchronisation of every device, median of 20",
               "checksum_s": s_val}
        for h in hs:
            if h.value:
                lib.db2_dist_decref(h)
        X.free()
        grp.close()
    finally:
        if store is not None:
            store.set("db2_scheduler_group_leg", "1")
    return out


LEGS = {}


def run_leg(args) -> dict:
    """One of the side workloads alone (`--leg NAME`), for profiling a single kernel on a small case: `--rows` below
    the full configuration scales the leg down (normal equations and k-means to rows / 16 rows)."""
    import daphne_b200.kernels as K
    from daphne_b200.dist import Comm
    from daphne_b200.lib import lib, require_device
    require_device()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    comm = Comm.from_env("nccl")
    ctx = K.Context(local_rank)
    comm.init_device(ctx)
    host, host_ptr = pinned_array(lib, max(args.rows // 16, 8192) * 512 // COLS + 1, COLS)
    out = LEGS[args.leg](ctx, comm, lib, host, world, args)
    lib.db2_free_host(host_ptr)
    return {"leg": args.leg, "n_gpus": world, **out} if comm.rank == 0 else {}


def _timed(lib, ctx, comm, fn, reps):
    """CUDA-event time of one call of fn in ms: `reps` calls are timed one by one after a warm-up call, the median is
    taken per rank and the max over ranks is returned (neighbouring jobs on the host share its power budget, so single
    repetitions of a power-hungry kernel scatter; the median is the robust figure)."""
    from daphne_b200.lib import check
    stream = C.c_void_p(ctx.stream)
    out = fn()
    comm.barrier()
    check(lib.db2_device_sync())
    times = []
    for _ in range(reps):
        e0, e1 = C.c_void_p(), C.c_void_p()
        check(lib.db2_event_create(C.byref(e0)))
        check(lib.db2_event_create(C.byref(e1)))
        check(lib.db2_event_record(e0, stream))
        out = fn()
        check(lib.db2_event_record(e1, stream))
        check(lib.db2_device_sync())
        ms = C.c_float()
        check(lib.db2_event_elapsed_ms(e0, e1, C.byref(ms)))
        times.append(ms.value)
        check(lib.db2_event_destroy(e0))
        check(lib.db2_event_destroy(e1))
    comm.barrier()
    return comm.max_float(float(np.median(times))), out


def kmeans_leg(ctx, comm, lib, host, world, args) -> dict:
    """K-means assignment + update, 10 iterations, on a 1,000,000 x 64 f64 row shard per GPU (U[0,1)), k = 50; the
    centroid sums and counts are combined across ranks every iteration.  Algorithmic work per row and iteration:
    520 bytes (the row and its assignment) and 6,464 flop (distances 2 k d + update d)."""
    import daphne_b200.kernels as K
    from daphne_b200 import pipelines
    n, d, k, iters = (1_000_000, 64, 50, 10) if args.rows >= ROWS_PER_GPU else (max(args.rows // 16, 4096), 64, 50, 10)
    # X = rand(n, d, 0.0, 1.0, 1, seed) as the DaphneDSL script would produce it (the reference's mt19937 stream),
    # generated straight into the device placement; the initial centroids are 50 rows of rank 0's block
    X = K.randMatrix(ctx, n, d, 0.0, 1.0, 1.0, 3 + comm.rank)
    picks = np.sort(np.random.default_rng(33).choice(n, k, replace=False))
    x0 = K.randMatrix(ctx, n, d, 0.0, 1.0, 1.0, 3).to_numpy() if comm.rank != 0 else X.to_numpy()
    C0 = K.DenseMatrix.from_numpy(ctx, np.ascontiguousarray(x0[picks]))
    del x0
    ms, res = _timed(lib, ctx, comm, lambda: pipelines.kmeans_native(ctx, X, C0, iters), 3)
    per_iter = ms / iters
    peak, kind = measured_peaks()
    return {"workload": f"k-means, {iters} iterations, f64 {n} x {d} per GPU, k = {k}, over {world} GPU(s)",
            "ms_per_iteration": per_iter, "rows_per_s": n * world * iters / (ms * 1e-3),
            "hbm_gbs_at_520B_per_row": n * 520 / (per_iter * 1e-3) / 1e9,
            "hbm_frac_of_" + kind: n * 520 / (per_iter * 1e-3) / 1e9 / peak,
            "fp64_tflops_at_6464_flop_per_row": n * 6464 / (per_iter * 1e-3) / 1e12,
            "fp64_frac_of_peak": n * 6464 / (per_iter * 1e-3) / 1e12 / FP64_PEAK_TFLOPS,
            "centroid_checksum": float(res.C.to_numpy().sum())}


def components_leg(ctx, comm, lib, host, world, args) -> dict:
    """Connected components by label propagation on a symmetric 0/1 CSR graph with 1,000,000 vertices and mean degree 8
    (seed 4), row-sharded over the ranks; the labels are all-gathered every iteration.  Algorithmic bytes per vertex and
    iteration on the reference's layout: 160 (8 entries x (8 + 8) + offsets + 3 vector passes)."""
    import scipy.sparse as sp
    import daphne_b200.kernels as K
    from daphne_b200 import pipelines
    from daphne_b200.dist import row_block
    n, deg = (1_000_000, 8) if args.rows >= ROWS_PER_GPU else (max(args.rows // 16, 4096), 8)
    rng = np.random.default_rng(4)
    m = n * deg // 2
    i, j = rng.integers(0, n, size=int(1.1 * m)), rng.integers(0, n, size=int(1.1 * m))
    keep = i != j
    key = np.unique(np.minimum(i[keep], j[keep]) * n + np.maximum(i[keep], j[keep]))[:m]
    lo, hi = key // n, key % n
    g = sp.csr_matrix((np.ones(2 * key.size), (np.concatenate([lo, hi]), np.concatenate([hi, lo]))), shape=(n, n))
    g.sort_indices()
    r0, r1 = row_block(n, comm.rank, world)
    G = K.CSRMatrix.from_scipy(ctx, g[r0:r1])
    blk = (r0, r1) if world > 1 else None
    ms, res = _timed(lib, ctx, comm, lambda: pipelines.connected_components_native(ctx, G, 1000, blk), 5)
    per_iter = ms / res.iterations
    labels = res.c.to_numpy().ravel()
    peak, kind = measured_peaks()
    # the labels of all shards against scipy's connected components of the same graph: every vertex must carry the
    # largest (1-based) vertex id of its component, so the sums over all vertices must be equal
    total = float(comm.allreduce_numpy(np.array([labels.sum()]), 3)[0]) if world > 1 else float(labels.sum())
    from scipy.sparse import csgraph
    ncomp, comp = csgraph.connected_components(g, directed=False)
    top = np.zeros(ncomp)
    np.maximum.at(top, comp, np.arange(1, n + 1, dtype=np.float64))
    expected = float(top[comp].sum())
    return {"workload": f"connected components, {n} vertices, {2 * key.size} stored entries, rows over {world} GPU(s)",
            "iterations": res.iterations, "ms_per_iteration": per_iter, "ms_total": ms,
            "vertices_per_s": n * res.iterations / (ms * 1e-3),
            "gbs_at_160B_per_vertex": n * 160 / (per_iter * 1e-3) / 1e9,
            "frac_of_" + kind + "_hbm": n * 160 / (per_iter * 1e-3) / 1e9 / peak,
            "components": int(ncomp), "label_checksum_all_ranks": total, "label_checksum_scipy": expected,
            "labels_equal_scipy": bool(total == expected and np.array_equal(labels, top[comp][r0:r1]))}


def f32_matmul_leg(ctx, comm, lib, host, world, args) -> dict:
    """f32 matMul through the tensor-core path (tcgen05 kind::tf32; three MMAs per product for single-precision
    accuracy): 8192^3 per GPU, replicated.  TFLOP/s counts 2 m n k once."""
    import daphne_b200.kernels as K
    m = 8192 if args.rows >= ROWS_PER_GPU else 4096
    rng = np.random.default_rng(7)
    a, b = rng.standard_normal((m, m), dtype=np.float32), rng.standard_normal((m, m), dtype=np.float32)
    A, B = K.DenseMatrix.from_numpy(ctx, a), K.DenseMatrix.from_numpy(ctx, b)
    A.device_ptr()
    B.device_ptr()
    keep = []

    def run():
        keep.clear()
        keep.append(K.matMul(A, B, False, True))
        return keep[0]
    ms, res = _timed(lib, ctx, comm, run, 7)
    got = res.to_numpy()[:64]
    ref = a[:64].astype(np.float64) @ b.astype(np.float64).T
    tf = 2.0 * m * m * m / (ms * 1e-3) / 1e12
    return {"workload": f"f32 {m} x {m} @ t({m} x {m}) per GPU", "ms": ms, "tflops": tf,
            "tf32_mma_tflops_issued": 3 * tf, "tf32_mma_frac_of_nominal_1125": 3 * tf / 1125.0,
            "max_abs_err_vs_f64_64_rows": float(np.abs(got - ref).max())}


def generic_chain_leg(ctx, comm, lib, host, world, args) -> dict:
    """A chain that has no compiled specialisation -- ((X - mu) * w) + 0.5 with rowSums and rowMins -- through the
    run-time form of the fused row pass.  Bytes: X read once (8 B per element) + two row results."""
    import daphne_b200.kernels as K
    from daphne_b200.kernels import AggOpCode as A, BinaryOpCode as B
    from daphne_b200.lib import check
    rows = min(args.rows, 1 << 23)
    cols = 32
    rng = np.random.default_rng(9)
    rows = max(1 << 16, rows >> 16 << 16)
    X = K.DenseMatrix.from_numpy(ctx, np.tile(5.0 + 2.0 * rng.standard_normal((1 << 16, cols)), (rows >> 16, 1)))
    X.device_ptr()
    mu = K.DenseMatrix.from_numpy(ctx, rng.standard_normal((1, cols)))
    w = K.DenseMatrix.from_numpy(ctx, rng.standard_normal((1, cols)) + 3.0)

    def run():
        Z = K.ewBinaryObjSca(B.ADD, K.ewBinaryMat(B.MUL, K.ewBinaryMat(B.SUB, X, mu), w), 0.5)
        r, m = K.aggRow(A.SUM, Z), K.aggRow(A.MIN, Z)
        r.device_ptr()
        return r, m
    # first with the chain read at run time (what serves the calls while the run-time compiler works), then with the
    # kernel the run-time compiler made for this chain
    check(lib.db2_rtc_set_mode(0))
    ms_rt, _ = _timed(lib, ctx, comm, run, 7)
    check(lib.db2_rtc_set_mode(1))
    t0 = time.perf_counter()
    run()
    check(lib.db2_rtc_wait())
    compile_s = time.perf_counter() - t0
    ms, (r, m) = _timed(lib, ctx, comm, run, 7)
    ready, failed = C.c_int(), C.c_int()
    check(lib.db2_rtc_counts(C.byref(ready), None, C.byref(failed)))
    # the same chain on 33 columns: rows that do not start on 16-byte boundaries (chunks copied element by element);
    # without the run-time compiler such layouts are served by the general interpreter
    rows33 = rows // 2
    X33 = K.DenseMatrix.from_numpy(ctx, np.tile(5.0 + 2.0 * rng.standard_normal((1 << 16, 33)), (rows33 >> 16, 1)))
    X33.device_ptr()
    mu33, w33 = (K.DenseMatrix.from_numpy(ctx, rng.standard_normal((1, 33)) + 3.0) for _ in range(2))

    def run33():
        Z = K.ewBinaryObjSca(B.ADD, K.ewBinaryMat(B.MUL, K.ewBinaryMat(B.SUB, X33, mu33), w33), 0.5)
        r33, m33 = K.aggRow(A.SUM, Z), K.aggRow(A.MIN, Z)
        r33.device_ptr()
        return r33, m33
    check(lib.db2_rtc_set_mode(0))
    ms33_interp, _ = _timed(lib, ctx, comm, run33, 5)
    check(lib.db2_rtc_set_mode(2))
    ms33, (r33, m33) = _timed(lib, ctx, comm, run33, 7)
    z33 = (X33.to_numpy()[:4096] - mu33.to_numpy()) * w33.to_numpy() + 0.5
    nbytes33 = rows33 * (33 * 8 + 16)
    nbytes = rows * (cols * 8 + 16)
    peak, _ = measured_peaks()
    xs = X.to_numpy()[:4096]
    z = (xs - mu.to_numpy()) * w.to_numpy() + 0.5
    return {"workload": f"((X - mu) * w) + 0.5 -> rowSums, rowMins on f64 {rows} x {cols} (no compiled-in specialisation)",
            "ms": ms, "hbm_gbs": nbytes / (ms * 1e-3) / 1e9, "hbm_frac_of_measured": nbytes / (ms * 1e-3) / 1e9 / peak,
            "kernel": "compiled at run time for this chain" if ready.value and not failed.value else "chain read at run time",
            "background_compile_s": compile_s,
            "ms_chain_read_at_run_time": ms_rt, "hbm_frac_chain_read_at_run_time": nbytes / (ms_rt * 1e-3) / 1e9 / peak,
            "columns_33": {"rows": rows33, "ms": ms33, "hbm_frac_of_measured": nbytes33 / (ms33 * 1e-3) / 1e9 / peak,
                           "ms_general_interpreter": ms33_interp,
                           "hbm_frac_general_interpreter": nbytes33 / (ms33_interp * 1e-3) / 1e9 / peak,
                           "row_mins_equal_numpy_4096_rows": bool(np.array_equal(m33.to_numpy()[:4096, 0], z33.min(1)))},
            "row_mins_equal_numpy_4096_rows": bool(np.array_equal(m.to_numpy()[:4096, 0], z.min(1))),
            "row_sums_max_rel_err_4096_rows": float(np.abs(r.to_numpy()[:4096, 0] / z.sum(1) - 1.0).max())}


def solve_leg(ctx, comm, lib, host, world, args) -> dict:
    """solve(A, b) alone on the 512 x 512 system of the normal equations (blocked LU with partial pivoting)."""
    import daphne_b200.kernels as K
    n = 512
    rng = np.random.default_rng(11)
    g = rng.standard_normal((4 * n, n))
    a = g.T @ g + 1e-3 * np.eye(n)
    b = rng.standard_normal((n, 1))
    Am, Bm = K.DenseMatrix.from_numpy(ctx, a), K.DenseMatrix.from_numpy(ctx, b)
    Am.device_ptr()
    Bm.device_ptr()
    ms, x = _timed(lib, ctx, comm, lambda: K.solve(Am, Bm), 15)
    xh = x.to_numpy()
    return {"workload": f"solve, f64 {n} x {n}, one right-hand side", "ms": ms,
            "residual_max_abs": float(np.abs(a @ xh - b).max()), "launches_per_solve": 3 * (n // 32) }


LEGS.update({"normal_equations_shard": normal_equations_leg, "normal_equations_full": normal_equations_full_leg,
             "kmeans_shard": kmeans_leg,
             "connected_components": components_leg, "f32_matmul_tcgen05": f32_matmul_leg,
             "scheduler_group": scheduler_group_leg, "generic_chain": generic_chain_leg, "solve_512": solve_leg})


def cpu_baseline(rows: int, cols: int, steps: int = 3, threads: int | None = None, X=None, budget_s: float = 1e9,
                 non_vectorized: bool = True) -> dict:
    """The reference's CPU implementation of the workload on the host cores.  When the reference's vectorized engine
    was built (oracle/_ref/libdaphne_ref_engine.so) it is that engine -- MTWrapper::executeCpuQueues with DAPHNE's
    defaults -- driving the reference's CPU kernels, one worker per host CPU, and beside it the same kernels called
    once on whole matrices (daphne without --vec).  Otherwise the reference's kernels (or their restatement) under a
    row-partitioning thread pool.  Steps are timed one by one (wall clock); the median is reported; after the first
    timed step the number of steps is cut so that the baseline stays inside `budget_s` seconds."""
    from oracle import cpu_pipelines, refengine
    if X is None:
        X = np.empty((rows, cols))
        make_input(rows, cols, SEED, X)
    if refengine.available():
        threads = threads or refengine.default_threads()
        run = lambda: refengine.standardise_aggregate(X, threads, True, results=False)[-1]  # noqa: E731
        kind, how = "reference", refengine.ENGINE
    else:
        k, kind = cpu_pipelines.backend()
        threads = threads or cpu_pipelines.host_threads()

        def run():
            t0 = time.perf_counter()
            cpu_pipelines.standardise_aggregate(X, threads, k)
            t = (time.perf_counter() - t0) * 1e3
            return (0.0, 0.0, 0.0, t)
        how = "the reference's CPU kernels under a row-partitioning thread pool (STATIC), the engine was not built"
    t_begin = time.perf_counter()
    run()  # warm-up
    parts = []
    for i in range(steps):
        parts.append(run())
        per = (time.perf_counter() - t_begin) / (len(parts) + 1)
        if (time.perf_counter() - t_begin) + per > budget_s:
            break
    tot = [p[3] for p in parts]
    t = float(np.median(tot)) * 1e-3
    med = parts[int(np.argsort(tot)[len(tot) // 2])]
    out = {"value": rows / t, "unit": "rows/s", "cores": threads, "kind": kind, "engine": how,
           "sample": f"first {rows} rows x {cols} cols of the N(5,2) seed-{SEED} input, {len(parts)} timed runs after 1 "
                     f"warm-up, median wall time",
           "ms_per_step": t * 1e3, "steps_run": len(parts),
           "ms_column_statistics": med[0], "ms_pipeline": med[1], "ms_idxmax": med[2]}
    if non_vectorized and refengine.available():
        ms = refengine.standardise_aggregate(X, threads, False, results=False)[-1]
        out["non_vectorized"] = {"value": rows / (ms[3] * 1e-3), "unit": "rows/s", "ms_per_step": ms[3], "cores": 1,
                                 "what": "the same kernel sequence called once on whole matrices (no --vec), 1 run"}
    return out


def run_reference(args) -> dict:
    """The reference arm: the reference's CPU engine on the SAME configuration (all rows of one GPU's block).  A step
    takes seconds on the host, so the number of timed steps is cut to what fits about three minutes; the line says
    how many ran."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return {}
    rows = args.rows if args.cpu_rows <= 0 else min(args.rows, args.cpu_rows)
    b = cpu_baseline(rows, COLS, steps=max(1, args.steps), threads=None, budget_s=170.0, non_vectorized=True)
    return {
        "impl": "reference", "metric": "pipeline_rows_per_s", "value": b["value"], "unit": "rows/s",
        "n_gpus": args.gpus, "steps": b["steps_run"], "steps_requested": args.steps, "warmup": 1,
        "ms_per_step": b["ms_per_step"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": {"workload": "cfg2 column standardisation + aggregation (mean, sd, Z=(X-mu)/sd, rowSums(Z^2), "
                               "sum, rowMaxs, idxMax) on f64 %d x %d, N(5,2) seed %d, host cores" % (rows, COLS, SEED),
                   "rows_per_gpu": rows, "cols": COLS, "same_rows_as_gpu_arm": rows == args.rows},
        "cpu_baseline": b,
        "e2e": {"value": b["value"], "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--rows", type=int, default=ROWS_PER_GPU, help="rows per GPU (default: the 4 GiB configuration)")
    ap.add_argument("--no-extra", action="store_true", help="skip the other workloads reported under `extra`")
    ap.add_argument("--cpu-rows", type=int, default=None,
                    help="rows of the CPU run: default 4,194,304 for the cpu_baseline of the GPU arm (a bounded "
                         "sample), all rows for --impl reference")
    ap.add_argument("--leg", default=None, choices=sorted(LEGS),
                    help="run only this side workload (profiling aid); prints its own JSON line")
    args = ap.parse_args()
    if args.cpu_rows is None:
        args.cpu_rows = 0 if args.impl == "reference" else 1 << 22
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.leg and args.impl == "ours":
        line = run_leg(args)
    else:
        line = run_reference(args) if args.impl == "reference" else run_ours(args)
    if line:
        print(json.dumps(line), flush=True)
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        import torch.distributed as dist
        if dist.is_initialized():
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
