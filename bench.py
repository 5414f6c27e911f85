#!/usr/bin/env python
"""Benchmark of the quantized sparse-matrix hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

One "step" is one pass of the hot path over the whole synthetic matrix that is resident on the
GPU.  Prints ONE JSON line (rank 0).  Workloads (seeded synthetic stand-ins for the benchmark
configurations; see cellerator_b200/synth.py):

    c2_forward    1,000,000 x 33,538 uint8 quantized CSR, W 33,538 x 64 bf16      (default)
    c3_transpose  same matrix, G 1,000,000 x 64 fp32 -> G' 33,538 x 64 (+ NCCL allreduce when N > 1)
    c4_4bit       4,000,000 x 4,000 nibble-packed CSR, W 4,000 x 128 bf16 (rows / 8 per GPU)
    c5_bell       2,000,000 x 8,192 Blocked-ELL 32x32, W 8,192 x 256 bf16 (rows / 8 per GPU)

With N > 1 (launched by torch.distributed.run, one rank per GPU) every rank holds its own
row shard of the same size (weak scaling: the per-GPU work is fixed); forward paths use no
collective, the transpose path all-reduces its gene x N partials over NCCL.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_HBM_GBS = 6650.0

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from the ncu
# captures summarised under profiles/ (bytes per stored entry, measured on a smaller case and
# scaled by the entries one launch processes).  None until a capture exists.
NCU_DRAM_BYTES_PER_NNZ = {
    ("c2_forward", "tensor_blocked"): 4.21,   # profiles/qcsr_fwd_blocked__c2_303104_rows.md
    ("c2_forward", "gene_tiled"): 5.32,       # profiles/qcsr_fwd_tiled__c2_75776_rows.md
    ("c2_forward", "warp_per_row"): 5.21,     # profiles/qcsr_fwd_warp_row__c2_60k_rows.md
    ("c4_4bit", "tensor_dense"): 12.8,        # profiles/qcsr_fwd_dense__c4_131072_rows.md
}


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def measured_tensor_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["bf16_tflops"]), "measured"
    except Exception:
        return 1590.0, "fallback"


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100", "-i",
                 str(index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                sm.append(float(parts[0]))
                smax.append(float(parts[1]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[4:8]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ---------------------------------------------------------------------------------------------
# workloads

def algorithmic_bytes(kind, m, k, n, nnz, bits, dense_bytes):
    """Compulsory HBM traffic of one launch (W / scale / offset counted once: they fit in L2)."""
    if kind == "bell":
        return None
    if kind == "transpose":
        return nnz * (bits / 8 + 4) + (m + 1) * 8 + m * n * 4 + k * n * 4 + k * 8
    return nnz * (bits / 8 + 4) + (m + 1) * 8 + m * n * 4 + k * n * dense_bytes + k * 8


def build_workload(name, device, rank, world, seed=0, rows_override=None, multiply="bf16", prepare_matrix=True,
                   persistent_limit_bytes=0, deterministic=False):
    import torch

    from cellerator_b200 import capi, ops, synth
    if name in ("c2_forward", "c3_transpose"):
        cfg = dict(synth.CONFIGS["c2_forward"])
    elif name == "c4_4bit":
        cfg = dict(synth.CONFIGS["c4_4bit"])
        cfg["rows"] //= 8                      # the configuration is an 8-GPU one: 500,000 cells per GPU
    elif name == "c5_bell":
        cfg = dict(synth.CONFIGS["c5_bell"])
        # 250,000 cells per GPU, rounded down to whole 32-cell block rows so that every rank's shard
        # starts on a block-row boundary (249,984)
        cfg["rows"] = cfg["rows"] // 8 // cfg["block_size"] * cfg["block_size"]
    else:
        raise SystemExit(f"unknown workload {name}")
    if rows_override:
        cfg["rows"] = rows_override
    rows = cfg["rows"]
    row_base = rank * rows                     # weak scaling: every rank owns `rows` cells of a world*rows matrix
    g = torch.Generator(device="cpu").manual_seed(1000 + seed)
    wl = {"name": name, "cfg": cfg, "rows": rows, "row_base": row_base}
    if name == "c5_bell":
        x = synth.make_qbell_device(**cfg, device=device, seed=seed, row_base=row_base)
        n = cfg["n"]
        w = (torch.randn(cfg["cols"], n, generator=g) * 0.02).to(torch.bfloat16).to(device)
        out = torch.empty(rows, n, dtype=torch.float32, device=device)
        op = ops.PreparedSpmm(capi.PROJECTION_BLOCKED_ELL, rows, cfg["cols"], n, rows * x.ell_cols, x.bits, x.policy,
                              w.dtype, device)
        units = rows * x.ell_cols              # dense slots of present blocks
        bytes_ = (x.block_col_idx.numel() * 4 + rows * x.row_stride_bytes + cfg["cols"] * n * 2 + cfg["cols"] * 8
                  + rows * n * 4)
        wl.update(x=x, dense=w, out=out, op=op, units=units, bytes=bytes_, kind="bell", n=n,
                  flops=2.0 * rows * x.ell_cols * n)
        return wl
    x = synth.make_qcsr_device(**cfg, device=device, seed=seed, row_base=row_base, total_rows=rows * world)
    torch.cuda.synchronize(device)
    if name == "c3_transpose":
        n = 64
        dense = torch.randn(rows, n, generator=g).to(device)
        out = torch.empty(cfg["cols"], n, dtype=torch.float32, device=device)
        # G is fp32, for which the contract's bound is 1e-4 * ||.||_1 * max|G|: the default arm asks for
        # fp32 products and hands the matrix to prepare, which selects the tensor-core schedule with
        # split products (three bf16 passes rebuild each product to ~3 * 2^-17; "tensor_blocked_x3").
        # --multiply bf16: one pass, values and G rounded to bf16 (1e-2 bound).  --no-prepare-matrix:
        # the fp32-FMA kernel with L2 vector reductions.  --deterministic: fp32 FMAs in a fixed order, gathered
        # gene by gene from a gene-major copy that prepare builds ("gene_gather").
        torch.cuda.synchronize(device)
        t_prepare = time.perf_counter()           # prepare is outside the timed region; its cost is reported
        op = ops.PreparedSpmm(capi.PROJECTION_TRANSPOSE, rows, cfg["cols"], n, x.nnz, x.bits, x.policy, dense.dtype,
                              device, multiply=capi.DTYPE_BF16 if multiply == "bf16" else capi.DTYPE_F32,
                              device_matrix=x if prepare_matrix else None, deterministic=deterministic)
        kind, dbytes = "transpose", 4
    else:
        n = cfg["n"]
        dense = (torch.randn(cfg["cols"], n, generator=g) * 0.02).to(torch.bfloat16).to(device)
        out = torch.empty(rows, n, dtype=torch.float32, device=device)
        # W is bf16 and the contract's tolerance for bf16 W is 1e-2 relative: bf16 products are
        # allowed (tensor-core schedule, one pass).  --multiply f32: fp32 products, rebuilt on the tensor
        # cores from two bf16 passes when the matrix is handed to prepare, or computed by the fp32-FMA
        # kernel with --no-prepare-matrix
        torch.cuda.synchronize(device)
        t_prepare = time.perf_counter()           # prepare is outside the timed region; its cost is reported
        op = ops.PreparedSpmm(capi.PROJECTION_CSR, rows, cfg["cols"], n, x.nnz, x.bits, x.policy, dense.dtype, device,
                              host_row_ptr=x.host_row_ptr,
                              multiply=capi.DTYPE_BF16 if multiply == "bf16" else capi.DTYPE_F32,
                              device_matrix=x if prepare_matrix else None, persistent_limit_bytes=persistent_limit_bytes)
        kind, dbytes = "forward", 2
    torch.cuda.synchronize(device)
    wl.update(x=x, dense=dense, out=out, op=op, units=x.nnz, kind=kind, n=n,
              bytes=algorithmic_bytes(kind, rows, cfg["cols"], n, x.nnz, x.bits, dbytes), flops=2.0 * x.nnz * n,
              prepare_ms=(time.perf_counter() - t_prepare) * 1e3)
    return wl


# ---------------------------------------------------------------------------------------------
# CPU baseline (the oracle is the checker and, here only, the thing timed)

def cpu_sample_from_device(wl, sample_rows):
    """Copies the first `sample_rows` rows of the resident matrix to the host (rebased to 0)."""
    x = wl["x"]
    rows = min(sample_rows, x.rows)
    rp = x.host_row_ptr[: rows + 1]
    hi = int(rp[-1])
    h = dict(rows=rows, cols=x.cols, bits=x.bits, policy=x.policy, row_ptr=rp.copy(),
             col_idx=x.col_idx[:hi].cpu().numpy(), scales=x.scales.cpu().numpy(), offsets=x.offsets.cpu().numpy())
    if x.bits == 8:
        h["packed"] = x.packed[:hi].cpu().numpy()
        h["packed_row_ptr"] = rp.copy()
    else:
        prp = x.packed_row_ptr[: rows + 1].cpu().numpy()
        h["packed"] = x.packed[: int(prp[-1])].cpu().numpy()
        h["packed_row_ptr"] = prp
    return h


def time_cpu_reference(h, dense_host, kind, threads, repeats=1):
    """Times decode + referee over the sample, split into `threads` contiguous row partitions
    (the reference's functions are single-threaded; one partition per host thread).  Uses the
    reference's own compiled sources when oracle/_ref exists, else the C restatement."""
    from concurrent.futures import ThreadPoolExecutor

    import oracle as orc
    use_ref = orc.Reference.available() and h["bits"] in (4, 8) and kind == "forward"
    port = orc.Oracle()
    ref = orc.Reference() if use_ref else None
    rows = h["rows"]
    bounds = np.linspace(0, rows, threads + 1).astype(np.int64)

    def work(i):
        r0, r1 = int(bounds[i]), int(bounds[i + 1])
        if r0 == r1:
            return
        if kind == "transpose":
            port.qcsr_transpose(h["bits"], h["policy"], h["row_ptr"], h["packed_row_ptr"], h["col_idx"], h["packed"],
                                h["scales"], h["offsets"], dense_host, h["cols"], r0, r1)
        elif ref is not None:
            lo, hi = int(h["row_ptr"][r0]), int(h["row_ptr"][r1])
            plo, phi = int(h["packed_row_ptr"][r0]), int(h["packed_row_ptr"][r1])
            rp = h["row_ptr"][r0:r1 + 1] - lo
            dec = ref.unpack_csr(h["bits"], h["policy"], rp, h["packed_row_ptr"][r0:r1 + 1] - plo, h["col_idx"][lo:hi],
                                 h["scales"], h["offsets"], h["packed"][plo:phi], cols=h["cols"])
            ref.spmm_reference(r1 - r0, h["cols"], dense_host.shape[1], rp.astype(np.uint64), h["col_idx"][lo:hi], dec,
                               dense_host)
        else:
            port.qcsr_forward(h["bits"], h["policy"], h["row_ptr"], h["packed_row_ptr"], h["col_idx"], h["packed"],
                              h["scales"], h["offsets"], dense_host, h["cols"], r0, r1)

    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        with ThreadPoolExecutor(max_workers=threads) as pool:
            list(pool.map(work, range(threads)))
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return best, ("reference" if ref is not None else "port")


def cpu_threads():
    try:
        return max(1, min(len(os.sched_getaffinity(0)), 64))
    except Exception:
        return max(1, min(os.cpu_count() or 1, 64))


# ---------------------------------------------------------------------------------------------

def run_ours(args):
    import torch
    import torch.distributed as dist

    from cellerator_b200 import capi, ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        args.gpus = world
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    if args.multiply is None:  # what the contract's tolerance for the workload's dense operand allows
        args.multiply = "f32" if args.workload == "c3_transpose" else "bf16"
    wl = build_workload(args.workload, device, rank, world, rows_override=args.rows, multiply=args.multiply,
                        prepare_matrix=not args.no_prepare_matrix, deterministic=args.deterministic,
                        persistent_limit_bytes=int(args.persistent_limit_gb * 1e9))
    op, x, dense, out = wl["op"], wl["x"], wl["dense"], wl["out"]
    launch = op.make_launch(x, dense, out)
    L = capi.lib()
    transpose_reduce = wl["kind"] == "transpose" and world > 1

    def step():
        op.run_launch(launch)
        if transpose_reduce:
            dist.all_reduce(out, op=dist.ReduceOp.SUM)

    # clocks are sampled from the warm-up on (nvidia-smi needs a moment to start); every sample is
    # taken with the GPU under this load
    sampler = ClockSampler(local) if rank == 0 else None
    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()

    launches0 = L.cb200_kernel_launch_count()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    kstart = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    kstop = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    start.record()
    for i in range(args.steps):
        kstart[i].record()
        op.run_launch(launch)
        kstop[i].record()
        if transpose_reduce:
            dist.all_reduce(out, op=dist.ReduceOp.SUM)
    stop.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    launches = L.cb200_kernel_launch_count() - launches0
    clocks = sampler.stop() if sampler else None
    elapsed_ms = start.elapsed_time(stop)
    kernel_ms = sum(a.elapsed_time(b) for a, b in zip(kstart, kstop)) / args.steps
    t = torch.tensor([elapsed_ms, kernel_ms], dtype=torch.float64, device=device)
    units = torch.tensor([float(wl["units"])], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(units, op=dist.ReduceOp.SUM)
    elapsed_ms, kernel_ms = (float(v) for v in t.tolist())
    total_units = float(units.item())
    ms_per_step = elapsed_ms / args.steps
    value = total_units / (ms_per_step * 1e-3) / 1e9

    # ---- end to end through the host-buffer call (H2D of the matrix + run + D2H of the result)
    e2e = None
    if wl["kind"] in ("forward",) and not args.no_e2e:
        host = ops.HostCsr.from_device(x)                 # pinned host copy of this rank's shard
        w_host = dense.cpu().pin_memory()
        y_host = torch.empty(out.shape, dtype=torch.float32).pin_memory()
        # The matrix arrives from the host on every call, so nothing prepared from its contents may be
        # used: the operation of this leg is prepared without the device matrix (no window-blocked copy;
        # CSR-only schedules on the freshly copied arrays).
        e2e_op = ops.PreparedSpmm(capi.PROJECTION_CSR, wl["rows"], wl["cfg"]["cols"], wl["n"], x.nnz, x.bits, x.policy,
                                  dense.dtype, device, host_row_ptr=x.host_row_ptr,
                                  multiply=capi.DTYPE_BF16 if args.multiply == "bf16" else capi.DTYPE_F32)
        runner = ops.HostForward(e2e_op, x, dense, out, host, w_host, y_host, chunks=args.e2e_chunks)
        runner.run()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e_steps = max(1, min(args.steps, args.e2e_steps))
        es, ee = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        es.record()
        for _ in range(e_steps):
            runner.run()
        ee.record()
        torch.cuda.synchronize()
        e_ms = torch.tensor([es.elapsed_time(ee) / e_steps], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(e_ms, op=dist.ReduceOp.MAX)
        e2e = {"value": total_units / (float(e_ms.item()) * 1e-3) / 1e9, "unit": "Gnnz/s",
               "h2d_bytes_per_step": int(runner.h2d_bytes), "d2h_bytes_per_step": int(runner.d2h_bytes),
               "ms_per_step": float(e_ms.item()), "steps": e_steps, "schedule": e2e_op.schedule}
        del host, runner

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak, peak_kind = measured_peak()
    result = {
        "metric": "quantized CSR SpMM throughput (fused dequant, fp32 accumulate)" if wl["kind"] != "bell"
        else "quantized Blocked-ELL projection throughput",
        "value": value, "unit": "Gnnz/s" if wl["kind"] != "bell" else "Gslot/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": f"u{x.bits} codes -> " + ("bf16 products (tcgen05), f32 accumulate"
                                           if op.schedule in ("tensor_windows", "tensor_blocked", "tensor_dense", "tcgen05_block_rows")
                                           else "split bf16 products (tcgen05, %s passes), f32 accumulate" % op.schedule[-1]
                                           if op.schedule in ("tensor_blocked_x2", "tensor_blocked_x3")
                                           else "f32 products, f32 accumulate"),
        "data": "synthetic (seeded, device-generated; shapes and value model of the named configuration)",
        "config": {"workload": args.workload, "cells_per_gpu": wl["rows"], "genes": wl["cfg"]["cols"], "n": wl["n"],
                   "units_per_gpu": int(wl["units"]), "bits": x.bits,
                   "dense": "bf16" if wl["kind"] != "transpose" else "f32",
                   "parallelism": f"row-sharded x{world}" + (" + NCCL allreduce" if transpose_reduce else ""),
                   "l2": "inputs larger than L2 (126 MB); no flush needed", "schedule": op.schedule,
                   "prepare_ms_once": round(wl.get("prepare_ms", 0.0), 2), "persistent_bytes": op.persistent_bytes},
        "gpu_launches": int(launches),
        "clocks": clocks,
    }
    if wl["kind"] == "bell":
        tpeak, tkind = measured_tensor_peak()
        hbm = wl["bytes"] / (kernel_ms * 1e-3) / 1e9
        result["roofline"] = {"bound": "hbm", "achieved": hbm, "peak": peak, "unit": "GB/s", "frac": hbm / peak,
                              "traffic": None, "peak_source": peak_kind, "kernel_ms": kernel_ms,
                              "tensor_tflops": wl["flops"] / (kernel_ms * 1e-3) / 1e12, "tensor_peak": tpeak,
                              "tensor_peak_source": tkind}
    else:
        achieved = wl["bytes"] / (kernel_ms * 1e-3) / 1e9
        per_nnz = NCU_DRAM_BYTES_PER_NNZ.get((args.workload, op.schedule)) if not args.rows else None
        result["roofline"] = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                              "frac": achieved / peak, "traffic": None if per_nnz is None else per_nnz * wl["units"],
                              "peak_source": peak_kind, "kernel_ms": kernel_ms,
                              "algorithmic_bytes_per_launch": wl["bytes"],
                              "useful_tflops": wl["flops"] / (kernel_ms * 1e-3) / 1e12}
    if e2e is not None:
        result["e2e"] = e2e

    # ---- CPU baseline on a bounded sample of the same workload (rank 0, N = 1 only)
    if world == 1 and wl["kind"] in ("forward", "transpose") and not args.no_cpu:
        threads = cpu_threads()
        sample_rows = min(wl["rows"], args.cpu_rows_per_thread * threads)
        h = cpu_sample_from_device(wl, sample_rows)
        dense_host = dense.float().cpu().numpy() if wl["kind"] == "forward" else dense[:sample_rows].cpu().numpy()
        dt, kind = time_cpu_reference(h, dense_host, wl["kind"], threads)
        nnz_s = int(h["row_ptr"][-1])
        result["cpu_baseline"] = {"value": nnz_s / dt / 1e9, "unit": "Gnnz/s", "cores": threads, "kind": kind,
                                  "sample": f"first {sample_rows} rows ({nnz_s} stored entries), decode + "
                                            f"double-precision referee, one row partition per thread",
                                  "seconds": dt}
    print(json.dumps(result))
    if world > 1:
        dist.destroy_process_group()


def lowering_cpu_seconds(sample):
    """query + materialize of one block size by the reference's host loops (compiled reference sources
    when oracle/_ref exists, else the restatement in oracle.c); single-threaded, as shipped."""
    import oracle as orc
    orc.build()
    lib, kind = (orc.Reference(), "reference") if orc.Reference.available() else (orc.Oracle(), "port")
    t0 = time.perf_counter()
    status, geo, _, _, _ = lib.bell_lowering(sample["row_offsets"], sample["feature_ids"], sample["values"], sample["features"],
                                             sample["fb_offsets"], sample["fperm"], sample["rperm"], sample["block_size"])
    dt = time.perf_counter() - t0
    if status != 0 or geo["state"] != 0:
        raise SystemExit(f"CPU lowering failed: status {status}, state {geo['state']}")
    return dt, kind


def lowering_sample(low_in, block_size, sample_rows):
    per_row = low_in["per_row"]
    return dict(row_offsets=low_in["row_offsets"][: sample_rows + 1].cpu().numpy().view(np.uint32),
                feature_ids=low_in["feature_ids"][: sample_rows * per_row].cpu().numpy().view(np.uint32),
                values=low_in["values"][: sample_rows * per_row].cpu().numpy(), features=low_in["features"],
                fb_offsets=low_in["fb_offsets"], fperm=low_in["fperm"].cpu().numpy().view(np.uint32),
                rperm=np.arange(sample_rows, dtype=np.uint32), block_size=block_size)


def run_lowering(args):
    """Workload c5_lowering: the CSR -> physical Blocked-ELL lowering (query + materialize, block size 32)
    of the Blocked-ELL configuration's shard, one-byte codes.  A step lowers the resident CSR once."""
    import torch
    import torch.distributed as dist

    from cellerator_b200 import capi, ops, synth
    rank, local = int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    cfg = dict(synth.CONFIGS["c5_bell"])
    bs = cfg["block_size"]
    rows = args.rows or cfg["rows"] // 8 // bs * bs
    low_in = synth.make_lowering_device(**{**cfg, "rows": rows}, device=device, seed=rank)
    low = ops.BellLowering(low_in["row_offsets"], low_in["feature_ids"], low_in["values"], low_in["features"],
                           low_in["fb_offsets"], low_in["fperm"], low_in["rperm"], device)
    L = capi.lib()
    state = {}

    def step():
        state["geo"] = low.query(bs)
        state["out"] = None                      # the previous step's buffers go back to the allocator first
        state["out"] = low.materialize(state["geo"])

    sampler = ClockSampler(local) if rank == 0 else None
    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    launches0 = L.cb200_kernel_launch_count()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        step()
    stop.record()
    torch.cuda.synchronize()
    launches = L.cb200_kernel_launch_count() - launches0
    clocks = sampler.stop() if sampler else None
    t = torch.tensor([start.elapsed_time(stop)], dtype=torch.float64, device=device)
    units = torch.tensor([float(low.nnz)], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(units, op=dist.ReduceOp.SUM)
    ms_per_step = float(t.item()) / args.steps
    geo = state["geo"]

    # ---- end to end: the CSR in pinned host memory -> device, lowered, the Blocked-ELL arrays back to the host
    e2e = None
    if not args.no_e2e:
        host_in = {k: low_in[k].cpu().pin_memory() for k in ("row_offsets", "feature_ids", "values")}
        dev_in = {k: torch.empty_like(low_in[k]) for k in host_in}
        low_e = ops.BellLowering(dev_in["row_offsets"], dev_in["feature_ids"], dev_in["values"], low_in["features"],
                                 low_in["fb_offsets"], low_in["fperm"], low_in["rperm"], device)
        host_cols = torch.empty(int(geo.column_index_count), dtype=torch.int32).pin_memory()
        host_vals = torch.empty(int(geo.value_bytes), dtype=torch.uint8).pin_memory()

        def e2e_step():
            for k in host_in:
                dev_in[k].copy_(host_in[k], non_blocking=True)
            g = low_e.query(bs)
            _, cols, vals = low_e.materialize(g)
            host_cols.copy_(cols, non_blocking=True)
            host_vals.copy_(vals, non_blocking=True)

        e2e_step()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e_steps = max(1, min(args.steps, args.e2e_steps))
        es, ee = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        es.record()
        for _ in range(e_steps):
            e2e_step()
        ee.record()
        torch.cuda.synchronize()
        e_ms = torch.tensor([es.elapsed_time(ee) / e_steps], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(e_ms, op=dist.ReduceOp.MAX)
        e2e = {"value": float(units.item()) / (float(e_ms.item()) * 1e-3) / 1e9, "unit": "Gnnz/s",
               "h2d_bytes_per_step": int(sum(v.numel() * v.element_size() for v in host_in.values())),
               "d2h_bytes_per_step": int(host_cols.numel() * 4 + host_vals.numel()), "ms_per_step": float(e_ms.item()),
               "steps": e_steps}
    if rank != 0:
        dist.destroy_process_group()
        return
    # compulsory traffic: offsets, ids (read by the query and again by the fill), codes, the zeroed and
    # written value array, the column indices
    bytes_ = (2 * (rows + 1) * 4 + 2 * low.nnz * 4 + low.nnz * low.value_size + geo.value_bytes
              + geo.column_index_count * 4)
    peak, peak_kind = measured_peak()
    achieved = bytes_ / (ms_per_step * 1e-3) / 1e9
    result = {
        "metric": "CSR -> Blocked-ELL lowering throughput (query + materialize)",
        "value": float(units.item()) / (ms_per_step * 1e-3) / 1e9, "unit": "Gnnz/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "u8 codes copied bytewise, u32 indices",
        "data": "synthetic (seeded, device-generated; shape of the Blocked-ELL configuration)",
        "config": {"workload": "c5_lowering", "cells_per_gpu": rows, "genes": cfg["cols"], "block_size": bs,
                   "ell_blocks_per_row": geo.ell_blocks_per_row, "units_per_gpu": low.nnz,
                   "value_bytes": int(geo.value_bytes), "parallelism": f"row-sharded x{world}",
                   "l2": "inputs and outputs larger than L2 (126 MB); no flush needed"},
        "gpu_launches": int(launches), "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": None, "peak_source": peak_kind, "kernel_ms": ms_per_step,
                     "algorithmic_bytes_per_launch": bytes_},
    }
    if e2e is not None:
        result["e2e"] = e2e
    if world == 1 and not args.no_cpu:
        sample_rows = min(rows, 20000 // bs * bs)
        dt, kind = lowering_cpu_seconds(lowering_sample(low_in, bs, sample_rows))
        nnz_s = sample_rows * low_in["per_row"]
        result["cpu_baseline"] = {"value": nnz_s / dt / 1e9, "unit": "Gnnz/s", "cores": 1, "kind": kind,
                                  "sample": f"first {sample_rows} rows ({nnz_s} stored entries), query + materialize, "
                                            f"the reference's single-threaded host loops", "seconds": dt}
    print(json.dumps(result))
    if world > 1:
        dist.destroy_process_group()


def run_reference(args):
    """The reference's CPU implementation of the path, timed on the host cores (rank 0 only)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    threads = cpu_threads()
    kind = "transpose" if args.workload == "c3_transpose" else "forward"
    if args.workload == "c5_lowering":
        # the reference's single-threaded host loops on a bounded sample of the Blocked-ELL configuration
        from cellerator_b200 import synth
        cfg = dict(synth.CONFIGS["c5_bell"])
        bs, sample_rows = cfg["block_size"], 20000 // cfg["block_size"] * cfg["block_size"]
        low_in = synth.make_lowering_device(**{**cfg, "rows": sample_rows}, device=torch.device("cpu"), seed=0)
        sample = lowering_sample(low_in, bs, sample_rows)
        nnz = sample_rows * low_in["per_row"]
        for _ in range(args.warmup):
            lowering_cpu_seconds(sample)
        times, impl_kind = [], "port"
        for _ in range(args.steps):
            dt, impl_kind = lowering_cpu_seconds(sample)
            times.append(dt)
        dt = sum(times) / len(times)
        value = nnz / dt / 1e9
        print(json.dumps({
            "impl": "reference", "metric": "CSR -> Blocked-ELL lowering throughput (query + materialize)",
            "value": value, "unit": "Gnnz/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "u8 codes copied bytewise, u32 indices", "data": "synthetic (same generator as the GPU arm)",
            "config": {"workload": "c5_lowering", "genes": cfg["cols"], "block_size": bs, "sample_rows": sample_rows,
                       "sample_nnz": nnz},
            "cpu_baseline": {"value": value, "unit": "Gnnz/s", "cores": 1, "kind": impl_kind,
                             "sample": f"first {sample_rows} rows ({nnz} stored entries) per step"},
            "e2e": {"value": value, "unit": "Gnnz/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0,
        }))
        return
    if args.workload == "c5_bell":
        print(json.dumps({"impl": "reference", "unavailable": "the CPU arm covers the CSR workloads and the lowering only"}))
        return
    sample_rows = args.cpu_rows_per_thread * threads
    if torch.cuda.is_available():
        device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
        wl = build_workload(args.workload, device, 0, 1, rows_override=max(sample_rows, 1024))
        h = cpu_sample_from_device(wl, sample_rows)
        dense_host = (wl["dense"].float().cpu().numpy() if kind == "forward" else wl["dense"][:sample_rows].cpu().numpy())
        cfg, n = wl["cfg"], wl["n"]
        del wl
        torch.cuda.empty_cache()
    else:
        from cellerator_b200 import synth
        cfg = dict(synth.CONFIGS["c4_4bit" if args.workload == "c4_4bit" else "c2_forward"])
        n = 64 if kind == "transpose" else cfg["n"]
        sample_rows = min(sample_rows, 2000)
        h = synth.make_qcsr_host(**{**cfg, "rows": sample_rows}, seed=0)
        rng = np.random.default_rng(1000)
        dense_host = (rng.normal(0, 0.02, size=(cfg["cols"], n)) if kind == "forward"
                      else rng.normal(0, 1, size=(sample_rows, n))).astype(np.float32)
    nnz = int(h["row_ptr"][-1])
    for _ in range(args.warmup):
        time_cpu_reference(h, dense_host, kind, threads)
    times, impl_kind = [], "port"
    for _ in range(args.steps):
        dt, impl_kind = time_cpu_reference(h, dense_host, kind, threads)
        times.append(dt)
    dt = sum(times) / len(times)
    value = nnz / dt / 1e9
    print(json.dumps({
        "impl": "reference", "metric": "quantized CSR SpMM throughput (fused dequant, fp32 accumulate)",
        "value": value, "unit": "Gnnz/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f64 accumulate (CPU referee)", "data": "synthetic (same generator as the GPU arm)",
        "config": {"workload": args.workload, "genes": cfg["cols"], "n": n, "sample_rows": h["rows"],
                   "sample_nnz": nnz},
        "cpu_baseline": {"value": value, "unit": "Gnnz/s", "cores": threads, "kind": impl_kind,
                         "sample": f"first {h['rows']} rows ({nnz} stored entries) per step"},
        "e2e": {"value": value, "unit": "Gnnz/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2_forward", choices=["c2_forward", "c3_transpose", "c4_4bit", "c5_bell", "c5_lowering"])
    ap.add_argument("--rows", type=int, default=0, help="override cells per GPU (profiling on a small case)")
    ap.add_argument("--deterministic", action="store_true",
                    help="c3_transpose: ask prepare for the schedule whose fp32 sums have a fixed order")
    ap.add_argument("--no-prepare-matrix", action="store_true",
                    help="do not hand the matrix to prepare: no window-blocked copy, CSR-only schedules")
    ap.add_argument("--persistent-limit-gb", type=float, default=0.0,
                    help="device memory prepare may keep per GPU (0 = no limit); below rows x genes x 2 bytes the forward "
                         "projection keeps the window-blocked copy (tensor_blocked) instead of dense tiles (tensor_dense)")
    ap.add_argument("--multiply", default=None, choices=["bf16", "f32"],
                    help="products: bf16 (tensor cores; default where the dense operand is bf16) or exact fp32 "
                         "(CUDA cores; default for the transpose, whose G is fp32)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--e2e-chunks", type=int, default=16)
    ap.add_argument("--cpu-rows-per-thread", type=int, default=4000,
                    help="rows of the CPU sample per host thread (4,000 rows x 16 threads: ~25 CPU-seconds per pass)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "c5_lowering":
        run_lowering(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
