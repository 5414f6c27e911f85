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
    ("c4_4bit", "tensor_codes"): 6.6,         # profiles/qcsr_fwd_codes__c4_131072_rows.md
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
                   persistent_limit_bytes=0, deterministic=False, strong=False, reuse_x=None):
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
    if strong:                                 # strong scaling: the configuration's cells divided over the ranks
        unit = cfg.get("block_size", 256)      # whole block rows / 256-row groups per rank
        cfg["rows"] = max(unit, cfg["rows"] // world // unit * unit)
    rows = cfg["rows"]
    row_base = rank * rows                     # every rank owns `rows` cells of a world*rows matrix
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
    # the transpose configuration is the forward one's matrix: a resident copy is used as it is
    x = reuse_x if reuse_x is not None else synth.make_qcsr_device(**cfg, device=device, seed=seed, row_base=row_base,
                                                                    total_rows=rows * world)
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
        def make_op():
            return ops.PreparedSpmm(capi.PROJECTION_TRANSPOSE, rows, cfg["cols"], n, x.nnz, x.bits, x.policy, dense.dtype,
                                    device, multiply=capi.DTYPE_BF16 if multiply == "bf16" else capi.DTYPE_F32,
                                    device_matrix=x if prepare_matrix else None, deterministic=deterministic)
        op = make_op()
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
        host_row_ptr = x.host_row_ptr

        def make_op():
            return ops.PreparedSpmm(capi.PROJECTION_CSR, rows, cfg["cols"], n, x.nnz, x.bits, x.policy, dense.dtype, device,
                                    host_row_ptr=host_row_ptr,
                                    multiply=capi.DTYPE_BF16 if multiply == "bf16" else capi.DTYPE_F32,
                                    device_matrix=x if prepare_matrix else None, persistent_limit_bytes=persistent_limit_bytes)
        op = make_op()
        kind, dbytes = "forward", 2
    torch.cuda.synchronize(device)
    first_ms = (time.perf_counter() - t_prepare) * 1e3
    # The first prepare of a process also pays for loading the library's kernels and the first large allocations.
    # What a matrix costs is the second one: the operation is destroyed and prepared again, and that time is reported
    # (the first one beside it).
    prepare_ms = first_ms
    if op.persistent_bytes > 0:
        op.close()
        torch.cuda.synchronize(device)
        t_prepare = time.perf_counter()
        op = make_op()
        torch.cuda.synchronize(device)
        prepare_ms = (time.perf_counter() - t_prepare) * 1e3
    wl.update(x=x, dense=dense, out=out, op=op, units=x.nnz, kind=kind, n=n,
              bytes=algorithmic_bytes(kind, rows, cfg["cols"], n, x.nnz, x.bits, dbytes), flops=2.0 * x.nnz * n,
              prepare_ms=prepare_ms, prepare_first_ms=first_ms)
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
# timing, statistics, parity of what was timed

def summary_stats(samples_ms):
    """median / MAD / p05 / p95 / mean of per-step device times, the summary the reference's benches print
    (bench/math/benchmark_support.hh:54-102)."""
    a = np.sort(np.asarray(samples_ms, dtype=np.float64))
    if a.size == 0:
        return {}
    med = float(np.median(a))
    return {"median_ms": med, "mad_ms": float(np.median(np.abs(a - med))), "p05_ms": float(np.percentile(a, 5)),
            "p95_ms": float(np.percentile(a, 95)), "mean_ms": float(a.mean()), "min_ms": float(a[0]), "samples": int(a.size)}


def timed_loop(step, steps, warmup, device, counter=None):
    """`warmup` untimed calls, then `steps` calls, each bracketed by CUDA events on the current stream.
    Returns (total ms over the timed calls, per-step ms list[, kernel launches inside the timed calls])."""
    import torch
    for _ in range(warmup):
        step()
    torch.cuda.synchronize(device)
    begin = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    end = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    count0 = counter() if counter else 0
    for i in range(steps):
        begin[i].record()
        step()
        end[i].record()
    torch.cuda.synchronize(device)
    times = (begin[0].elapsed_time(end[-1]), [a.elapsed_time(b) for a, b in zip(begin, end)])
    return times + (counter() - count0,) if counter else times


def host_rows(x, r0, r1):
    """Rows [r0, r1) of a device-resident quantized CSR as a host matrix of its own (offsets rebased)."""
    rp = x.host_row_ptr
    lo, hi = int(rp[r0]), int(rp[r1])
    h = dict(rows=r1 - r0, cols=x.cols, bits=x.bits, policy=x.policy, row_ptr=rp[r0:r1 + 1] - lo,
             col_idx=x.col_idx[lo:hi].cpu().numpy(), scales=x.scales.cpu().numpy(), offsets=x.offsets.cpu().numpy())
    if x.bits == 8:
        h["packed"], h["packed_row_ptr"] = x.packed[lo:hi].cpu().numpy(), h["row_ptr"]
    else:
        prp = x.packed_row_ptr[r0:r1 + 1].cpu().numpy()
        h["packed"], h["packed_row_ptr"] = x.packed[int(prp[0]):int(prp[-1])].cpu().numpy(), prp - prp[0]
    return h


def parity_of_what_ran(wl, op, bf16_products, rows_per_site=16):
    """Checks the output the timed loop left behind (forward, Blocked-ELL) or a row-range relaunch of the same
    prepared operation (transpose) against the CPU oracle, outside the timed region, and reads the status
    word of the kernels' bounded waits.  -> dict for the JSON line; "ok" False fails the run."""
    import oracle as orc
    checker = orc.Oracle()
    x, dense, out = wl["x"], wl["dense"], wl["out"]
    try:
        word = op.status()
    except Exception as e:                       # CB200_STATUS_DEVICE_WAIT_TIMEOUT
        return {"ok": False, "status_word": 1, "error": str(e)}
    rel_bound = 1e-2 if bf16_products else 1e-4
    worst_rel, worst_scaled, rows_checked = 0.0, 0.0, 0
    if wl["kind"] == "bell":
        bs, width = x.block_size, x.ell_cols // x.block_size
        w_host = dense.float().cpu().numpy()
        bci = x.block_col_idx.view(-1, width)
        for b0 in (0, x.rows // bs // 2, x.rows // bs - 1):
            r0, r1 = b0 * bs, min(x.rows, (b0 + 1) * bs)
            packed = x.packed[r0 * x.row_stride_bytes: r1 * x.row_stride_bytes].cpu().numpy()
            ro, cols, vals = checker.bell_to_csr(x.bits, x.policy, r1 - r0, x.cols, bs, x.ell_cols, x.row_stride_bytes,
                                                 bci[b0:b0 + 1].cpu().numpy().view(np.uint32).ravel(), x.scales.cpu().numpy(),
                                                 x.offsets.cpu().numpy(), packed)
            ref = checker.spmm_reference(r1 - r0, x.cols, wl["n"], ro, cols, vals, w_host)
            l1 = np.add.reduceat(np.abs(vals.astype(np.float64)), ro[:-1].astype(np.int64))
            scale = l1[:, None] * float(np.abs(w_host).max()) + 1e-30
            err = np.abs(out[r0:r1].cpu().numpy().astype(np.float64) - ref)
            worst_scaled = max(worst_scaled, float(np.max(err / scale)))
            worst_rel = max(worst_rel, float(np.max(err / np.maximum(np.abs(ref), 1e-2 * scale))))
            rows_checked += r1 - r0
        ok = word == 0 and worst_rel <= 1e-2
        return {"ok": ok, "status_word": word, "rows": rows_checked, "max_rel": worst_rel, "bound": 1e-2,
                "max_over_row_l1_scale": worst_scaled, "against": "CPU oracle (decode + double-precision referee), sampled block rows of the timed output"}
    if wl["kind"] == "transpose":
        # a partial over 1,024 cells, relaunched on the same prepared operation
        import torch
        r0 = (x.rows // 2 // 256) * 256 + 77 if x.rows > 4096 else 0
        r1 = min(x.rows, r0 + 1024)
        part = torch.empty_like(out)
        op.run(x, dense, part, row_begin=r0, row_end=r1)
        try:
            word = max(word, op.status())
        except Exception as e:
            return {"ok": False, "status_word": 1, "error": str(e)}
        h = host_rows(x, r0, r1)
        g_host = dense[r0:r1].cpu().numpy()
        ref = checker.qcsr_transpose(h["bits"], h["policy"], h["row_ptr"], h["packed_row_ptr"], h["col_idx"], h["packed"], h["scales"],
                                     h["offsets"], g_host, x.cols)
        dec = checker.unpack_csr(h["bits"], h["policy"], h["row_ptr"], h["packed_row_ptr"], h["col_idx"], h["scales"], h["offsets"],
                                 h["packed"])
        cl1 = np.zeros(x.cols)
        np.add.at(cl1, h["col_idx"], np.abs(dec.astype(np.float64)))
        scale = cl1[:, None] * float(np.abs(g_host).max()) + 1e-30
        worst_scaled = float(np.max(np.abs(part.cpu().numpy().astype(np.float64) - ref) / scale))
        ok = word == 0 and worst_scaled <= rel_bound
        return {"ok": ok, "status_word": word, "rows": r1 - r0, "max_over_column_l1_scale": worst_scaled, "bound": rel_bound,
                "against": f"CPU oracle partial over cells [{r0},{r1}), relaunched on the timed prepared operation"}
    w_host = dense.float().cpu().numpy()
    wmax = float(np.abs(w_host).max())
    sites = sorted({0, x.rows // 3, (2 * x.rows) // 3, max(0, x.rows - rows_per_site)})
    for r0 in sites:
        r1 = min(x.rows, r0 + rows_per_site)
        h = host_rows(x, r0, r1)
        ref = checker.qcsr_forward(h["bits"], h["policy"], h["row_ptr"], h["packed_row_ptr"], h["col_idx"], h["packed"], h["scales"],
                                   h["offsets"], w_host, x.cols)
        dec = checker.unpack_csr(h["bits"], h["policy"], h["row_ptr"], h["packed_row_ptr"], h["col_idx"], h["scales"], h["offsets"],
                                 h["packed"])
        l1 = np.zeros(r1 - r0)
        counts = np.diff(h["row_ptr"])
        if len(dec):
            l1[counts > 0] = np.add.reduceat(np.abs(dec.astype(np.float64)), h["row_ptr"][:-1][counts > 0])
        scale = l1[:, None] * wmax + 1e-30
        err = np.abs(out[r0:r1].cpu().numpy().astype(np.float64) - ref)
        worst_scaled = max(worst_scaled, float(np.max(err / scale)))
        worst_rel = max(worst_rel, float(np.max(err / np.maximum(np.abs(ref), 1e-2 * scale))))
        rows_checked += r1 - r0
    # bf16 products: the contract's 1e-2 relative (floor 1e-2 * ||row||_1 * max|W|); fp32 products: 1e-4 * ||row||_1 * max|W|
    ok = word == 0 and (worst_rel <= 1e-2 if bf16_products else worst_scaled <= 1e-4)
    return {"ok": ok, "status_word": word, "rows": rows_checked, "max_rel": worst_rel, "bound": 1e-2 if bf16_products else 1e-4,
            "max_over_row_l1_scale": worst_scaled, "against": "CPU oracle (decode + double-precision referee), sampled rows of the timed output"}


class TransposeFleet:
    """One slot of the product's multi-GPU layer per process: the transpose partial and its NCCL all-reduce are one
    call of the C ABI (cb200_fleet_run_transpose), on torch's current stream.  torch.distributed only carries the
    128-byte unique id from rank 0 to the others."""

    def __init__(self, device, rank, world):
        import ctypes as C

        import torch
        import torch.distributed as dist

        from cellerator_b200 import capi
        self.C, self.capi, self.L = C, capi, capi.lib()
        uid = torch.zeros(128, dtype=torch.uint8, device=device)
        if world > 1:
            if rank == 0:
                raw = (C.c_uint8 * 128)()
                capi.check(self.L.cb200_fleet_unique_id(None, raw))
                uid.copy_(torch.frombuffer(bytearray(raw), dtype=torch.uint8))
            dist.broadcast(uid, src=0)
        self._uid = (C.c_uint8 * 128).from_buffer_copy(uid.cpu().numpy().tobytes())
        o = capi.header(capi.FleetOptions())
        self._devs = (C.c_int32 * 1)(device.index)
        self._streams = (C.c_void_p * 1)(torch.cuda.current_stream(device).cuda_stream)
        o.device_count, o.devices, o.streams = 1, self._devs, self._streams
        o.world_size, o.world_rank = world, rank
        o.nccl_unique_id = C.cast(self._uid, C.c_void_p) if world > 1 else None
        self.handle = C.c_void_p()
        capi.check(self.L.cb200_fleet_create(C.byref(o), C.byref(self.handle)))
        if world > 1 and not self.L.cb200_fleet_communicator_ready(self.handle):
            raise SystemExit("the fleet's NCCL communicator is not ready")
        self.slots = (C.c_uint32 * 1)(0)

    def run_transpose(self, op, launch):
        prepared = (self.C.c_void_p * 1)(op.handle.value)
        launches = (self.capi.Launch * 1)(launch)
        self.capi.check(self.L.cb200_fleet_run_transpose(self.handle, self.slots, 1, prepared, launches))

    def allreduce(self, t):
        bufs = (self.C.c_void_p * 1)(t.data_ptr())
        self.capi.check(self.L.cb200_fleet_allreduce_sum_f32(self.handle, self.slots, 1, bufs, bufs, t.numel()))

    def close(self):
        if self.handle:
            self.L.cb200_fleet_destroy(self.handle)
            self.handle = self.C.c_void_p()


def measure_workload(name, args, device, rank, world, steps, warmup, fleet, multiply=None, prepare_matrix=True, check=True,
                     reuse_x=None):
    """Builds one workload, times `steps` passes with per-step events, checks what ran.  -> (record, workload)."""
    import torch
    import torch.distributed as dist

    from cellerator_b200 import capi
    if multiply is None:
        multiply = "f32" if name == "c3_transpose" else "bf16"
    wl = build_workload(name, device, rank, world, rows_override=args.rows, multiply=multiply, prepare_matrix=prepare_matrix,
                        deterministic=args.deterministic and name == "c3_transpose",
                        persistent_limit_bytes=int(args.persistent_limit_gb * 1e9), strong=args.scaling == "strong", reuse_x=reuse_x)
    op, x, dense, out = wl["op"], wl["x"], wl["dense"], wl["out"]
    launch = op.make_launch(x, dense, out)
    transpose = wl["kind"] == "transpose"
    if transpose:
        step = lambda: fleet.run_transpose(op, launch)          # partial + NCCL all-reduce, one C-ABI call
    else:
        step = lambda: op.run_launch(launch)
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    L = capi.lib()
    total_ms, per_step, launches = timed_loop(step, steps, max(warmup, 3), device, counter=L.cb200_kernel_launch_count)
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    rec = {"schedule": op.schedule, "steps": steps, "ms_per_step": total_ms / steps, "step_ms": summary_stats(per_step),
           "rows": wl["rows"], "cols": wl["cfg"]["cols"], "n": wl["n"], "bits": x.bits,
           "units_per_gpu": int(wl["units"]), "gpu_launches": int(launches),
           "prepare_ms_once": round(wl.get("prepare_ms", 0.0), 2), "prepare_ms_first_in_process": round(wl.get("prepare_first_ms", 0.0), 2),
           "persistent_bytes": op.persistent_bytes}
    if transpose:
        # the two halves of a step, timed apart: the partial alone, and the all-reduce alone (back to back)
        _, k_ms = timed_loop(lambda: op.run_launch(launch), min(steps, 5), 1, device)
        rec["ms_kernel"] = float(np.median(k_ms))
        if world > 1:
            _, a_ms = timed_loop(lambda: fleet.allreduce(out), 20, 3, device)
            rec["ms_allreduce"] = float(np.median(a_ms))
            rec["allreduce_bytes"] = int(out.numel() * 4)
    t = torch.tensor([rec["ms_per_step"], rec["step_ms"]["median_ms"], rec.get("ms_kernel", 0.0), rec.get("ms_allreduce", 0.0)],
                     dtype=torch.float64, device=device)
    units = torch.tensor([float(wl["units"])], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(units, op=dist.ReduceOp.SUM)
    rec["ms_per_step"], median_ms = float(t[0]), float(t[1])
    if transpose:
        rec["ms_kernel"] = float(t[2])
        if world > 1:
            rec["ms_allreduce"] = float(t[3])
    rec["total_units"] = float(units.item())
    rec["value"] = rec["total_units"] / (rec["ms_per_step"] * 1e-3) / 1e9
    rec["value_at_median"] = rec["total_units"] / (median_ms * 1e-3) / 1e9
    peak, peak_kind = measured_peak()
    kernel_ms = rec["ms_kernel"] if transpose else median_ms
    rec["kernel_ms"] = kernel_ms
    if wl["kind"] == "bell":
        tpeak, tkind = measured_tensor_peak()
        hbm = wl["bytes"] / (kernel_ms * 1e-3) / 1e9
        rec["roofline"] = {"bound": "hbm", "achieved": hbm, "peak": peak, "unit": "GB/s", "frac": hbm / peak, "traffic": None,
                           "peak_source": peak_kind, "kernel_ms": kernel_ms, "algorithmic_bytes_per_launch": wl["bytes"],
                           "tensor_tflops": wl["flops"] / (kernel_ms * 1e-3) / 1e12, "tensor_peak": tpeak, "tensor_peak_source": tkind}
    else:
        achieved = wl["bytes"] / (kernel_ms * 1e-3) / 1e9
        per_nnz = NCU_DRAM_BYTES_PER_NNZ.get((name, op.schedule)) if not args.rows else None
        rec["roofline"] = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                           "traffic": None if per_nnz is None else per_nnz * wl["units"], "peak_source": peak_kind,
                           "kernel_ms": kernel_ms, "algorithmic_bytes_per_launch": wl["bytes"],
                           "useful_tflops": wl["flops"] / (kernel_ms * 1e-3) / 1e12}
    rec["frac"] = rec["roofline"]["frac"]
    if check and rank == 0:
        bf16_products = op.schedule in ("tensor_windows", "tensor_blocked", "tensor_dense", "tensor_codes", "tcgen05_block_rows")
        rec["parity_check"] = parity_of_what_ran(wl, op, bf16_products)
    return rec, wl


def run_ours(args):
    import ctypes as C

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
    fleet = TransposeFleet(device, rank, world)
    L = capi.lib()

    # clocks are sampled from the warm-up on (nvidia-smi needs a moment to start); every sample is taken with
    # the GPU under this load
    sampler = ClockSampler(local) if rank == 0 else None
    main, wl = measure_workload(args.workload, args, device, rank, world, args.steps, args.warmup, fleet, multiply=args.multiply,
                                prepare_matrix=not args.no_prepare_matrix)
    clocks = sampler.stop() if sampler else None
    op, x, dense, out = wl["op"], wl["x"], wl["dense"], wl["out"]
    total_units = main["total_units"]
    default_arm = args.workload == "c2_forward" and args.multiply in (None, "bf16") and not args.no_prepare_matrix

    # ---- the same pass with the north star's arithmetic: codes and indices read at launch, scale and zero-point
    # applied in registers, fp32 products on the CUDA cores (no prepared copy)
    exact_arm = None
    if default_arm and not args.no_extras:
        ex = ops.PreparedSpmm(capi.PROJECTION_CSR, wl["rows"], wl["cfg"]["cols"], wl["n"], x.nnz, x.bits, x.policy, dense.dtype, device,
                              host_row_ptr=x.host_row_ptr, multiply=capi.DTYPE_F32)
        ex_out = torch.empty_like(out)
        ex_launch = ex.make_launch(x, dense, ex_out)
        _, ex_ms = timed_loop(lambda: ex.run_launch(ex_launch), 5, 2, device)
        t = torch.tensor([float(np.median(ex_ms))], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ex_med = float(t.item())
        peak, _ = measured_peak()
        exact_arm = {"schedule": ex.schedule, "products": "fp32 FMA, decode in registers at launch", "steps": 5,
                     "ms_per_step": ex_med, "value": total_units / (ex_med * 1e-3) / 1e9, "unit": "Gnnz/s",
                     "frac": wl["bytes"] / (ex_med * 1e-3) / 1e9 / peak}
        if rank == 0:
            exact_arm["parity_check"] = parity_of_what_ran(dict(wl, out=ex_out), ex, False)
        ex.close()
        del ex_out, ex_launch

    # ---- strong-scaling point: the configuration's cells split over the ranks (rows / world of this rank's shard,
    # whole 256-row groups), same prepared operation
    strong = None
    if world > 1 and wl["kind"] == "forward" and not args.no_extras and args.scaling == "weak":
        part_rows = max(256, (wl["rows"] // world) // 256 * 256)
        part = op.make_launch(x, dense, out, row_begin=0, row_end=part_rows)
        _, s_ms = timed_loop(lambda: op.run_launch(part), 10, 3, device)
        part_units = float(x.host_row_ptr[part_rows])
        t = torch.tensor([float(np.median(s_ms))], dtype=torch.float64, device=device)
        u = torch.tensor([part_units], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(u, op=dist.ReduceOp.SUM)
        del part
        strong = {"cells_per_gpu": part_rows, "ms_per_step": float(t.item()), "value": float(u.item()) / (float(t.item()) * 1e-3) / 1e9,
                  "unit": "Gnnz/s", "note": "the configuration's cells divided by the GPU count: whole-job rate at fixed total work"}

    # ---- end to end through the C ABI's host-buffer call (H2D of the matrix + run + D2H of the result)
    e2e = None
    if wl["kind"] == "forward" and not args.no_e2e:
        host = ops.HostCsr.from_device(x)                 # pinned host copy of this rank's shard
        w_host = dense.cpu().pin_memory()
        y_host = torch.empty(out.shape, dtype=torch.float32).pin_memory()
        chunks = max(1, args.e2e_chunks)
        so = capi.header(capi.HostStageOptions())
        so.device, so.k, so.n, so.bits, so.policy = device.index, x.cols, wl["n"], x.bits, x.policy
        so.dense_dtype = capi.DTYPE_BF16
        so.multiply = capi.DTYPE_F32
        so.max_chunk_rows = -(-x.rows // chunks)
        counts = np.diff(x.host_row_ptr[:: so.max_chunk_rows].tolist() + [int(x.host_row_ptr[-1])])
        so.max_chunk_nnz = int(counts.max()) + 1
        so.chunk_buffers = max(2, min(4, args.e2e_buffers))
        # the ranks of a box share its cores: each stage narrows gene indices with its share of them
        so.host_threads = max(1, len(os.sched_getaffinity(0)) // max(1, int(os.environ.get("LOCAL_WORLD_SIZE", world))))
        stage = C.c_void_p()
        capi.check(L.cb200_host_stage_create(C.byref(so), C.byref(stage)))
        hd = capi.header(capi.QCsr())
        hd.rows, hd.cols, hd.nnz, hd.bits, hd.policy = x.rows, x.cols, x.nnz, x.bits, x.policy
        hd.row_ptr, hd.col_idx, hd.packed_values = host.row_ptr.data_ptr(), host.col_idx.data_ptr(), host.packed.data_ptr()
        hd.scales, hd.offsets = host.scales.data_ptr(), host.offsets.data_ptr()
        hd.packed_row_ptr = None if host.packed_row_ptr is None else host.packed_row_ptr.data_ptr()
        h2d, d2h = C.c_uint64(), C.c_uint64()

        def host_call():
            capi.check(L.cb200_host_forward(stage, C.byref(hd), w_host.data_ptr(), wl["n"], y_host.data_ptr(), wl["n"], 1.0,
                                            C.byref(h2d), C.byref(d2h)))
        host_call()
        if world > 1:
            dist.barrier()
        e_steps = max(1, min(args.steps, args.e2e_steps))
        t0 = time.perf_counter()                          # the call returns when y has landed: host clock around it
        for _ in range(e_steps):
            host_call()
        e_ms_local = (time.perf_counter() - t0) * 1e3 / e_steps
        e_ms = torch.tensor([e_ms_local], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(e_ms, op=dist.ReduceOp.MAX)
        e_ms = float(e_ms.item())
        e2e = {"value": total_units / (e_ms * 1e-3) / 1e9, "unit": "Gnnz/s", "h2d_bytes_per_step": int(h2d.value),
               "d2h_bytes_per_step": int(d2h.value), "ms_per_step": e_ms, "steps": e_steps,
               "call": "cb200_host_forward (C ABI, pinned host buffers, %d chunk buffers of %d rows; gene indices cross as gap bytes "
                       "while the host rewrites them fast enough)" % (so.chunk_buffers, so.max_chunk_rows),
               "h2d_bytes_per_entry": float(h2d.value) / max(1.0, float(x.nnz)),
               "schedule": "gene_tiled (codes read at launch)", "stage_device_bytes": int(L.cb200_host_stage_device_bytes(stage)),
               "aggregate_h2d_gbs": world * h2d.value / (e_ms * 1e-3) / 1e9}
        if rank == 0:   # the host result against the device-resident result of the exact schedule, sampled rows vs the oracle
            e2e["parity_check"] = parity_of_what_ran(dict(wl, out=y_host), _NoStatus(), False)
        L.cb200_host_stage_destroy(stage)
        # The same call sequence with the matrix RESIDENT, as the reference's prepared operations hold it (the shard
        # stays on its GPU between steps; a step brings W and takes Y): the prepared operation of the timed loop above,
        # W from pinned host memory, Y back to pinned host memory, all inside the timed region.  Reported beside the
        # end-to-end number, not instead of it.
        launch_r = op.make_launch(x, dense, out)

        def resident_call():
            dense.copy_(w_host, non_blocking=True)
            op.run_launch(launch_r)
            y_host.copy_(out, non_blocking=True)
            torch.cuda.synchronize(device)
        resident_call()
        if world > 1:
            dist.barrier()
        r_steps = max(3, min(args.steps, 10))
        t0 = time.perf_counter()
        for _ in range(r_steps):
            resident_call()
        r_ms = torch.tensor([(time.perf_counter() - t0) * 1e3 / r_steps], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(r_ms, op=dist.ReduceOp.MAX)
        r_ms = float(r_ms.item())
        e2e["resident_matrix"] = {"value": total_units / (r_ms * 1e-3) / 1e9, "unit": "Gnnz/s", "ms_per_step": r_ms, "steps": r_steps,
                                  "h2d_bytes_per_step": int(w_host.numel() * w_host.element_size()),
                                  "d2h_bytes_per_step": int(y_host.numel() * 4), "schedule": op.schedule,
                                  "call": "cb200_spmm_run on the prepared operation; W from and Y to pinned host memory every step"}
        del host, y_host

    # ---- the other configurations on the same line (short runs; the headline workload's memory is released first)
    others = None
    if default_arm and not args.no_extras and not args.rows:
        others = {}
        keep_x = x
        op.close()
        x = op = out = wl = None
        torch.cuda.empty_cache()
        for name in ("c3_transpose", "c4_4bit", "c5_bell"):
            try:
                rec, owl = measure_workload(name, args, device, rank, world, 5, 3, fleet, reuse_x=keep_x if name == "c3_transpose" else None)
            except Exception as e:                         # a configuration that cannot run is reported, not hidden
                others[name] = {"error": str(e)}
                continue
            keys = ("schedule", "ms_per_step", "step_ms", "value", "frac", "kernel_ms", "ms_kernel", "ms_allreduce", "allreduce_bytes",
                    "prepare_ms_once", "persistent_bytes", "units_per_gpu", "parity_check")
            others[name] = {k: rec[k] for k in keys if k in rec}
            others[name]["unit"] = "Gslot/s" if name == "c5_bell" else "Gnnz/s"
            others[name]["roofline"] = rec["roofline"]
            owl["op"].close()
            del owl, rec
            if name == "c3_transpose":
                keep_x = None
            torch.cuda.empty_cache()

    fleet.close()
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    kind_bell = args.workload == "c5_bell"
    schedule = main["schedule"]
    baked = schedule in ("tensor_blocked", "tensor_blocked_x2", "tensor_blocked_x3", "tensor_dense", "gene_gather")
    result = {
        "metric": ("quantized Blocked-ELL projection throughput" if kind_bell else
                   "quantized CSR SpMM throughput (dequant fused into the multiply, fp32 accumulate)"),
        "value": main["value"], "unit": "Gslot/s" if kind_bell else "Gnnz/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": main["ms_per_step"],
        "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
        "dtype": f"u{main['bits']} codes -> " + ("bf16 products (tcgen05), f32 accumulate"
                                                 if schedule == "tensor_windows"
                                                 else "fp16 products (tcgen05), f32 accumulate"
                                                 if schedule in ("tensor_blocked", "tensor_dense", "tensor_codes", "tcgen05_block_rows")
                                                 else "split bf16 products (tcgen05, %s passes), f32 accumulate" % schedule[-1]
                                                 if schedule in ("tensor_blocked_x2", "tensor_blocked_x3")
                                                 else "f32 products, f32 accumulate"),
        "data": "synthetic (seeded, device-generated; shapes and value model of the named configuration)",
        "config": {"workload": args.workload, "cells_per_gpu": main["rows"], "genes": main["cols"], "n": main["n"],
                   "units_per_gpu": main["units_per_gpu"], "bits": main["bits"],
                   "dense": "bf16" if args.workload != "c3_transpose" else "f32",
                   "parallelism": f"row-sharded x{world}" + (" + NCCL allreduce (cb200_fleet_run_transpose)" if args.workload == "c3_transpose" and world > 1 else ""),
                   "l2": "inputs larger than L2 (126 MB); no flush needed", "schedule": schedule,
                   "dequantisation": ("at prepare: the timed kernel streams {fp16 decoded value, tile position} words that prepare "
                                      "wrote from the codes, scales and offsets; a change of any of them needs a new prepare"
                                      if baked else
                                      "at launch, in registers: the timed kernel streams dense tiles of codes (a byte per slot) that "
                                      "prepare laid out; scales and offsets are read at every launch"
                                      if schedule == "tensor_codes" else "at launch: codes, scales and offsets are read by the timed kernel"),
                   "prepare_ms_once": main["prepare_ms_once"], "persistent_bytes": main["persistent_bytes"],
                   "summation_order": ("atomic (order of arrival at L2)" if schedule in ("vector_reductions",) else
                                       "fixed: the same bits on every launch")},
        "step_ms": main["step_ms"], "value_at_median": main["value_at_median"],
        "gpu_launches": main["gpu_launches"],
        "clocks": clocks,
        "roofline": main["roofline"],
    }
    if "parity_check" in main:
        result["parity_check"] = main["parity_check"]
    if main["prepare_ms_once"] > 0 and main["persistent_bytes"] > 0:
        amortised_ms = main["ms_per_step"] + main["prepare_ms_once"] / args.steps
        result["prepared"] = {"prepare_ms": main["prepare_ms_once"], "first_prepare_of_the_process_ms": main.get("prepare_ms_first_in_process"),
                              "persistent_bytes": main["persistent_bytes"],
                              "amortised_value_at_steps": {"steps": args.steps, "value": total_units / (amortised_ms * 1e-3) / 1e9}}
    if "ms_kernel" in main:
        result["transpose"] = {k: main[k] for k in ("ms_kernel", "ms_allreduce", "allreduce_bytes") if k in main}
        result["transpose"]["ms_step"] = main["ms_per_step"]
    if exact_arm is not None:
        result["exact_arm"] = exact_arm
    if strong is not None:
        result["strong_scaling"] = strong
    if others is not None:
        result["other_workloads"] = others
    if e2e is not None:
        result["e2e"] = e2e

    # ---- CPU baseline on a bounded sample of the same workload (rank 0, N = 1 only)
    if world == 1 and args.workload in ("c2_forward", "c3_transpose", "c4_4bit") and not args.no_cpu:
        threads = cpu_threads()
        sample = reference_sample(args.workload, args.cpu_rows_per_thread * threads, device)
        dt, kind = time_cpu_reference(sample["h"], sample["dense_host"], sample["kind"], threads)
        nnz_s = int(sample["h"]["row_ptr"][-1])
        result["cpu_baseline"] = {"value": nnz_s / dt / 1e9, "unit": "Gnnz/s", "cores": threads, "kind": kind,
                                  "sample": f"first {sample['h']['rows']} rows ({nnz_s} stored entries), decode + "
                                            f"double-precision referee, one row partition per thread",
                                  "seconds": dt}
    print(json.dumps(result))
    failed = [k for k, v in (("main", result.get("parity_check")), ("exact_arm", (exact_arm or {}).get("parity_check")),
                             ("e2e", (e2e or {}).get("parity_check"))) if v is not None and not v.get("ok", False)]
    if others:
        failed += [n for n, r in others.items() if isinstance(r.get("parity_check"), dict) and not r["parity_check"].get("ok", False)]
    if world > 1:
        dist.destroy_process_group()
    if failed:
        print("parity check failed: " + ", ".join(failed), file=sys.stderr)
        sys.exit(1)


class _NoStatus:
    """Stands in for a prepared operation where the call itself has already checked the kernels' status words."""
    def status(self):
        return 0


def reference_sample(workload, sample_rows, device):
    """The first `sample_rows` rows of the workload's matrix on the host, with its dense operand: generated by the seeded
    generator alone (no operation of the product is prepared for it)."""
    import torch

    from cellerator_b200 import synth
    kind = "transpose" if workload == "c3_transpose" else "forward"
    cfg = dict(synth.CONFIGS["c4_4bit" if workload == "c4_4bit" else "c2_forward"])
    n = 64 if kind == "transpose" else cfg["n"]
    if device is not None:
        full_rows = cfg["rows"] // (8 if workload == "c4_4bit" else 1)
        x = synth.make_qcsr_device(**{**cfg, "rows": max(sample_rows, 1024)}, device=device, seed=0, row_base=0, total_rows=full_rows)
        torch.cuda.synchronize(device)
        h = host_rows(x, 0, min(sample_rows, x.rows))
        del x
        torch.cuda.empty_cache()
    else:
        sample_rows = min(sample_rows, 2000)
        h = synth.make_qcsr_host(**{**cfg, "rows": sample_rows}, seed=0)
    g = torch.Generator(device="cpu").manual_seed(1000)
    if kind == "forward":
        dense_host = (torch.randn(cfg["cols"], n, generator=g) * 0.02).to(torch.bfloat16).float().numpy()
    else:
        dense_host = torch.randn(h["rows"], n, generator=g).numpy()
    return {"h": h, "dense_host": dense_host, "kind": kind, "cfg": cfg, "n": n}


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
    sample = reference_sample(args.workload, args.cpu_rows_per_thread * threads,
                              torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))) if torch.cuda.is_available() else None)
    h, dense_host, cfg, n = sample["h"], sample["dense_host"], sample["cfg"], sample["n"]
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
        "impl": "reference", "metric": "quantized CSR SpMM throughput (dequant fused into the multiply, fp32 accumulate)",
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
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="weak: every GPU holds the configuration's per-GPU shard; strong: the configuration's cells are "
                         "divided over the GPUs")
    ap.add_argument("--no-extras", action="store_true",
                    help="headline workload only: no exact arm, strong-scaling point or other configurations")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--e2e-chunks", type=int, default=16)
    ap.add_argument("--e2e-buffers", type=int, default=3, help="chunk buffers of the host stage's ring (2..4)")
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
