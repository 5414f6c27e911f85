"""Seeded synthetic cells x genes workloads shaped like the benchmark configurations.

Two generators with the same statistical recipe:

* `make_qcsr_host` / `make_qbell_host`: numpy, for the small configurations, the tests and the
  golden fixtures (bit-reproducible across machines for a given numpy version).
* `make_qcsr_device` / `make_qbell_device`: CUDA (libcb200_synth.so), for the full-size
  benchmark matrices that are too large to build on a host.

Recipe: nnz per row ~ round(lognormal(median, sigma)) clipped; genes uniform without
replacement, ascending; counts ~ negative binomial(mean mu_g ~ lognormal(0, 1.5), dispersion
0.5) forced >= 1; value = log1p(count / rowsum * 1e4); per-gene affine calibration with
offset = min, scale = max((max - min) / (2^bits - 1), 1e-6), unseen genes scale 1 offset 0;
codes by true division and round-half-away-from-zero, clamped.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import capi

CONFIGS = {
    # name: rows, cols, median nnz/row, sigma, clip lo, clip hi, bits, n, dense dtype
    "c1_cpu_ref": dict(rows=20_000, cols=2_000, median=300, sigma=0.5, lo=50, hi=1_500, bits=8, n=32, dense="f32"),
    "c2_forward": dict(rows=1_000_000, cols=33_538, median=1_500, sigma=0.6, lo=1, hi=33_538, bits=8, n=64,
                       dense="bf16"),
    "c4_4bit": dict(rows=4_000_000, cols=4_000, median=600, sigma=0.5, lo=1, hi=4_000, bits=4, n=128, dense="bf16"),
    "c5_bell": dict(rows=2_000_000, cols=8_192, block_size=32, ell_blocks=16, fill=0.6, bits=8, n=256, dense="bf16"),
}


def row_nnz(rows, median, sigma, lo, hi, rng) -> np.ndarray:
    raw = np.rint(np.exp(rng.normal(np.log(median), sigma, size=rows)))
    return np.clip(raw, lo, hi).astype(np.int64)


def quantize_codes(values, scale, offset, bits) -> np.ndarray:
    """The quantisation rule in float32 numpy: scale == 0 -> 0, q = (v - offset) / scale,
    round half away from zero (by truncating q +- 0.5), clamp to [0, 2^bits - 1]."""
    values = values.astype(np.float32)
    scale = scale.astype(np.float32)
    offset = offset.astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        q = (values - offset) / scale
    shifted = np.where(q >= 0, q + np.float32(0.5), q - np.float32(0.5)).astype(np.float32)
    # a conversion that overflows int32 (or a NaN) gives INT_MIN on the x86-64 hosts the host
    # codec runs on, which the rule maps to code 0
    overflow = ~(shifted < np.float32(2147483648.0))
    shifted = np.nan_to_num(shifted, nan=0.0, posinf=0.0, neginf=-3e9)
    rounded = np.trunc(np.clip(shifted, -2.0e9, 2.2e9)).astype(np.int64)
    rounded = np.clip(rounded, 0, (1 << bits) - 1)
    rounded[(scale == 0) | overflow] = 0
    return rounded.astype(np.uint8)


def pack_codes(codes, row_ptr, bits):
    """codes (one per entry) -> packed bytes + packed_row_ptr; low lane first, rows byte-aligned."""
    row_ptr = np.asarray(row_ptr, dtype=np.int64)
    cpb = 8 // bits
    counts = np.diff(row_ptr)
    row_bytes = (counts + cpb - 1) // cpb
    prp = np.zeros(len(row_ptr), dtype=np.int64)
    np.cumsum(row_bytes, out=prp[1:])
    if bits == 8:
        return codes.astype(np.uint8).copy(), prp
    packed = np.zeros(int(prp[-1]), dtype=np.uint8)
    rows_of = np.repeat(np.arange(len(counts)), counts)
    local = np.arange(len(codes), dtype=np.int64) - row_ptr[rows_of]
    byte = prp[rows_of] + local // cpb
    shift = ((local % cpb) * bits).astype(np.uint8)
    np.bitwise_or.at(packed, byte, (codes.astype(np.uint8) << shift).astype(np.uint8))
    return packed, prp


def calibrate(values, genes, cols, bits):
    lo = np.full(cols, np.inf, dtype=np.float32)
    hi = np.full(cols, -np.inf, dtype=np.float32)
    np.minimum.at(lo, genes, values)
    np.maximum.at(hi, genes, values)
    seen = np.isfinite(lo)
    scales = np.ones(cols, dtype=np.float32)
    offsets = np.zeros(cols, dtype=np.float32)
    levels = np.float32((1 << bits) - 1)
    scales[seen] = np.maximum((hi[seen] - lo[seen]) / levels, np.float32(1e-6))
    offsets[seen] = lo[seen]
    return scales, offsets


def make_qcsr_host(rows, cols, median, sigma, lo, hi, bits, seed=0, **_) -> dict:
    rng = np.random.default_rng(seed)
    counts = row_nnz(rows, median, sigma, lo, min(hi, cols), rng)
    row_ptr = np.zeros(rows + 1, dtype=np.int64)
    np.cumsum(counts, out=row_ptr[1:])
    nnz = int(row_ptr[-1])
    col_idx = np.empty(nnz, dtype=np.int32)
    for r in range(rows):
        col_idx[row_ptr[r]:row_ptr[r + 1]] = np.sort(rng.choice(cols, size=int(counts[r]), replace=False))
    gene_mean = np.exp(rng.normal(0.0, 1.5, size=cols))
    mu = gene_mean[col_idx]
    shape = 2.0  # 1 / dispersion
    cnt = np.maximum(rng.negative_binomial(shape, shape / (shape + mu)), 1).astype(np.float64)
    rowsum = np.add.reduceat(cnt, row_ptr[:-1][counts > 0]) if nnz else np.zeros(0)
    rs = np.zeros(rows)
    rs[counts > 0] = rowsum
    values = np.log1p(cnt / np.repeat(rs, counts) * 1e4).astype(np.float32)
    scales, offsets = calibrate(values, col_idx, cols, bits)
    codes = quantize_codes(values, scales[col_idx], offsets[col_idx], bits)
    packed, prp = pack_codes(codes, row_ptr, bits)
    return dict(rows=rows, cols=cols, bits=bits, policy=capi.DECODE_PER_GENE_AFFINE, row_ptr=row_ptr,
                packed_row_ptr=prp, col_idx=col_idx, packed=packed, scales=scales, offsets=offsets,
                values=values, codes=codes)


def make_qbell_host(rows, cols, block_size, ell_blocks, fill, bits, seed=0, row_stride_align=16, **_) -> dict:
    rng = np.random.default_rng(seed)
    block_rows = -(-rows // block_size)
    block_cols = -(-cols // block_size)
    ell_cols = ell_blocks * block_size
    bci = np.empty((block_rows, ell_blocks), dtype=np.uint32)
    for b in range(block_rows):
        bci[b] = np.sort(rng.choice(block_cols, size=ell_blocks, replace=False))
    genes = (bci[np.arange(rows) // block_size][:, :, None].astype(np.int64) * block_size
             + np.arange(block_size)[None, None, :]).reshape(rows, ell_cols)
    gene_mean = np.exp(rng.normal(0.0, 1.5, size=block_cols * block_size))
    present = (rng.random((rows, ell_cols)) < fill) & (genes < cols)
    shape = 2.0
    cnt = np.maximum(rng.negative_binomial(shape, shape / (shape + gene_mean[genes])), 1) * present
    rowsum = cnt.sum(axis=1, keepdims=True).astype(np.float64)
    rowsum[rowsum == 0] = 1.0
    values = np.log1p(cnt / rowsum * 1e4).astype(np.float32)
    in_range = genes < cols
    scales, offsets = calibrate(values[in_range], genes[in_range], cols, bits)
    # metadata padded to whole block columns; the padding repeats gene 0's entry, which is what
    # slots of a ragged last block column are coded with
    pad = block_cols * block_size - cols
    scales = np.concatenate([scales, np.full(pad, scales[0], dtype=np.float32)])
    offsets = np.concatenate([offsets, np.full(pad, offsets[0], dtype=np.float32)])
    safe = np.where(in_range, genes, 0)
    codes = quantize_codes(values.ravel(), scales[safe.ravel()], offsets[safe.ravel()], bits).reshape(rows, ell_cols)
    cpb = 8 // bits
    raw = -(-ell_cols // cpb)
    stride = -(-raw // row_stride_align) * row_stride_align
    packed = np.zeros((rows, stride), dtype=np.uint8)
    for lane in range(cpb):
        part = codes[:, lane::cpb]
        packed[:, : part.shape[1]] |= (part << (lane * bits)).astype(np.uint8)
    return dict(rows=rows, cols=cols, block_size=block_size, ell_cols=ell_cols, row_stride_bytes=stride, bits=bits,
                policy=capi.DECODE_PER_GENE_AFFINE, block_col_idx=bci.ravel(), packed=packed.ravel(), scales=scales,
                offsets=offsets, values_by_slot=values, genes_by_slot=genes)


# ---- device generators ---------------------------------------------------------------

def make_lowering_host(rows, features, feature_blocks, mean_nnz, seed=0, value_dtype=np.float32, clustered=True) -> dict:
    """A canonical CSR with uint32 offsets plus a row order and a feature order, the inputs of the
    CSR -> Blocked-ELL lowering: `feature_blocks` semantic blocks of random widths, random feature and
    row permutations (feature_permutation[execution] = canonical, row_permutation[execution row] =
    canonical row).  clustered: a row draws most of its features from two of the semantic blocks, so
    that block rows share block columns as ordered single-cell data does."""
    rng = np.random.default_rng(seed)
    cuts = np.sort(rng.choice(np.arange(1, features), size=feature_blocks - 1, replace=False)) if feature_blocks > 1 else []
    fb_offsets = np.concatenate([[0], cuts, [features]]).astype(np.uint32)
    fperm = rng.permutation(features).astype(np.uint32)
    rperm = rng.permutation(rows).astype(np.uint32)
    finv = np.empty(features, dtype=np.uint32)
    finv[fperm] = np.arange(features, dtype=np.uint32)
    counts = np.minimum(rng.poisson(mean_nnz, size=rows), features)
    counts[rng.random(rows) < 0.05] = 0                       # some empty rows
    row_offsets = np.zeros(rows + 1, dtype=np.uint32)
    np.cumsum(counts, out=row_offsets[1:])
    ids = np.empty(int(row_offsets[-1]), dtype=np.uint32)
    for r in range(rows):
        k = int(counts[r])
        if k == 0:
            continue
        if clustered and feature_blocks > 1:
            a, b = rng.integers(0, feature_blocks, size=2)
            pool = np.concatenate([np.arange(fb_offsets[a], fb_offsets[a + 1]), np.arange(fb_offsets[b], fb_offsets[b + 1])])
            pool = np.unique(pool)
            take = min(k, len(pool))
            execution = rng.choice(pool, size=take, replace=False)
            if take < k:
                rest = np.setdiff1d(np.arange(features), execution)
                execution = np.concatenate([execution, rng.choice(rest, size=k - take, replace=False)])
        else:
            execution = rng.choice(features, size=k, replace=False)
        ids[row_offsets[r]:row_offsets[r + 1]] = np.sort(fperm[execution])
    if np.issubdtype(value_dtype, np.floating):
        values = rng.uniform(0.5, 9.0, size=len(ids)).astype(value_dtype)
    else:
        values = rng.integers(1, np.iinfo(value_dtype).max, size=len(ids), endpoint=True).astype(value_dtype)
    return dict(rows=rows, features=features, row_offsets=row_offsets, feature_ids=ids, values=values,
                fb_offsets=fb_offsets, fperm=fperm, finv=finv, rperm=rperm)


def make_lowering_device(rows, cols, block_size, ell_blocks, fill, device, seed=0, **_):
    """The Blocked-ELL configuration as a canonical CSR of one-byte codes on the device (uint32 offsets
    and feature ids, held as int32 tensors): every block row of `block_size` cells touches `ell_blocks`
    distinct block columns, and a cell stores round(fill * ell_blocks * block_size) of those slots.
    Identity row and feature orders, one semantic feature block."""
    import torch
    g = torch.Generator(device="cpu").manual_seed(seed)
    per_row = int(round(fill * ell_blocks * block_size))
    block_rows = (rows + block_size - 1) // block_size
    patterns = torch.stack([torch.randperm(cols // block_size, generator=g)[:ell_blocks] for _ in range(256)])
    pattern = patterns[torch.randint(0, 256, (block_rows,), generator=g)].repeat_interleave(block_size, dim=0)[:rows].to(device)
    gd = torch.Generator(device=device).manual_seed(seed + 1)
    pick = torch.rand(rows, ell_blocks * block_size, device=device, generator=gd).argsort(dim=1)[:, :per_row]
    feature = (pattern.gather(1, pick // block_size) * block_size + pick % block_size).sort(dim=1).values.to(torch.int32)
    del pick, pattern
    row_offsets = (torch.arange(rows + 1, device=device, dtype=torch.int64) * per_row).to(torch.int32)
    values = torch.randint(1, 256, (rows * per_row,), device=device, dtype=torch.uint8, generator=gd)
    return dict(row_offsets=row_offsets, feature_ids=feature.reshape(-1), values=values, features=cols,
                fb_offsets=np.array([0, cols], dtype=np.uint32),
                fperm=torch.arange(cols, dtype=torch.int32, device=device),
                rperm=torch.arange(rows, dtype=torch.int32, device=device), per_row=per_row)


def make_qcsr_device(rows, cols, median, sigma, lo, hi, bits, device, seed=0, row_base=0, total_rows=None, **_):
    """Rows [row_base, row_base+rows) of the seeded matrix, generated on `device`.
    Row lengths and per-gene means come from numpy (cheap), everything per-entry from CUDA.
    Returns an ops.QuantizedCsr."""
    import torch

    from .ops import QuantizedCsr

    S = capi.synth_lib()
    dev = torch.device(device)
    total_rows = rows + row_base if total_rows is None else total_rows
    rng = np.random.default_rng(seed)
    counts_all = row_nnz(total_rows, median, sigma, lo, min(hi, cols), rng)
    gene_mean_h = np.exp(rng.normal(0.0, 1.5, size=cols)).astype(np.float32)
    counts = counts_all[row_base:row_base + rows]
    row_ptr_h = np.zeros(rows + 1, dtype=np.int64)
    np.cumsum(counts, out=row_ptr_h[1:])
    nnz = int(row_ptr_h[-1])
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev).cuda_stream
        row_ptr = torch.from_numpy(row_ptr_h).to(dev)
        gene_mean = torch.from_numpy(gene_mean_h).to(dev)
        col_idx = torch.empty(nnz, dtype=torch.int32, device=dev)
        values = torch.empty(nnz, dtype=torch.float32, device=dev)
        rc = S.cb200_synth_columns(C.c_int64(rows), C.c_int32(cols), C.c_void_p(row_ptr.data_ptr()),
                                   C.c_void_p(col_idx.data_ptr()), C.c_uint64(seed), C.c_int64(row_base),
                                   C.c_void_p(stream))
        assert rc == 0, rc
        rc = S.cb200_synth_values(C.c_int64(rows), C.c_void_p(row_ptr.data_ptr()), C.c_void_p(col_idx.data_ptr()),
                                  C.c_void_p(gene_mean.data_ptr()), C.c_void_p(values.data_ptr()), C.c_uint64(seed),
                                  C.c_int64(row_base), C.c_void_p(stream))
        assert rc == 0, rc
        gmin = torch.empty(cols, dtype=torch.int32, device=dev)
        gmax = torch.empty(cols, dtype=torch.int32, device=dev)
        scales = torch.empty(cols, dtype=torch.float32, device=dev)
        offsets = torch.empty(cols, dtype=torch.float32, device=dev)
        S.cb200_synth_calibrate_init(C.c_int32(cols), C.c_void_p(gmin.data_ptr()), C.c_void_p(gmax.data_ptr()),
                                     C.c_void_p(stream))
        S.cb200_synth_calibrate_accumulate(C.c_int64(nnz), C.c_void_p(col_idx.data_ptr()),
                                           C.c_void_p(values.data_ptr()), C.c_void_p(gmin.data_ptr()),
                                           C.c_void_p(gmax.data_ptr()), C.c_void_p(stream))
        S.cb200_synth_calibrate_finish(C.c_int32(cols), C.c_int(bits), C.c_void_p(gmin.data_ptr()),
                                       C.c_void_p(gmax.data_ptr()), C.c_void_p(scales.data_ptr()),
                                       C.c_void_p(offsets.data_ptr()), C.c_void_p(stream))
        cpb = 8 // bits
        prp_h = np.zeros(rows + 1, dtype=np.int64)
        np.cumsum((counts + cpb - 1) // cpb, out=prp_h[1:])
        packed = torch.zeros(max(int(prp_h[-1]), 1), dtype=torch.uint8, device=dev)
        x = QuantizedCsr(rows=rows, cols=cols, bits=bits, policy=capi.DECODE_PER_GENE_AFFINE, row_ptr=row_ptr,
                         col_idx=col_idx, packed=packed, scales=scales, offsets=offsets,
                         packed_row_ptr=None if bits == 8 else torch.from_numpy(prp_h).to(dev),
                         host_row_ptr=row_ptr_h)
        x.quantize_(values)
        torch.cuda.synchronize(dev)
        del values
    return x


def make_qbell_device(rows, cols, block_size, ell_blocks, fill, bits, device, seed=0, row_base=0, **_):
    """Rows [row_base, row_base+rows) of the seeded Blocked-ELL matrix (row_base a multiple of
    block_size), generated and packed on `device`.  Returns an ops.QuantizedBell."""
    import torch

    from .ops import QuantizedBell, quantize_bell_

    S = capi.synth_lib()
    dev = torch.device(device)
    assert row_base % block_size == 0
    block_rows = -(-rows // block_size)
    block_cols = -(-cols // block_size)
    ell_cols = ell_blocks * block_size
    rng = np.random.default_rng(seed)
    gene_mean_h = np.exp(rng.normal(0.0, 1.5, size=block_cols * block_size)).astype(np.float32)
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev).cuda_stream
        gene_mean = torch.from_numpy(gene_mean_h).to(dev)
        bci = torch.empty(block_rows * ell_blocks, dtype=torch.int32, device=dev)
        S.cb200_synth_bell_blocks(C.c_int64(block_rows), C.c_int(ell_blocks), C.c_int(block_cols),
                                  C.c_void_p(bci.data_ptr()), C.c_uint64(seed), C.c_int64(row_base // block_size),
                                  C.c_void_p(stream))
        values = torch.empty(rows * ell_cols, dtype=torch.float32, device=dev)
        genes = torch.empty(rows * ell_cols, dtype=torch.int32, device=dev)
        S.cb200_synth_bell_values(C.c_int64(rows), C.c_int(block_size), C.c_int(ell_cols), C.c_void_p(bci.data_ptr()),
                                  C.c_void_p(gene_mean.data_ptr()), C.c_float(fill), C.c_void_p(values.data_ptr()),
                                  C.c_void_p(genes.data_ptr()), C.c_uint64(seed), C.c_int64(row_base),
                                  C.c_void_p(stream))
        gmin = torch.empty(cols, dtype=torch.int32, device=dev)
        gmax = torch.empty(cols, dtype=torch.int32, device=dev)
        scales = torch.empty(cols, dtype=torch.float32, device=dev)
        offsets = torch.empty(cols, dtype=torch.float32, device=dev)
        S.cb200_synth_calibrate_init(C.c_int32(cols), C.c_void_p(gmin.data_ptr()), C.c_void_p(gmax.data_ptr()),
                                     C.c_void_p(stream))
        S.cb200_synth_calibrate_accumulate(C.c_int64(rows * ell_cols), C.c_void_p(genes.data_ptr()),
                                           C.c_void_p(values.data_ptr()), C.c_void_p(gmin.data_ptr()),
                                           C.c_void_p(gmax.data_ptr()), C.c_void_p(stream))
        S.cb200_synth_calibrate_finish(C.c_int32(cols), C.c_int(bits), C.c_void_p(gmin.data_ptr()),
                                       C.c_void_p(gmax.data_ptr()), C.c_void_p(scales.data_ptr()),
                                       C.c_void_p(offsets.data_ptr()), C.c_void_p(stream))
        del genes
        cpb = 8 // bits
        stride = -(-(-(-ell_cols // cpb)) // 16) * 16
        packed = torch.zeros(rows * stride, dtype=torch.uint8, device=dev)
        x = QuantizedBell(rows=rows, cols=cols, block_size=block_size, ell_cols=ell_cols, row_stride_bytes=stride,
                          bits=bits, policy=capi.DECODE_PER_GENE_AFFINE, block_col_idx=bci, packed=packed,
                          scales=scales, offsets=offsets)
        quantize_bell_(x, values)
        torch.cuda.synchronize(dev)
        del values
    return x
