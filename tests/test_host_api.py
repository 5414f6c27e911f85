"""CPU checks of the C ABI: the library loads, exports every declared symbol, its host helpers
equal the oracle, the capability query answers as documented, and compute entry points fail
loudly (status + message) when no CUDA device is usable."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from cellerator_b200 import capi, ops, synth
from conftest import ROOT, random_csr


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "cellerator_b200.h")).read()
    declared = set(re.findall(r"\b(cb200_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    L = capi.lib()
    for name in sorted(declared):
        assert hasattr(L, name), f"{name} declared in the header but not exported"
    assert declared == set(capi.EXPORTED_SYMBOLS)
    assert L.cb200_abi_version() == capi.ABI_VERSION
    assert L.cb200_status_string(capi.STALE_STRUCTURE) == b"stale structure"


@pytest.mark.parametrize("bits", [1, 2, 4, 8])
def test_layout_helpers_equal_oracle(oracle, bits):
    rng = np.random.default_rng(bits)
    for _ in range(5):
        c = random_csr(rng, rows=int(rng.integers(0, 50)), cols=64, max_nnz=40, bits=bits)
        prp, total = ops.build_packed_row_ptr(bits, c["row_ptr"])
        prp_o, total_o = oracle.build_packed_row_ptr(bits, c["row_ptr"])
        assert np.array_equal(prp, prp_o) and total == total_o
        for rpb in (1, 4, 9, 1000):
            brp = ops.build_uniform_block_row_ptr(c["rows"], rpb)
            brp_o, count_o = oracle.build_uniform_block_row_ptr(c["rows"], rpb)
            assert np.array_equal(brp, brp_o) and len(brp) - 1 == count_o
            for b in (-1, 0, count_o - 1, count_o):
                if c["rows"] == 0:
                    continue
                assert ops.get_block(c["row_ptr"], prp, brp, b) == oracle.get_block(c["row_ptr"], prp_o, brp_o, b)
        if c["rows"]:
            assert ops.get_block(c["row_ptr"], prp, None, 3) == oracle.get_block(c["row_ptr"], prp_o, None, 3)
    assert capi.lib().cb200_build_packed_row_ptr(3, None, 0, None) == -1
    assert capi.lib().cb200_build_uniform_block_row_ptr(10, 0, None) == -1


def test_partition_rows_matches_reference_rule(oracle):
    for rows, parts in ((1_000_000, 8), (1_000_003, 8), (5, 8), (20_000, 2), (7, 1)):
        brp = ops.partition_rows(rows, parts)
        assert len(brp) == parts + 1 and brp[0] == 0 and brp[-1] == rows
        per = -(-rows // parts)
        ref, count = oracle.build_uniform_block_row_ptr(rows, per)
        assert np.array_equal(brp[:count + 1], ref)
        assert np.all(brp[count:] == rows)


def test_numpy_quantiser_equals_oracle_pack(oracle):
    for bits in (4, 8):
        h = synth.make_qcsr_host(rows=300, cols=400, median=40, sigma=0.6, lo=0, hi=200, bits=bits, seed=bits)
        packed = oracle.pack_csr(bits, 1, h["row_ptr"], h["packed_row_ptr"], h["col_idx"], h["scales"], h["offsets"],
                                 h["values"])
        assert np.array_equal(packed, h["packed"])
        assert np.array_equal(oracle.extract_codes(bits, h["row_ptr"], h["packed_row_ptr"], packed), h["codes"])
    b = synth.make_qbell_host(rows=70, cols=250, block_size=32, ell_blocks=3, fill=0.6, bits=8, seed=3)
    packed = oracle.bell_pack(8, 1, 70, 250, 32, b["ell_cols"], b["row_stride_bytes"], b["block_col_idx"], b["scales"],
                              b["offsets"], b["values_by_slot"])
    assert np.array_equal(packed, b["packed"])


def test_backend_query_capabilities():
    fwd = ops.backend_query(capi.PROJECTION_CSR)
    assert fwd["supported"] and fwd["flags"] & capi.CAP_DETERMINISTIC and fwd["name"].startswith("cb200.qcsr.forward")
    assert ops.backend_query(capi.PROJECTION_CSR, dense=capi.DTYPE_F32)["supported"]
    assert ops.backend_query(capi.PROJECTION_CSR, sparse=capi.DTYPE_U4)["supported"]
    assert not ops.backend_query(capi.PROJECTION_CSR, dense=capi.DTYPE_F16)["supported"]
    assert not ops.backend_query(capi.PROJECTION_CSR, quantized=0)["supported"]
    assert not ops.backend_query(capi.PROJECTION_CSR, accumulation=capi.DTYPE_BF16)["supported"]
    tr = ops.backend_query(capi.PROJECTION_TRANSPOSE, dense=capi.DTYPE_F32)
    assert tr["supported"] and not (tr["flags"] & capi.CAP_DETERMINISTIC)
    assert not ops.backend_query(capi.PROJECTION_TRANSPOSE, dense=capi.DTYPE_BF16)["supported"]
    assert ops.backend_query(capi.PROJECTION_BLOCKED_ELL, multiply=capi.DTYPE_BF16)["supported"]
    with pytest.raises(capi.Cb200Error) as e:
        ops.backend_query(99)
    assert e.value.status == capi.UNSUPPORTED


def test_bad_descriptors_are_rejected_before_any_device_call():
    L = capi.lib()
    pr = capi.SpmmProblem()            # version / size left at 0
    handle = C.c_void_p()
    assert L.cb200_spmm_prepare(C.byref(pr), C.byref(handle)) == capi.INVALID_ARGUMENT
    assert b"header" in L.cb200_last_error()
    pr = capi.header(capi.SpmmProblem())
    pr.projection, pr.m, pr.k, pr.n, pr.bits, pr.policy, pr.dense_dtype = capi.PROJECTION_CSR, 4, 4, 8, 8, 1, capi.DTYPE_F32
    assert L.cb200_spmm_prepare(C.byref(pr), C.byref(handle)) == capi.STALE_STRUCTURE      # epoch 0
    pr.structure_epoch = 1
    pr.bits = 3
    assert L.cb200_spmm_prepare(C.byref(pr), C.byref(handle)) == capi.UNSUPPORTED
    pr.bits = 8
    pr.projection, pr.deterministic = capi.PROJECTION_TRANSPOSE, 1
    assert L.cb200_spmm_prepare(C.byref(pr), C.byref(handle)) == capi.UNSUPPORTED          # deterministic transpose without the device matrix
    assert L.cb200_spmm_run(None, None) == capi.INVALID_ARGUMENT


def test_no_cpu_fallback_without_a_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    L = capi.lib()
    pr = capi.header(capi.SpmmProblem())
    pr.projection, pr.m, pr.k, pr.n, pr.bits, pr.policy, pr.dense_dtype = capi.PROJECTION_CSR, 4, 4, 8, 8, 1, capi.DTYPE_F32
    pr.structure_epoch = 1
    handle = C.c_void_p()
    assert L.cb200_spmm_prepare(C.byref(pr), C.byref(handle)) == capi.CUDA_ERROR
    assert not handle.value and L.cb200_last_error() != b""
    opts = capi.header(capi.SessionOptions())
    opts.owned_stream_count = 1
    sess = C.c_void_p()
    assert L.cb200_session_create(C.byref(opts), C.byref(sess)) == capi.CUDA_ERROR
    m = capi.header(capi.QCsr())
    assert L.cb200_dequantize_rows(C.byref(m), 0, 0, None, 0, None) == capi.CUDA_ERROR


def _decode_gene_gaps(gaps, row_ptr, positions, genes):
    """What the device does with the gap form: gene = previous gene of the row + gap + 1 (-1 before a row's first
    entry); a listed entry takes its gene from the list, and the entries behind it count on from there."""
    listed = dict(zip(positions.tolist(), genes.tolist()))
    out = np.empty(len(gaps), dtype=np.int64)
    base = int(row_ptr[0])
    for r in range(len(row_ptr) - 1):
        gene = -1
        for i in range(int(row_ptr[r]) - base, int(row_ptr[r + 1]) - base):
            if gaps[i] == 255:
                gene = listed[i]
            else:
                gene += int(gaps[i]) + 1
            out[i] = gene
    return out


@pytest.mark.parametrize("case", ["dense_rows", "long_gaps", "descending", "offset_rows"])
@pytest.mark.parametrize("threads", [1, 5])
def test_gene_gap_encoding_round_trip(case, threads):
    """cb200_host_encode_gene_gaps (the host half of cb200_host_forward's short index form) against a decode in plain
    Python: every entry comes back, whatever the gaps; marked entries are exactly those whose gap does not fit a byte;
    a list that is too short is reported."""
    L = capi.lib()
    rng = np.random.default_rng(len(case) + threads)
    rows = 300
    cols = {"dense_rows": 3000, "long_gaps": 400_000, "descending": 3000, "offset_rows": 70_000}[case]
    counts = rng.integers(0, 260, size=rows)
    counts[rng.integers(0, rows, size=5)] = 0                          # empty rows
    counts[7] = 1                                                       # a single entry
    row_ptr = np.zeros(rows + 1, dtype=np.int64)
    np.cumsum(counts, out=row_ptr[1:])
    col = np.concatenate([np.sort(rng.choice(cols, size=int(c), replace=False)) for c in counts] + [np.zeros(0, dtype=np.int64)]).astype(np.int32)
    if case == "descending":
        for r in rng.choice(rows, size=30, replace=False):
            lo, hi = row_ptr[r], row_ptr[r + 1]
            col[lo:hi] = rng.permutation(col[lo:hi])
        col[row_ptr[3]:row_ptr[4]] = -5                                 # indices the kernels would leave out survive too
    first_row = 40 if case == "offset_rows" else 0                      # a chunk in the middle of the caller's arrays
    ptr = np.ascontiguousarray(row_ptr[first_row:])
    n = int(ptr[-1] - ptr[0])
    gaps = np.full(n + 64, 0xEE, dtype=np.uint8)
    positions, genes = np.zeros(n + 1, dtype=np.int32), np.zeros(n + 1, dtype=np.int32)
    count = L.cb200_host_encode_gene_gaps(col.ctypes.data, ptr.ctypes.data, len(ptr) - 1, gaps.ctypes.data, positions.ctypes.data,
                                          genes.ctypes.data, n + 1, threads)
    assert count >= 0
    assert np.all(gaps[n:] == 0xEE)                                     # nothing written past the last entry
    assert np.all(np.diff(positions[:count]) > 0)                       # ascending positions, no sort needed on the device
    chunk = col[ptr[0]:ptr[-1]].astype(np.int64)
    assert np.array_equal(_decode_gene_gaps(gaps[:n], ptr, positions[:count], genes[:count]), chunk)
    previous = np.concatenate([[-1], chunk[:-1]])
    previous[(ptr[:-1] - ptr[0])[np.diff(ptr) > 0]] = -1                # a row's first entry counts from -1
    gap = chunk - previous - 1
    assert np.array_equal(np.flatnonzero(gaps[:n] == 255), np.flatnonzero((gap < 0) | (gap >= 255)))
    assert count == int(np.sum((gap < 0) | (gap >= 255)))
    if count > 0:
        assert L.cb200_host_encode_gene_gaps(col.ctypes.data, ptr.ctypes.data, len(ptr) - 1, gaps.ctypes.data, positions.ctypes.data,
                                             genes.ctypes.data, count - 1, threads) == -1
    assert L.cb200_host_encode_gene_gaps(col.ctypes.data, ptr.ctypes.data, len(ptr) - 1, gaps.ctypes.data, positions.ctypes.data,
                                         genes.ctypes.data, n + 1, 0) == -2
