"""Gene-major copy (device CSR -> CSC of the codes) and the deterministic transpose that gathers from
it, through the C-ABI, against the oracle bit for bit."""
import numpy as np
import pytest
import torch

from cellerator_b200 import capi, ops, synth
from conftest import random_csr
from gpu_util import dense, host_pack, to_dev

pytestmark = pytest.mark.gpu


def bits_of(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


@pytest.mark.parametrize("bits,rows,cols,max_nnz", [(8, 2500, 300, 40), (4, 2500, 300, 41), (8, 1024, 3000, 2600),
                                                    (4, 1500, 2200, 2100), (8, 5, 7, 3), (8, 3000, 1, 1)])
def test_gene_major_copy_is_the_stable_transposition(cuda_device, oracle, bits, rows, cols, max_nnz):
    """Ragged and empty rows, a row count that is no multiple of the 1,024-row blocks, rows longer
    than the 1,024 threads that place a row, a single gene: the same arrays as the oracle."""
    rng = np.random.default_rng(bits * 1000 + rows + cols)
    c = host_pack(oracle, random_csr(rng, rows=rows, cols=cols, max_nnz=max_nnz, bits=bits))
    x = to_dev(c, cuda_device)
    col_ptr, row_idx, codes = ops.qcsr_gene_major(x)
    rc, e_ptr, e_rows, e_codes = oracle.qcsr_gene_major(bits, cols, c["row_ptr"], c["packed_row_ptr"], c["col_idx"], c["packed"])
    assert rc == 0
    assert np.array_equal(col_ptr.cpu().numpy(), e_ptr)
    assert np.array_equal(row_idx.cpu().numpy(), e_rows)
    assert np.array_equal(codes.cpu().numpy(), e_codes)


def test_gene_major_copy_reports_a_bad_column(cuda_device, oracle):
    rng = np.random.default_rng(3)
    c = host_pack(oracle, random_csr(rng, rows=40, cols=20, max_nnz=6, bits=8, empty_rows=False))
    c["col_idx"] = c["col_idx"].copy()
    c["col_idx"][-1] = 20
    with pytest.raises(ValueError):
        ops.qcsr_gene_major(to_dev(c, cuda_device))
    assert capi.lib().cb200_qcsr_gene_major_workspace(10, 20) == 256 + 20 * 4
    assert capi.lib().cb200_qcsr_gene_major_workspace(10, 0) == 0


@pytest.mark.parametrize("bits", [8, 4])
def test_gene_major_copy_of_a_wide_matrix(cuda_device, oracle, bits):
    """More genes than one launch of the counting pass covers (57,344): two gene ranges there, thirty
    in the placing pass; cells in three row blocks."""
    rng = np.random.default_rng(60 + bits)
    rows, cols = 2100, 120_000
    c = host_pack(oracle, random_csr(rng, rows=rows, cols=cols, max_nnz=60, bits=bits))
    x = to_dev(c, cuda_device)
    col_ptr, row_idx, codes = ops.qcsr_gene_major(x)
    rc, e_ptr, e_rows, e_codes = oracle.qcsr_gene_major(bits, cols, c["row_ptr"], c["packed_row_ptr"], c["col_idx"], c["packed"])
    assert rc == 0
    assert np.array_equal(col_ptr.cpu().numpy(), e_ptr)
    assert np.array_equal(row_idx.cpu().numpy(), e_rows)
    assert np.array_equal(codes.cpu().numpy(), e_codes)
    g, g_host = dense(rng, rows, 32, torch.float32, cuda_device, std=1.0)
    out = ops.spmm_transpose(x, g, deterministic=True).cpu().numpy()
    want = oracle.qcsr_transpose_ordered(1, e_ptr, e_rows, e_codes, c["scales"], c["offsets"], g_host, 0, rows)
    assert np.array_equal(bits_of(out), bits_of(want))


def test_gene_major_copy_at_scale_sorted_and_complete(cuda_device):
    """Genes as in the benchmark configuration, 1/16 of its cells: every gene's cells ascend strictly,
    the segment sizes are the column histogram, and the codes are a permutation of the source's."""
    cfg = dict(synth.CONFIGS["c2_forward"])
    cfg["rows"] //= 16
    x = synth.make_qcsr_device(**cfg, device=cuda_device, seed=2)
    col_ptr, row_idx, codes = ops.qcsr_gene_major(x)
    hist = torch.bincount(x.col_idx.long(), minlength=x.cols)
    assert torch.equal(col_ptr[1:] - col_ptr[:-1], hist)
    assert int(col_ptr[0]) == 0 and int(col_ptr[-1]) == x.nnz
    rising = row_idx[1:] > row_idx[:-1]
    starts = torch.zeros(x.nnz, dtype=torch.bool, device=cuda_device)
    inner = col_ptr[1:-1]
    starts[inner[inner < x.nnz]] = True
    assert bool(torch.all(rising | starts[1:]))
    assert torch.equal(torch.bincount(codes.long(), minlength=256), torch.bincount(x.packed.long(), minlength=256))
    # entry by entry on a sample of genes: the source holds that (cell, gene) with that code
    rows_of = torch.repeat_interleave(torch.arange(x.rows, device=cuda_device), x.row_ptr[1:] - x.row_ptr[:-1])
    for gene in (0, 17, x.cols // 2, x.cols - 1):
        lo, hi = int(col_ptr[gene]), int(col_ptr[gene + 1])
        mask = x.col_idx == gene
        assert torch.equal(row_idx[lo:hi].long(), rows_of[mask])
        assert torch.equal(codes[lo:hi], x.packed[mask])


@pytest.mark.parametrize("bits,policy,n", [(8, 1, 64), (8, 2, 32), (4, 1, 128), (4, 2, 64)])
def test_deterministic_transpose_matches_the_fixed_order_bit_for_bit(cuda_device, oracle, bits, policy, n):
    """deterministic = 1 with the matrix handed to prepare: schedule gene_gather; whole range, a row
    range, alpha / beta, all equal to the oracle's fixed order in every bit; a second run repeats
    them.  Genes hold up to thousands of entries, so all eight runs and ragged chunks occur."""
    rng = np.random.default_rng(bits * 10 + policy + n)
    rows, cols = 6000, 23
    c = host_pack(oracle, random_csr(rng, rows=rows, cols=cols, max_nnz=20, bits=bits, policy=policy))
    x = to_dev(c, cuda_device)
    g, g_host = dense(rng, rows, n, torch.float32, cuda_device, std=1.0)
    op = ops.PreparedSpmm(capi.PROJECTION_TRANSPOSE, rows, cols, n, x.nnz, bits, policy, g.dtype, cuda_device,
                          deterministic=True, device_matrix=x)
    assert op.schedule == "gene_gather"
    assert op.persistent_bytes >= 5 * x.nnz
    rc, col_ptr, row_idx, codes = oracle.qcsr_gene_major(bits, cols, c["row_ptr"], c["packed_row_ptr"], c["col_idx"], c["packed"])
    assert rc == 0 and np.diff(col_ptr).max() > 8 * 256
    for lo, hi in [(0, rows), (777, 4100), (50, 50)]:
        want = oracle.qcsr_transpose_ordered(policy, col_ptr, row_idx, codes, c["scales"], c["offsets"], g_host, lo, hi)
        first = op.run(x, g, torch.full((cols, n), float("nan"), device=cuda_device), row_begin=lo, row_end=hi).cpu().numpy()
        again = op.run(x, g, torch.full((cols, n), float("nan"), device=cuda_device), row_begin=lo, row_end=hi).cpu().numpy()
        assert np.array_equal(bits_of(first), bits_of(want))
        assert np.array_equal(bits_of(first), bits_of(again))
    init = rng.normal(size=(cols, n)).astype(np.float32)
    want = oracle.qcsr_transpose_ordered(policy, col_ptr, row_idx, codes, c["scales"], c["offsets"], g_host, 0, rows,
                                         alpha=-1.5, beta=0.25, out=init)
    got = op.run(x, g, torch.from_numpy(init).to(cuda_device), alpha=-1.5, beta=0.25).cpu().numpy()
    assert np.array_equal(bits_of(got), bits_of(want))
    # and it is the transpose: the double-precision referee within the fp32 bound
    ref = oracle.qcsr_transpose(bits, policy, c["row_ptr"], c["packed_row_ptr"], c["col_idx"], c["packed"], c["scales"],
                                c["offsets"], g_host, cols)
    whole = op.run(x, g, torch.empty(cols, n, device=cuda_device)).cpu().numpy()
    assert np.allclose(whole, ref, rtol=1e-4, atol=1e-2)
    op.close()


def test_deterministic_transpose_unaligned_dense_rows(cuda_device, oracle):
    """G with a leading dimension that breaks the vector loads: scalar loads, same bits."""
    rng = np.random.default_rng(77)
    rows, cols, n = 900, 50, 64
    c = host_pack(oracle, random_csr(rng, rows=rows, cols=cols, max_nnz=30, bits=8))
    x = to_dev(c, cuda_device)
    g, g_host = dense(rng, rows, n, torch.float32, cuda_device, std=1.0, ld=n + 1)
    out = ops.spmm_transpose(x, g, deterministic=True).cpu().numpy()
    rc, col_ptr, row_idx, codes = oracle.qcsr_gene_major(8, cols, c["row_ptr"], c["packed_row_ptr"], c["col_idx"], c["packed"])
    want = oracle.qcsr_transpose_ordered(1, col_ptr, row_idx, codes, c["scales"], c["offsets"], np.ascontiguousarray(g_host), 0, rows)
    assert np.array_equal(bits_of(out), bits_of(want))


def test_deterministic_transpose_needs_the_matrix_and_a_covered_shape(cuda_device, oracle):
    rng = np.random.default_rng(9)
    c = host_pack(oracle, random_csr(rng, rows=64, cols=16, max_nnz=5, bits=8))
    x = to_dev(c, cuda_device)
    with pytest.raises(capi.Cb200Error):   # no matrix at prepare time
        ops.PreparedSpmm(capi.PROJECTION_TRANSPOSE, 64, 16, 64, x.nnz, 8, 1, torch.float32, cuda_device, deterministic=True)
    with pytest.raises(capi.Cb200Error):   # N outside {32, 64, 128}
        ops.PreparedSpmm(capi.PROJECTION_TRANSPOSE, 64, 16, 48, x.nnz, 8, 1, torch.float32, cuda_device, deterministic=True,
                         device_matrix=x)
    with pytest.raises(capi.Cb200Error):   # the copy does not fit the caller's limit
        ops.PreparedSpmm(capi.PROJECTION_TRANSPOSE, 64, 16, 64, x.nnz, 8, 1, torch.float32, cuda_device, deterministic=True,
                         device_matrix=x, persistent_limit_bytes=64)


def test_deterministic_transpose_at_scale_against_the_atomic_kernel(cuda_device):
    """Genes as in the benchmark configuration, 1/16 of its cells: the gather schedule against the
    atomic kernel within the fp32 bound, and two runs equal in every bit."""
    cfg = dict(synth.CONFIGS["c2_forward"])
    cfg["rows"] //= 16
    x = synth.make_qcsr_device(**cfg, device=cuda_device, seed=1)
    n = 64
    g = torch.randn(x.rows, n, device=cuda_device)
    op = ops.PreparedSpmm(capi.PROJECTION_TRANSPOSE, x.rows, x.cols, n, x.nnz, x.bits, x.policy, g.dtype, cuda_device,
                          deterministic=True, device_matrix=x)
    a = op.run(x, g, torch.empty(x.cols, n, device=cuda_device))
    b = op.run(x, g, torch.empty(x.cols, n, device=cuda_device))
    assert torch.equal(a.view(torch.int32), b.view(torch.int32))
    exact = ops.spmm_transpose(x, g)
    vals = x.dequantize().abs().double()
    col_l1 = torch.zeros(x.cols, dtype=torch.float64, device=cuda_device).index_add_(0, x.col_idx.long(), vals)
    gmax = float(g.abs().max())
    assert torch.all((a - exact).abs() <= 1e-4 * (col_l1[:, None] * gmax).float() + 1e-30)
    op.close()


def test_deterministic_transpose_skewed_genes(cuda_device, oracle):
    """One gene present in every cell, the others rare: the long gene is handed out first (genes go to
    CTAs in descending order of their entry count), the result is still the fixed-order one."""
    rng = np.random.default_rng(123)
    rows, cols, n = 7000, 60, 64
    counts = rng.integers(0, 4, size=rows)
    row_ptr = np.zeros(rows + 1, dtype=np.int64)
    np.cumsum(counts + 1, out=row_ptr[1:])
    others = np.array([g for g in range(cols) if g != 41])
    col_idx = np.concatenate([np.sort(np.append(rng.choice(others, size=int(k), replace=False), 41)) for k in counts]).astype(np.int32)
    c = dict(rows=rows, cols=cols, bits=8, policy=1, row_ptr=row_ptr, col_idx=col_idx,
             scales=rng.uniform(0.01, 0.5, size=cols).astype(np.float32), offsets=rng.uniform(-1, 1, size=cols).astype(np.float32),
             values=rng.uniform(-2.0, 40.0, size=len(col_idx)).astype(np.float32))
    c = host_pack(oracle, c)
    x = to_dev(c, cuda_device)
    g, g_host = dense(rng, rows, n, torch.float32, cuda_device, std=1.0)
    out = ops.spmm_transpose(x, g, deterministic=True).cpu().numpy()
    rc, col_ptr, row_idx, codes = oracle.qcsr_gene_major(8, cols, c["row_ptr"], c["packed_row_ptr"], c["col_idx"], c["packed"])
    assert rc == 0 and col_ptr[42] - col_ptr[41] == rows
    want = oracle.qcsr_transpose_ordered(1, col_ptr, row_idx, codes, c["scales"], c["offsets"], g_host, 0, rows)
    assert np.array_equal(bits_of(out), bits_of(want))
