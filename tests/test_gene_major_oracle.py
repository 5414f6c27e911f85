"""CPU checks of the oracle's gene-major copy (stable CSR -> CSC of the codes) and of its order-fixed
transpose: a hand-made case, numpy's stable sort as a second statement of the placement, and the
double-precision referee (pinned to the reference elsewhere in this suite) for the sums."""
import numpy as np
import pytest

from conftest import random_csr


def pack(oracle, c):
    prp, _ = oracle.build_packed_row_ptr(c["bits"], c["row_ptr"])
    c = dict(c)
    c["packed_row_ptr"] = prp
    c["packed"] = oracle.pack_csr(c["bits"], c["policy"], c["row_ptr"], prp, c["col_idx"], c["scales"], c["offsets"], c["values"])
    return c


def test_gene_major_by_hand(oracle):
    # rows: {1: a, 3: b}, {}, {0: c, 1: d}, {3: e}   with 8-bit codes 10, 20, 30, 40, 50
    row_ptr = np.array([0, 2, 2, 4, 5], dtype=np.int64)
    col_idx = np.array([1, 3, 0, 1, 3], dtype=np.int32)
    packed = np.array([10, 20, 30, 40, 50], dtype=np.uint8)
    rc, col_ptr, row_idx, codes = oracle.qcsr_gene_major(8, 4, row_ptr, row_ptr, col_idx, packed)
    assert rc == 0
    assert col_ptr.tolist() == [0, 1, 3, 3, 5]
    assert row_idx.tolist() == [2, 0, 2, 0, 3]
    assert codes.tolist() == [30, 10, 40, 20, 50]
    bad = col_idx.copy()
    bad[4] = 4
    assert oracle.qcsr_gene_major(8, 4, row_ptr, row_ptr, bad, packed)[0] == 1


@pytest.mark.parametrize("bits", [8, 4])
def test_gene_major_is_numpys_stable_sort(oracle, bits):
    rng = np.random.default_rng(5 + bits)
    c = pack(oracle, random_csr(rng, rows=700, cols=37, max_nnz=30, bits=bits))
    rc, col_ptr, row_idx, codes = oracle.qcsr_gene_major(bits, c["cols"], c["row_ptr"], c["packed_row_ptr"], c["col_idx"], c["packed"])
    assert rc == 0
    src_codes = oracle.extract_codes(bits, c["row_ptr"], c["packed_row_ptr"], c["packed"])
    rows_of = np.repeat(np.arange(c["rows"], dtype=np.int32), np.diff(c["row_ptr"]))
    order = np.argsort(c["col_idx"], kind="stable")
    assert np.array_equal(row_idx, rows_of[order])
    assert np.array_equal(codes, src_codes[order])
    assert np.array_equal(col_ptr, np.concatenate([[0], np.cumsum(np.bincount(c["col_idx"], minlength=c["cols"]))]))


@pytest.mark.parametrize("policy", [1, 2])
def test_ordered_transpose_agrees_with_the_referee(oracle, policy):
    """Genes with more than 8 * 256 entries, so every run of the fixed order is exercised."""
    rng = np.random.default_rng(40 + policy)
    rows, cols, n = 5000, 9, 32
    c = pack(oracle, random_csr(rng, rows=rows, cols=cols, max_nnz=9, bits=8, policy=policy))
    g = rng.normal(size=(rows, n)).astype(np.float32)
    rc, col_ptr, row_idx, codes = oracle.qcsr_gene_major(8, cols, c["row_ptr"], c["packed_row_ptr"], c["col_idx"], c["packed"])
    assert rc == 0 and np.diff(col_ptr).max() > 8 * 256
    for lo, hi in [(0, rows), (1234, 4321), (10, 10)]:
        ref = oracle.qcsr_transpose(8, policy, c["row_ptr"], c["packed_row_ptr"], c["col_idx"], c["packed"], c["scales"],
                                    c["offsets"], g, cols, lo, hi)
        got = oracle.qcsr_transpose_ordered(policy, col_ptr, row_idx, codes, c["scales"], c["offsets"], g, lo, hi)
        assert np.allclose(got, ref, rtol=1e-4, atol=1e-2)
    init = rng.normal(size=(cols, n)).astype(np.float32)
    ref = oracle.qcsr_transpose(8, policy, c["row_ptr"], c["packed_row_ptr"], c["col_idx"], c["packed"], c["scales"],
                                c["offsets"], g, cols)
    got = oracle.qcsr_transpose_ordered(policy, col_ptr, row_idx, codes, c["scales"], c["offsets"], g, 0, rows,
                                        alpha=-1.5, beta=0.25, out=init)
    assert np.allclose(got, -1.5 * ref + 0.25 * init, rtol=1e-4, atol=1e-2)
