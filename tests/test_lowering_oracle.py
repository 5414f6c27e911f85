"""The oracle's CSR -> physical Blocked-ELL lowering (oracle.c, orc_bell_lowering) pinned against the
reference: the fixture and expected numbers of the reference's own test
(tests/math_bell_lowering_test.cc), a golden case written by the reference's compiled sources, and --
where oracle/_ref is built -- random cases run through both."""
import os

import numpy as np
import pytest

from cellerator_b200 import synth
from conftest import GOLDEN


def kat_inputs(k):
    rows, features = k["rows"], k["features"]
    fperm, rperm = k["feature_permutation"], k["row_permutation"]
    canonical = [None] * rows
    for er, pair in enumerate(k["execution_features_by_execution_row"]):
        canonical[rperm[er]] = sorted(fperm[e] for e in pair)
    ro, ids, vals = [0], [], []
    for row in range(rows):
        for f in canonical[row]:
            ids.append(f)
            vals.append(float(row * 100 + f + 1))
        ro.append(len(ids))
    return ro, ids, np.array(vals, dtype=np.float32), features, k["feature_block_offsets"], fperm, rperm


def independent_decode(rows, features, fb_offsets, fperm, rperm, bs, padded_offsets, columns, values, ell_blocks):
    """Dense canonical matrix from a block-major physical BELL, the way the reference's test decodes it
    (tests/math_bell_lowering_test.cc:137-200); asserts that padding holds zeros."""
    dense = np.zeros((rows, features), dtype=values.dtype)
    block_rows = len(columns) // max(ell_blocks, 1) if ell_blocks else 0
    v = values.reshape(block_rows, ell_blocks, bs, bs) if ell_blocks else values.reshape(0, 0, bs, bs)
    c = columns.reshape(block_rows, ell_blocks)
    for br in range(block_rows):
        for slot in range(ell_blocks):
            pb = int(c[br, slot])
            blk = v[br, slot]
            if pb < 0:
                assert not blk.any()
                continue
            for lane in range(bs):
                er = br * bs + lane
                for local in range(bs):
                    val = blk[lane, local]
                    pf = pb * bs + local
                    if er >= rows:
                        assert val == 0
                        continue
                    semantic = int(np.searchsorted(padded_offsets, pf, side="right")) - 1
                    within = pf - int(padded_offsets[semantic])
                    if within >= fb_offsets[semantic + 1] - fb_offsets[semantic]:
                        assert val == 0
                        continue
                    dense[rperm[er], fperm[fb_offsets[semantic] + within]] = val
    return dense


def dense_of(rows, features, ro, ids, vals):
    d = np.zeros((rows, features), dtype=np.asarray(vals).dtype)
    for r in range(rows):
        d[r, ids[ro[r]:ro[r + 1]]] = vals[ro[r]:ro[r + 1]]
    return d


def test_kat_reference_fixture(oracle, kats):
    k = kats["bell_lowering_9x13"]
    ro, ids, vals, features, fbo, fperm, rperm = kat_inputs(k)
    want = dense_of(k["rows"], features, ro, np.array(ids), vals)
    for i, bs in enumerate(k["block_sizes"]):
        status, geo, pfo, cols, out = oracle.bell_lowering(ro, ids, vals, features, fbo, fperm, rperm, bs,
                                                           max_value_expansion=1000.0, max_storage_expansion=1000.0)
        assert status == 0 and geo["state"] == 0
        assert geo["padded_features"] == k["padded_features"][i] and geo["dense_value_slots"] == k["dense_value_slots"][i]
        got = independent_decode(k["rows"], features, fbo, fperm, rperm, bs, pfo, cols, out.view(np.float32), geo["ell_blocks_per_row"])
        assert np.array_equal(got, want)
        default = oracle.bell_lowering(ro, ids, vals, features, fbo, fperm, rperm, bs, materialize=False)[1]
        assert default["state"] == k["default_policy_states"][i]
        if bs == 8:
            assert abs(default["ell_slot_utilization"] - k["bell8_ell_slot_utilization"]) < 1e-12


def test_kat_rejections(oracle, kats):
    """The failure cases of the reference's test (tests/math_bell_lowering_test.cc:260-330): unsorted
    features, maps that are not inverses, capacity."""
    k = kats["bell_lowering_9x13"]
    ro, ids, vals, features, fbo, fperm, rperm = kat_inputs(k)
    bad = list(ids)
    bad[0], bad[1] = bad[1], bad[0]
    assert oracle.bell_lowering(ro, bad, vals, features, fbo, fperm, rperm, 8)[0] == 2          # invalid_source
    twice = list(fperm)
    twice[1] = twice[0]
    assert oracle.bell_lowering(ro, ids, vals, features, fbo, twice, rperm, 8)[0] == 3          # incompatible_plan
    rtwice = list(rperm)
    rtwice[3] = rtwice[2]
    assert oracle.bell_lowering(ro, ids, vals, features, fbo, fperm, rtwice, 8)[0] == 4         # incompatible_order
    assert oracle.bell_lowering(ro, ids, vals, features, [0, 3, 3, 13], fperm, rperm, 8)[0] == 3  # empty feature block


def test_golden_from_reference_sources(oracle):
    z = np.load(os.path.join(GOLDEN, "bell_lowering_small.npz"))
    for bs in (8, 16, 32):
        status, geo, pfo, cols, vals = oracle.bell_lowering(z["row_offsets"], z["feature_ids"], z["values"], int(z["features"]),
                                                            z["fb_offsets"], z["fperm"], z["rperm"], bs,
                                                            max_value_expansion=1e9, max_storage_expansion=1e9)
        assert status == 0
        assert [geo[k] for k in oracle.BELL_GEOMETRY] == z[f"geometry{bs}"].tolist()
        assert [geo[k] for k in oracle.BELL_METRICS] == z[f"metrics{bs}"].tolist()
        assert np.array_equal(pfo, z[f"padded_offsets{bs}"]) and np.array_equal(cols, z[f"columns{bs}"])
        assert np.array_equal(vals, z[f"values{bs}"])


@pytest.mark.parametrize("seed", range(6))
def test_oracle_equals_reference_random(oracle, reference, seed):
    dtype = [np.float32, np.uint8, np.float64, np.uint16][seed % 4]
    h = synth.make_lowering_host(rows=70 + seed * 13, features=300 + seed * 50, feature_blocks=1 + seed, mean_nnz=12,
                                 seed=seed, value_dtype=dtype, clustered=seed % 2 == 0)
    for bs in (8, 16, 32):
        for limits in ({}, dict(max_value_expansion=1e9, max_storage_expansion=1e9)):
            a = oracle.bell_lowering(h["row_offsets"], h["feature_ids"], h["values"], h["features"], h["fb_offsets"],
                                     h["fperm"], h["rperm"], bs, **limits)
            b = reference.bell_lowering(h["row_offsets"], h["feature_ids"], h["values"], h["features"], h["fb_offsets"],
                                        h["fperm"], h["rperm"], bs, **limits)
            assert a[0] == b[0] and a[1] == b[1]
            for x, y in zip(a[2:], b[2:]):
                assert (x is None and y is None) or np.array_equal(x, y)


def test_row_major_layout_is_the_block_major_one_transposed(oracle):
    """values_layout 1 (rows of the quantized Blocked-ELL matrices) holds the same values as the
    reference's block-major layout, at r * stride + slot * bs + column."""
    h = synth.make_lowering_host(rows=90, features=200, feature_blocks=3, mean_nnz=9, seed=5, value_dtype=np.uint8)
    for bs in (8, 32):
        args = (h["row_offsets"], h["feature_ids"], h["values"], h["features"], h["fb_offsets"], h["fperm"], h["rperm"], bs)
        _, geo, _, cols, blk = oracle.bell_lowering(*args, max_value_expansion=1e9, max_storage_expansion=1e9)
        stride = geo["ell_columns"] + 16
        st, _, _, cols2, row = oracle.bell_lowering(*args, max_value_expansion=1e9, max_storage_expansion=1e9,
                                                    values_layout=1, row_stride_bytes=stride)
        assert st == 0 and np.array_equal(cols, cols2)
        ell = geo["ell_blocks_per_row"]
        b = blk.reshape(geo["block_rows"], ell, bs, bs).transpose(0, 2, 1, 3).reshape(geo["padded_rows"], ell * bs)
        r = row.reshape(geo["padded_rows"], stride)
        assert np.array_equal(r[:, :ell * bs], b) and not r[:, ell * bs:].any()


def ordered_partition(rng, rows, features, feature_blocks, mean_nnz):
    """An ordered plan partition: per entry (semantic block, position in block, canonical id), rows in
    ascending execution order; plus the plan's block offsets and feature permutation."""
    h = synth.make_lowering_host(rows=rows, features=features, feature_blocks=feature_blocks, mean_nnz=mean_nnz,
                                 seed=int(rng.integers(1 << 30)), value_dtype=np.uint8)
    fbo, fperm, finv = h["fb_offsets"], h["fperm"], h["finv"]
    ro = h["row_offsets"]
    execution = finv[h["feature_ids"]]
    for r in range(rows):                                   # a row's entries ascend in execution order
        execution[ro[r]:ro[r + 1]] = np.sort(execution[ro[r]:ro[r + 1]])
    block = (np.searchsorted(fbo, execution, side="right") - 1).astype(np.uint32)
    return dict(row_offsets=ro, block_ids=block, local_ids=(execution - fbo[block]).astype(np.uint32),
                canonical_ids=fperm[execution], features=features, fb_offsets=fbo, fperm=fperm, execution=execution)


def test_execution_csr_kat_and_reference(oracle, reference):
    """The fixture of the reference's test (tests/math_execution_csr_test.cu:30-33,57-86): execution ids
    0..3; then random partitions and one violation of each kind through both implementations."""
    fixture = ([0, 2, 4], [0, 0, 1, 1], [0, 1, 0, 1], [2, 0, 3, 1], 4, [0, 2, 4], [2, 0, 3, 1])
    for lib in (oracle, reference):
        status, ids = lib.build_execution_csr(*fixture)
        assert status == 0 and ids.tolist() == [0, 1, 2, 3]
    rng = np.random.default_rng(4)
    for blocks in (1, 3, 9):
        p = ordered_partition(rng, rows=120, features=500, feature_blocks=blocks, mean_nnz=15)
        args = [p["row_offsets"], p["block_ids"], p["local_ids"], p["canonical_ids"], p["features"], p["fb_offsets"], p["fperm"]]
        a, b = oracle.build_execution_csr(*args), reference.build_execution_csr(*args)
        assert a[0] == b[0] == 0 and np.array_equal(a[1], b[1]) and np.array_equal(a[1], p["execution"])
        for field, make_bad in ((3, lambda v: (v + 1) % p["features"]), (1, lambda v: v + blocks), (2, lambda v: v + 10_000)):
            bad = list(args)
            bad[field] = args[field].copy()
            bad[field][7] = make_bad(bad[field][7])
            assert oracle.build_execution_csr(*bad)[0] == reference.build_execution_csr(*bad)[0] != 0
