"""GPU parity of the CSR -> physical Blocked-ELL lowering, through the C ABI, against the oracle
(bit-exact: geometry, metrics, padded feature-block offsets, column indices, values)."""
import os

import numpy as np
import pytest
import torch

from cellerator_b200 import capi, ops, synth
from conftest import GOLDEN
from test_lowering_oracle import kat_inputs

pytestmark = pytest.mark.gpu

GEO_FIELDS = ("state", "padded_rows", "padded_features", "block_rows", "ell_blocks_per_row", "ell_columns",
              "column_index_count", "value_bytes", "occupied_blocks", "stored_blocks", "dense_value_slots",
              "persistent_bytes", "source_bytes", "scalar_occupancy", "ell_slot_utilization", "value_slot_expansion",
              "storage_expansion")


def assert_same(oracle, low, args, bs, **limits):
    status, want, pfo, cols, vals = oracle.bell_lowering(*args, bs, **limits)
    assert status == 0
    geo = low.query(bs, **limits)
    assert {f: getattr(geo, f) for f in GEO_FIELDS} == want
    if want["state"] != 0:
        with pytest.raises(capi.Cb200Error):
            low.materialize(geo)
        return geo
    g_pfo, g_cols, g_vals = low.materialize(geo)
    torch.cuda.synchronize()
    assert np.array_equal(g_pfo.cpu().numpy().view(np.uint32), pfo)
    assert np.array_equal(g_cols.cpu().numpy(), cols)
    assert np.array_equal(g_vals.cpu().numpy(), vals)
    return geo


def test_kat_reference_fixture(cuda_device, oracle, kats):
    k = kats["bell_lowering_9x13"]
    ro, ids, vals, features, fbo, fperm, rperm = kat_inputs(k)
    low = ops.BellLowering(ro, ids, vals, features, fbo, fperm, rperm, cuda_device)
    for i, bs in enumerate(k["block_sizes"]):
        geo = assert_same(oracle, low, (ro, ids, vals, features, fbo, fperm, rperm), bs,
                          max_value_expansion=1000.0, max_storage_expansion=1000.0)
        assert geo.padded_features == k["padded_features"][i] and geo.dense_value_slots == k["dense_value_slots"][i]
        assert low.query(bs).state == k["default_policy_states"][i]


def test_golden_from_reference_sources(cuda_device):
    z = np.load(os.path.join(GOLDEN, "bell_lowering_small.npz"))
    low = ops.BellLowering(z["row_offsets"], z["feature_ids"], z["values"], int(z["features"]), z["fb_offsets"], z["fperm"],
                           z["rperm"], cuda_device)
    for bs in (8, 16, 32):
        geo = low.query(bs, max_value_expansion=1e9, max_storage_expansion=1e9)
        assert geo.state == 0 and geo.ell_blocks_per_row == int(z[f"geometry{bs}"][4])
        pfo, cols, vals = low.materialize(geo)
        assert np.array_equal(pfo.cpu().numpy().view(np.uint32), z[f"padded_offsets{bs}"])
        assert np.array_equal(cols.cpu().numpy(), z[f"columns{bs}"])
        assert np.array_equal(vals.cpu().numpy(), z[f"values{bs}"])


@pytest.mark.parametrize("seed", range(8))
def test_random_against_oracle(cuda_device, oracle, seed):
    """Value sizes 1..16 bytes, one to eight semantic blocks, clustered and uniform rows, empty rows, a
    ragged last block row; default and relaxed policy."""
    dtype = [np.float32, np.uint8, np.float64, np.uint16][seed % 4]
    h = synth.make_lowering_host(rows=301 + seed * 37, features=900 + seed * 211, feature_blocks=1 + seed, mean_nnz=25,
                                 seed=100 + seed, value_dtype=dtype, clustered=seed % 2 == 0)
    values = h["values"]
    if seed == 7:                                  # 12-byte values: the bytewise path
        values = np.ascontiguousarray(np.stack([values, values + 1, values + 2], axis=1))
    args = (h["row_offsets"], h["feature_ids"], values, h["features"], h["fb_offsets"], h["fperm"], h["rperm"])
    low = ops.BellLowering(*args, cuda_device)
    for bs in (8, 16, 32):
        assert_same(oracle, low, args, bs)
        assert_same(oracle, low, args, bs, max_value_expansion=1e9, max_storage_expansion=1e9)


def test_rejections(cuda_device, oracle, kats):
    k = kats["bell_lowering_9x13"]
    ro, ids, vals, features, fbo, fperm, rperm = kat_inputs(k)
    swapped = list(ids)
    swapped[0], swapped[1] = swapped[1], swapped[0]
    with pytest.raises(capi.Cb200Error, match="invalid source"):
        ops.BellLowering(ro, swapped, vals, features, fbo, fperm, rperm, cuda_device).query(8)
    low = ops.BellLowering(ro, ids, vals, features, fbo, fperm, rperm, cuda_device)
    low.finv[0], low.finv[1] = low.finv[1].clone(), low.finv[0].clone()
    with pytest.raises(capi.Cb200Error, match="incompatible plan"):
        low.query(8)
    low = ops.BellLowering(ro, ids, vals, features, fbo, fperm, rperm, cuda_device)
    low.rinv[2], low.rinv[3] = low.rinv[3].clone(), low.rinv[2].clone()
    with pytest.raises(capi.Cb200Error, match="incompatible order"):
        low.query(8)
    with pytest.raises(capi.Cb200Error, match="feature block is empty"):
        ops.BellLowering(ro, ids, vals, features, [0, 3, 3, 13], fperm, rperm, cuda_device).query(8)
    low = ops.BellLowering(ro, ids, vals, features, fbo, fperm, rperm, cuda_device)
    with pytest.raises(capi.Cb200Error):
        low.query(12)                                                           # not 8, 16 or 32
    geo = low.query(8, max_value_expansion=1000.0, max_storage_expansion=1000.0)
    geo.ell_blocks_per_row -= 1                                                 # a modified geometry is refused
    with pytest.raises(capi.Cb200Error, match="candidate mismatch"):
        low.materialize(geo)


def test_lowered_codes_feed_the_blocked_ell_projection(cuda_device, oracle):
    """Row-major layout with one-byte codes is a cb200_qbell: lowering a quantized CSR (zero offsets,
    so that empty slots decode to zero) and projecting it gives what the CSR projection gives."""
    rng = np.random.default_rng(3)
    rows, genes, n, bs = 32 * 40 + 7, 2048, 128, 32
    h = synth.make_lowering_host(rows=rows, features=genes, feature_blocks=1, mean_nnz=60, seed=9, value_dtype=np.uint8)
    ident_f, ident_r = np.arange(genes, dtype=np.uint32), np.arange(rows, dtype=np.uint32)
    low = ops.BellLowering(h["row_offsets"], h["feature_ids"], h["values"], genes, [0, genes], ident_f, ident_r, cuda_device)
    geo = low.query(bs, max_value_expansion=1e9, max_storage_expansion=1e9)
    stride = (geo.ell_columns + 15) // 16 * 16
    _, cols, codes = low.materialize(geo, layout=capi.BELL_VALUES_ROW_MAJOR, row_stride_bytes=stride)
    scales = rng.uniform(0.01, 0.05, genes).astype(np.float32)
    bell = ops.QuantizedBell.from_host(dict(rows=rows, cols=genes, block_size=bs, ell_cols=geo.ell_columns,
                                            row_stride_bytes=stride, bits=8, policy=1,
                                            block_col_idx=cols.cpu().numpy().view(np.uint32),
                                            packed=codes.cpu().numpy()[:rows * stride], scales=scales, offsets=None), cuda_device)
    csr = ops.QuantizedCsr.from_host(dict(rows=rows, cols=genes, bits=8, policy=1, row_ptr=h["row_offsets"].astype(np.int64),
                                          packed_row_ptr=None, col_idx=h["feature_ids"].astype(np.int32), packed=h["values"],
                                          scales=scales, offsets=None), cuda_device)
    w = torch.from_numpy(rng.normal(0, 0.02, (genes, n)).astype(np.float32)).to(cuda_device)
    y_bell = ops.bell_forward(bell, w)
    y_csr = ops.spmm_forward(csr, w)
    assert torch.allclose(y_bell, y_csr, rtol=1e-4, atol=1e-5)


def test_full_scale_properties(cuda_device):
    """250,000 cells x 8,192 genes (the Blocked-ELL configuration's shard), block size 32: properties that
    need no oracle -- every stored value lands exactly once (sum and count preserved), slots ascend,
    empty slots hold -1 and zeros, the ELL width is the largest block-row demand."""
    rows, genes, bs = 250_000, 8192, 32
    g = torch.Generator(device="cpu").manual_seed(0)
    # 16 of 256 block columns per block row, each slot of a present block stored with probability 0.6
    per_row = 300
    block_rows = (rows + bs - 1) // bs
    chosen = torch.stack([torch.randperm(genes // bs, generator=g)[:16] for _ in range(64)])       # 64 patterns
    pattern = chosen[torch.randint(0, 64, (block_rows,), generator=g)]                             # per block row
    pattern = pattern.repeat_interleave(bs, dim=0)[:rows].to(cuda_device)                          # per row
    pick = torch.rand(rows, 16 * bs, device=cuda_device).argsort(dim=1)[:, :per_row]
    feature = (pattern.gather(1, pick // bs) * bs + pick % bs).sort(dim=1).values.to(torch.int32)
    assert bool((feature[:, 1:] > feature[:, :-1]).all())
    row_offsets = (torch.arange(rows + 1, device=cuda_device, dtype=torch.int64) * per_row).to(torch.int32)
    values = torch.randint(1, 256, (rows * per_row,), device=cuda_device, dtype=torch.uint8)
    ident_f = torch.arange(genes, dtype=torch.int32, device=cuda_device)
    rperm = torch.arange(rows, dtype=torch.int32, device=cuda_device)                              # identity keeps the patterns
    low = ops.BellLowering(row_offsets, feature.reshape(-1), values, genes, [0, genes], ident_f, rperm, cuda_device)
    geo = low.query(bs)
    assert geo.state == 0 and geo.ell_blocks_per_row == 16 and geo.block_rows == block_rows
    assert geo.occupied_blocks == 16 * block_rows and abs(geo.scalar_occupancy - per_row / (16 * bs)) < 1e-3
    _, cols, vals = low.materialize(geo)
    c = cols.view(block_rows, 16)
    assert bool((c >= 0).all()) and bool((c[:, 1:] > c[:, :-1]).all())
    assert int((vals != 0).sum()) == rows * per_row
    assert int(vals.sum(dtype=torch.int64)) == int(values.sum(dtype=torch.int64))


def test_pack_dense_operand_kat_and_random(cuda_device, oracle):
    """pack_dense_operand_cuda's contract: the reference test's vector (tests/math_execution_csr_test.cu:93-112),
    then random shapes, value sizes, both source layouts, strided sources, and the padded physical order."""
    src = torch.arange(1, 9, dtype=torch.float32, device=cuda_device).reshape(4, 2)
    perm = torch.tensor([2, 0, 3, 1], dtype=torch.int32, device=cuda_device)
    assert ops.pack_dense_operand(src, perm).flatten().tolist() == [5.0, 6.0, 1.0, 2.0, 7.0, 8.0, 3.0, 4.0]
    assert ops.pack_dense_operand(src.t().contiguous(), perm, col_major=True).flatten().tolist() == [5.0, 6.0, 1.0, 2.0, 7.0, 8.0, 3.0, 4.0]
    rng = np.random.default_rng(0)
    for features, columns, dtype, pad in [(1000, 64, torch.bfloat16, 0), (333, 7, torch.float32, 3), (257, 128, torch.float64, 0),
                                          (512, 33, torch.uint8, 5), (4096, 256, torch.bfloat16, 8)]:
        full = torch.from_numpy(rng.integers(0, 200, size=(features, columns + pad)).astype(np.float32)).to(cuda_device).to(dtype)
        view = full[:, :columns]
        fperm = rng.permutation(features).astype(np.uint32)
        d_perm = torch.from_numpy(fperm.view(np.int32)).to(cuda_device)
        host = view.cpu().contiguous().view(torch.uint8).numpy().reshape(features, -1)       # bytes of every row
        want = oracle.pack_dense_operand(host, fperm)
        got = ops.pack_dense_operand(view, d_perm)
        assert np.array_equal(got.cpu().view(torch.uint8).numpy().reshape(features, -1), want)
        col = view.t().contiguous()                                                          # [columns][features]
        got_c = ops.pack_dense_operand(col, d_perm, col_major=True)
        assert torch.equal(got_c, got)
        cuts = np.sort(rng.choice(np.arange(1, features), size=3, replace=False))
        fbo = np.concatenate([[0], cuts, [features]]).astype(np.uint32)
        widths = np.diff(fbo.astype(np.int64))
        pfo = np.concatenate([[0], np.cumsum((widths + 31) // 32 * 32)]).astype(np.uint32)
        want_p = oracle.pack_dense_operand(host, fperm, fb_offsets=fbo, padded_offsets=pfo)
        got_p = ops.pack_dense_operand(view, d_perm, fb_offsets=fbo, padded_offsets=pfo)
        assert np.array_equal(got_p.cpu().view(torch.uint8).numpy().reshape(int(pfo[-1]), -1), want_p)
    bad = torch.tensor([2, 0, 9, 1], dtype=torch.int32, device=cuda_device)
    with pytest.raises(capi.Cb200Error, match="invalid geometry"):
        ops.pack_dense_operand(src, bad)


def test_permuted_lowering_and_packed_operand_project_like_the_csr(cuda_device, oracle):
    """The two prepare-time steps together, under random row and feature orders and three semantic blocks:
    lowered codes (row-major) x W packed in the padded physical order = the CSR projection, with the rows
    of the result in execution order."""
    rng = np.random.default_rng(17)
    rows, genes, n, bs = 32 * 30 + 11, 1500, 128, 32
    h = synth.make_lowering_host(rows=rows, features=genes, feature_blocks=3, mean_nnz=50, seed=4, value_dtype=np.uint8)
    low = ops.BellLowering(h["row_offsets"], h["feature_ids"], h["values"], genes, h["fb_offsets"], h["fperm"], h["rperm"], cuda_device)
    geo = low.query(bs, max_value_expansion=1e9, max_storage_expansion=1e9)
    stride = (geo.ell_columns + 15) // 16 * 16
    pfo, cols, codes = low.materialize(geo, layout=capi.BELL_VALUES_ROW_MAJOR, row_stride_bytes=stride)
    scales = rng.uniform(0.01, 0.05, genes).astype(np.float32)
    w = torch.from_numpy(rng.normal(0, 0.02, (genes, n)).astype(np.float32)).to(cuda_device)
    pfo_host = pfo.cpu().numpy().view(np.uint32)
    w_phys = ops.pack_dense_operand(w, low.fperm, fb_offsets=h["fb_offsets"], padded_offsets=pfo_host)
    s_phys = ops.pack_dense_operand(torch.from_numpy(scales).to(cuda_device)[:, None].contiguous(), low.fperm,
                                    fb_offsets=h["fb_offsets"], padded_offsets=pfo_host)[:, 0].contiguous()
    bell = ops.QuantizedBell.from_host(dict(rows=rows, cols=geo.padded_features, block_size=bs, ell_cols=geo.ell_columns,
                                            row_stride_bytes=stride, bits=8, policy=1,
                                            block_col_idx=cols.cpu().numpy().view(np.uint32),
                                            packed=codes.cpu().numpy()[:rows * stride], scales=s_phys.cpu().numpy(),
                                            offsets=None), cuda_device)
    csr = ops.QuantizedCsr.from_host(dict(rows=rows, cols=genes, bits=8, policy=1, row_ptr=h["row_offsets"].astype(np.int64),
                                          packed_row_ptr=None, col_idx=h["feature_ids"].astype(np.int32), packed=h["values"],
                                          scales=scales, offsets=None), cuda_device)
    y_bell = ops.bell_forward(bell, w_phys)                      # rows in execution order
    y_csr = ops.spmm_forward(csr, w)                             # rows in canonical order
    assert torch.allclose(y_bell, y_csr[low.rperm.long()], rtol=1e-4, atol=1e-5)


def test_edge_shapes(cuda_device, oracle):
    """No stored entry at all (state empty_source, nothing to materialize), fewer rows than a block,
    one feature block narrower than a block, 16-byte values."""
    ro = np.zeros(6, dtype=np.uint32)
    empty = ops.BellLowering(ro, np.zeros(0, dtype=np.uint32), np.zeros(0, dtype=np.float32), 7, [0, 7],
                             np.arange(7, dtype=np.uint32), np.arange(5, dtype=np.uint32), cuda_device)
    geo = empty.query(8)
    assert geo.state == 1 and geo.ell_blocks_per_row == 0 and geo.value_bytes == 0
    want = oracle.bell_lowering(ro, [], np.zeros(0, dtype=np.float32), 7, [0, 7], np.arange(7), np.arange(5), 8, materialize=False)[1]
    assert want["state"] == 1 and geo.padded_rows == want["padded_rows"] and geo.padded_features == want["padded_features"]
    with pytest.raises(capi.Cb200Error):
        empty.materialize(geo)
    # three rows, features [0,3) | [3,5): every semantic block narrower than the smallest block size
    ro = np.array([0, 2, 2, 5], dtype=np.uint32)
    ids = np.array([1, 4, 0, 2, 3], dtype=np.uint32)
    vals = np.arange(5 * 4, dtype=np.float32).reshape(5, 4)          # 16 bytes per stored entry
    args = (ro, ids, vals, 5, [0, 3, 5], np.array([2, 0, 4, 1, 3], dtype=np.uint32), np.array([1, 2, 0], dtype=np.uint32))
    low = ops.BellLowering(*args, cuda_device)
    for bs in (8, 16, 32):
        geo = assert_same(oracle, low, args, bs, max_value_expansion=1e9, max_storage_expansion=1e9)
        assert geo.block_rows == 1 and geo.padded_features == 2 * bs


def test_execution_csr_ids(cuda_device, oracle):
    """cb200_build_execution_csr: the reference test's fixture, random partitions against the oracle, and
    the violation flags (1 geometry, 2 identity)."""
    from test_lowering_oracle import ordered_partition
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.uint32).view(np.int32)).to(cuda_device)
    flags, ids = ops.build_execution_csr(dev([0, 2, 4]), dev([0, 0, 1, 1]), dev([0, 1, 0, 1]), dev([2, 0, 3, 1]), 4, [0, 2, 4],
                                         dev([2, 0, 3, 1]))
    assert flags == 0 and ids.tolist() == [0, 1, 2, 3]
    rng = np.random.default_rng(12)
    for blocks, rows, mean in ((1, 300, 40), (4, 1000, 70), (16, 257, 5)):
        p = ordered_partition(rng, rows=rows, features=2000, feature_blocks=blocks, mean_nnz=mean)
        host = [p["row_offsets"], p["block_ids"], p["local_ids"], p["canonical_ids"]]
        status, want = oracle.build_execution_csr(*host, p["features"], p["fb_offsets"], p["fperm"])
        assert status == 0
        flags, ids = ops.build_execution_csr(*[dev(a) for a in host], p["features"], p["fb_offsets"], dev(p["fperm"]))
        assert flags == 0 and np.array_equal(ids.cpu().numpy().view(np.uint32), want)
        for field, make_bad, flag in ((3, lambda v: (v + 1) % p["features"], 2), (1, lambda v: v + blocks, 1),
                                      (2, lambda v: v + 10_000, 1)):
            bad = [a.copy() for a in host]
            bad[field][11] = make_bad(bad[field][11])
            assert oracle.build_execution_csr(*bad, p["features"], p["fb_offsets"], p["fperm"])[0] == {1: 3, 2: 2}[flag]
            assert ops.build_execution_csr(*[dev(a) for a in bad], p["features"], p["fb_offsets"], dev(p["fperm"]))[0] & flag
        swapped = [a.copy() for a in host]                 # two neighbours of one row out of order
        r = int(np.argmax(np.diff(p["row_offsets"].astype(np.int64)) >= 2))
        i = int(p["row_offsets"][r])
        for a in swapped[1:]:
            a[i], a[i + 1] = a[i + 1], a[i]
        assert ops.build_execution_csr(*[dev(a) for a in swapped], p["features"], p["fb_offsets"], dev(p["fperm"]))[0] == 2
