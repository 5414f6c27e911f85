"""Pins the C restatement (oracle/oracle.c) against (1) the known-answer vectors held by the
reference's own tests, (2) golden outputs produced by the reference's sources compiled in
place (tests/golden/*.npz, made by tests/golden/make_golden.py), and (3) where the reference
tree is present, the compiled reference itself on random inputs."""
import hashlib
import os

import numpy as np
import pytest

from conftest import GOLDEN, random_csr


def rule_codes(k, bits):
    max_code = (1 << bits) - 1
    row_ptr, col = k["row_ptr"], k["col_idx"]
    codes = []
    for r in range(k["rows"]):
        for i in range(row_ptr[r], row_ptr[r + 1]):
            codes.append((i + r + col[i]) % (max_code + 1))
    return np.array(codes, dtype=np.uint8)


def pack_by_rule(codes, row_ptr, bits):
    """Byte layout written out longhand: code i of a row -> byte i // cpb, shift (i % cpb) * bits."""
    cpb = 8 // bits
    out = []
    for r in range(len(row_ptr) - 1):
        row = codes[row_ptr[r]:row_ptr[r + 1]]
        for b in range(0, len(row), cpb):
            byte = 0
            for lane, c in enumerate(row[b:b + cpb]):
                byte |= int(c) << (lane * bits)
            out.append(byte)
    return np.array(out, dtype=np.uint8)


@pytest.mark.parametrize("bits", [1, 2, 4, 8])
@pytest.mark.parametrize("policy", [1, 2])
def test_kat_quantized_csr_4x8(oracle, kats, bits, policy):
    k = kats["quantized_csr_4x8"]
    row_ptr = np.array(k["row_ptr"], dtype=np.int64)
    col = np.array(k["col_idx"], dtype=np.int32)
    scales = np.array(k["gene_scales"], dtype=np.float32)
    offsets = np.array(k["gene_offsets"] if policy == 1 else k["row_offsets"], dtype=np.float32)
    codes = rule_codes(k, bits)
    rows_of = np.repeat(np.arange(k["rows"]), np.diff(row_ptr))
    off = offsets[col] if policy == 1 else offsets[rows_of]
    values = (off + scales[col] * codes.astype(np.float32)).astype(np.float32)

    prp, total = oracle.build_packed_row_ptr(bits, row_ptr)
    cpb = 8 // bits
    assert prp.tolist() == np.concatenate([[0], np.cumsum(-(-np.diff(row_ptr) // cpb))]).tolist()
    packed = oracle.pack_csr(bits, policy, row_ptr, prp, col, scales, offsets, values)
    assert packed.tolist() == pack_by_rule(codes, row_ptr, bits).tolist()
    assert oracle.extract_codes(bits, row_ptr, prp, packed).tolist() == codes.tolist()
    back = oracle.unpack_csr(bits, policy, row_ptr, prp, col, scales, offsets, packed)
    assert np.max(np.abs(back - values)) <= k["roundtrip_eps"]

    brp, count = oracle.build_uniform_block_row_ptr(k["rows"], k["rows_per_block"])
    assert count == 2 and brp.tolist() == [0, 2, 4]
    blk = oracle.get_block(row_ptr, prp, brp, 1)
    assert (blk["row_begin"], blk["row_end"], blk["nnz_begin"], blk["nnz_end"]) == (2, 4, 7, 12)
    assert (blk["packed_begin"], blk["packed_end"]) == (int(prp[2]), int(prp[4]))
    # block-local pack: values rebased to the block's first entry (packing.cuh:294-310)
    part = oracle.pack_csr(bits, policy, row_ptr, prp, col, scales, offsets, values[7:], row_begin=2, row_end=4,
                           value_base=7)
    assert part[prp[2]:].tolist() == packed[prp[2]:].tolist()


def test_kat_referee_forward_and_transposed(oracle, kats):
    k = kats["referee_2x3"]
    y = oracle.spmm_reference(k["m"], k["k"], k["n"], k["row_offsets"], k["columns"], k["values"],
                              np.array(k["rhs"]).reshape(3, 2), alpha=k["alpha"], beta=k["beta"],
                              initial=np.array(k["initial"]).reshape(2, 2), initial_ld=2, epilogue=k["epilogue"],
                              bias=k["bias"])
    assert np.max(np.abs(y.ravel() - np.array(k["expected"]))) < 1e-12
    t = k["transposed"]
    yt = oracle.spmm_reference(k["m"], k["k"], k["n"], t["row_offsets"], t["columns"], t["values"],
                               np.array(t["rhs"]).reshape(2, 3), transpose_sparse=True, transpose_dense=True,
                               rhs_ld=t["rhs_ld"], alpha=k["alpha"], beta=k["beta"],
                               initial=np.array(k["initial"]).reshape(2, 2), initial_ld=2, epilogue=k["epilogue"],
                               bias=k["bias"])
    assert np.max(np.abs(yt.ravel() - np.array(k["expected"]))) < 1e-12


def test_kat_csr_3x3_forward_and_bwd_rhs(oracle, kats):
    k = kats["csr_3x3"]
    rhs = np.array(k["rhs"], dtype=np.float32).reshape(3, 2)
    y = oracle.spmm_reference(3, 3, 2, k["major_ptr"], k["minor_idx"], k["values"], rhs)
    assert y.ravel().tolist() == k["spmm_fwd"]
    g = np.array(k["grad_out"], dtype=np.float32).reshape(3, 2)
    gt = oracle.spmm_reference(3, 3, 2, k["major_ptr"], k["minor_idx"], k["values"], g, transpose_sparse=True)
    assert gt.ravel().tolist() == k["bwd_rhs"]


@pytest.mark.parametrize("bits,policy", [(8, 1), (4, 2)])
def test_kat_bell_3x3(oracle, kats, bits, policy):
    k = kats["bell_3x3"]
    bci = np.array(k["block_col_idx"], dtype=np.uint32)
    scales = np.array(k["per_gene_scales"] if policy == 1 else k["column_scales"], dtype=np.float32)
    offsets = None if policy == 1 else np.array(k["row_offsets"], dtype=np.float32)
    stride = -(-k["ell_cols"] * bits // 8)
    packed = oracle.bell_pack(bits, policy, 3, 3, 1, 2, stride, bci, scales, offsets, k["slot_values"])
    ro, cols, vals = oracle.bell_to_csr(bits, policy, 3, 3, 1, 2, stride, bci, scales, offsets, packed)
    assert ro.tolist() == [0, 2, 4, 5]
    y = oracle.spmm_reference(3, 3, 2, ro, cols, vals, np.array(k["rhs"], dtype=np.float32).reshape(3, 2))
    assert np.allclose(y.ravel(), k["expected"], atol=1e-4)
    dec = oracle.bell_unpack(bits, policy, 3, 3, 1, 2, stride, bci, scales, offsets, packed)
    assert dec.ravel().tolist() == k["slot_values"]  # the slot of the empty block decodes to exactly 0


@pytest.mark.parametrize("name", ["csr8_small", "csr4_small"])
def test_golden_csr_from_reference_sources(oracle, name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    bits, rows, cols, n = int(z["bits"]), int(z["rows"]), int(z["cols"]), int(z["n"])
    prp, total = oracle.build_packed_row_ptr(bits, z["row_ptr"])
    assert np.array_equal(prp, z["packed_row_ptr"]) and total == len(z["packed"])
    packed = oracle.pack_csr(bits, 1, z["row_ptr"], prp, z["col_idx"], z["scales"], z["offsets"], z["values"])
    assert np.array_equal(packed, z["packed"])                      # integer parity: bit-exact
    decoded = oracle.unpack_csr(bits, 1, z["row_ptr"], prp, z["col_idx"], z["scales"], z["offsets"], packed)
    assert np.array_equal(decoded, z["decoded"])                    # same unfused product-then-sum
    y = oracle.spmm_reference(rows, cols, n, z["row_ptr"], z["col_idx"], decoded, z["w"])
    assert np.array_equal(y, z["y"])                                # same order of double sums
    gt = oracle.spmm_reference(cols, rows, n, z["row_ptr"], z["col_idx"], decoded, z["g"], transpose_sparse=True)
    assert np.array_equal(gt, z["gt"])
    # the composed range helpers used by the GPU parity tests
    y2 = oracle.qcsr_forward(bits, 1, z["row_ptr"], prp, z["col_idx"], packed, z["scales"], z["offsets"], z["w"],
                             cols, row_begin=5, row_end=rows - 3)
    assert np.array_equal(y2, z["y"][5:rows - 3])
    half = rows // 2
    part = (oracle.qcsr_transpose(bits, 1, z["row_ptr"], prp, z["col_idx"], packed, z["scales"], z["offsets"], z["g"],
                                  cols, 0, half)
            + oracle.qcsr_transpose(bits, 1, z["row_ptr"], prp, z["col_idx"], packed, z["scales"], z["offsets"],
                                    z["g"], cols, half, rows))
    assert np.allclose(part, z["gt"], rtol=1e-12, atol=1e-12)


@pytest.mark.parametrize("name", ["bell8_small", "bell4_small"])
def test_golden_bell_from_reference_sources(oracle, name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    a = (int(z["bits"]), 1, int(z["rows"]), int(z["cols"]), int(z["block_size"]), int(z["ell_cols"]),
         int(z["row_stride_bytes"]), z["block_col_idx"], z["scales"], z["offsets"])
    packed = oracle.bell_pack(*a, z["values_by_slot"])
    assert np.array_equal(packed, z["packed"])
    assert np.array_equal(oracle.bell_unpack(*a, packed), z["decoded"])
    ro, cols, vals = oracle.bell_to_csr(*a, packed)
    y = oracle.spmm_reference(int(z["rows"]), int(z["cols"]), int(z["n"]), ro, cols, vals, z["w"])
    assert np.array_equal(y, z["y"])


def test_golden_config1_full(oracle):
    """Configuration 1 (20,000 x 2,000, N = 32 fp32) end to end on the CPU against the
    reference-built summary: same inputs (hashes), same Y (head rows bit-equal, digest equal)."""
    from cellerator_b200 import synth
    z = np.load(os.path.join(GOLDEN, "c1_summary.npz"))
    cfg = synth.CONFIGS["c1_cpu_ref"]
    h = synth.make_qcsr_host(**cfg, seed=0)
    sha = lambda a: hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()  # noqa: E731
    if sha(h["row_ptr"]) != str(z["sha_row_ptr"]) or sha(h["col_idx"]) != str(z["sha_col_idx"]):
        pytest.skip("numpy on this machine draws a different random stream than the fixture's")
    assert sha(h["packed"]) == str(z["sha_packed"])      # numpy quantiser == reference pack_nnz_values
    w = np.random.default_rng(1000).normal(0.0, 0.02, size=(cfg["cols"], cfg["n"])).astype(np.float32)
    assert sha(w) == str(z["sha_w"])
    y = oracle.qcsr_forward(8, 1, h["row_ptr"], h["packed_row_ptr"], h["col_idx"], h["packed"], h["scales"],
                            h["offsets"], w, cfg["cols"])
    assert np.array_equal(y[:64], z["y_head"])
    assert np.array_equal(y.sum(axis=1), z["y_rowsum"])
    assert list(oracle.digest_f32(y.astype(np.float32))) == z["y_digest"].tolist()


# ---- against the compiled reference itself (only where the reference tree is present) ---------------

@pytest.mark.parametrize("bits", [1, 2, 4, 8])
@pytest.mark.parametrize("policy", [1, 2])
def test_oracle_equals_reference_codec_random(oracle, reference, bits, policy):
    rng = np.random.default_rng(100 * bits + policy)
    for trial in range(6):
        c = random_csr(rng, rows=int(rng.integers(1, 40)), cols=int(rng.integers(4, 90)), max_nnz=70, bits=bits,
                       policy=policy)
        prp_o, tot_o = oracle.build_packed_row_ptr(bits, c["row_ptr"])
        prp_r, tot_r = reference.build_packed_row_ptr(bits, c["row_ptr"])
        assert np.array_equal(prp_o, prp_r) and tot_o == tot_r
        if len(c["col_idx"]) == 0:
            continue
        po = oracle.pack_csr(bits, policy, c["row_ptr"], prp_o, c["col_idx"], c["scales"], c["offsets"], c["values"])
        pr = reference.pack_csr(bits, policy, c["row_ptr"], prp_o, c["col_idx"], c["scales"], c["offsets"],
                                c["values"], cols=c["cols"])
        assert np.array_equal(po, pr)
        uo = oracle.unpack_csr(bits, policy, c["row_ptr"], prp_o, c["col_idx"], c["scales"], c["offsets"], po)
        ur = reference.unpack_csr(bits, policy, c["row_ptr"], prp_o, c["col_idx"], c["scales"], c["offsets"], po,
                                  cols=c["cols"])
        assert np.array_equal(uo, ur)
        for rpb in (1, 3, 7, 64):
            bo, co = oracle.build_uniform_block_row_ptr(c["rows"], rpb)
            br, cr = reference.build_uniform_block_row_ptr(c["rows"], rpb)
            assert co == cr and np.array_equal(bo, br)
            for b in (-1, 0, co - 1, co):
                assert oracle.get_block(c["row_ptr"], prp_o, bo, b) == reference.get_block(c["row_ptr"], prp_o, bo, b)
        assert oracle.get_block(c["row_ptr"], prp_o, None, 5) == reference.get_block(c["row_ptr"], prp_o, None, 5)


def test_oracle_equals_reference_scalar_rules(oracle, reference):
    rng = np.random.default_rng(7)
    for bits in (1, 2, 4, 8):
        for _ in range(400):
            v, s, o = (float(np.float32(x)) for x in (rng.uniform(-5, 60), rng.choice([0.0, 0.1, 0.25, 1e-6, 3.0]),
                                                      rng.uniform(-2, 2)))
            assert oracle.quantize_code(bits, v, s, o) == reference.quantize_code(bits, v, s, o)
        # exact .5 ties round away from zero
        assert oracle.quantize_code(bits, 0.5, 1.0, 0.0) == reference.quantize_code(bits, 0.5, 1.0, 0.0) == 1
        # magnitudes that overflow the int conversion, and NaN: the host result is code 0
        # (the reference's scalar helper may return INT_MIN as unsigned there; what its pack stores
        # is that value masked to the code width, i.e. 0)
        for v in (1e12, -1e12, 3e9, float("nan"), float("inf")):
            assert oracle.quantize_code(bits, v, 0.5, 0.0) == 0
            assert reference.quantize_code(bits, v, 0.5, 0.0) & ((1 << bits) - 1) == 0
    rng2 = np.random.default_rng(8)
    c = dict(row_ptr=np.array([0, 6], dtype=np.int64), col_idx=np.arange(6, dtype=np.int32),
             scales=np.full(6, 0.5, dtype=np.float32), offsets=np.zeros(6, dtype=np.float32),
             values=np.array([1e12, -1e12, 3e9, np.nan, np.inf, 3.0], dtype=np.float32))
    for bits in (1, 2, 4, 8):
        prp, _ = oracle.build_packed_row_ptr(bits, c["row_ptr"])
        a = oracle.pack_csr(bits, 1, c["row_ptr"], prp, c["col_idx"], c["scales"], c["offsets"], c["values"])
        b = reference.pack_csr(bits, 1, c["row_ptr"], prp, c["col_idx"], c["scales"], c["offsets"], c["values"], cols=6)
        assert np.array_equal(a, b)
    del rng2
    for _ in range(400):
        code, s, o = int(rng.integers(0, 256)), float(np.float32(rng.uniform(0, 1))), float(np.float32(rng.uniform(-1, 1)))
        assert oracle.dequantize_code(code, s, o) == reference.dequantize_code(code, s, o)


def test_oracle_equals_reference_referee_random(oracle, reference):
    rng = np.random.default_rng(21)
    for trial in range(8):
        m, k, n = (int(x) for x in rng.integers(1, 24, size=3))
        ts, td = bool(trial & 1), bool(trial & 2)
        srows, scols = (k, m) if ts else (m, k)
        c = random_csr(rng, srows, scols, max_nnz=min(scols, 12), bits=8)
        vals = rng.normal(size=len(c["col_idx"])).astype(np.float32)
        rr, rc = (n, k) if td else (k, n)
        col_major = bool(trial & 4)
        ld = (rr if col_major else rc) + 2
        rhs = rng.normal(size=((rc if col_major else rr), ld)).astype(np.float32)
        init = rng.normal(size=(m, n)).astype(np.float32)
        bias = rng.normal(size=n).astype(np.float32)
        for epi in ("none", "bias", "relu", "gelu_erf", "gelu_tanh", "bias_relu", "bias_gelu_erf", "bias_gelu_tanh"):
            kw = dict(transpose_sparse=ts, transpose_dense=td, rhs_col_major=col_major, rhs_ld=ld, alpha=1.5,
                      beta=-0.25, initial=init, initial_ld=n, epilogue=epi, bias=bias if "bias" in epi else None)
            a = oracle.spmm_reference(m, k, n, c["row_ptr"], c["col_idx"], vals, rhs, **kw)
            b = reference.spmm_reference(m, k, n, c["row_ptr"], c["col_idx"], vals, rhs, **kw)
            assert np.array_equal(a, b), (trial, epi)
        y32 = a.astype(np.float32)
        assert oracle.digest_f32(y32) == reference.digest_f32(y32)


@pytest.mark.parametrize("bits,policy,bs", [(8, 1, 32), (4, 2, 8), (2, 1, 4), (1, 2, 16)])
def test_oracle_equals_reference_bell_random(oracle, reference, bits, policy, bs):
    rng = np.random.default_rng(bits * 10 + policy)
    rows, width = 3 * bs - 5, 3
    cols = 5 * bs - 3                       # last block column is ragged: genes >= cols are skipped
    block_rows = -(-rows // bs)
    bci = np.stack([np.sort(rng.choice(5, size=width, replace=False)) for _ in range(block_rows)]).astype(np.uint32)
    bci[1, 1] = 0xFFFFFFFF                  # an empty block
    ell = width * bs
    stride = -(-(-(-ell * bits // 8)) // 16) * 16
    scales = rng.uniform(0.05, 0.4, size=5 * bs).astype(np.float32)
    scales[cols:] = scales[0]               # metadata padding repeats gene 0 (see oracle.c)
    offsets = rng.uniform(-1, 1, size=5 * bs if policy == 1 else rows).astype(np.float32)
    if policy == 1:
        offsets[cols:] = offsets[0]
    vals = rng.uniform(-1, 20, size=(rows, ell)).astype(np.float32)
    a = (bits, policy, rows, cols, bs, ell, stride, bci.ravel(), scales, offsets)
    po, pr = oracle.bell_pack(*a, vals), reference.bell_pack(*a, vals)
    assert np.array_equal(po, pr)
    assert np.array_equal(oracle.bell_unpack(*a, po), reference.bell_unpack(*a, po))


def test_compare_reports_mismatches(oracle):
    ref = np.array([0.0, 30.0, 29.0, 74.0])
    cand = np.array([0.0, 30.0, 29.25, 74.0], dtype=np.float32)
    out = oracle.compare(ref, cand, tol_abs=1e-6, tol_rel=1e-6, rel_floor=1e-12)
    assert out["mismatch_count"] == 1 and out["worst_index"] == 2 and abs(out["max_abs"] - 0.25) < 1e-12
    cand[1] = np.inf
    assert oracle.compare(ref, cand)["status"] == 6
