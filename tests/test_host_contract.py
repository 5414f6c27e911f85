"""CPU checks of the host-side pieces of the C ABI that need no device: element look-up against the
reference's 4x8 known-answer matrix, the SpMM request contract (validation, trivial cases, 128-bit
signature) against the reference's golden value and, where the compiled reference is at hand, against
the reference itself on random requests; the host container of a quantized Blocked-ELL matrix; the
fleet's row partition; and the fleet's behaviour without a usable NCCL or device."""
import ctypes as C
import json
import os
import struct

import numpy as np
import pytest

import oracle as orc
from cellerator_b200 import capi, ops, synth
from conftest import ROOT, random_csr

KATS = json.load(open(os.path.join(ROOT, "tests", "golden", "kats.json")))


def _host_qcsr(c, keep):
    """cb200_qcsr over HOST numpy arrays (kept alive in `keep`)."""
    d = capi.header(capi.QCsr())
    arrays = {"row_ptr": np.ascontiguousarray(c["row_ptr"], dtype=np.int64),
              "col_idx": np.ascontiguousarray(c["col_idx"], dtype=np.int32),
              "packed": np.ascontiguousarray(c["packed"], dtype=np.uint8),
              "scales": None if c.get("scales") is None else np.ascontiguousarray(c["scales"], dtype=np.float32),
              "offsets": None if c.get("offsets") is None else np.ascontiguousarray(c["offsets"], dtype=np.float32),
              "prp": None if c.get("packed_row_ptr") is None else np.ascontiguousarray(c["packed_row_ptr"], dtype=np.int64)}
    keep.append(arrays)
    d.rows, d.cols, d.nnz, d.bits, d.policy = c["rows"], c["cols"], len(arrays["col_idx"]), c["bits"], c["policy"]
    d.row_ptr, d.col_idx, d.packed_values = arrays["row_ptr"].ctypes.data, arrays["col_idx"].ctypes.data, arrays["packed"].ctypes.data
    d.scales = None if arrays["scales"] is None else arrays["scales"].ctypes.data
    d.offsets = None if arrays["offsets"] is None else arrays["offsets"].ctypes.data
    d.packed_row_ptr = None if arrays["prp"] is None else arrays["prp"].ctypes.data
    return d


# ---- element look-up (access.cuh:47-79,133-153) on the reference's 4x8 fixture ---------------------

@pytest.mark.parametrize("bits", [1, 2, 4, 8])
@pytest.mark.parametrize("policy", [1, 2])
def test_element_lookup_on_the_4x8_fixture(oracle, bits, policy):
    k = KATS["quantized_csr_4x8"]
    row_ptr, col = np.array(k["row_ptr"], dtype=np.int64), np.array(k["col_idx"], dtype=np.int32)
    max_code = (1 << bits) - 1
    codes = np.array([(i + r + col[i]) % (max_code + 1) for r in range(4) for i in range(row_ptr[r], row_ptr[r + 1])])
    scales = np.array(k["gene_scales"], dtype=np.float32)
    offsets = np.array(k["gene_offsets"] if policy == 1 else k["row_offsets"], dtype=np.float32)
    prp, _ = oracle.build_packed_row_ptr(bits, row_ptr)
    # values whose codes are exactly the rule's, packed by the host codec
    off_of = lambda r, g: offsets[g] if policy == 1 else offsets[r]
    values = np.array([codes[i] * scales[col[i]] + off_of(r, col[i]) for r in range(4) for i in range(row_ptr[r], row_ptr[r + 1])],
                      dtype=np.float32)
    packed = oracle.pack_csr(bits, policy, row_ptr, prp, col, scales, offsets, values)
    keep = []
    m = _host_qcsr(dict(rows=4, cols=8, bits=bits, policy=policy, row_ptr=row_ptr, col_idx=col, packed=packed, scales=scales,
                        offsets=offsets, packed_row_ptr=prp), keep)
    L = capi.lib()
    dec = oracle.unpack_csr(bits, policy, row_ptr, prp, col, scales, offsets, packed)
    for r in range(4):
        for g in range(8):
            hit = [i for i in range(row_ptr[r], row_ptr[r + 1]) if col[i] == g]
            assert L.cb200_find_in_row(C.byref(m), r, g) == (hit[0] if hit else -1)
            got = L.cb200_get_value(C.byref(m), r, g)
            if hit:
                local = hit[0] - row_ptr[r]
                assert L.cb200_get_code(C.byref(m), r, local) == codes[hit[0]]
                assert np.float32(got) == dec[hit[0]], (r, g)          # the bits of the host decode
            else:
                assert got == 0.0
    # out of range: the reference's answers
    assert L.cb200_find_in_row(C.byref(m), -1, 0) == -1 and L.cb200_find_in_row(C.byref(m), 4, 0) == -1
    assert L.cb200_get_value(C.byref(m), 0, 8) == 0.0 and L.cb200_get_value(C.byref(m), 9, 1) == 0.0
    assert L.cb200_get_code(C.byref(m), 0, 99) == 0


def test_element_lookup_on_random_matrices(oracle):
    rng = np.random.default_rng(5)
    L = capi.lib()
    for bits in (4, 8):
        c = random_csr(rng, rows=30, cols=50, max_nnz=25, bits=bits, policy=1)
        prp, _ = oracle.build_packed_row_ptr(bits, c["row_ptr"])
        packed = oracle.pack_csr(bits, 1, c["row_ptr"], prp, c["col_idx"], c["scales"], c["offsets"], c["values"])
        dec = oracle.unpack_csr(bits, 1, c["row_ptr"], prp, c["col_idx"], c["scales"], c["offsets"], packed)
        keep = []
        m = _host_qcsr(dict(c, packed=packed, packed_row_ptr=prp), keep)
        dense = np.zeros((30, 50), dtype=np.float32)
        for r in range(30):
            lo, hi = c["row_ptr"][r], c["row_ptr"][r + 1]
            dense[r, c["col_idx"][lo:hi]] = dec[lo:hi]
        got = np.array([[L.cb200_get_value(C.byref(m), r, g) for g in range(50)] for r in range(30)], dtype=np.float32)
        assert np.array_equal(got, dense)


# ---- request contract (operation.hh:136-221, operation.cc:119-292, operation_signature.cc:30-68) -----

def _fixture_request():
    """request_fixture() of tests/math_operation_contract_test.cc:28-50."""
    r = capi.SpmmRequest()
    r.schema_version, r.operation = 1, 1
    r.m, r.k, r.n, r.sparse_nnz = 8, 16, 32, 24
    r.structure_schema_version, r.structure_identity_version, r.structure_value = 1, 1, 0xc511e7a70
    r.dense_rhs_layout = r.output_layout = 1
    r.dense_rhs_leading_dimension = r.output_leading_dimension = 32
    r.sparse_storage_type_code = r.dense_storage_type_code = capi.TYPE_F16
    r.output_storage_type_code = r.compute_type_code = r.accumulation_type_code = capi.TYPE_F32
    r.alpha.type_code = r.beta.type_code = capi.TYPE_F32
    r.alpha.bits = struct.unpack("<I", struct.pack("<f", 1.0))[0]
    r.beta.bits = 0
    r.workspace_kind, r.reuse_kind, r.reuse_expected_run_count = 1, 1, 1
    for o in (r.sparse_feature_order, r.dense_feature_order):
        o.schema_version, o.kind, o.feature_count, o.feature_axis_identity_version, o.feature_axis_identity = 1, 1, 16, 1, 0x12345678
    return r


def _signature(r):
    sig = (C.c_uint64 * 2)()
    capi.check(capi.lib().cb200_spmm_request_signature(C.byref(r), C.byref(sig)))
    return int(sig[0]), int(sig[1])


def _fields(r):
    """The 48 values of the request in declaration order (what oracle.Reference.request_contract takes)."""
    o = lambda x: [x.schema_version, x.kind, x.feature_count, x.feature_axis_identity_version, x.feature_axis_identity,
                   x.packing_geometry_identity]
    return [r.schema_version, r.operation, r.m, r.k, r.n, r.sparse_nnz, r.structure_schema_version, r.structure_identity_version,
            r.structure_value, r.transpose_sparse, r.transpose_dense, r.dense_rhs_layout, r.output_layout,
            r.dense_rhs_leading_dimension, r.output_leading_dimension, r.sparse_storage_type_code, r.dense_storage_type_code,
            r.output_storage_type_code, r.compute_type_code, r.accumulation_type_code, r.alpha.type_code, r.alpha.reserved,
            r.alpha.bits, r.beta.type_code, r.beta.reserved, r.beta.bits, r.determinism, r.workspace_kind, r.workspace_reserved,
            r.workspace_byte_limit, r.reuse_kind, r.reuse_reserved, r.reuse_expected_run_count, r.epilogue_kind,
            r.epilogue_bias_type_code, r.epilogue_bias_element_count] + o(r.sparse_feature_order) + o(r.dense_feature_order)


def test_operation_signature_golden_value():
    """The golden of tests/math_operation_contract_test.cc:62-72."""
    r = _fixture_request()
    L = capi.lib()
    assert L.cb200_spmm_request_validate(C.byref(r)) == 0
    assert L.cb200_spmm_request_classify(C.byref(r)) == 0
    assert _signature(r) == (0xa7e9d18214be8880, 0xc02e69bb5dae6efb)
    assert _signature(r) == _signature(r)
    base = _signature(r)
    r.dense_rhs_layout = 2
    assert _signature(r) != base                     # the dense layout is part of the identity
    r = _fixture_request()
    r.structure_value += 1
    assert _signature(r) != base                     # so is the sparse structure
    r = _fixture_request()
    r.sparse_feature_order.feature_axis_identity += 1
    assert _signature(r) != base


def test_request_validation_codes():
    """One violation per rule of validate_spmm_request, with the reference's codes (operation.hh:63-80)."""
    L = capi.lib()

    def code(mutate):
        r = _fixture_request()
        mutate(r)
        return L.cb200_spmm_request_validate(C.byref(r))

    def set_(**kw):
        def go(r):
            for k, v in kw.items():
                obj, name = r, k
                while "__" in name:
                    head, name = name.split("__", 1)
                    obj = getattr(obj, head)
                setattr(obj, name, v)
        return go

    assert code(set_(schema_version=2)) == 1
    assert code(set_(m=0)) == 2                                   # nnz without rows
    assert code(set_(sparse_nnz=8 * 16 + 1)) == 2
    assert code(set_(transpose_sparse=2)) == 11
    assert code(set_(dense_rhs_layout=3)) == 11
    assert code(set_(dense_rhs_leading_dimension=31)) == 11
    assert code(set_(output_leading_dimension=31)) == 11
    assert code(set_(dense_storage_type_code=99)) == 3
    assert code(set_(alpha__type_code=capi.TYPE_F64)) == 4         # scalars use the compute type
    assert code(set_(alpha__bits=1 << 40)) == 4                    # an f32 scalar has no high word
    assert code(set_(determinism=2)) == 14
    assert code(set_(workspace_kind=2)) == 5                       # a caller limit needs a byte limit
    assert code(set_(workspace_byte_limit=64)) == 5
    assert code(set_(reuse_expected_run_count=2)) == 6
    assert code(set_(reuse_kind=3)) == 6                           # persistent reuse has run count 0
    assert code(set_(structure_value=0)) == 12
    assert code(set_(sparse_feature_order__feature_count=15)) == 7
    assert code(set_(dense_feature_order__feature_axis_identity=0x99)) == 8
    assert code(set_(epilogue_kind=8)) == 15
    assert code(set_(epilogue_kind=1)) == 9                        # bias epilogue without bias storage
    assert code(set_(epilogue_bias_element_count=32)) == 10
    assert code(set_(epilogue_kind=5, epilogue_bias_element_count=32, epilogue_bias_type_code=capi.TYPE_F32)) == 0
    # trivial cases (operation.cc:283-292)
    for mutate, kind in ((set_(n=0, dense_rhs_leading_dimension=0, output_leading_dimension=0), 1),
                         (set_(sparse_nnz=0), 2), (set_(alpha__bits=0), 2)):
        r = _fixture_request()
        mutate(r)
        assert L.cb200_spmm_request_classify(C.byref(r)) == kind


@pytest.mark.skipif(not orc.Reference.available(), reason="needs the compiled reference sources (oracle/_ref)")
def test_request_contract_equals_the_compiled_reference():
    ref = orc.Reference()
    L = capi.lib()
    rng = np.random.default_rng(11)
    assert ref.request_contract(_fields(_fixture_request()))[2:] == (0xa7e9d18214be8880, 0xc02e69bb5dae6efb)
    names = [n for n, t in capi.SpmmRequest._fields_ if t in (C.c_uint32, C.c_uint64)]
    for trial in range(400):
        r = _fixture_request()
        for _ in range(int(rng.integers(0, 4))):   # a few random field edits: most leave the request invalid in one way
            name = names[int(rng.integers(0, len(names)))]
            setattr(r, name, int(rng.choice([0, 1, 2, 3, 4, 7, 9, 16, 31, 32, 33, 128, 1 << 33, (1 << 64) - 1])))
        if trial % 3 == 0:
            r.alpha.bits = int(rng.integers(0, 1 << 32))
            r.epilogue_kind = int(rng.integers(0, 9))
        want = ref.request_contract(_fields(r))
        got = (L.cb200_spmm_request_validate(C.byref(r)), L.cb200_spmm_request_classify(C.byref(r)), *_signature(r))
        assert got == want, (trial, _fields(r))


def test_request_from_problem_validates_and_signs():
    pr = capi.header(capi.SpmmProblem())
    pr.projection, pr.m, pr.k, pr.n, pr.nnz, pr.bits, pr.policy = capi.PROJECTION_CSR, 1000, 2000, 64, 30000, 8, 1
    pr.dense_dtype, pr.structure_epoch = capi.DTYPE_BF16, 1
    ln = capi.header(capi.Launch())
    ln.dense_ld = ln.out_ld = 64
    ln.alpha, ln.beta, ln.epilogue = 1.0, 0.0, capi.EPILOGUE["bias_relu"]
    r = capi.SpmmRequest()
    L = capi.lib()
    capi.check(L.cb200_spmm_request_from_problem(C.byref(pr), C.byref(ln), 0xabc, 0xdef, C.byref(r)))
    assert L.cb200_spmm_request_validate(C.byref(r)) == 0
    assert (r.m, r.k, r.n, r.transpose_sparse, r.dense_storage_type_code, r.epilogue_bias_element_count) == (1000, 2000, 64, 0, capi.TYPE_BF16, 64)
    fwd = _signature(r)
    pr.projection = capi.PROJECTION_TRANSPOSE
    pr.dense_dtype = capi.DTYPE_F32
    ln.epilogue = 0
    capi.check(L.cb200_spmm_request_from_problem(C.byref(pr), C.byref(ln), 0xabc, 0xdef, C.byref(r)))
    assert L.cb200_spmm_request_validate(C.byref(r)) == 0
    assert (r.m, r.k, r.transpose_sparse) == (2000, 1000, 1)       # logical shape after the declared transpose
    assert _signature(r) != fwd


# ---- host container of a quantized Blocked-ELL matrix (matrix/quantized_blocked_ell.cuh:27-220) --------

def test_qbell_aux_word_and_row_bytes():
    L = capi.lib()
    aux = L.cb200_qbell_pack_aux(4, 32, 16)
    assert aux == (16 << 24) | (4 << 16) | 32
    bits, bs, cols = C.c_uint32(), C.c_uint32(), C.c_uint32()
    width = C.c_uint64()
    L.cb200_qbell_unpack_aux(aux, C.byref(bits), C.byref(bs), C.byref(width), C.byref(cols))
    assert (bits.value, bs.value, width.value, cols.value) == (4, 32, 16, 512)
    assert L.cb200_qbell_row_bytes(8, 512) == 512 and L.cb200_qbell_row_bytes(4, 513) == 257 and L.cb200_qbell_row_bytes(0, 9) == 0
    assert L.cb200_qbell_aligned_row_bytes(4, 513, 16) == 272 and L.cb200_qbell_aligned_row_bytes(4, 513, 1) == 257


@pytest.mark.parametrize("policy", [1, 2])
def test_qbell_host_container_is_one_slab(policy):
    L = capi.lib()
    b = synth.make_qbell_host(rows=70, cols=256, block_size=32, ell_blocks=3, fill=0.6, bits=8, seed=2)
    offsets = b["offsets"] if policy == 1 else np.linspace(-1.0, 1.0, 70, dtype=np.float32)    # per gene / per row
    m = capi.QBellHost()
    L.cb200_qbell_host_init(C.byref(m), 70, 256, 0, 32, b["ell_cols"], 8, policy, 0)
    assert m.row_stride_bytes == b["row_stride_bytes"] == 96
    assert L.cb200_qbell_host_allocate(C.byref(m)) == 1
    idx_bytes = 3 * 3 * 4
    packed_bytes = 70 * 96
    scales_at = (idx_bytes + packed_bytes + 3) // 4 * 4
    assert m.block_col_idx == m.storage and m.packed_values == m.storage + idx_bytes
    assert m.column_scales == m.storage + scales_at and m.column_offsets == m.column_scales + 256 * 4
    assert m.row_offsets == m.column_offsets + 256 * 4
    assert L.cb200_qbell_host_bytes(C.byref(m)) == C.sizeof(capi.QBellHost) + scales_at + 2 * 256 * 4 + 70 * 4
    # fill the slab and read it back through the view
    C.memmove(m.block_col_idx, b["block_col_idx"].ctypes.data, idx_bytes)
    C.memmove(m.packed_values, b["packed"].ctypes.data, packed_bytes)
    C.memmove(m.column_scales, b["scales"].ctypes.data, 256 * 4)
    C.memmove(m.row_offsets if policy == 2 else m.column_offsets, offsets.ctypes.data, offsets.nbytes)
    view = capi.QBell()
    capi.check(L.cb200_qbell_host_view(C.byref(m), C.byref(view)))
    assert (view.rows, view.cols, view.block_size, view.ell_cols, view.row_stride_bytes, view.bits, view.policy) == (70, 256, 32, 96, 96, 8, policy)
    assert view.offsets == (m.row_offsets if policy == 2 else m.column_offsets) and view.scales == m.column_scales
    got = np.ctypeslib.as_array(C.cast(view.packed_values, C.POINTER(C.c_uint8)), shape=(packed_bytes,))
    assert np.array_equal(got, b["packed"])
    got_off = np.ctypeslib.as_array(C.cast(view.offsets, C.POINTER(C.c_float)), shape=(offsets.size,))
    assert np.array_equal(got_off, offsets)
    L.cb200_qbell_host_clear(C.byref(m))
    assert not m.storage and m.rows == 0 and m.flags == 0


# ---- fleet: row partition and failure without a communicator ----------------------------------------

@pytest.mark.parametrize("bits", [4, 8])
def test_fleet_partition_equals_the_reference_rule(oracle, bits):
    rng = np.random.default_rng(3)
    L = capi.lib()
    for rows, parts in ((1000, 8), (1003, 8), (5, 8), (16, 2), (7, 1), (0, 4)):
        c = random_csr(rng, rows=rows, cols=64, max_nnz=30, bits=bits)
        prp, _ = oracle.build_packed_row_ptr(bits, c["row_ptr"])
        blocks = (capi.CsrBlock * parts)()
        rp = np.ascontiguousarray(c["row_ptr"], dtype=np.int64)
        capi.check(L.cb200_fleet_partition(rows, parts, rp.ctypes.data, prp.ctypes.data if bits != 8 else None, blocks))
        per = max(1, -(-rows // parts))
        brp, count = oracle.build_uniform_block_row_ptr(rows, per)
        covered = 0
        for b in range(parts):
            got = {n: getattr(blocks[b], n) for n, _ in capi.CsrBlock._fields_}
            if b < count:
                assert got == oracle.get_block(c["row_ptr"], prp, brp, b)
            else:                                     # empty trailing shard at the end of the matrix
                assert got["row_begin"] == got["row_end"] == rows and got["nnz_begin"] == got["nnz_end"] == int(rp[-1])
            assert got["row_begin"] == covered
            covered = got["row_end"]
        assert covered == rows
    assert L.cb200_fleet_partition(10, 0, rp.ctypes.data, None, blocks) == capi.INVALID_ARGUMENT


def test_fleet_without_nccl_or_device_fails_with_a_status(tmp_path):
    L = capi.lib()
    uid = (C.c_uint8 * 128)()
    # a library that is not NCCL: the unique id cannot be made, and says so
    assert L.cb200_fleet_unique_id(str(tmp_path / "libnot_there.so").encode(), uid) == capi.COMM_NOT_READY
    assert b"dlopen" in L.cb200_last_error()
    assert L.cb200_fleet_unique_id(capi.LIB_PATH.encode(), uid) == capi.COMM_NOT_READY     # loads, but has no NCCL entry point
    assert b"NCCL entry point" in L.cb200_last_error()
    o = capi.header(capi.FleetOptions())
    handle = C.c_void_p()
    o.device_count = 0
    assert L.cb200_fleet_create(C.byref(o), C.byref(handle)) == capi.INVALID_ARGUMENT
    o.device_count, o.world_size, o.world_rank = 1, 2, 1
    assert L.cb200_fleet_create(C.byref(o), C.byref(handle)) == capi.INVALID_ARGUMENT      # a job across processes needs the id
    import torch
    if not torch.cuda.is_available():
        o.world_size, o.world_rank = 1, 0
        assert L.cb200_fleet_create(C.byref(o), C.byref(handle)) == capi.CUDA_ERROR       # no device: no fallback
        assert not handle.value
    assert L.cb200_fleet_slot_count(None) == 0 and L.cb200_fleet_communicator_ready(None) == 0
