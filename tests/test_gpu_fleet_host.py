"""GPU checks of the multi-GPU layer on one device, the host-buffer forward entry, the device element
look-up, session-borrowed persistent memory, the status readers and the bounded-wait path, all through
the C ABI."""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest
import torch

from cellerator_b200 import capi, ops, synth
from conftest import ROOT, random_csr
from gpu_util import assert_forward_close, dense, host_pack, row_l1, to_dev

pytestmark = pytest.mark.gpu


def _fleet(device, **kw):
    o = capi.header(capi.FleetOptions())
    o.device_count = 1
    devs = (C.c_int32 * 1)(device.index)
    o.devices = devs
    for k, v in kw.items():
        setattr(o, k, v)
    handle = C.c_void_p()
    st = capi.lib().cb200_fleet_create(C.byref(o), C.byref(handle))
    return st, handle, (o, devs)


def _run_fleet(fn, fleet, op, launch):
    slots = (C.c_uint32 * 1)(0)
    prepared = (C.c_void_p * 1)(op.handle.value)
    launches = (capi.Launch * 1)(launch)
    return fn(fleet, slots, 1, prepared, launches)


def test_one_gpu_fleet_equals_the_single_device_calls(cuda_device, oracle):
    """A fleet of one slot in a job of one rank: forward and transpose are bit-equal to cb200_spmm_run, the
    transpose needs no communicator, and the launches run on the fleet's own stream."""
    L = capi.lib()
    rng = np.random.default_rng(3)
    c = host_pack(oracle, random_csr(rng, rows=700, cols=900, max_nnz=120, bits=8, policy=1))
    x = to_dev(c, cuda_device)
    w, _ = dense(rng, 900, 64, torch.bfloat16, cuda_device)
    g, _ = dense(rng, 700, 64, torch.float32, cuda_device, std=1.0)
    st, fleet, keep = _fleet(cuda_device, enable_peer_access=1)
    assert st == capi.SUCCESS, L.cb200_last_error()
    try:
        assert L.cb200_fleet_slot_count(fleet) == 1 and L.cb200_fleet_world_size(fleet) == 1
        assert L.cb200_fleet_device(fleet, 0) == cuda_device.index and L.cb200_fleet_device(fleet, 1) == -1
        assert L.cb200_fleet_communicator_ready(fleet) == 1       # nothing to communicate with
        assert L.cb200_fleet_stream(fleet, 0) and not L.cb200_fleet_stream(fleet, 3)
        fwd = ops.PreparedSpmm(capi.PROJECTION_CSR, 700, 900, 64, x.nnz, 8, 1, w.dtype, cuda_device, host_row_ptr=c["row_ptr"])
        want = fwd.run(x, w, torch.empty(700, 64, device=cuda_device))
        torch.cuda.synchronize()
        got = torch.full((700, 64), float("nan"), device=cuda_device)
        capi.check(_run_fleet(L.cb200_fleet_run_forward, fleet, fwd, fwd.make_launch(x, w, got)))
        slots = (C.c_uint32 * 1)(0)
        capi.check(L.cb200_fleet_synchronize(fleet, slots, 1))
        assert torch.equal(got, want)
        tr = ops.PreparedSpmm(capi.PROJECTION_TRANSPOSE, 700, 900, 64, x.nnz, 8, 1, g.dtype, cuda_device, deterministic=True,
                              device_matrix=x)
        want_t = tr.run(x, g, torch.empty(900, 64, device=cuda_device))
        torch.cuda.synchronize()
        got_t = torch.full((900, 64), float("nan"), device=cuda_device)
        capi.check(_run_fleet(L.cb200_fleet_run_transpose, fleet, tr, tr.make_launch(x, g, got_t)))
        capi.check(L.cb200_fleet_synchronize(fleet, slots, 1))
        assert torch.equal(got_t, want_t)
        # a partial with a leading dimension cannot be all-reduced in place
        wide = torch.empty(900, 80, device=cuda_device)
        assert _run_fleet(L.cb200_fleet_run_transpose, fleet, tr, tr.make_launch(x, g, wide[:, :64])) == capi.INVALID_SHAPE
        # grow-only scratch
        p1, p2 = C.c_void_p(), C.c_void_p()
        capi.check(L.cb200_fleet_request_scratch(fleet, 0, 1 << 20, C.byref(p1)))
        capi.check(L.cb200_fleet_request_scratch(fleet, 0, 1 << 10, C.byref(p2)))
        assert p1.value == p2.value and p1.value
        bad = (C.c_uint32 * 1)(5)
        assert L.cb200_fleet_synchronize(fleet, bad, 1) == capi.INVALID_ARGUMENT
    finally:
        L.cb200_fleet_destroy(fleet)


def test_a_communicator_that_is_not_ready_is_a_status_not_a_fallback(cuda_device, oracle, tmp_path):
    """Rank 0 of a two-rank job whose NCCL cannot initialise (a stand-in library that refuses): the fleet is
    created, reports the communicator as not ready, the transpose returns CB200_STATUS_COMM_NOT_READY before
    anything is enqueued (the output keeps its canary), and the forward path, which needs no collective, runs."""
    L = capi.lib()
    fake = str(tmp_path / "libfake_nccl.so")
    subprocess.run(["gcc", "-shared", "-fPIC", "-O1", "-o", fake, os.path.join(ROOT, "tests", "fake_nccl.c")], check=True)
    uid = (C.c_uint8 * 128)()
    capi.check(L.cb200_fleet_unique_id(fake.encode(), uid))
    assert bytes(uid) == b"\x07" * 128
    st, fleet, keep = _fleet(cuda_device, world_size=2, world_rank=0, nccl_unique_id=C.cast(uid, C.c_void_p), nccl_library=fake.encode())
    assert st == capi.SUCCESS, L.cb200_last_error()
    try:
        assert L.cb200_fleet_world_size(fleet) == 2 and L.cb200_fleet_communicator_ready(fleet) == 0
        rng = np.random.default_rng(4)
        c = host_pack(oracle, random_csr(rng, rows=300, cols=400, max_nnz=60, bits=8, policy=1))
        x = to_dev(c, cuda_device)
        g, _ = dense(rng, 300, 32, torch.float32, cuda_device, std=1.0)
        tr = ops.PreparedSpmm(capi.PROJECTION_TRANSPOSE, 300, 400, 32, x.nnz, 8, 1, g.dtype, cuda_device)
        out = torch.full((400, 32), 123.0, device=cuda_device)
        assert _run_fleet(L.cb200_fleet_run_transpose, fleet, tr, tr.make_launch(x, g, out)) == capi.COMM_NOT_READY
        assert b"not ready" in L.cb200_last_error()
        torch.cuda.synchronize()
        assert torch.all(out == 123.0)                            # nothing ran
        sends = (C.c_void_p * 1)(out.data_ptr())
        slots = (C.c_uint32 * 1)(0)
        assert L.cb200_fleet_allreduce_sum_f32(fleet, slots, 1, sends, sends, out.numel()) == capi.COMM_NOT_READY
        w, _ = dense(rng, 400, 32, torch.bfloat16, cuda_device)
        fwd = ops.PreparedSpmm(capi.PROJECTION_CSR, 300, 400, 32, x.nnz, 8, 1, w.dtype, cuda_device)
        y = torch.empty(300, 32, device=cuda_device)
        capi.check(_run_fleet(L.cb200_fleet_run_forward, fleet, fwd, fwd.make_launch(x, w, y)))
        capi.check(L.cb200_fleet_synchronize(fleet, slots, 1))
        assert torch.equal(y, fwd.run(x, w, torch.empty_like(y)))
    finally:
        L.cb200_fleet_destroy(fleet)


def _host_desc(c, keep):
    t = {k: torch.from_numpy(np.ascontiguousarray(c[k], dtype=dt)).pin_memory()
         for k, dt in (("row_ptr", np.int64), ("col_idx", np.int32), ("packed", np.uint8), ("scales", np.float32), ("offsets", np.float32))}
    if c["bits"] != 8:
        t["prp"] = torch.from_numpy(np.ascontiguousarray(c["packed_row_ptr"], dtype=np.int64)).pin_memory()
    keep.append(t)
    d = capi.header(capi.QCsr())
    d.rows, d.cols, d.nnz, d.bits, d.policy = c["rows"], c["cols"], len(c["col_idx"]), c["bits"], c["policy"]
    d.row_ptr, d.col_idx, d.packed_values = t["row_ptr"].data_ptr(), t["col_idx"].data_ptr(), t["packed"].data_ptr()
    d.scales, d.offsets = t["scales"].data_ptr(), t["offsets"].data_ptr()
    d.packed_row_ptr = t["prp"].data_ptr() if "prp" in t else None
    return d


@pytest.mark.parametrize("bits,policy,dtype,n", [(8, 1, torch.bfloat16, 64), (4, 1, torch.bfloat16, 128), (8, 2, torch.float32, 32),
                                                  (4, 2, torch.float32, 24)])
def test_host_buffer_forward_through_the_chunk_ring(cuda_device, oracle, bits, policy, dtype, n):
    """cb200_host_forward: host arrays in, host Y out, the matrix crossing in ragged chunks through a ring of
    two or three device buffers; equal to the oracle's bound and bit-equal to the device-resident call."""
    L = capi.lib()
    rng = np.random.default_rng(40 + bits + policy)
    rows, cols = 1500, 4100
    c = host_pack(oracle, random_csr(rng, rows=rows, cols=cols, max_nnz=400, bits=bits, policy=policy))
    keep = []
    xd = _host_desc(c, keep)
    w, w_host = dense(rng, cols, n, dtype, cuda_device)
    w_pinned = w.cpu().contiguous().pin_memory()
    y_host = torch.full((rows, n), float("nan")).pin_memory()
    o = capi.header(capi.HostStageOptions())
    o.device, o.k, o.n, o.bits, o.policy = cuda_device.index, cols, n, bits, policy
    o.dense_dtype = capi.DTYPE_BF16 if dtype == torch.bfloat16 else capi.DTYPE_F32
    o.max_chunk_rows, o.max_chunk_nnz, o.chunk_buffers = 211, 50_000, 3
    stage = C.c_void_p()
    capi.check(L.cb200_host_stage_create(C.byref(o), C.byref(stage)))
    try:
        assert 0 < L.cb200_host_stage_device_bytes(stage) < 8 << 20       # three chunk buffers and W, not the matrix
        h2d, d2h = C.c_uint64(), C.c_uint64()
        launches0 = L.cb200_kernel_launch_count()
        for _ in range(2):                                         # the ring's events are reused by a second call
            capi.check(L.cb200_host_forward(stage, C.byref(xd), w_pinned.data_ptr(), n, y_host.data_ptr(), n, 1.0, C.byref(h2d), C.byref(d2h)))
        assert L.cb200_kernel_launch_count() - launches0 >= 2 * 2 * (rows // 211)
        # (gene indices may cross as 16-bit words where the host narrows them fast enough: k = 4,100 allows it)
        assert d2h.value == rows * n * 4 and h2d.value >= len(c["col_idx"]) * 2 + c["packed"].nbytes
        ref = oracle.qcsr_forward(bits, policy, c["row_ptr"], c["packed_row_ptr"], c["col_idx"], c["packed"], c["scales"],
                                  c["offsets"], w_host, cols)
        l1, _ = row_l1(oracle, c)
        assert_forward_close(y_host.numpy(), ref, l1, float(np.abs(w_host).max()), bf16=dtype == torch.bfloat16)
        # a row longer than a chunk buffer is refused with a status, nothing is computed
        o2 = capi.header(capi.HostStageOptions())
        for name, _ in capi.HostStageOptions._fields_[2:]:
            setattr(o2, name, getattr(o, name))
        o2.max_chunk_nnz = 10
        small = C.c_void_p()
        capi.check(L.cb200_host_stage_create(C.byref(o2), C.byref(small)))
        assert L.cb200_host_forward(small, C.byref(xd), w_pinned.data_ptr(), n, y_host.data_ptr(), n, 1.0, None, None) == capi.INSUFFICIENT_WORKSPACE
        L.cb200_host_stage_destroy(small)
    finally:
        L.cb200_host_stage_destroy(stage)
    # the device-resident call on the same matrix (exact schedules): same kernels per row -> same bits where the
    # schedule is the same; the warp-per-row kernel sums a row in one fixed order whatever the chunking
    x = to_dev(c, cuda_device)
    y_dev = ops.spmm_forward(x, w, schedule="warp_per_row")
    if n == 24:                                                    # no tiled shape: both paths run warp per row
        assert np.array_equal(y_dev.cpu().numpy(), y_host.numpy())


def _host_forward_all_forms(cuda_device, c, w_pinned, n, modes, chunk_rows=300, chunk_nnz=120_000):
    """cb200_host_forward over the same host matrix with each form of the gene indices on the link: {mode: (Y, bytes
    moved host -> device)}; every stage is called twice (staging buffers and events are reused)."""
    L = capi.lib()
    keep = []
    xd = _host_desc(c, keep)
    out = {}
    for mode in modes:
        o = capi.header(capi.HostStageOptions())
        o.device, o.k, o.n, o.bits, o.policy = cuda_device.index, c["cols"], n, c["bits"], c["policy"]
        o.dense_dtype = capi.DTYPE_BF16
        o.max_chunk_rows, o.max_chunk_nnz, o.chunk_buffers, o.narrow_indices = chunk_rows, chunk_nnz, 3, mode
        stage = C.c_void_p()
        capi.check(L.cb200_host_stage_create(C.byref(o), C.byref(stage)))
        try:
            y_host = torch.full((c["rows"], n), float("nan")).pin_memory()
            h2d = C.c_uint64()
            for _ in range(2):
                capi.check(L.cb200_host_forward(stage, C.byref(xd), w_pinned.data_ptr(), n, y_host.data_ptr(), n, 1.0, C.byref(h2d), None))
            out[mode] = (y_host.clone(), h2d.value)
        finally:
            L.cb200_host_stage_destroy(stage)
    return out


@pytest.mark.parametrize("bits", [8, 4])
def test_host_buffer_forward_with_shorter_index_forms(cuda_device, oracle, bits):
    """The gene indices cross the link as gap bytes (narrow_indices = 2), 16-bit words (1), 32-bit words (-1), or as
    the stage decides per call (0): the results are bit-identical, and the bytes on the link are what each form needs."""
    rng = np.random.default_rng(70 + bits)
    rows, cols, n = 2100, 4100, 64
    c = host_pack(oracle, random_csr(rng, rows=rows, cols=cols, max_nnz=700, bits=bits, policy=1))
    w, w_host = dense(rng, cols, n, torch.bfloat16, cuda_device)
    w_pinned = w.cpu().contiguous().pin_memory()
    nnz = len(c["col_idx"])
    got = _host_forward_all_forms(cuda_device, c, w_pinned, n, (2, 1, -1, 0))
    for mode in (2, 1, 0):
        assert torch.equal(got[mode][0], got[-1][0])
    slack = 16 * (rows // 300 + 2)                                       # 16-byte padding per chunk
    gaps_over = int(np.sum(np.diff(c["col_idx"].astype(np.int64)) - 1 >= 255))   # an upper bound of the listed entries
    assert got[-1][1] - got[1][1] >= 2 * nnz - slack                      # two bytes per entry saved
    assert got[-1][1] - got[2][1] >= 3 * nnz - slack - 8 * (gaps_over + rows)   # three, less the list of long gaps
    assert got[2][1] <= got[0][1] <= got[-1][1]
    ref = oracle.qcsr_forward(bits, 1, c["row_ptr"], c["packed_row_ptr"], c["col_idx"], c["packed"], c["scales"], c["offsets"],
                              w_host, cols)
    l1, _ = row_l1(oracle, c)
    assert_forward_close(got[2][0].numpy(), ref, l1, float(np.abs(w_host).max()), bf16=True)


@pytest.mark.parametrize("cols,max_nnz,shuffled_rows", [(65536, 700, 0), (20_000, 400, 40), (200_000, 300, 0)])
def test_host_buffer_forward_gap_bytes_with_long_gaps(cuda_device, oracle, cols, max_nnz, shuffled_rows):
    """Gap bytes where gaps do not fit a byte: a few per chunk (listed), rows whose genes do not ascend (every descent is
    listed), and so many that the list overflows and the chunk goes as 32-bit indices.  Always the same bits as the
    32-bit form."""
    rng = np.random.default_rng(cols % 1000 + max_nnz)
    rows, n = 1500, 32
    c = random_csr(rng, rows=rows, cols=cols, max_nnz=max_nnz, bits=8, policy=1)
    c["col_idx"][-1] = cols - 1                                           # the top index, in the last row's last entry
    for r in rng.choice(rows, size=shuffled_rows, replace=False):         # rows in arbitrary gene order
        lo, hi = int(c["row_ptr"][r]), int(c["row_ptr"][r + 1])
        order = rng.permutation(hi - lo)
        c["col_idx"][lo:hi] = c["col_idx"][lo:hi][order]
        c["values"][lo:hi] = c["values"][lo:hi][order]
    c = host_pack(oracle, c)
    w, w_host = dense(rng, cols, n, torch.bfloat16, cuda_device)
    w_pinned = w.cpu().contiguous().pin_memory()
    got = _host_forward_all_forms(cuda_device, c, w_pinned, n, (2, -1, 0), chunk_rows=211, chunk_nnz=60_000)
    assert torch.equal(got[2][0], got[-1][0]) and torch.equal(got[0][0], got[-1][0])
    assert got[2][1] <= got[-1][1] + 16 * (rows // 211 + 2)
    if shuffled_rows == 0:      # (the kernels behind the call take a row's genes in ascending order, like the reference's CSR)
        ref = oracle.qcsr_forward(8, 1, c["row_ptr"], c["packed_row_ptr"], c["col_idx"], c["packed"], c["scales"], c["offsets"], w_host, cols)
        l1, _ = row_l1(oracle, c)
        assert_forward_close(got[2][0].numpy(), ref, l1, float(np.abs(w_host).max()), bf16=True)


def test_host_stage_refuses_unknown_index_forms(cuda_device):
    L = capi.lib()
    o = capi.header(capi.HostStageOptions())
    o.device, o.k, o.n, o.bits, o.policy, o.dense_dtype = cuda_device.index, 70_000, 64, 8, 1, capi.DTYPE_BF16
    o.max_chunk_rows, o.max_chunk_nnz, o.chunk_buffers, o.narrow_indices = 300, 120_000, 3, 1
    stage = C.c_void_p()
    capi.check(L.cb200_host_stage_create(C.byref(o), C.byref(stage)))        # 16-bit words asked for, k too large: 32-bit copies
    L.cb200_host_stage_destroy(stage)
    for bad in (3, -2):
        o.narrow_indices = bad
        assert L.cb200_host_stage_create(C.byref(o), C.byref(stage)) == capi.INVALID_ARGUMENT
    o.narrow_indices, o.host_threads = 0, -1
    assert L.cb200_host_stage_create(C.byref(o), C.byref(stage)) == capi.INVALID_ARGUMENT


@pytest.mark.parametrize("bits,policy", [(8, 1), (4, 2), (2, 1), (1, 2)])
def test_device_element_lookup(cuda_device, oracle, bits, policy):
    """cb200_get_values on the device equals cb200_get_value on the host, bit for bit."""
    L = capi.lib()
    rng = np.random.default_rng(bits * 7 + policy)
    c = host_pack(oracle, random_csr(rng, rows=60, cols=90, max_nnz=40, bits=bits, policy=policy))
    x = to_dev(c, cuda_device)
    rr, cc = np.meshgrid(np.arange(-1, 61), np.arange(-1, 91), indexing="ij")
    rows_d = torch.from_numpy(rr.ravel().astype(np.int64)).to(cuda_device)
    cols_d = torch.from_numpy(cc.ravel().astype(np.int32)).to(cuda_device)
    vals = torch.full((rows_d.numel(),), float("nan"), device=cuda_device)
    codes = torch.full((rows_d.numel(),), -7, dtype=torch.int32, device=cuda_device)
    d = x.desc()
    capi.check(L.cb200_get_values(C.byref(d), rows_d.data_ptr(), cols_d.data_ptr(), rows_d.numel(), vals.data_ptr(), codes.data_ptr(),
                                  cuda_device.index, torch.cuda.current_stream().cuda_stream))
    dec = oracle.unpack_csr(bits, policy, c["row_ptr"], c["packed_row_ptr"], c["col_idx"], c["scales"], c["offsets"], c["packed"])
    want = np.zeros((62, 92), dtype=np.float32)
    stored = np.zeros((62, 92), dtype=bool)
    for r in range(60):
        lo, hi = c["row_ptr"][r], c["row_ptr"][r + 1]
        want[r + 1, c["col_idx"][lo:hi] + 1] = dec[lo:hi]
        stored[r + 1, c["col_idx"][lo:hi] + 1] = True
    got = vals.cpu().numpy().reshape(62, 92)
    assert np.array_equal(got, want)
    assert np.array_equal(codes.cpu().numpy().reshape(62, 92) >= 0, stored)


@pytest.mark.parametrize("kind", ["tensor_blocked", "tensor_blocked_x2", "tensor_dense", "gene_gather", "transpose_x3", "row_order"])
def test_prepare_builds_in_session_memory_without_allocating(cuda_device, oracle, kind):
    """The session reserves cb200_spmm_persistent_requirement bytes before sealing; prepare builds its copies
    inside that block on the given stream, allocates nothing, and the launches equal those of a prepared
    operation that allocated for itself.  A block that is too small is refused with a status."""
    L = capi.lib()
    rng = np.random.default_rng(21)
    rows, cols, n = 256 * 4 + 19, 1000, 64
    c = host_pack(oracle, random_csr(rng, rows=rows, cols=cols, max_nnz=260, bits=8, policy=1))
    x = to_dev(c, cuda_device)
    transpose = kind in ("gene_gather", "transpose_x3")
    if transpose:
        d, _ = dense(rng, rows, n, torch.float32, cuda_device, std=1.0)
        args = dict(projection=capi.PROJECTION_TRANSPOSE, multiply=0, deterministic=kind == "gene_gather",
                    schedule=None if kind == "gene_gather" else "tensor_blocked", matrix=x)
        out_shape = (cols, n)
    else:
        d, _ = dense(rng, cols, n, torch.bfloat16, cuda_device)
        args = dict(projection=capi.PROJECTION_CSR, multiply=0 if kind in ("tensor_blocked_x2", "row_order") else capi.DTYPE_BF16,
                    deterministic=False, schedule={"tensor_blocked_x2": "tensor_blocked", "row_order": "gene_tiled"}.get(kind, kind),
                    matrix=None if kind == "row_order" else x)
        out_shape = (rows, n)
    common = dict(host_row_ptr=c["row_ptr"], multiply=args["multiply"], device_matrix=args["matrix"], deterministic=args["deterministic"],
                  schedule=args["schedule"])
    need = ops.PreparedSpmm.persistent_requirement(args["projection"], rows, cols, n, x.nnz, 8, 1, d.dtype, cuda_device.index, **common)
    assert need > 0
    sess_opts = capi.header(capi.SessionOptions())
    sess_opts.device, sess_opts.owned_stream_count = cuda_device.index, 1
    sess = C.c_void_p()
    capi.check(L.cb200_session_create(C.byref(sess_opts), C.byref(sess)))
    try:
        block = C.c_void_p()
        capi.check(L.cb200_session_reserve_persistent(sess, need, C.byref(block)))
        capi.check(L.cb200_session_reserve_transient(sess, 0, 1 << 22))
        capi.check(L.cb200_session_seal(sess))
        binding = L.cb200_session_bind(sess, 0, 0)
        assert binding.status == capi.SUCCESS

        class Borrowed:                                            # what PreparedSpmm needs of a tensor
            def data_ptr(self): return block.value
            def numel(self): return need
            def element_size(self): return 1

        # the self-allocating operation first: it also loads the build kernels, so that the measurement below sees
        # allocations only
        own = ops.PreparedSpmm(args["projection"], rows, cols, n, x.nnz, 8, 1, d.dtype, cuda_device, **common)
        torch.cuda.synchronize()
        free0, _ = torch.cuda.mem_get_info(cuda_device)
        reserved0 = torch.cuda.memory_reserved(cuda_device)
        op = ops.PreparedSpmm(args["projection"], rows, cols, n, x.nnz, 8, 1, d.dtype, cuda_device, persistent=Borrowed(),
                              prepare_stream=binding.stream, **common)
        free1, _ = torch.cuda.mem_get_info(cuda_device)
        # the only allocation is the workspace tensor of the Python wrapper (through torch's cache)
        assert free0 - free1 <= max(0, torch.cuda.memory_reserved(cuda_device) - reserved0)
        assert 0 < op.persistent_bytes <= need
        expected = {"transpose_x3": "tensor_blocked_x3", "row_order": "gene_tiled"}.get(kind, kind)
        assert op.schedule == own.schedule == expected
        a = op.run(x, d, torch.full(out_shape, float("nan"), device=cuda_device))
        b = own.run(x, d, torch.full(out_shape, float("nan"), device=cuda_device))
        torch.cuda.synchronize()
        assert op.status() == 0 and own.status() == 0
        if kind in ("transpose_x3",):                             # atomic order of the flush: equal to rounding
            assert torch.allclose(a, b, rtol=1e-4, atol=1e-3)
        else:
            assert torch.equal(a, b)
        op.close()                                                 # frees nothing of the session's block
        own.close()
        # too small a block: a status, and nothing half-built is left behind
        class Small(Borrowed):
            def numel(self): return 4096
        with pytest.raises(capi.Cb200Error) as e:
            ops.PreparedSpmm(args["projection"], rows, cols, n, x.nnz, 8, 1, d.dtype, cuda_device, persistent=Small(),
                             prepare_stream=binding.stream, **common)
        assert e.value.status == capi.INSUFFICIENT_WORKSPACE
    finally:
        L.cb200_session_destroy(sess)


def test_status_readers_and_the_bounded_wait_path(cuda_device, oracle):
    """The status word has a reader on every path.  With the test hook armed the tensor-core kernel's W loader
    withholds its copies and every wait gives up after a few thousand polls: the launch ends at once, the reader
    returns CB200_STATUS_DEVICE_WAIT_TIMEOUT, the context stays usable (TMEM freed), and the next launch on the
    same stream, hook disarmed, is correct."""
    L = capi.lib()
    rng = np.random.default_rng(8)
    rows, cols, n = 256 * 6, 128 * 9, 64
    # about 1,400 entries per 256 x 128 segment: one entry chunk each, so the two-group kernel (the one with the hook) runs
    c = host_pack(oracle, random_csr(rng, rows=rows, cols=cols, max_nnz=100, bits=8, policy=1, empty_rows=False))
    x = to_dev(c, cuda_device)
    w, w_host = dense(rng, cols, n, torch.bfloat16, cuda_device)
    op = ops.PreparedSpmm(capi.PROJECTION_CSR, rows, cols, n, x.nnz, 8, 1, w.dtype, cuda_device, multiply=capi.DTYPE_BF16,
                          device_matrix=x, schedule="tensor_blocked")
    assert op.schedule == "tensor_blocked"
    good = op.run(x, w, torch.empty(rows, n, device=cuda_device)).clone()
    assert op.status() == 0
    L.cb200_test_arm_wait_timeout(4096)
    try:
        op.run(x, w, torch.empty(rows, n, device=cuda_device))
    finally:
        L.cb200_test_disarm_wait_timeout()
    with pytest.raises(capi.Cb200Error) as e:
        op.status()
    assert e.value.status == capi.DEVICE_WAIT_TIMEOUT
    torch.cuda.synchronize()                                       # no fault: the context answers
    again = op.run(x, w, torch.full((rows, n), float("nan"), device=cuda_device))
    assert op.status() == 0
    assert torch.equal(again, good)
    # the routed public calls: status block at the start of the caller's scratch
    y = ops.public_projection(x, w.float())
    assert torch.isfinite(y).all()
    op.close()


def test_an_empty_first_shard_is_a_no_op(cuda_device, oracle):
    """[0, 0) is an empty row range, not "all rows": the forward launch writes nothing, the transpose scales by beta."""
    rng = np.random.default_rng(2)
    c = host_pack(oracle, random_csr(rng, rows=90, cols=70, max_nnz=30, bits=8, policy=1))
    x = to_dev(c, cuda_device)
    w, _ = dense(rng, 70, 32, torch.bfloat16, cuda_device)
    g, _ = dense(rng, 90, 32, torch.float32, cuda_device, std=1.0)
    fwd = ops.PreparedSpmm(capi.PROJECTION_CSR, 90, 70, 32, x.nnz, 8, 1, w.dtype, cuda_device)
    y = torch.full((90, 32), 5.0, device=cuda_device)
    fwd.run(x, w, y, row_begin=0, row_end=0)
    assert torch.all(y == 5.0)
    full = fwd.run(x, w, torch.empty(90, 32, device=cuda_device))          # the default is CB200_ALL_ROWS
    assert torch.equal(full, fwd.run(x, w, torch.empty(90, 32, device=cuda_device), row_begin=0, row_end=90))
    tr = ops.PreparedSpmm(capi.PROJECTION_TRANSPOSE, 90, 70, 32, x.nnz, 8, 1, g.dtype, cuda_device)
    out = torch.full((70, 32), 4.0, device=cuda_device)
    tr.run(x, g, out, row_begin=0, row_end=0, beta=0.5)
    assert torch.all(out == 2.0)
    blocks = (capi.CsrBlock * 8)()
    rp = np.ascontiguousarray(c["row_ptr"][:4], dtype=np.int64)            # 3 rows over 8 ranks: trailing shards are empty
    capi.check(capi.lib().cb200_fleet_partition(3, 8, rp.ctypes.data, None, blocks))
    assert [(b.row_begin, b.row_end) for b in blocks] == [(0, 1), (1, 2), (2, 3)] + [(3, 3)] * 5
