"""Prepared-operation and session lifecycle on a real device: validation happens on the host
before anything is enqueued, and a failed call leaves the context usable."""
import ctypes as C

import numpy as np
import pytest
import torch

from cellerator_b200 import capi, ops
from conftest import random_csr
from gpu_util import dense, host_pack, to_dev

pytestmark = pytest.mark.gpu


@pytest.fixture()
def problem(cuda_device, oracle):
    rng = np.random.default_rng(1)
    c = host_pack(oracle, random_csr(rng, rows=50, cols=90, max_nnz=40, bits=8, policy=1))
    x = to_dev(c, cuda_device)
    w, w_host = dense(rng, 90, 32, torch.float32, cuda_device)
    ref = oracle.qcsr_forward(8, 1, c["row_ptr"], c["packed_row_ptr"], c["col_idx"], c["packed"], c["scales"],
                              c["offsets"], w_host, 90)
    return x, w, ref


def test_prepare_run_lifecycle_and_rejections(cuda_device, problem):
    x, w, ref = problem
    op = ops.PreparedSpmm(capi.PROJECTION_CSR, x.rows, x.cols, 32, x.nnz, 8, 1, w.dtype, cuda_device,
                          structure_epoch=7, host_row_ptr=x.host_row_ptr, deterministic=True)
    assert op.schedule in ("warp_per_row", "gene_tiled")
    out = torch.zeros(x.rows, 32, device=cuda_device)
    before = capi.lib().cb200_kernel_launch_count()
    op.run(x, w, out)
    assert capi.lib().cb200_kernel_launch_count() > before
    assert np.allclose(out.cpu().numpy(), ref, rtol=1e-4, atol=1e-5)

    def status_of(**kw):
        ln = op.make_launch(x, w, out, **{k: v for k, v in kw.items() if k in ("epoch", "row_begin", "row_end")})
        for k, v in kw.items():
            if k not in ("epoch", "row_begin", "row_end"):
                setattr(ln, k, v)
        return capi.lib().cb200_spmm_run(op.handle, C.byref(ln))

    launches = capi.lib().cb200_kernel_launch_count()
    assert status_of(epoch=8) == capi.STALE_STRUCTURE                     # structure epoch moved on
    assert status_of(device=3) == capi.INVALID_STREAM                     # not the prepared device
    assert status_of(workspace_device=1) == capi.INVALID_STREAM           # workspace on another device
    assert status_of(row_begin=10, row_end=x.rows + 1) == capi.INVALID_SHAPE
    assert status_of(out=None) == capi.INVALID_ARGUMENT
    assert status_of(out=w.data_ptr()) == capi.INVALID_ARGUMENT           # output aliases an input
    assert status_of(dense_ld=8) == capi.INVALID_SHAPE
    x.bits = 4
    assert status_of() == capi.INVALID_SHAPE                              # matrix disagrees with the preparation
    x.bits = 8
    assert capi.lib().cb200_kernel_launch_count() == launches             # nothing was enqueued
    assert capi.lib().cb200_last_error() != b""
    op.run(x, w, out)                                                     # still usable afterwards
    op.close()


def test_session_reserve_seal_bind(cuda_device, problem):
    x, w, ref = problem
    L = capi.lib()
    ext = torch.cuda.Stream(device=cuda_device)
    arr = (C.c_void_p * 1)(ext.cuda_stream)
    opts = capi.header(capi.SessionOptions())
    opts.device, opts.owned_stream_count, opts.external_stream_count = cuda_device.index, 1, 1
    opts.external_streams = arr
    sess = C.c_void_p()
    capi.check(L.cb200_session_create(C.byref(opts), C.byref(sess)))
    pers = C.c_void_p()
    capi.check(L.cb200_session_reserve_persistent(sess, 4096, C.byref(pers)))
    assert pers.value and pers.value % 256 == 0
    capi.check(L.cb200_session_reserve_transient(sess, 1, 1 << 20))
    assert L.cb200_session_bind(sess, 1, 16).status == capi.SEALED            # bind needs a sealed session
    capi.check(L.cb200_session_seal(sess))
    assert L.cb200_session_reserve_persistent(sess, 16, C.byref(pers)) == capi.SEALED
    assert L.cb200_session_reserve_transient(sess, 0, 1 << 21) == capi.SEALED
    assert L.cb200_session_bind(sess, 5, 0).status == capi.INVALID_ARGUMENT
    assert L.cb200_session_bind(sess, 1, 1 << 22).status == capi.INSUFFICIENT_WORKSPACE
    b = L.cb200_session_bind(sess, 0, 0)
    assert b.status == capi.SUCCESS and b.stream == ext.cuda_stream and b.device == cuda_device.index
    b1 = L.cb200_session_bind(sess, 1, 1 << 20)
    assert b1.status == capi.SUCCESS and b1.workspace and b1.workspace_bytes == 1 << 20
    # run on the session's own stream with its workspace
    op = ops.PreparedSpmm(capi.PROJECTION_CSR, x.rows, x.cols, 32, x.nnz, 8, 1, w.dtype, cuda_device)
    out = torch.zeros(x.rows, 32, device=cuda_device)
    torch.cuda.synchronize(cuda_device)
    ln = op.make_launch(x, w, out, stream=b1.stream)
    ln.workspace, ln.workspace_bytes = b1.workspace, b1.workspace_bytes
    op.run_launch(ln)
    capi.check(L.cb200_session_synchronize(sess))
    assert np.allclose(out.cpu().numpy(), ref, rtol=1e-4, atol=1e-5)
    L.cb200_session_destroy(sess)


def test_session_lifetimes_accounting_and_caches(cuda_device):
    """persistent_lifetime classes, session_accounting and the fixed caches of the reference's execution_session
    (include/Cellerator/runtime/session.cuh:28-90,147-177)."""
    L = capi.lib()
    opts = capi.header(capi.SessionOptions())
    opts.device, opts.owned_stream_count = cuda_device.index, 2
    sess = C.c_void_p()
    capi.check(L.cb200_session_create(C.byref(opts), C.byref(sess)))
    try:
        a, b, c = C.c_void_p(), C.c_void_p(), C.c_void_p()
        capi.check(L.cb200_session_reserve_persistent_as(sess, capi.LIFETIME_STRUCTURE, 1 << 20, C.byref(a)))
        capi.check(L.cb200_session_reserve_persistent_as(sess, capi.LIFETIME_PLAN, 1 << 16, C.byref(b)))
        capi.check(L.cb200_session_reserve_persistent_as(sess, capi.LIFETIME_GRAPH_STABLE, 4096, C.byref(c)))
        assert L.cb200_session_reserve_persistent_as(sess, 7, 16, C.byref(c)) == capi.INVALID_ARGUMENT
        capi.check(L.cb200_session_reserve_transient(sess, 0, 1 << 12))
        capi.check(L.cb200_session_reserve_transient(sess, 0, 1 << 14))       # grows: the old block is replaced
        capi.check(L.cb200_session_prepare_stream_libraries(sess, 1))
        assert L.cb200_session_prepare_stream_libraries(sess, 9) == capi.INVALID_ARGUMENT
        assert L.cb200_session_graph_stable_address(sess, c, 4096) == 1
        assert L.cb200_session_graph_stable_address(sess, C.c_void_p(c.value + 4000), 200) == 0     # runs past the reservation
        assert L.cb200_session_graph_stable_address(sess, a, 16) == 0                                # structure memory is not graph-stable
        entry = capi.SessionCacheEntry(0xabc, 0xdef, a, 3, 5)
        capi.check(L.cb200_session_cache_insert(sess, 1, C.byref(entry)))
        entry.generation = 6
        capi.check(L.cb200_session_cache_insert(sess, 1, C.byref(entry)))    # same key: replaced
        found = L.cb200_session_cache_find(sess, 1, 0xabc, 0xdef)
        assert found and found.contents.generation == 6 and found.contents.state == a.value
        assert not L.cb200_session_cache_find(sess, 0, 0xabc, 0xdef)         # another cache kind
        for i in range(63):
            e = capi.SessionCacheEntry(1, 100 + i, a, 1, 1)
            capi.check(L.cb200_session_cache_insert(sess, 1, C.byref(e)))
        e = capi.SessionCacheEntry(1, 999, a, 1, 1)
        assert L.cb200_session_cache_insert(sess, 1, C.byref(e)) == capi.INSUFFICIENT_WORKSPACE      # 64 entries
        capi.check(L.cb200_session_seal(sess))
        assert L.cb200_session_prepare_stream_libraries(sess, 0) == capi.SEALED
        for _ in range(3):
            assert L.cb200_session_bind(sess, 0, 1 << 14).status == capi.SUCCESS
        capi.check(L.cb200_session_synchronize(sess))
        acc = capi.SessionAccounting()
        capi.check(L.cb200_session_get_accounting(sess, C.byref(acc)))
        assert (acc.structure.current_bytes, acc.plan.current_bytes, acc.graph_stable.current_bytes) == (1 << 20, 1 << 16, 4096)
        assert acc.structure.allocation_count == acc.plan.allocation_count == acc.graph_stable.allocation_count == 1
        assert acc.transient.current_bytes == 1 << 14 and acc.transient.high_water_bytes == 1 << 14 and acc.transient.allocation_count == 2
        assert (acc.handle_prepare_count, acc.launch_bind_count, acc.synchronization_count) == (1, 3, 1)
    finally:
        L.cb200_session_destroy(sess)
