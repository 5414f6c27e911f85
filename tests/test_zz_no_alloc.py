"""The allocation-free forward entry point, cb200_qcsr_forward_static.

It exists for callers that cannot call cudaMalloc (allocator-free regions, fixed and policed
device-memory budgets, foreign-language shims without a device allocator): the kernel's scratch is
a fixed array inside the library instead of a caller-provided workspace.  This file is named so
that pytest collects it last; the test passes on its own in a fresh process and after the rest of
the suite.  It calls the entry point twice in a row through the C ABI (the second call finds the
array holding the first call's contents) and compares both results with the existing
prepare/run entry point, which runs the same kernel on a caller-provided workspace.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from cellerator_b200 import capi, ops
from conftest import random_csr
from gpu_util import assert_forward_close, dense, host_pack, row_l1, to_dev

pytestmark = pytest.mark.gpu


def forward_static(x, w, y, alpha=1.0, beta=0.0):
    dev = x.device
    dtype = capi.DTYPE_BF16 if w.dtype == torch.bfloat16 else capi.DTYPE_F32
    return capi.lib().cb200_qcsr_forward_static(C.byref(x.desc()), w.data_ptr(), dtype, w.shape[1], y.data_ptr(),
                                                y.stride(0), alpha, beta, dev.index,
                                                torch.cuda.current_stream(dev).cuda_stream)


def static_status(device):
    """cb200_qcsr_forward_static_status: the status word of the last static call (it lives in the library's array)."""
    word = C.c_int32(-1)
    st = capi.lib().cb200_qcsr_forward_static_status(device.index, torch.cuda.current_stream(device).cuda_stream, C.byref(word))
    return st, word.value


@pytest.mark.parametrize("bits,dtype,n,policy", [(8, torch.bfloat16, 64, 1), (4, torch.bfloat16, 128, 1), (8, torch.float32, 32, 1),
                                                 (8, torch.bfloat16, 64, 2), (4, torch.float32, 64, 2)])
def test_static_scratch_entry_matches_prepared_entry_twice(cuda_device, oracle, monkeypatch, bits, dtype, n, policy):
    monkeypatch.setitem(ops.SCHEDULE_REQUEST, capi.PROJECTION_CSR, "gene_tiled")
    rng = np.random.default_rng(900 + bits + n + policy)
    rows, cols = 128 * 2 + 19, 2600
    c = host_pack(oracle, random_csr(rng, rows=rows, cols=cols, max_nnz=500, bits=bits, policy=policy))
    x = to_dev(c, cuda_device)
    w, w_host = dense(rng, cols, n, dtype, cuda_device)

    # the existing entry point: prepared operation + caller workspace
    op = ops.PreparedSpmm(capi.PROJECTION_CSR, rows, cols, n, x.nnz, bits, policy, w.dtype, cuda_device,
                          host_row_ptr=x.host_row_ptr)
    assert op.schedule == "gene_tiled"
    expected = op.run(x, w, torch.empty(rows, n, device=cuda_device))
    torch.cuda.synchronize(cuda_device)

    # two calls in a row of the allocation-free entry point; no device memory may be taken
    first = torch.full((rows, n), float("nan"), device=cuda_device)
    second = torch.full((rows, n), float("nan"), device=cuda_device)
    capi.check(forward_static(x, w, first))          # also does the one-time address look-up
    torch.cuda.synchronize(cuda_device)
    free_before, _ = torch.cuda.mem_get_info(cuda_device)
    capi.check(forward_static(x, w, second))
    torch.cuda.synchronize(cuda_device)
    free_after, _ = torch.cuda.mem_get_info(cuda_device)
    assert free_after == free_before
    assert static_status(cuda_device) == (capi.SUCCESS, 0)       # no bounded wait ran out; the reader allocates nothing either
    assert torch.cuda.mem_get_info(cuda_device)[0] == free_before

    ref = oracle.qcsr_forward(bits, policy, c["row_ptr"], c["packed_row_ptr"], c["col_idx"], c["packed"], c["scales"],
                              c["offsets"], w_host, cols)
    l1, _ = row_l1(oracle, c)
    for got in (first, second):
        assert torch.equal(got, expected)            # same kernel, same summation order
        assert_forward_close(got.cpu().numpy(), ref, l1, float(np.abs(w_host).max()), bf16=dtype == torch.bfloat16)

    # alpha / beta through the same entry
    third = expected.clone()
    capi.check(forward_static(x, w, third, alpha=0.5, beta=2.0))
    assert torch.allclose(third, 2.5 * expected, rtol=1e-5, atol=1e-6)


def test_static_scratch_entry_rejects_what_it_does_not_cover(cuda_device, oracle):
    rng = np.random.default_rng(5)
    c = host_pack(oracle, random_csr(rng, rows=40, cols=200, max_nnz=50, bits=8, policy=1))
    x = to_dev(c, cuda_device)
    w24, _ = dense(rng, 200, 24, torch.bfloat16, cuda_device)
    y = torch.zeros(40, 24, device=cuda_device)
    assert forward_static(x, w24, y) == capi.UNSUPPORTED
    assert b"allocation-free" in capi.lib().cb200_last_error()
    w64, _ = dense(rng, 200, 64, torch.bfloat16, cuda_device)
    y_odd = torch.zeros(40, 66, device=cuda_device)[:, 1:65]                # Y rows not 16-byte aligned
    assert forward_static(x, w64, y_odd) == capi.UNSUPPORTED
    assert capi.lib().cb200_qcsr_forward_static(None, w64.data_ptr(), capi.DTYPE_BF16, 64, y.data_ptr(), 64, 1.0, 0.0,
                                                0, None) == capi.INVALID_ARGUMENT
    assert torch.all(y == 0)
