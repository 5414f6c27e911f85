"""The reference's public projection calls (cellerator_sparse_projection_forward / _backward,
src/abi/abi.cu:278-396) routed to this backend for the quantized layouts: same results as the
operation-core path and as the oracle, same rejections as the public ABI makes."""
import ctypes as C

import numpy as np
import pytest
import torch

from cellerator_b200 import capi, ops, synth
from conftest import random_csr
from gpu_util import assert_forward_close, dense, host_pack, row_l1, to_dev

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("policy", [1, 2])
@pytest.mark.parametrize("n", [32, 64, 40])
@pytest.mark.parametrize("bits", [8, 4])
def test_quantized_csr_forward_and_backward(cuda_device, oracle, policy, n, bits):
    """(4-bit codes: the public descriptor carries no packed row offsets; the call derives them on the stream.)"""
    rng = np.random.default_rng(50 + n + policy + bits)
    c = host_pack(oracle, random_csr(rng, rows=700 if bits == 8 else 2300, cols=900, max_nnz=220, bits=bits, policy=policy))
    x = to_dev(c, cuda_device)
    w, w_host = dense(rng, c["cols"], n, torch.float32, cuda_device, ld=n + 4)       # explicit leading dimension
    y = ops.public_projection(x, w)
    ref = oracle.qcsr_forward(bits, policy, c["row_ptr"], c["packed_row_ptr"], c["col_idx"], c["packed"], c["scales"],
                              c["offsets"], w_host, c["cols"])
    l1, _ = row_l1(oracle, c)
    assert_forward_close(y.cpu().numpy(), ref, l1, float(np.abs(w_host).max()))
    assert torch.equal(y, ops.spmm_forward(x, w))                                    # the operation-core path, bit for bit
    g, _ = dense(rng, c["rows"], n, torch.float32, cuda_device, std=1.0)
    gr = ops.public_projection(x, g, backward=True)
    # the same fp32 reductions in another order (L2 atomics): equal to summation error, which scales with
    # the largest partial sums (~600 here), not with the element
    direct = ops.spmm_transpose(x, g)
    assert float((gr - direct).abs().max()) <= 1e-5 * float(direct.abs().max())


def test_quantized_blocked_ell_forward(cuda_device, oracle):
    rng = np.random.default_rng(8)
    h = synth.make_qbell_host(32 * 9 + 5, 1000, 32, 4, 0.6, 8, seed=3)
    x = ops.QuantizedBell.from_host(h, cuda_device)
    w, _ = dense(rng, 1000, 64, torch.float32, cuda_device)
    assert torch.equal(ops.public_projection(x, w), ops.bell_forward(x, w))


def test_rejections(cuda_device, oracle):
    rng = np.random.default_rng(1)
    c = host_pack(oracle, random_csr(rng, rows=50, cols=80, max_nnz=20, bits=8, policy=1))
    x = to_dev(c, cuda_device)
    w, _ = dense(rng, 80, 32, torch.float32, cuda_device)
    l = ops.public_layout(x)
    out = torch.empty(50, 32, device=cuda_device)
    scratch = torch.empty(4096, dtype=torch.uint8, device=cuda_device)
    call = lambda lay, sbytes=4096: capi.lib().cb200_public_projection_forward(
        C.byref(lay), C.c_void_p(w.data_ptr()), C.c_int64(32), C.c_int64(32), C.c_void_p(out.data_ptr()), C.c_int64(32),
        C.c_int32(0), C.c_void_p(0), C.c_void_p(scratch.data_ptr()), C.c_uint64(sbytes))
    assert call(l) == 0
    assert call(l, 128) == 7                                       # scratch too small: insufficient workspace
    l.layout = 1                                                   # CELLERATOR_LAYOUT_CSR (fp16 values): not this backend's
    assert call(l) == 3
    l = ops.public_layout(x)
    l.bits = 2                                                     # 8- and 4-bit codes only
    assert call(l) == 3
    l = ops.public_layout(x)
    l.size = 8
    assert call(l) == 1
    bell = ops.QuantizedBell.from_host(synth.make_qbell_host(64, 128, 32, 2, 0.5, 8, seed=1), cuda_device)
    with pytest.raises(capi.Cb200Error):                           # backward of the Blocked-ELL layout is not served
        ops.public_projection(bell, torch.zeros(64, 32, device=cuda_device), backward=True)
