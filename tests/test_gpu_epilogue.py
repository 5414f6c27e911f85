"""GPU parity of the composed epilogue of the forward projections, through the C ABI:

    out = act(alpha * deq(X) W + beta * out + bias[column]),

the rule of the reference's referee (src/compute/math/referee.cc:81-97), for every epilogue kind of
the request contract (include/Cellerator/compute/math/operation.hh:49-61) and every forward schedule.

Two checks per case.  (1) The epilogue alone: the kernel's output with the epilogue against the
oracle's epilogue applied to the same kernel's output without it (the oracle's referee run on an
empty matrix with beta = 1); fp32 erff / tanhf against double erf / tanh, tolerance 2e-6 absolute
plus 2e-6 relative.  (2) End to end against the oracle's referee on the decoded matrix; the
activations have slope <= 1.13, so the forward bound is widened by 1.2."""
import numpy as np
import pytest
import torch

from cellerator_b200 import capi, ops, synth
from conftest import random_csr
from gpu_util import dense, host_pack, row_l1, to_dev

pytestmark = pytest.mark.gpu

KINDS = ["bias", "relu", "gelu_erf", "gelu_tanh", "bias_relu", "bias_gelu_erf", "bias_gelu_tanh"]


def oracle_epilogue(oracle, plain, kind, bias):
    """The oracle's epilogue applied to `plain`: referee on an empty matrix, beta = 1, initial = plain."""
    m, n = plain.shape
    return oracle.spmm_reference(m, 1, n, np.zeros(m + 1, dtype=np.uint64), np.zeros(0, dtype=np.uint32),
                                 np.zeros(0, dtype=np.float32), np.zeros((1, n), dtype=np.float32), beta=1.0,
                                 initial=plain, initial_ld=n, epilogue=kind, bias=bias)


def assert_epilogue_only(oracle, y_epi, y_plain, kind, bias_host):
    want = oracle_epilogue(oracle, y_plain, kind, bias_host if kind.startswith("bias") else None)
    got = np.asarray(y_epi, dtype=np.float64)
    assert np.all(np.abs(got - want) <= 2e-6 + 2e-6 * np.abs(want)), f"{kind}: {np.max(np.abs(got - want)):.3e}"


# schedule, W dtype, N, multiply, matrix handed to prepare, tolerance against the referee
FORWARD_CASES = [
    ("warp_per_row", torch.float32, 64, 0, False, 1e-4),
    ("warp_per_row", torch.bfloat16, 128, 0, False, 1e-4),
    ("warp_per_row", torch.float32, 40, 0, False, 1e-4),          # any-N kernel
    ("gene_tiled", torch.bfloat16, 128, 0, False, 1e-4),
    ("gene_tiled", torch.float32, 64, 0, False, 1e-4),
    ("tensor_windows", torch.bfloat16, 64, capi.DTYPE_BF16, False, 1e-2),
    ("tensor_blocked", torch.bfloat16, 128, capi.DTYPE_BF16, True, 1e-2),
    ("tensor_dense", torch.bfloat16, 64, capi.DTYPE_BF16, True, 1e-2),
    ("tensor_codes", torch.bfloat16, 128, capi.DTYPE_BF16, True, 1e-2),   # 4-bit codes
    ("tensor_blocked_x2", torch.bfloat16, 64, 0, True, 1e-4),     # the epilogue runs once, on the last pass
    ("tensor_blocked_x3", torch.float32, 32, 0, True, 1e-4),
]


@pytest.mark.parametrize("schedule,dtype,n,multiply,hand_matrix,tol", FORWARD_CASES)
def test_forward_epilogues(cuda_device, oracle, monkeypatch, schedule, dtype, n, multiply, hand_matrix, tol):
    monkeypatch.setitem(ops.SCHEDULE_REQUEST, capi.PROJECTION_CSR, schedule.split("_x")[0])
    rng = np.random.default_rng(len(schedule) * 131 + n)
    rows, cols, bits, policy = 2 * 1024 + 77, 900, 4 if schedule == "tensor_codes" else 8, 1
    c = host_pack(oracle, random_csr(rng, rows=rows, cols=cols, max_nnz=280, bits=bits, policy=policy))
    x = to_dev(c, cuda_device)
    w, w_host = dense(rng, cols, n, dtype, cuda_device, std=0.05)
    bias_host = rng.normal(0.0, 0.5, n).astype(np.float32)
    bias = torch.from_numpy(bias_host).to(cuda_device)
    init_host = rng.normal(0.0, 1.0, (rows, n)).astype(np.float32)
    init = torch.from_numpy(init_host).to(cuda_device)
    op = ops.PreparedSpmm(capi.PROJECTION_CSR, rows, cols, n, x.nnz, bits, policy, w.dtype, cuda_device,
                          host_row_ptr=x.host_row_ptr, multiply=multiply, device_matrix=x if hand_matrix else None)
    assert op.schedule == schedule
    _, dec = row_l1(oracle, c)
    l1, _ = row_l1(oracle, c)
    wmax = float(np.abs(w_host).max())
    alpha, beta = 1.5, 0.25
    plain = op.run(x, w, init.clone(), alpha=alpha, beta=beta).cpu().numpy()
    for kind in KINDS:
        y = op.run(x, w, init.clone(), alpha=alpha, beta=beta, epilogue=kind, bias=bias).cpu().numpy()
        assert_epilogue_only(oracle, y, plain, kind, bias_host)
        ref = oracle.spmm_reference(rows, cols, n, c["row_ptr"], c["col_idx"], dec, w_host, alpha=alpha, beta=beta,
                                    initial=init_host, initial_ld=n, epilogue=kind,
                                    bias=bias_host if kind.startswith("bias") else None)
        bound = 1.2 * tol * alpha * l1[:, None] * wmax + 1e-5
        assert np.all(np.abs(y - ref) <= bound), f"{kind}: {np.max(np.abs(y - ref) / bound):.3e} of the bound"
    # a row range leaves the other rows alone, epilogue included
    out = init.clone()
    op.run(x, w, out, row_begin=256, row_end=1024, epilogue="bias_relu", bias=bias)
    assert torch.equal(out[:256], init[:256]) and torch.equal(out[1024:], init[1024:])
    assert torch.all(out[256:1024] >= 0.0)
    op.close()


def test_epilogue_validation(cuda_device, oracle):
    rng = np.random.default_rng(9)
    c = host_pack(oracle, random_csr(rng, rows=40, cols=100, max_nnz=20, bits=8, policy=1))
    x = to_dev(c, cuda_device)
    w, _ = dense(rng, 100, 32, torch.float32, cuda_device)
    y = torch.zeros(40, 32, device=cuda_device)
    op = ops.PreparedSpmm(capi.PROJECTION_CSR, 40, 100, 32, x.nnz, 8, 1, w.dtype, cuda_device)
    with pytest.raises(capi.Cb200Error):                       # a bias kind without its vector
        op.run(x, w, y, epilogue="bias_relu")
    with pytest.raises(capi.Cb200Error):                       # not one of the eight kinds
        op.run(x, w, y, epilogue=8)
    op.run(x, w, y, epilogue="relu")                           # no bias needed
    assert torch.all(y >= 0.0)
    op.close()
    g = torch.zeros(40, 32, device=cuda_device)
    tr = ops.PreparedSpmm(capi.PROJECTION_TRANSPOSE, 40, 100, 32, x.nnz, 8, 1, g.dtype, cuda_device)
    with pytest.raises(capi.Cb200Error):                       # the transpose composes no epilogue
        tr.run(x, g, torch.zeros(100, 32, device=cuda_device), epilogue="relu")
    tr.close()


@pytest.mark.parametrize("block_size,ell_blocks,cols,n,dtype,bits", [
    (32, 8, 2048, 256, torch.bfloat16, 8),      # tcgen05 kernel
    (32, 3, 250, 64, torch.float32, 8),         # CUDA-core vector kernel
    (16, 5, 333, 40, torch.float32, 4),         # any-N kernel
])
def test_bell_epilogues(cuda_device, oracle, block_size, ell_blocks, cols, n, dtype, bits):
    rng = np.random.default_rng(block_size + n)
    rows = 6 * block_size + 3
    h = synth.make_qbell_host(rows, cols, block_size, ell_blocks, 0.6, bits, seed=block_size)
    x = ops.QuantizedBell.from_host(h, cuda_device)
    w, _ = dense(rng, cols, n, dtype, cuda_device, std=0.05)
    bias_host = rng.normal(0.0, 0.5, n).astype(np.float32)
    bias = torch.from_numpy(bias_host).to(cuda_device)
    init = torch.from_numpy(rng.normal(size=(rows, n)).astype(np.float32)).to(cuda_device)
    plain = ops.bell_forward(x, w, out=init.clone(), alpha=0.75, beta=0.5).cpu().numpy()
    for kind in KINDS:
        y = ops.bell_forward(x, w, out=init.clone(), alpha=0.75, beta=0.5, epilogue=kind, bias=bias).cpu().numpy()
        assert_epilogue_only(oracle, y, plain, kind, bias_host)
