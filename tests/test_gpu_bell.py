"""GPU parity of the quantized Blocked-ELL projection, through the C ABI."""
import os

import numpy as np
import pytest
import torch

from cellerator_b200 import capi, ops, synth
from conftest import GOLDEN
from gpu_util import dense

pytestmark = pytest.mark.gpu


def bell_reference(oracle, h, w_host):
    a = (h["bits"], h["policy"], h["rows"], h["cols"], h["block_size"], h["ell_cols"], h["row_stride_bytes"],
         h["block_col_idx"], h["scales"], h["offsets"])
    ro, cols, vals = oracle.bell_to_csr(*a, h["packed"])
    y = oracle.spmm_reference(h["rows"], h["cols"], w_host.shape[1], ro, cols, vals, w_host)
    l1 = np.zeros(h["rows"])
    counts = np.diff(ro.astype(np.int64))
    nz = counts > 0
    if len(vals):
        l1[nz] = np.add.reduceat(np.abs(vals.astype(np.float64)), ro[:-1][nz].astype(np.int64))
    return y, l1


def assert_bell_close(y, ref, l1, wmax, bf16_multiply):
    """CUDA-core kernel: the forward bound 1e-4 * ||row||_1 * max|W|.  Tensor-core kernel (values and W rounded
    to fp16, eleven significant bits, before the multiply): 2e-3 of ||row||_1 * max|W|, five times inside the
    1e-2 tolerance the benchmark contract gives 16-bit products (two roundings of 2^-12 each bound it by 5e-4)."""
    err = np.abs(np.asarray(y, dtype=np.float64) - ref)
    scale = l1[:, None] * wmax + 1e-30
    tol = 2e-3 if bf16_multiply else 1e-4
    assert np.all(err <= tol * scale), f"max err/scale {np.max(err / scale):.3e}"


@pytest.mark.parametrize("bits,policy", [(8, 1), (4, 2)])
def test_kat_bell_3x3(cuda_device, oracle, kats, bits, policy):
    k = kats["bell_3x3"]
    bci = np.array(k["block_col_idx"], dtype=np.uint32)
    scales = np.array(k["per_gene_scales"] if policy == 1 else k["column_scales"], dtype=np.float32)
    offsets = None if policy == 1 else np.array(k["row_offsets"], dtype=np.float32)
    stride = -(-k["ell_cols"] * bits // 8)
    packed = oracle.bell_pack(bits, policy, 3, 3, 1, 2, stride, bci, scales, offsets, k["slot_values"])
    x = ops.QuantizedBell.from_host(dict(rows=3, cols=3, block_size=1, ell_cols=2, row_stride_bytes=stride, bits=bits,
                                         policy=policy, block_col_idx=bci, packed=packed, scales=scales,
                                         offsets=offsets), cuda_device)
    w = torch.tensor(k["rhs"], dtype=torch.float32, device=cuda_device).reshape(3, 2)
    y = ops.bell_forward(x, w).cpu().numpy()
    assert np.allclose(y.ravel(), k["expected"], atol=1e-4)


@pytest.mark.parametrize("name", ["bell8_small", "bell4_small"])
def test_golden_bell_forward(cuda_device, oracle, name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    h = dict(rows=int(z["rows"]), cols=int(z["cols"]), block_size=int(z["block_size"]), ell_cols=int(z["ell_cols"]),
             row_stride_bytes=int(z["row_stride_bytes"]), bits=int(z["bits"]), policy=1,
             block_col_idx=z["block_col_idx"], packed=z["packed"], scales=z["scales"], offsets=z["offsets"])
    x = ops.QuantizedBell.from_host(h, cuda_device)
    w = torch.from_numpy(z["w"]).to(cuda_device)
    y = ops.bell_forward(x, w).cpu().numpy()
    _, l1 = bell_reference(oracle, h, z["w"])
    assert_bell_close(y, z["y"], l1, float(np.abs(z["w"]).max()), bf16_multiply=False)


@pytest.mark.parametrize("block_size,ell_blocks,cols,n,dtype,bits", [
    (32, 4, 1000, 256, torch.bfloat16, 8),
    (32, 16, 8192, 256, torch.bfloat16, 8),
    (32, 3, 250, 64, torch.float32, 8),
    (16, 5, 333, 40, torch.float32, 4),
    (8, 6, 100, 128, torch.bfloat16, 4),
])
def test_random_bell_forward(cuda_device, oracle, block_size, ell_blocks, cols, n, dtype, bits):
    rng = np.random.default_rng(block_size + n)
    rows = 4 * block_size + 5          # last block row is ragged
    h = synth.make_qbell_host(rows, cols, block_size, ell_blocks, 0.6, bits, seed=block_size)
    bci = h["block_col_idx"].reshape(-1, ell_blocks).copy()
    bci[1, -1] = 0xFFFFFFFF            # an empty block: skipped
    h["block_col_idx"] = bci.ravel()
    x = ops.QuantizedBell.from_host(h, cuda_device)
    w, w_host = dense(rng, cols, n, dtype, cuda_device)
    ref, l1 = bell_reference(oracle, h, w_host)
    y = ops.bell_forward(x, w)
    tensor_core = dtype == torch.bfloat16 and block_size == 32
    assert_bell_close(y.cpu().numpy(), ref, l1, float(np.abs(w_host).max()), bf16_multiply=tensor_core)
    y2 = ops.bell_forward(x, w)
    assert torch.equal(y, y2)          # deterministic
    init = torch.from_numpy(rng.normal(size=(rows, n)).astype(np.float32)).to(cuda_device)
    y3 = ops.bell_forward(x, w, out=init.clone(), alpha=0.5, beta=2.0)
    assert torch.allclose(y3, 0.5 * y + 2.0 * init, rtol=1e-4, atol=1e-4)


def test_device_generated_bell_matches_oracle(cuda_device, oracle):
    cfg = dict(synth.CONFIGS["c5_bell"])
    cfg["rows"] = 32 * 40
    x = synth.make_qbell_device(**cfg, device=cuda_device, seed=0)
    rng = np.random.default_rng(2)
    w, w_host = dense(rng, x.cols, cfg["n"], torch.bfloat16, cuda_device)
    y = ops.bell_forward(x, w).cpu().numpy()
    h = dict(rows=x.rows, cols=x.cols, block_size=x.block_size, ell_cols=x.ell_cols,
             row_stride_bytes=x.row_stride_bytes, bits=x.bits, policy=x.policy,
             block_col_idx=x.block_col_idx.cpu().numpy().view(np.uint32), packed=x.packed.cpu().numpy(),
             scales=x.scales.cpu().numpy(), offsets=x.offsets.cpu().numpy())
    ref, l1 = bell_reference(oracle, h, w_host)
    assert_bell_close(y, ref, l1, float(np.abs(w_host).max()), bf16_multiply=True)
    bci = h["block_col_idx"].reshape(-1, cfg["ell_blocks"])
    assert np.all(np.diff(bci.astype(np.int64), axis=1) > 0) and bci.max() < 256
    dec = ops.dequantize_bell(x).cpu().numpy()
    frac = float((dec != 0).mean())
    assert 0.5 < frac < 0.7            # about 60 % of the slots of present blocks are non-zero


def test_bell_configuration_at_one_eighth_scale(cuda_device, oracle):
    """The Blocked-ELL configuration's genes, block geometry and N = 256 on 1/8 of a GPU's shard (31,232 cells,
    976 block rows), device-generated: block rows sampled at the start, the middle and the end against the
    reference's decode + double-precision referee, repeat runs bit-identical, shards equal to the whole."""
    cfg = dict(synth.CONFIGS["c5_bell"])
    bs = cfg["block_size"]
    cfg["rows"] = cfg["rows"] // 8 // 8 // bs * bs
    x = synth.make_qbell_device(**cfg, device=cuda_device, seed=0)
    rng = np.random.default_rng(6)
    w, w_host = dense(rng, x.cols, cfg["n"], torch.bfloat16, cuda_device)
    op = ops.PreparedSpmm(capi.PROJECTION_BLOCKED_ELL, x.rows, x.cols, cfg["n"], x.rows * x.ell_cols, x.bits, x.policy, w.dtype, cuda_device)
    assert op.schedule == "tcgen05_block_rows"
    y = op.run(x, w, torch.full((x.rows, cfg["n"]), float("nan"), device=cuda_device))
    assert op.status() == 0
    assert torch.equal(y, op.run(x, w, torch.empty_like(y)))
    bci = x.block_col_idx.cpu().numpy().view(np.uint32).reshape(-1, cfg["ell_blocks"])
    packed = x.packed.cpu().numpy().reshape(x.rows, x.row_stride_bytes)
    wmax = float(np.abs(w_host).max())
    block_rows = x.rows // bs
    for b0 in (0, block_rows // 2 - 1, block_rows - 3):
        r0, r1 = b0 * bs, (b0 + 3) * bs
        h = dict(rows=r1 - r0, cols=x.cols, block_size=bs, ell_cols=x.ell_cols, row_stride_bytes=x.row_stride_bytes, bits=x.bits,
                 policy=x.policy, block_col_idx=bci[b0:b0 + 3].ravel().copy(), packed=packed[r0:r1].ravel().copy(),
                 scales=x.scales.cpu().numpy(), offsets=x.offsets.cpu().numpy())
        ref, l1 = bell_reference(oracle, h, w_host)
        assert_bell_close(y[r0:r1].cpu().numpy(), ref, l1, wmax, bf16_multiply=True)
    out = torch.empty_like(y)
    cut = (block_rows // 3) * bs
    op.run(x, w, out, row_begin=0, row_end=cut)
    op.run(x, w, out, row_begin=cut, row_end=x.rows)
    assert torch.equal(out, y)
    op.close()


@pytest.mark.parametrize("value_factor,w_factor", [(1.0e-6, 1.0e4), (3.0e5, 1.0e-5), (0.0, 1.0), (1.0, 0.0)])
def test_bell_tensor_kernel_keeps_its_accuracy_over_magnitudes(cuda_device, oracle, value_factor, w_factor):
    """The tensor-core kernel multiplies fp16 operands stored times powers of two found at launch (largest |W|,
    bound of the decoded magnitudes): tiny and huge scales, offsets and W, and all-zero operands, give the same
    relative accuracy."""
    rng = np.random.default_rng(41)
    rows, cols, n, ell_blocks = 4 * 32 + 7, 1000, 256, 5
    h = synth.make_qbell_host(rows, cols, 32, ell_blocks, 0.6, 8, seed=3)
    h["scales"] = (h["scales"] * value_factor).astype(np.float32)
    h["offsets"] = (h["offsets"] * value_factor).astype(np.float32)
    x = ops.QuantizedBell.from_host(h, cuda_device)
    w, w_host = dense(rng, cols, n, torch.bfloat16, cuda_device)
    w = (w.float() * w_factor).to(torch.bfloat16)
    w_host = w.float().cpu().numpy()
    op = ops.PreparedSpmm(capi.PROJECTION_BLOCKED_ELL, rows, cols, n, rows * x.ell_cols, x.bits, x.policy, w.dtype, cuda_device)
    assert op.schedule == "tcgen05_block_rows"
    y = op.run(x, w, torch.full((rows, n), float("nan"), device=cuda_device))
    assert op.status() == 0
    ref, l1 = bell_reference(oracle, h, w_host)
    if value_factor == 0.0 or w_factor == 0.0:
        assert torch.all(y == 0.0)
    else:
        assert_bell_close(y.cpu().numpy(), ref, l1, float(np.abs(w_host).max()), bf16_multiply=True)
