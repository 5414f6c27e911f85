"""GPU parity of the fused dequant-SpMM forward path, through the C ABI, against the oracle."""
import os

import numpy as np
import pytest
import torch

from cellerator_b200 import capi, ops, synth
from conftest import GOLDEN, random_csr
from gpu_util import assert_forward_close, dense, host_pack, row_l1, to_dev

pytestmark = pytest.mark.gpu


def test_kat_csr_3x3(cuda_device, kats):
    k = kats["csr_3x3"]
    vals = np.array(k["values"], dtype=np.float32)
    h = dict(rows=3, cols=3, bits=8, policy=1, row_ptr=np.array(k["major_ptr"]), packed_row_ptr=None,
             col_idx=np.array(k["minor_idx"]), packed=vals.astype(np.uint8), scales=None, offsets=None)
    x = to_dev(h, cuda_device)
    w = torch.tensor(k["rhs"], dtype=torch.float32, device=cuda_device).reshape(3, 2)
    y = ops.spmm_forward(x, w)
    assert y.cpu().numpy().ravel().tolist() == k["spmm_fwd"]


@pytest.mark.parametrize("name", ["csr8_small", "csr4_small"])
def test_golden_forward(cuda_device, oracle, name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    h = dict(rows=int(z["rows"]), cols=int(z["cols"]), bits=int(z["bits"]), policy=1, row_ptr=z["row_ptr"],
             packed_row_ptr=z["packed_row_ptr"], col_idx=z["col_idx"], packed=z["packed"], scales=z["scales"],
             offsets=z["offsets"])
    x = to_dev(h, cuda_device)
    w = torch.from_numpy(z["w"]).to(cuda_device)
    y = ops.spmm_forward(x, w).cpu().numpy()
    l1, _ = row_l1(oracle, h)
    assert_forward_close(y, z["y"], l1, float(np.abs(z["w"]).max()))


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n", [1, 2, 8, 16, 24, 32, 40, 64, 128, 256])
def test_random_forward_all_widths(cuda_device, oracle, bits, dtype, n):
    rng = np.random.default_rng(1000 * bits + n)
    policy = 1 + (n % 3 == 0)
    c = host_pack(oracle, random_csr(rng, rows=83, cols=700, max_nnz=260, bits=bits, policy=policy))
    x = to_dev(c, cuda_device)
    w, w_host = dense(rng, c["cols"], n, dtype, cuda_device, ld=n + (8 if n % 16 == 0 else 0))
    y = ops.spmm_forward(x, w).cpu().numpy()
    ref = oracle.qcsr_forward(bits, policy, c["row_ptr"], c["packed_row_ptr"], c["col_idx"], c["packed"], c["scales"],
                              c["offsets"], w_host, c["cols"])
    l1, _ = row_l1(oracle, c)
    assert_forward_close(y, ref, l1, float(np.abs(w_host).max()), bf16=dtype == torch.bfloat16)


def test_edge_rows_alpha_beta_and_ranges(cuda_device, oracle):
    rng = np.random.default_rng(5)
    rows, cols, n = 64, 333, 64
    counts = np.array([0, 1, 31, 32, 33, 63, 64, 65, 0, 0, 200, 1] + [int(v) for v in rng.integers(0, 120, rows - 12)])
    row_ptr = np.concatenate([[0], np.cumsum(counts)]).astype(np.int64)
    col = np.concatenate([np.sort(rng.choice(cols, size=int(k), replace=False)) for k in counts]).astype(np.int32)
    c = dict(rows=rows, cols=cols, bits=8, policy=1, row_ptr=row_ptr, col_idx=col,
             scales=rng.uniform(0.01, 0.3, cols).astype(np.float32), offsets=rng.uniform(-1, 1, cols).astype(np.float32),
             values=rng.uniform(0, 30, len(col)).astype(np.float32))
    c = host_pack(oracle, c)
    x = to_dev(c, cuda_device)
    w, w_host = dense(rng, cols, n, torch.bfloat16, cuda_device)
    ref = oracle.qcsr_forward(8, 1, row_ptr, c["packed_row_ptr"], col, c["packed"], c["scales"], c["offsets"], w_host, cols)
    l1, _ = row_l1(oracle, c)
    wmax = float(np.abs(w_host).max())
    y = ops.spmm_forward(x, w).cpu().numpy()
    assert_forward_close(y, ref, l1, wmax, bf16=True)
    assert np.all(y[counts == 0] == 0.0)                                   # empty rows write exact zeros
    # alpha / beta
    y0 = torch.from_numpy(rng.normal(size=(rows, n)).astype(np.float32)).to(cuda_device)
    y1 = ops.spmm_forward(x, w, out=y0.clone(), alpha=0.5, beta=-2.0).cpu().numpy()
    assert np.allclose(y1, 0.5 * ref - 2.0 * y0.cpu().numpy(), rtol=1e-5, atol=1e-5 * wmax * (l1.max() + 1))
    # beta == 0 must not read the output (NaN-filled destination)
    nan_out = torch.full((rows, n), float("nan"), device=cuda_device)
    assert np.array_equal(ops.spmm_forward(x, w, out=nan_out).cpu().numpy(), y)
    # row ranges: only the rows of the range are written, bit-identical to the full run
    op = ops.PreparedSpmm(capi.PROJECTION_CSR, rows, cols, n, x.nnz, 8, 1, w.dtype, cuda_device)
    out = torch.full((rows, n), -7.0, device=cuda_device)
    op.run(x, w, out, row_begin=10, row_end=37)
    got = out.cpu().numpy()
    assert np.array_equal(got[10:37], y[10:37]) and np.all(got[:10] == -7.0) and np.all(got[37:] == -7.0)
    op.run(x, w, out, row_begin=20, row_end=20)                             # empty range: no-op
    assert np.array_equal(out.cpu().numpy(), got)


def test_config1_full_parity_and_determinism(cuda_device, oracle):
    """Configuration 1: 20,000 x 2,000, N = 32, fp32 W, against the oracle on every row."""
    cfg = synth.CONFIGS["c1_cpu_ref"]
    h = synth.make_qcsr_host(**cfg, seed=0)
    x = to_dev(h, cuda_device)
    w_host = np.random.default_rng(1000).normal(0.0, 0.02, size=(cfg["cols"], cfg["n"])).astype(np.float32)
    w = torch.from_numpy(w_host).to(cuda_device)
    y = ops.spmm_forward(x, w)
    ref = oracle.qcsr_forward(8, 1, h["row_ptr"], h["packed_row_ptr"], h["col_idx"], h["packed"], h["scales"],
                              h["offsets"], w_host, cfg["cols"])
    l1, _ = row_l1(oracle, h)
    assert_forward_close(y.cpu().numpy(), ref, l1, float(np.abs(w_host).max()))
    z = np.load(os.path.join(GOLDEN, "c1_summary.npz"))
    if int(z["nnz"]) == len(h["col_idx"]):
        assert_forward_close(y[:64].cpu().numpy(), z["y_head"], l1[:64], float(np.abs(w_host).max()))
    y2 = ops.spmm_forward(x, w)
    assert torch.equal(y, y2)                                               # advertised as deterministic
    assert oracle.digest_f32(y.cpu().numpy()) == oracle.digest_f32(y2.cpu().numpy())


@pytest.mark.parametrize("bits,n", [(8, 64), (4, 128)])
def test_full_scale_properties(cuda_device, oracle, bits, n):
    """A large device-generated matrix (genes as in the benchmark configuration, 1/8 of its
    cells): sampled rows against the oracle, linearity in W, and row-partition invariance."""
    cfg = dict(synth.CONFIGS["c2_forward" if bits == 8 else "c4_4bit"])
    cfg["rows"] //= 8
    x = synth.make_qcsr_device(**{**cfg, "bits": bits}, device=cuda_device, seed=0)
    rng = np.random.default_rng(9)
    w1, _ = dense(rng, x.cols, n, torch.bfloat16, cuda_device)
    w2, _ = dense(rng, x.cols, n, torch.bfloat16, cuda_device)
    op = ops.PreparedSpmm(capi.PROJECTION_CSR, x.rows, x.cols, n, x.nnz, bits, x.policy, w1.dtype, cuda_device,
                          host_row_ptr=x.host_row_ptr)
    y1 = op.run(x, w1, torch.empty(x.rows, n, device=cuda_device))
    # linearity: Y(W1) + Y(W2) == Y computed with beta accumulation
    y12 = op.run(x, w2, y1.clone(), beta=1.0)
    y2 = op.run(x, w2, torch.empty(x.rows, n, device=cuda_device))
    assert torch.allclose(y12, y1 + y2, rtol=1e-5, atol=1e-5)
    # row-partition invariance (1/2/4/8 shards): bit-identical to the single launch
    for parts in (2, 4, 8):
        brp = ops.partition_rows(x.rows, parts)
        out = torch.empty(x.rows, n, device=cuda_device)
        for p in range(parts):
            op.run(x, w1, out, row_begin=int(brp[p]), row_end=int(brp[p + 1]))
        assert torch.equal(out, y1)
    # sampled rows vs the oracle
    rp = x.host_row_ptr
    w_host = w1.float().cpu().numpy()
    for r0 in (0, x.rows // 2 - 3, x.rows - 40):
        r1 = r0 + 40
        lo, hi = int(rp[r0]), int(rp[r1])
        sub = dict(rows=40, cols=x.cols, bits=bits, policy=1, row_ptr=rp[r0:r1 + 1] - lo,
                   col_idx=x.col_idx[lo:hi].cpu().numpy(), scales=x.scales.cpu().numpy(), offsets=x.offsets.cpu().numpy())
        if bits == 8:
            sub["packed"] = x.packed[lo:hi].cpu().numpy()
            sub["packed_row_ptr"] = sub["row_ptr"]
        else:
            prp = x.packed_row_ptr[r0:r1 + 1].cpu().numpy()
            sub["packed"] = x.packed[int(prp[0]):int(prp[-1])].cpu().numpy()
            sub["packed_row_ptr"] = prp - prp[0]
        ref = oracle.qcsr_forward(bits, 1, sub["row_ptr"], sub["packed_row_ptr"], sub["col_idx"], sub["packed"],
                                  sub["scales"], sub["offsets"], w_host, x.cols)
        l1, _ = row_l1(oracle, sub)
        assert_forward_close(y1[r0:r1].cpu().numpy(), ref, l1, float(np.abs(w_host).max()), bf16=True)
        assert np.all(np.diff(sub["col_idx"][: int(sub["row_ptr"][1])]) > 0)   # genes ascending, distinct


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("dtype,n", [(torch.bfloat16, 64), (torch.bfloat16, 128), (torch.bfloat16, 32),
                                     (torch.float32, 32), (torch.float32, 64)])
@pytest.mark.parametrize("policy", [1, 2])
def test_gene_tiled_schedule(cuda_device, oracle, monkeypatch, bits, dtype, n, policy):
    """The shared-memory-staged kernel, forced on a small matrix that still spans several gene
    tiles, several row groups per CTA and a ragged last group; bit-identical across row ranges
    and to a second run, and the bounded-wait status word stays 0."""
    monkeypatch.setitem(ops.SCHEDULE_REQUEST, capi.PROJECTION_CSR, "gene_tiled")
    rng = np.random.default_rng(31 * bits + n + policy)
    rows, cols = 128 * 3 + 37, 4100
    c = host_pack(oracle, random_csr(rng, rows=rows, cols=cols, max_nnz=700, bits=bits, policy=policy))
    x = to_dev(c, cuda_device)
    w, w_host = dense(rng, cols, n, dtype, cuda_device)
    op = ops.PreparedSpmm(capi.PROJECTION_CSR, rows, cols, n, x.nnz, bits, policy, w.dtype, cuda_device,
                          host_row_ptr=x.host_row_ptr)
    assert op.schedule == "gene_tiled"
    y = op.run(x, w, torch.full((rows, n), float("nan"), device=cuda_device))
    assert int(op.workspace[:4].view(torch.int32).item()) == 0
    ref = oracle.qcsr_forward(bits, policy, c["row_ptr"], c["packed_row_ptr"], c["col_idx"], c["packed"], c["scales"],
                              c["offsets"], w_host, cols)
    l1, _ = row_l1(oracle, c)
    assert_forward_close(y.cpu().numpy(), ref, l1, float(np.abs(w_host).max()), bf16=dtype == torch.bfloat16)
    assert torch.equal(y, op.run(x, w, torch.empty_like(y)))
    out = torch.full((rows, n), -3.0, device=cuda_device)
    op.run(x, w, out, row_begin=100, row_end=300)
    assert torch.equal(out[100:300], y[100:300]) and torch.all(out[:100] == -3.0) and torch.all(out[300:] == -3.0)
    y0 = torch.from_numpy(rng.normal(size=(rows, n)).astype(np.float32)).to(cuda_device)
    y1 = op.run(x, w, y0.clone(), alpha=2.0, beta=0.5)
    assert torch.allclose(y1, 2.0 * y + 0.5 * y0, rtol=1e-5, atol=1e-6)
    # the warp-per-row kernel agrees to rounding (different summation order)
    monkeypatch.setitem(ops.SCHEDULE_REQUEST, capi.PROJECTION_CSR, "warp_per_row")
    op2 = ops.PreparedSpmm(capi.PROJECTION_CSR, rows, cols, n, x.nnz, bits, policy, w.dtype, cuda_device)
    assert op2.schedule == "warp_per_row"
    y2 = op2.run(x, w, torch.empty_like(y))
    assert_forward_close(y2.cpu().numpy(), ref, l1, float(np.abs(w_host).max()), bf16=dtype == torch.bfloat16)
