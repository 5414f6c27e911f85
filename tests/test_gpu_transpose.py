"""GPU parity of the gene-side transpose G' = deq(X)^T G, through the C ABI."""
import os

import numpy as np
import pytest
import torch

from cellerator_b200 import capi, ops, synth
from conftest import GOLDEN, random_csr
from gpu_util import dense, host_pack, to_dev

pytestmark = pytest.mark.gpu


def assert_transpose_close(got, ref, col_l1, g_abs_max):
    """max|d| <= 1e-4 * (||gene column||_1 * max|G|): the forward bound with the roles of the
    axes exchanged (the sum for gene g runs over the entries of column g)."""
    bound = 1e-4 * col_l1[:, None] * g_abs_max + 1e-30
    err = np.abs(np.asarray(got, dtype=np.float64) - ref)
    assert np.all(err <= bound), f"max excess {np.max(err - bound):.3e}"


def col_l1_of(oracle, c):
    dec = oracle.unpack_csr(c["bits"], c["policy"], c["row_ptr"], c["packed_row_ptr"], c["col_idx"], c["scales"],
                            c["offsets"], c["packed"])
    out = np.zeros(c["cols"])
    np.add.at(out, c["col_idx"], np.abs(dec.astype(np.float64)))
    return out


def test_kat_bwd_rhs_3x3(cuda_device, kats):
    k = kats["csr_3x3"]
    vals = np.array(k["values"], dtype=np.float32)
    x = to_dev(dict(rows=3, cols=3, bits=8, policy=1, row_ptr=np.array(k["major_ptr"]), packed_row_ptr=None,
                    col_idx=np.array(k["minor_idx"]), packed=vals.astype(np.uint8), scales=None, offsets=None),
               cuda_device)
    g = torch.tensor(k["grad_out"], dtype=torch.float32, device=cuda_device).reshape(3, 2)
    out = ops.spmm_transpose(x, g)
    assert out.cpu().numpy().ravel().tolist() == k["bwd_rhs"]


@pytest.mark.parametrize("name", ["csr8_small", "csr4_small"])
def test_golden_transpose(cuda_device, oracle, name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    c = dict(rows=int(z["rows"]), cols=int(z["cols"]), bits=int(z["bits"]), policy=1, row_ptr=z["row_ptr"],
             packed_row_ptr=z["packed_row_ptr"], col_idx=z["col_idx"], packed=z["packed"], scales=z["scales"],
             offsets=z["offsets"])
    x = to_dev(c, cuda_device)
    g = torch.from_numpy(z["g"]).to(cuda_device)
    out = ops.spmm_transpose(x, g).cpu().numpy()
    assert_transpose_close(out, z["gt"], col_l1_of(oracle, c), float(np.abs(z["g"]).max()))


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("n", [1, 3, 8, 16, 32, 64, 128, 24])
def test_random_transpose(cuda_device, oracle, bits, n):
    rng = np.random.default_rng(77 * bits + n)
    policy = 1 + (n % 16 == 0)
    c = host_pack(oracle, random_csr(rng, rows=120, cols=257, max_nnz=150, bits=bits, policy=policy))
    x = to_dev(c, cuda_device)
    g, g_host = dense(rng, c["rows"], n, torch.float32, cuda_device, std=1.0)
    ref = oracle.qcsr_transpose(bits, policy, c["row_ptr"], c["packed_row_ptr"], c["col_idx"], c["packed"],
                                c["scales"], c["offsets"], g_host, c["cols"])
    cl1 = col_l1_of(oracle, c)
    gmax = float(np.abs(g_host).max())
    out = ops.spmm_transpose(x, g).cpu().numpy()
    assert_transpose_close(out, ref, cl1, gmax)
    # alpha / beta, with a destination that must be honoured
    init = torch.from_numpy(rng.normal(size=(c["cols"], n)).astype(np.float32)).to(cuda_device)
    out2 = ops.spmm_transpose(x, g, out=init.clone(), alpha=2.0, beta=0.5).cpu().numpy()
    assert np.allclose(out2, 2.0 * ref + 0.5 * init.cpu().numpy(), rtol=1e-4, atol=1e-4 * gmax * (cl1.max() + 1))
    # beta == 0 never reads the destination
    nan_out = torch.full((c["cols"], n), float("nan"), device=cuda_device)
    assert np.isfinite(ops.spmm_transpose(x, g, out=nan_out).cpu().numpy()).all()


def test_row_shards_sum_to_whole(cuda_device, oracle):
    """The multi-GPU rule: per-shard partials over the uniform row partition add up to the
    whole-matrix result (what the allreduce computes)."""
    rng = np.random.default_rng(12)
    c = host_pack(oracle, random_csr(rng, rows=301, cols=190, max_nnz=120, bits=8, policy=1))
    x = to_dev(c, cuda_device)
    g, g_host = dense(rng, c["rows"], 64, torch.float32, cuda_device, std=1.0)
    whole = ops.spmm_transpose(x, g)
    ref = oracle.qcsr_transpose(8, 1, c["row_ptr"], c["packed_row_ptr"], c["col_idx"], c["packed"], c["scales"],
                                c["offsets"], g_host, c["cols"])
    for parts in (2, 4, 8):
        brp = ops.partition_rows(c["rows"], parts)
        total = torch.zeros_like(whole)
        for p in range(parts):
            r0, r1 = int(brp[p]), int(brp[p + 1])
            if r0 == r1:
                continue
            part = ops.spmm_transpose(x, g, row_begin=r0, row_end=r1)
            pref = oracle.qcsr_transpose(8, 1, c["row_ptr"], c["packed_row_ptr"], c["col_idx"], c["packed"],
                                         c["scales"], c["offsets"], g_host, c["cols"], r0, r1)
            assert np.allclose(part.cpu().numpy(), pref, rtol=1e-4, atol=1e-3)
            total += part
        assert torch.allclose(total, whole, rtol=1e-4, atol=1e-3)
    assert_transpose_close(whole.cpu().numpy(), ref, col_l1_of(oracle, c), float(np.abs(g_host).max()))


def test_transpose_rejects_deterministic_and_bf16(cuda_device):
    with pytest.raises(capi.Cb200Error) as e:
        ops.PreparedSpmm(capi.PROJECTION_TRANSPOSE, 8, 8, 8, 8, 8, 1, torch.float32, cuda_device, deterministic=True)
    assert e.value.status == capi.UNSUPPORTED
    with pytest.raises(capi.Cb200Error):
        ops.PreparedSpmm(capi.PROJECTION_TRANSPOSE, 8, 8, 8, 8, 8, 1, torch.bfloat16, cuda_device)


def assert_tensor_transpose_close(got, ref, col_l1, g_abs_max):
    """bf16 products: decoded values and G both rounded to bf16 (2^-9 each), fp32 accumulation:
    1e-2 relative to ||gene column||_1 * max|G|, the benchmark contract's bf16 tolerance."""
    err = np.abs(np.asarray(got, dtype=np.float64) - ref)
    scale = col_l1[:, None] * g_abs_max + 1e-30
    assert np.all(err <= 1e-2 * scale), f"max err/scale {np.max(err / scale):.3e}"
    assert np.median(err / scale) < 2e-3


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("n", [32, 64])
@pytest.mark.parametrize("policy", [1, 2])
def test_tensor_transpose_parity(cuda_device, oracle, monkeypatch, bits, n, policy):
    """The tcgen05 schedule over the window-blocked copy, forced on a small matrix: several row
    groups, more than one set of eight gene windows with a ragged last set and a ragged last window,
    row ranges (rows outside the range contribute nothing), alpha / beta."""
    monkeypatch.setitem(ops.SCHEDULE_REQUEST, capi.PROJECTION_TRANSPOSE, "tensor_blocked")
    rng = np.random.default_rng(91 * bits + n + policy)
    rows, cols = 256 * 5, 1300
    c = host_pack(oracle, random_csr(rng, rows=rows, cols=cols, max_nnz=200, bits=bits, policy=policy))
    x = to_dev(c, cuda_device)
    g, g_host = dense(rng, rows, n, torch.float32, cuda_device, std=1.0)
    op = ops.PreparedSpmm(capi.PROJECTION_TRANSPOSE, rows, cols, n, x.nnz, bits, policy, g.dtype, cuda_device,
                          multiply=capi.DTYPE_BF16, device_matrix=x)
    assert op.schedule == "tensor_blocked"
    out = op.run(x, g, torch.full((cols, n), float("nan"), device=cuda_device))
    torch.cuda.synchronize()
    assert int(op.workspace[:4].view(torch.int32).item()) == 0          # no bounded wait ran out
    ref = oracle.qcsr_transpose(bits, policy, c["row_ptr"], c["packed_row_ptr"], c["col_idx"], c["packed"],
                                c["scales"], c["offsets"], g_host, cols)
    cl1 = col_l1_of(oracle, c)
    gmax = float(np.abs(g_host).max())
    assert_tensor_transpose_close(out.cpu().numpy(), ref, cl1, gmax)
    # a row range that starts and ends inside groups
    r0, r1 = 300, 1000
    part = op.run(x, g, torch.empty(cols, n, device=cuda_device), row_begin=r0, row_end=r1)
    pref = oracle.qcsr_transpose(bits, policy, c["row_ptr"], c["packed_row_ptr"], c["col_idx"], c["packed"],
                                 c["scales"], c["offsets"], g_host, cols, r0, r1)
    assert_tensor_transpose_close(part.cpu().numpy(), pref, cl1, gmax)
    # alpha / beta
    init = torch.from_numpy(rng.normal(size=(cols, n)).astype(np.float32)).to(cuda_device)
    out2 = op.run(x, g, init.clone(), alpha=2.0, beta=0.5).cpu().numpy()
    assert np.allclose(out2, 2.0 * out.cpu().numpy() + 0.5 * init.cpu().numpy(), rtol=1e-4, atol=1e-4 * gmax * (cl1.max() + 1))
    # without the opt-in the exact kernel runs
    exact = ops.PreparedSpmm(capi.PROJECTION_TRANSPOSE, rows, cols, n, x.nnz, bits, policy, g.dtype, cuda_device)
    assert exact.schedule == "vector_reductions"
    assert_transpose_close(exact.run(x, g, torch.empty(cols, n, device=cuda_device)).cpu().numpy(), ref, cl1, gmax)
    op.close()
    exact.close()


def test_tensor_transpose_full_scale(cuda_device):
    """Genes as in the benchmark configuration, 1/8 of its cells: the tensor schedule against the
    exact kernel on every gene, and the shard rule (partials of row halves add up)."""
    cfg = dict(synth.CONFIGS["c2_forward"])
    cfg["rows"] //= 8
    x = synth.make_qcsr_device(**cfg, device=cuda_device, seed=0)
    n = 64
    g = torch.randn(x.rows, n, device=cuda_device)
    op = ops.PreparedSpmm(capi.PROJECTION_TRANSPOSE, x.rows, x.cols, n, x.nnz, x.bits, x.policy, g.dtype, cuda_device,
                          multiply=capi.DTYPE_BF16, device_matrix=x)
    assert op.schedule == "tensor_blocked"
    out = op.run(x, g, torch.empty(x.cols, n, device=cuda_device))
    torch.cuda.synchronize()
    assert int(op.workspace[:4].view(torch.int32).item()) == 0
    exact = ops.spmm_transpose(x, g)
    vals = x.dequantize().abs().double()
    col_l1 = torch.zeros(x.cols, dtype=torch.float64, device=cuda_device).index_add_(0, x.col_idx.long(), vals)
    del vals
    gmax = float(g.abs().max())
    assert torch.all((out - exact).abs() <= 1e-2 * (col_l1[:, None] * gmax).float() + 1e-30)
    for _ in range(3):      # every CTA's sums go to a slot of their own and are added in a fixed order: the same bits every time
        assert torch.equal(op.run(x, g, torch.empty(x.cols, n, device=cuda_device)), out)
    half = (x.rows // 2 // 256) * 256 + 77
    a = op.run(x, g, torch.empty(x.cols, n, device=cuda_device), row_begin=0, row_end=half)
    b = op.run(x, g, a, row_begin=half, row_end=x.rows, beta=1.0)
    assert torch.allclose(b, out, rtol=1e-3, atol=1e-3 * gmax)
    op.close()


@pytest.mark.parametrize("bits,policy", [(8, 1), (4, 2)])
def test_tensor_transpose_split_products_meet_the_fp32_bound(cuda_device, oracle, monkeypatch, bits, policy):
    """fp32 products requested and the matrix handed to prepare: three bf16 passes (hi*hi + hi*lo +
    lo*hi) rebuild each product; the result meets the fp32 bound 1e-4 * ||gene column||_1 * max|G|
    with a wide margin, also on a row range and with alpha / beta."""
    monkeypatch.setitem(ops.SCHEDULE_REQUEST, capi.PROJECTION_TRANSPOSE, "tensor_blocked")
    rng = np.random.default_rng(17 * bits + policy)
    rows, cols, n = 256 * 4, 1100, 64
    c = host_pack(oracle, random_csr(rng, rows=rows, cols=cols, max_nnz=220, bits=bits, policy=policy))
    x = to_dev(c, cuda_device)
    g, g_host = dense(rng, rows, n, torch.float32, cuda_device, std=1.0)
    op = ops.PreparedSpmm(capi.PROJECTION_TRANSPOSE, rows, cols, n, x.nnz, bits, policy, g.dtype, cuda_device,
                          device_matrix=x)
    assert op.schedule == "tensor_blocked_x3"
    out = op.run(x, g, torch.full((cols, n), float("nan"), device=cuda_device))
    torch.cuda.synchronize()
    assert int(op.workspace[:4].view(torch.int32).item()) == 0
    ref = oracle.qcsr_transpose(bits, policy, c["row_ptr"], c["packed_row_ptr"], c["col_idx"], c["packed"],
                                c["scales"], c["offsets"], g_host, cols)
    cl1 = col_l1_of(oracle, c)
    gmax = float(np.abs(g_host).max())
    assert_transpose_close(out.cpu().numpy(), ref, cl1, gmax)
    err = np.abs(out.cpu().numpy().astype(np.float64) - ref) / (cl1[:, None] * gmax + 1e-30)
    assert err.max() < 3e-5                                             # ~3 * 2^-17 per product, fp32 sums
    part = op.run(x, g, torch.empty(cols, n, device=cuda_device), row_begin=130, row_end=777)
    pref = oracle.qcsr_transpose(bits, policy, c["row_ptr"], c["packed_row_ptr"], c["col_idx"], c["packed"],
                                 c["scales"], c["offsets"], g_host, cols, 130, 777)
    assert_transpose_close(part.cpu().numpy(), pref, cl1, gmax)
    init = torch.from_numpy(rng.normal(size=(cols, n)).astype(np.float32)).to(cuda_device)
    out2 = op.run(x, g, init.clone(), alpha=2.0, beta=0.5).cpu().numpy()
    assert np.allclose(out2, 2.0 * ref + 0.5 * init.cpu().numpy(), rtol=1e-4, atol=1e-4 * gmax * (cl1.max() + 1))
    op.close()


def test_tensor_transpose_respects_the_memory_limit(cuda_device, oracle, monkeypatch):
    """persistent_limit_bytes with room for one word per entry but not two: the split passes decode
    the code words at launch and still meet the fp32 bound; below one word per entry the exact
    kernel runs.  The limit is prepare_policy.persistent_memory_limit of the reference."""
    monkeypatch.setitem(ops.SCHEDULE_REQUEST, capi.PROJECTION_TRANSPOSE, "tensor_blocked")
    rng = np.random.default_rng(91)
    rows, cols, n = 256 * 3, 900, 64
    c = host_pack(oracle, random_csr(rng, rows=rows, cols=cols, max_nnz=200, bits=8, policy=1))
    x = to_dev(c, cuda_device)
    g, g_host = dense(rng, rows, n, torch.float32, cuda_device, std=1.0)
    ref = oracle.qcsr_transpose(8, 1, c["row_ptr"], c["packed_row_ptr"], c["col_idx"], c["packed"],
                                c["scales"], c["offsets"], g_host, cols)
    cl1 = col_l1_of(oracle, c)
    gmax = float(np.abs(g_host).max())
    one_word = ops.PreparedSpmm(capi.PROJECTION_TRANSPOSE, rows, cols, n, x.nnz, 8, 1, g.dtype, cuda_device,
                                device_matrix=x, persistent_limit_bytes=6 * x.nnz)
    assert one_word.schedule == "tensor_blocked_x3"
    out = one_word.run(x, g, torch.full((cols, n), float("nan"), device=cuda_device))
    torch.cuda.synchronize()
    assert int(one_word.workspace[:4].view(torch.int32).item()) == 0
    assert_transpose_close(out.cpu().numpy(), ref, cl1, gmax)
    one_word.close()
    none = ops.PreparedSpmm(capi.PROJECTION_TRANSPOSE, rows, cols, n, x.nnz, 8, 1, g.dtype, cuda_device,
                            device_matrix=x, persistent_limit_bytes=2 * x.nnz)
    assert none.schedule == "vector_reductions"
    out = none.run(x, g, torch.full((cols, n), float("nan"), device=cuda_device))
    assert_transpose_close(out.cpu().numpy(), ref, cl1, gmax)
    none.close()


def _row_range_on_host(x, r0, r1):
    """Rows [r0, r1) of a device matrix as a host matrix of its own (offsets rebased to 0)."""
    rp = x.host_row_ptr
    lo, hi = int(rp[r0]), int(rp[r1])
    sub = dict(rows=r1 - r0, cols=x.cols, bits=x.bits, policy=x.policy, row_ptr=rp[r0:r1 + 1] - lo,
               col_idx=x.col_idx[lo:hi].cpu().numpy(), scales=x.scales.cpu().numpy(), offsets=x.offsets.cpu().numpy())
    if x.bits == 8:
        sub["packed"], sub["packed_row_ptr"] = x.packed[lo:hi].cpu().numpy(), sub["row_ptr"]
    else:
        prp = x.packed_row_ptr[r0:r1 + 1].cpu().numpy()
        sub["packed"], sub["packed_row_ptr"] = x.packed[int(prp[0]):int(prp[-1])].cpu().numpy(), prp - prp[0]
    return sub


def test_deterministic_request_may_name_the_tensor_schedule(cuda_device, oracle, monkeypatch):
    """deterministic = 1 selects the gather schedule by default and the tensor-core schedule when the request names it:
    both give the same bits on every run (the tensor kernel's CTAs write their sums to slots of their own, which a
    second kernel adds in a fixed order), both inside the fp32 bound."""
    rng = np.random.default_rng(12)
    rows, cols, n = 256 * 40 + 19, 128 * 9 + 30, 64
    c = host_pack(oracle, random_csr(rng, rows=rows, cols=cols, max_nnz=150, bits=8, policy=1))
    x = to_dev(c, cuda_device)
    g = torch.randn(rows, n, device=cuda_device)
    ref = oracle.qcsr_transpose(8, 1, c["row_ptr"], c["packed_row_ptr"], c["col_idx"], c["packed"], c["scales"], c["offsets"],
                                g.cpu().numpy(), cols)
    cl1 = col_l1_of(oracle, c)
    gmax = float(g.abs().max())
    for hint, expected in ((None, "gene_gather"), ("tensor_blocked", "tensor_blocked_x3")):
        monkeypatch.setitem(ops.SCHEDULE_REQUEST, capi.PROJECTION_TRANSPOSE, hint)
        op = ops.PreparedSpmm(capi.PROJECTION_TRANSPOSE, rows, cols, n, x.nnz, 8, 1, g.dtype, cuda_device, deterministic=True,
                              device_matrix=x)
        assert op.schedule == expected
        first = op.run(x, g, torch.empty(cols, n, device=cuda_device))
        assert op.status() == 0
        for _ in range(4):
            assert torch.equal(op.run(x, g, torch.empty(cols, n, device=cuda_device)), first)
        assert_transpose_close(first.cpu().numpy(), ref, cl1, gmax)
        op.close()


@pytest.mark.parametrize("schedule", ["tensor_blocked_x3", "tensor_blocked", "gene_gather", "vector_reductions"])
def test_transpose_schedules_against_the_oracle_at_scale(cuda_device, oracle, schedule):
    """Genes as in the benchmark configuration, 1/8 of its cells, the schedule prepare chooses for each kind of
    request: row-range partials over 2,048 cells at the start and in the middle of the matrix against the
    oracle's double-precision partial of the same rows: 1e-4 * ||gene column||_1 * max|G| for fp32 products
    (exact, split, ordered), 1e-2 for the single bf16 pass."""
    cfg = dict(synth.CONFIGS["c2_forward"])
    cfg["rows"] //= 8
    x = synth.make_qcsr_device(**cfg, device=cuda_device, seed=0)
    n = 64
    g = torch.randn(x.rows, n, device=cuda_device)
    kw = {"tensor_blocked_x3": dict(device_matrix=x), "tensor_blocked": dict(device_matrix=x, multiply=capi.DTYPE_BF16),
          "gene_gather": dict(device_matrix=x, deterministic=True), "vector_reductions": {}}[schedule]
    op = ops.PreparedSpmm(capi.PROJECTION_TRANSPOSE, x.rows, x.cols, n, x.nnz, x.bits, x.policy, g.dtype, cuda_device, **kw)
    assert op.schedule == schedule
    mid = x.rows // 2 + 77                                         # inside a 256-row group
    for r0 in (0, mid):
        r1 = r0 + 2048
        part = op.run(x, g, torch.full((x.cols, n), float("nan"), device=cuda_device), row_begin=r0, row_end=r1)
        assert op.status() == 0
        sub = _row_range_on_host(x, r0, r1)
        g_host = g[r0:r1].cpu().numpy()
        ref = oracle.qcsr_transpose(sub["bits"], sub["policy"], sub["row_ptr"], sub["packed_row_ptr"], sub["col_idx"], sub["packed"],
                                    sub["scales"], sub["offsets"], g_host, x.cols)
        cl1 = col_l1_of(oracle, sub)
        gmax = float(np.abs(g_host).max())
        got = part.cpu().numpy()
        if schedule == "tensor_blocked":
            assert_tensor_transpose_close(got, ref, cl1, gmax)
        else:
            assert_transpose_close(got, ref, cl1, gmax)
        worst = np.max(np.abs(got.astype(np.float64) - ref) / (cl1[:, None] * gmax + 1e-30))
        print(f"{schedule} rows [{r0},{r1}): max |d| / (||column||_1 max|G|) = {worst:.3e}")
    if schedule in ("tensor_blocked_x3", "tensor_blocked", "gene_gather"):      # fixed summation order: repeatable to the bit
        whole = op.run(x, g, torch.empty(x.cols, n, device=cuda_device))
        for _ in range(2):
            assert torch.equal(op.run(x, g, torch.empty(x.cols, n, device=cuda_device)), whole)
    op.close()
