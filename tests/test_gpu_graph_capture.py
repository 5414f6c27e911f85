"""cb200_spmm_run under CUDA stream capture: every schedule the candidates offer with
candidate_graph_capture (operation_core.hh:63-68) is recorded into a graph -- a launch enqueues
kernels and memsets only -- and a replay into a cleared output gives the eager result (the same bits
for the schedules with a fixed summation order, the contract's bound for the atomic ones)."""
import numpy as np
import pytest
import torch

from cellerator_b200 import capi, ops, synth
from conftest import random_csr
from gpu_util import dense, host_pack, to_dev

pytestmark = pytest.mark.gpu


def capture_and_replay(op, x, d, out, stream, **kw):
    """eager run on `stream`, capture of the same launch, replay into a poisoned output"""
    with torch.cuda.stream(stream):
        launch = op.make_launch(x, d, out, **kw)
        op.run_launch(launch)               # also sets the kernels' one-time attributes outside the capture
        stream.synchronize()
        eager = out.clone()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            op.run_launch(launch)
        out.fill_(float("nan"))
        graph.replay()
        stream.synchronize()
        first = out.clone()
        out.fill_(float("nan"))
        graph.replay()
        stream.synchronize()
    return eager, first, out.clone()


@pytest.mark.parametrize("schedule,multiply", [("warp_per_row", 0), ("gene_tiled", 0), ("tensor_blocked", capi.DTYPE_BF16)])
def test_forward_schedules_are_capturable(cuda_device, oracle, monkeypatch, schedule, multiply):
    monkeypatch.setitem(ops.SCHEDULE_REQUEST, capi.PROJECTION_CSR, schedule)
    rng = np.random.default_rng(len(schedule))
    rows, cols, n = 256 * 20, 700, 64
    c = host_pack(oracle, random_csr(rng, rows=rows, cols=cols, max_nnz=90, bits=8))
    x = to_dev(c, cuda_device)
    w, _ = dense(rng, cols, n, torch.bfloat16, cuda_device)
    op = ops.PreparedSpmm(capi.PROJECTION_CSR, rows, cols, n, x.nnz, 8, 1, w.dtype, cuda_device, host_row_ptr=c["row_ptr"],
                          multiply=multiply, device_matrix=x if multiply else None)
    assert op.schedule == schedule
    stream = torch.cuda.Stream(cuda_device)
    eager, first, second = capture_and_replay(op, x, w, torch.empty(rows, n, device=cuda_device), stream)
    assert torch.equal(eager.view(torch.int32), first.view(torch.int32))   # a row has one owner: fixed order
    assert torch.equal(first.view(torch.int32), second.view(torch.int32))
    op.close()


@pytest.mark.parametrize("mode", ["vector_reductions", "tensor_blocked", "gene_gather"])
def test_transpose_schedules_are_capturable(cuda_device, oracle, monkeypatch, mode):
    if mode == "tensor_blocked":
        monkeypatch.setitem(ops.SCHEDULE_REQUEST, capi.PROJECTION_TRANSPOSE, "tensor_blocked")
    rng = np.random.default_rng(len(mode))
    rows, cols, n = 256 * 6, 500, 64
    c = host_pack(oracle, random_csr(rng, rows=rows, cols=cols, max_nnz=80, bits=8))
    x = to_dev(c, cuda_device)
    g, _ = dense(rng, rows, n, torch.float32, cuda_device, std=1.0)
    op = ops.PreparedSpmm(capi.PROJECTION_TRANSPOSE, rows, cols, n, x.nnz, 8, 1, g.dtype, cuda_device,
                          multiply=capi.DTYPE_BF16 if mode == "tensor_blocked" else 0,
                          device_matrix=None if mode == "vector_reductions" else x, deterministic=mode == "gene_gather")
    assert op.schedule == mode
    stream = torch.cuda.Stream(cuda_device)
    eager, first, second = capture_and_replay(op, x, g, torch.empty(cols, n, device=cuda_device), stream)
    if mode == "gene_gather":
        assert torch.equal(eager.view(torch.int32), first.view(torch.int32))
        assert torch.equal(first.view(torch.int32), second.view(torch.int32))
    else:                                   # atomic order: equal up to the reassociation of fp32 sums
        scale = float(eager.abs().max())
        assert torch.allclose(eager, first, rtol=0, atol=1e-4 * scale) and torch.allclose(first, second, rtol=0, atol=1e-4 * scale)
    op.close()


def test_blocked_ell_is_capturable(cuda_device):
    cfg = dict(synth.CONFIGS["c5_bell"])
    cfg["rows"] = 32 * 64
    x = synth.make_qbell_device(**cfg, device=cuda_device, seed=4)
    n = cfg["n"]
    w = (torch.randn(cfg["cols"], n, device=cuda_device) * 0.02).to(torch.bfloat16)
    op = ops.PreparedSpmm(capi.PROJECTION_BLOCKED_ELL, x.rows, cfg["cols"], n, x.rows * x.ell_cols, x.bits, x.policy, w.dtype,
                          cuda_device)
    stream = torch.cuda.Stream(cuda_device)
    eager, first, second = capture_and_replay(op, x, w, torch.empty(x.rows, n, device=cuda_device), stream)
    assert torch.equal(eager.view(torch.int32), first.view(torch.int32))
    assert torch.equal(first.view(torch.int32), second.view(torch.int32))
    op.close()
