"""The N > 1 host logic on CPU ranks (gloo, world_size 2 and 4): the uniform row partition gives
every rank a contiguous cell range; forward needs no collective (the ranks' Y rows tile the whole
Y exactly); the transpose partials, summed by an all-reduce, equal the whole-matrix result.  The
per-rank compute is done by the oracle here; on GPUs the same ranges go to cb200_spmm_run."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle as orc
        from cellerator_b200 import ops, synth
        checker = orc.Oracle()
        h = synth.make_qcsr_host(rows=203, cols=300, median=40, sigma=0.7, lo=0, hi=200, bits=8, seed=5)
        rng = np.random.default_rng(6)
        w = rng.normal(0, 0.02, size=(300, 16)).astype(np.float32)
        g = rng.normal(0, 1.0, size=(203, 16)).astype(np.float32)
        brp = ops.partition_rows(h["rows"], world)
        r0, r1 = int(brp[rank]), int(brp[rank + 1])
        blk = ops.get_block(h["row_ptr"], h["packed_row_ptr"], brp, rank)
        assert (blk["row_begin"], blk["row_end"]) == (r0, r1)
        assert blk["nnz_begin"] == int(h["row_ptr"][r0]) and blk["nnz_end"] == int(h["row_ptr"][r1])
        args = (8, 1, h["row_ptr"], h["packed_row_ptr"], h["col_idx"], h["packed"], h["scales"], h["offsets"])
        # forward: my rows only, no collective on the data path
        y_mine = checker.qcsr_forward(*args, w, 300, r0, r1)
        full = torch.zeros(h["rows"], 16, dtype=torch.float64)
        full[r0:r1] = torch.from_numpy(y_mine)
        dist.all_reduce(full)                     # test-side assembly only
        # transpose: partial over my rows, then the all-reduce the GPU path issues
        part = torch.from_numpy(checker.qcsr_transpose(*args, g, 300, r0, r1))
        dist.all_reduce(part, op=dist.ReduceOp.SUM)
        if rank == 0:
            y_ref = checker.qcsr_forward(*args, w, 300)
            gt_ref = checker.qcsr_transpose(*args, g, 300)
            np.save(os.path.join(result_dir, "fwd_ok.npy"), np.array([np.array_equal(full.numpy(), y_ref)]))
            np.save(os.path.join(result_dir, "tr_err.npy"), np.array([np.abs(part.numpy() - gt_ref).max()]))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_row_sharding_and_allreduce_on_cpu_ranks(tmp_path, world):
    port = _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert bool(np.load(tmp_path / "fwd_ok.npy")[0])          # forward shards tile Y bit-exactly
    assert float(np.load(tmp_path / "tr_err.npy")[0]) < 1e-9   # double sums regrouped by shard


def test_empty_trailing_shards():
    from cellerator_b200 import ops
    brp = ops.partition_rows(5, 8)                              # more ranks than row blocks
    assert brp.tolist() == [0, 1, 2, 3, 4, 5, 5, 5, 5]
    assert ops.partition_rows(0, 2).tolist() == [0, 0, 0]
