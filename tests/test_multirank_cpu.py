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
        # deterministic transpose: fixed-order fp32 partial over my row range of the gene-major copy,
        # summed by the same all-reduce; a second round repeats every bit
        rc, col_ptr, row_idx, codes = checker.qcsr_gene_major(8, 300, h["row_ptr"], h["packed_row_ptr"], h["col_idx"], h["packed"])
        assert rc == 0
        rounds = []
        for _ in range(2):
            mine = torch.from_numpy(checker.qcsr_transpose_ordered(1, col_ptr, row_idx, codes, h["scales"], h["offsets"], g, r0, r1))
            dist.all_reduce(mine, op=dist.ReduceOp.SUM)
            rounds.append(mine.numpy().copy())
        if rank == 0:
            gt64 = checker.qcsr_transpose(*args, g, 300)
            np.save(os.path.join(result_dir, "ordered.npy"),
                    np.array([float(np.array_equal(rounds[0].view(np.uint32), rounds[1].view(np.uint32))),
                              float(np.abs(rounds[0] - gt64).max() / (np.abs(gt64).max() + 1e-30))]))
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
    same_bits, rel_err = np.load(tmp_path / "ordered.npy")
    assert same_bits == 1.0 and rel_err < 1e-5                 # fixed-order fp32 partials, summed across ranks


def test_empty_trailing_shards():
    from cellerator_b200 import ops
    brp = ops.partition_rows(5, 8)                              # more ranks than row blocks
    assert brp.tolist() == [0, 1, 2, 3, 4, 5, 5, 5, 5]
    assert ops.partition_rows(0, 2).tolist() == [0, 0, 0]


def _lowering_worker(rank, world, port, result_dir):
    """Row-sharded CSR -> Blocked-ELL lowering: shards on block-row boundaries lower on their own; the
    common ELL width is the all-reduce MAX of the shards' widths, and with it the shards' column
    indices and values tile the whole-matrix result."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle as orc
        from cellerator_b200 import synth
        checker = orc.Oracle()
        bs = 16
        h = synth.make_lowering_host(rows=bs * 13 + 5, features=400, feature_blocks=3, mean_nnz=10, seed=2,
                                     value_dtype=np.uint8)
        relaxed = dict(max_value_expansion=1e9, max_storage_expansion=1e9)
        # execution rows [e0, e1) of the row order, whole block rows per rank
        block_rows = (h["rows"] + bs - 1) // bs
        per = (block_rows + world - 1) // world
        e0, e1 = min(h["rows"], rank * per * bs), min(h["rows"], (rank + 1) * per * bs)
        # the shard as a CSR of its own: rows = the canonical rows its execution rows name, local order identity
        canon = h["rperm"][e0:e1].astype(np.int64)
        counts = (h["row_offsets"][canon + 1] - h["row_offsets"][canon]).astype(np.int64)
        ro = np.concatenate([[0], np.cumsum(counts)]).astype(np.uint32)
        take = np.concatenate([np.arange(h["row_offsets"][c], h["row_offsets"][c + 1]) for c in canon]).astype(np.int64) \
            if len(canon) else np.zeros(0, dtype=np.int64)
        shard = (ro, h["feature_ids"][take], h["values"][take], h["features"], h["fb_offsets"], h["fperm"],
                 np.arange(len(canon), dtype=np.uint32))
        _, geo, _, cols, vals = checker.bell_lowering(*shard, bs, **relaxed)
        width = torch.tensor([geo["ell_blocks_per_row"]], dtype=torch.int64)
        occupied = torch.tensor([geo["occupied_blocks"]], dtype=torch.int64)
        dist.all_reduce(width, op=dist.ReduceOp.MAX)
        dist.all_reduce(occupied, op=dist.ReduceOp.SUM)
        whole = checker.bell_lowering(h["row_offsets"], h["feature_ids"], h["values"], h["features"], h["fb_offsets"],
                                      h["fperm"], h["rperm"], bs, **relaxed)
        ok = int(width) == whole[1]["ell_blocks_per_row"] and int(occupied) == whole[1]["occupied_blocks"]
        # my block rows of the whole result, cut to my own width, are my shard's result
        w_all, w_mine = whole[1]["ell_blocks_per_row"], geo["ell_blocks_per_row"]
        b0, b1 = e0 // bs, (e1 + bs - 1) // bs
        ref_cols = whole[3].reshape(-1, w_all)[b0:b1]
        ok = ok and np.array_equal(ref_cols[:, :w_mine], cols.reshape(-1, max(w_mine, 1))[:, :w_mine] if w_mine else ref_cols[:, :0])
        ok = ok and bool((ref_cols[:, w_mine:] == -1).all())
        ref_vals = whole[4].reshape(-1, w_all, bs * bs)[b0:b1]
        ok = ok and np.array_equal(ref_vals[:, :w_mine].ravel(), vals) and not ref_vals[:, w_mine:].any()
        flag = torch.tensor([int(ok)])
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if rank == 0:
            np.save(os.path.join(result_dir, "lowering_ok.npy"), np.array([int(flag)]))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_row_sharded_lowering_on_cpu_ranks(tmp_path, world):
    port = _free_port()
    mp.spawn(_lowering_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert int(np.load(tmp_path / "lowering_ok.npy")[0]) == 1
