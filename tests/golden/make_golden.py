"""Generates tests/golden/*.npz from the UNMODIFIED reference sources.

Run on a machine that has the Cellerator tree (CELLERATOR_REFERENCE, or a checkout called `reference` beside this repository):

    make -C oracle ref && python tests/golden/make_golden.py

Every array written here is produced by oracle/_ref/libcellerator_ref.so, i.e. by the
reference's own pack_nnz_values / unpack_nnz_values / build_spmm_reference /
blocked_ell::pack_row_major_values compiled in place; the inputs come from the seeded numpy
generator in cellerator_b200/synth.py.  The fixtures are small (a few hundred KB) and are
what the CPU test-suite pins oracle.c against on machines without the reference tree.
"""
import hashlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import oracle as orc  # noqa: E402
from cellerator_b200 import synth  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))


def csr_case(ref, name, rows, cols, median, sigma, lo, hi, bits, n, seed):
    h = synth.make_qcsr_host(rows, cols, median, sigma, lo, hi, bits, seed=seed)
    prp, total = ref.build_packed_row_ptr(bits, h["row_ptr"])
    packed = ref.pack_csr(bits, 1, h["row_ptr"], prp, h["col_idx"], h["scales"], h["offsets"], h["values"], cols=cols)
    decoded = ref.unpack_csr(bits, 1, h["row_ptr"], prp, h["col_idx"], h["scales"], h["offsets"], packed, cols=cols)
    rng = np.random.default_rng(seed + 1000)
    w = rng.normal(0.0, 0.02, size=(cols, n)).astype(np.float32)
    g = rng.normal(0.0, 1.0, size=(rows, n)).astype(np.float32)
    ro = h["row_ptr"].astype(np.uint64)
    y = ref.spmm_reference(rows, cols, n, ro, h["col_idx"], decoded, w)
    gt = ref.spmm_reference(cols, rows, n, ro, h["col_idx"], decoded, g, transpose_sparse=True)
    np.savez_compressed(os.path.join(OUT, name + ".npz"), rows=rows, cols=cols, bits=bits, n=n, seed=seed,
                        row_ptr=h["row_ptr"], col_idx=h["col_idx"], scales=h["scales"], offsets=h["offsets"],
                        values=h["values"], packed_row_ptr=prp, packed=packed, decoded=decoded, w=w, g=g, y=y, gt=gt)
    print(name, "nnz", len(h["col_idx"]), "packed bytes", total)


def c1_case(ref):
    """Configuration 1 in full (20,000 x 2,000, N = 32, fp32 W): too large to commit as arrays,
    so the fixture keeps hashes of the inputs, the first 64 rows of Y and the determinism digest."""
    cfg = synth.CONFIGS["c1_cpu_ref"]
    h = synth.make_qcsr_host(**cfg, seed=0)
    rows, cols, n = cfg["rows"], cfg["cols"], cfg["n"]
    prp, _ = ref.build_packed_row_ptr(8, h["row_ptr"])
    packed = ref.pack_csr(8, 1, h["row_ptr"], prp, h["col_idx"], h["scales"], h["offsets"], h["values"], cols=cols)
    decoded = ref.unpack_csr(8, 1, h["row_ptr"], prp, h["col_idx"], h["scales"], h["offsets"], packed, cols=cols)
    w = np.random.default_rng(1000).normal(0.0, 0.02, size=(cols, n)).astype(np.float32)
    y = ref.spmm_reference(rows, cols, n, h["row_ptr"].astype(np.uint64), h["col_idx"], decoded, w)
    sha = lambda a: hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()  # noqa: E731
    digest = ref.digest_f32(y.astype(np.float32))
    np.savez_compressed(os.path.join(OUT, "c1_summary.npz"), nnz=len(h["col_idx"]), sha_row_ptr=sha(h["row_ptr"]),
                        sha_col_idx=sha(h["col_idx"]), sha_packed=sha(packed), sha_w=sha(w), y_head=y[:64],
                        y_rowsum=y.sum(axis=1), y_digest=np.array(digest, dtype=np.uint64),
                        row_l1=np.add.reduceat(np.abs(decoded), h["row_ptr"][:-1]))
    print("c1 nnz", len(h["col_idx"]))


def bell_case(ref, name, rows, cols, block_size, ell_blocks, fill, bits, n, seed):
    h = synth.make_qbell_host(rows, cols, block_size, ell_blocks, fill, bits, seed=seed)
    packed = ref.bell_pack(bits, 1, rows, cols, block_size, h["ell_cols"], h["row_stride_bytes"], h["block_col_idx"],
                           h["scales"], h["offsets"], h["values_by_slot"])
    decoded = ref.bell_unpack(bits, 1, rows, cols, block_size, h["ell_cols"], h["row_stride_bytes"],
                              h["block_col_idx"], h["scales"], h["offsets"], packed)
    # CSR over every slot of a present block (the slots the reference's fused kernel multiplies)
    genes = h["genes_by_slot"]
    keep = genes < cols
    ro = np.zeros(rows + 1, dtype=np.uint64)
    np.cumsum(keep.sum(axis=1), out=ro[1:])
    w = np.random.default_rng(seed + 1000).normal(0.0, 0.02, size=(cols, n)).astype(np.float32)
    y = ref.spmm_reference(rows, cols, n, ro, genes[keep].astype(np.uint32), decoded[keep], w)
    np.savez_compressed(os.path.join(OUT, name + ".npz"), rows=rows, cols=cols, block_size=block_size,
                        ell_cols=h["ell_cols"], row_stride_bytes=h["row_stride_bytes"], bits=bits, n=n,
                        block_col_idx=h["block_col_idx"], scales=h["scales"], offsets=h["offsets"],
                        values_by_slot=h["values_by_slot"], packed=packed, decoded=decoded, w=w, y=y)
    print(name, "slots", rows * h["ell_cols"])


def lowering_case(ref, name, seed):
    """CSR -> physical Blocked-ELL lowering by the reference's query_bell_candidates_host /
    materialize_bell_candidate_host, for the three block sizes."""
    h = synth.make_lowering_host(rows=150, features=420, feature_blocks=5, mean_nnz=14, seed=seed)
    out = dict(rows=h["rows"], features=h["features"], row_offsets=h["row_offsets"], feature_ids=h["feature_ids"],
               values=h["values"], fb_offsets=h["fb_offsets"], fperm=h["fperm"], rperm=h["rperm"])
    for bs in (8, 16, 32):
        status, geo, pfo, cols, vals = ref.bell_lowering(h["row_offsets"], h["feature_ids"], h["values"], h["features"],
                                                         h["fb_offsets"], h["fperm"], h["rperm"], bs,
                                                         max_value_expansion=1e9, max_storage_expansion=1e9)
        assert status == 0 and geo["state"] == 0
        out[f"geometry{bs}"] = np.array([geo[k] for k in ref.BELL_GEOMETRY], dtype=np.uint64)
        out[f"metrics{bs}"] = np.array([geo[k] for k in ref.BELL_METRICS], dtype=np.float64)
        out[f"padded_offsets{bs}"], out[f"columns{bs}"], out[f"values{bs}"] = pfo, cols, vals
    np.savez_compressed(os.path.join(OUT, name + ".npz"), **out)
    print(name, "nnz", len(h["feature_ids"]))


if __name__ == "__main__":
    orc.build(ref=True)
    ref = orc.Reference()
    csr_case(ref, "csr8_small", rows=192, cols=640, median=60, sigma=0.6, lo=0, hi=400, bits=8, n=32, seed=11)
    csr_case(ref, "csr4_small", rows=160, cols=512, median=45, sigma=0.7, lo=0, hi=300, bits=4, n=16, seed=12)
    bell_case(ref, "bell8_small", rows=96, cols=250, block_size=32, ell_blocks=3, fill=0.6, bits=8, n=32, seed=13)
    bell_case(ref, "bell4_small", rows=64, cols=128, block_size=8, ell_blocks=4, fill=0.5, bits=4, n=8, seed=14)
    c1_case(ref)
    lowering_case(ref, "bell_lowering_small", seed=21)
