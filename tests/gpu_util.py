"""Helpers shared by the GPU parity tests (imported only from tests marked gpu)."""
import numpy as np
import torch

from cellerator_b200 import capi, ops


def to_dev(h, device):
    return ops.QuantizedCsr.from_host(h, device)


def row_l1(oracle, h):
    """||row||_1 of the decoded matrix, from the oracle's decode."""
    dec = oracle.unpack_csr(h["bits"], h["policy"], h["row_ptr"], h["packed_row_ptr"], h["col_idx"], h["scales"],
                            h["offsets"], h["packed"])
    out = np.zeros(h["rows"])
    counts = np.diff(h["row_ptr"])
    if len(dec):
        nz = counts > 0
        out[nz] = np.add.reduceat(np.abs(dec.astype(np.float64)), h["row_ptr"][:-1][nz])
    return out, dec


def assert_forward_close(y_gpu, y_ref, l1, w_abs_max, bf16=False):
    """fp32 W: max|d| <= 1e-4 * (||row||_1 * max|W|) per row.  bf16 W: additionally 1e-2 relative
    (the operand is widened exactly, so the tighter absolute bound holds as well)."""
    y_gpu = np.asarray(y_gpu, dtype=np.float64)
    bound = 1e-4 * l1[:, None] * w_abs_max + 1e-30
    err = np.abs(y_gpu - y_ref)
    worst = np.unravel_index(np.argmax(err - bound), err.shape)
    assert np.all(err <= bound), f"row {worst[0]} col {worst[1]}: |d|={err[worst]:.3e} bound={bound[worst[0], 0]:.3e}"
    if bf16:
        rel = err / np.maximum(np.abs(y_ref), 1e-2 * l1[:, None] * w_abs_max + 1e-30)
        assert np.max(rel, initial=0.0) <= 1e-2


def host_pack(oracle, c):
    """random_csr dict -> adds packed_row_ptr / packed via the oracle (the checker)."""
    prp, _ = oracle.build_packed_row_ptr(c["bits"], c["row_ptr"])
    c = dict(c)
    c["packed_row_ptr"] = prp
    c["packed"] = oracle.pack_csr(c["bits"], c["policy"], c["row_ptr"], prp, c["col_idx"], c["scales"], c["offsets"],
                                  c["values"])
    return c


def dense(rng, rows, n, dtype, device, std=0.02, ld=None):
    ld = n if ld is None else ld
    full = torch.from_numpy(rng.normal(0.0, std, size=(rows, ld)).astype(np.float32)).to(device).to(dtype)
    view = full[:, :n]
    return view, view.float().cpu().numpy()
