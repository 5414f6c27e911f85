"""GPU codec parity through the C ABI: packed bytes and decoded floats must be bit-identical
to the host codec (oracle / golden fixtures from the reference's sources)."""
import os

import numpy as np
import pytest
import torch

from cellerator_b200 import capi, ops
from conftest import GOLDEN, random_csr
from test_oracle import pack_by_rule, rule_codes

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("bits", [1, 2, 4, 8])
@pytest.mark.parametrize("policy", [1, 2])
def test_kat_4x8_device_bytes_equal_host_bytes(cuda_device, oracle, kats, bits, policy):
    k = kats["quantized_csr_4x8"]
    row_ptr = np.array(k["row_ptr"], dtype=np.int64)
    col = np.array(k["col_idx"], dtype=np.int32)
    scales = np.array(k["gene_scales"], dtype=np.float32)
    offsets = np.array(k["gene_offsets"] if policy == 1 else k["row_offsets"], dtype=np.float32)
    codes = rule_codes(k, bits)
    rows_of = np.repeat(np.arange(k["rows"]), np.diff(row_ptr))
    off = offsets[col] if policy == 1 else offsets[rows_of]
    values = (off + scales[col] * codes.astype(np.float32)).astype(np.float32)
    prp, total = ops.build_packed_row_ptr(bits, row_ptr)
    x = ops.QuantizedCsr.from_host(dict(rows=4, cols=8, bits=bits, policy=policy, row_ptr=row_ptr, packed_row_ptr=prp,
                                        col_idx=col, packed=np.full(total, 0xEE, dtype=np.uint8), scales=scales,
                                        offsets=offsets), cuda_device)
    x.quantize_(torch.from_numpy(values).to(cuda_device))
    assert x.packed.cpu().numpy().tolist() == pack_by_rule(codes, row_ptr, bits).tolist()
    back = x.dequantize().cpu().numpy()
    assert np.max(np.abs(back - values)) <= k["roundtrip_eps"]
    host = oracle.unpack_csr(bits, policy, row_ptr, prp, col, scales, offsets, x.packed.cpu().numpy())
    assert np.array_equal(back, host)
    # block-local calls, blocks of 2 rows (get_block + launch_*_block in the reference)
    brp = ops.build_uniform_block_row_ptr(4, k["rows_per_block"])
    x.packed.fill_(0)
    for b in range(len(brp) - 1):
        blk = ops.get_block(row_ptr, prp, brp, b)
        part = torch.from_numpy(values[blk["nnz_begin"]:blk["nnz_end"]].copy()).to(cuda_device)
        x.quantize_(part, blk["row_begin"], blk["row_end"])
        got = x.dequantize(blk["row_begin"], blk["row_end"]).cpu().numpy()
        assert np.array_equal(got, host[blk["nnz_begin"]:blk["nnz_end"]])
    assert x.packed.cpu().numpy().tolist() == pack_by_rule(codes, row_ptr, bits).tolist()


@pytest.mark.parametrize("name", ["csr8_small", "csr4_small"])
def test_golden_csr_codec(cuda_device, name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    bits = int(z["bits"])
    x = ops.QuantizedCsr.from_host(dict(rows=int(z["rows"]), cols=int(z["cols"]), bits=bits, policy=1,
                                        row_ptr=z["row_ptr"], packed_row_ptr=z["packed_row_ptr"], col_idx=z["col_idx"],
                                        packed=np.zeros_like(z["packed"]), scales=z["scales"], offsets=z["offsets"]),
                                   cuda_device)
    x.quantize_(torch.from_numpy(z["values"]).to(cuda_device))
    assert np.array_equal(x.packed.cpu().numpy(), z["packed"])
    assert np.array_equal(x.dequantize().cpu().numpy(), z["decoded"])


@pytest.mark.parametrize("bits", [1, 2, 4, 8])
@pytest.mark.parametrize("policy", [1, 2])
def test_random_codec_equals_oracle(cuda_device, oracle, bits, policy):
    rng = np.random.default_rng(50 + bits * 2 + policy)
    for rows, cols, max_nnz in ((1, 5, 5), (37, 300, 130), (200, 2000, 900)):
        c = random_csr(rng, rows, cols, max_nnz, bits, policy)
        # exact .5 ties and out-of-range values exercise rounding and clamping
        if len(c["values"]) > 8:
            c["values"][:4] = [1e9, -1e9, 0.0, 0.5]
        prp, total = oracle.build_packed_row_ptr(bits, c["row_ptr"])
        expect = oracle.pack_csr(bits, policy, c["row_ptr"], prp, c["col_idx"], c["scales"], c["offsets"], c["values"])
        h = dict(c, packed_row_ptr=prp, packed=np.full(max(total, 1), 0x55, dtype=np.uint8)[:total])
        x = ops.QuantizedCsr.from_host(h, cuda_device)
        if total == 0:
            continue
        x.quantize_(torch.from_numpy(c["values"]).to(cuda_device))
        assert np.array_equal(x.packed.cpu().numpy(), expect)
        dec = oracle.unpack_csr(bits, policy, c["row_ptr"], prp, c["col_idx"], c["scales"], c["offsets"], expect)
        assert np.array_equal(x.dequantize().cpu().numpy(), dec)


def test_codec_null_metadata_and_bad_arguments(cuda_device, oracle):
    rng = np.random.default_rng(3)
    c = random_csr(rng, 20, 40, 20, 8, 1)
    c["scales"], c["offsets"] = None, None            # null scales -> 1, null offsets -> 0
    c["values"] = rng.integers(0, 256, size=len(c["col_idx"])).astype(np.float32)
    prp, total = oracle.build_packed_row_ptr(8, c["row_ptr"])
    x = ops.QuantizedCsr.from_host(dict(c, packed_row_ptr=None, packed=np.zeros(total, dtype=np.uint8)), cuda_device)
    x.quantize_(torch.from_numpy(c["values"]).to(cuda_device))
    assert np.array_equal(x.packed.cpu().numpy(), c["values"].astype(np.uint8))
    assert np.array_equal(x.dequantize().cpu().numpy(), c["values"])
    with pytest.raises(capi.Cb200Error) as e:
        x.quantize_(torch.from_numpy(c["values"]).to(cuda_device), 5, 100)
    assert e.value.status == capi.INVALID_SHAPE
    x.bits = 3
    with pytest.raises(capi.Cb200Error):
        x.dequantize()


@pytest.mark.parametrize("name", ["bell8_small", "bell4_small"])
def test_golden_bell_codec(cuda_device, name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    x = ops.QuantizedBell.from_host(dict(rows=int(z["rows"]), cols=int(z["cols"]), block_size=int(z["block_size"]),
                                         ell_cols=int(z["ell_cols"]), row_stride_bytes=int(z["row_stride_bytes"]),
                                         bits=int(z["bits"]), policy=1, block_col_idx=z["block_col_idx"],
                                         packed=np.full_like(z["packed"], 0xCC), scales=z["scales"],
                                         offsets=z["offsets"]), cuda_device)
    ops.quantize_bell_(x, torch.from_numpy(z["values_by_slot"]).to(cuda_device))
    assert np.array_equal(x.packed.cpu().numpy(), z["packed"])          # padding bytes included
    assert np.array_equal(ops.dequantize_bell(x).cpu().numpy(), z["decoded"])
