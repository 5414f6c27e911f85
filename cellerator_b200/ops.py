"""Driver-side objects over the C ABI: device-resident quantized matrices and prepared SpMM
operations.  torch supplies device memory and streams only; every computation is a call into
libcellerator_b200.so through `capi`.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field

import numpy as np
import torch

from . import capi

_TORCH_DENSE = {torch.float32: capi.DTYPE_F32, torch.bfloat16: capi.DTYPE_BF16}


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream_handle(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


# ---- host helpers (no device) ----------------------------------------------------------

def build_packed_row_ptr(bits: int, row_ptr: np.ndarray):
    row_ptr = np.ascontiguousarray(row_ptr, dtype=np.int64)
    out = np.zeros_like(row_ptr)
    total = capi.lib().cb200_build_packed_row_ptr(bits, row_ptr.ctypes.data, len(row_ptr) - 1, out.ctypes.data)
    if total < 0:
        raise capi.Cb200Error(capi.INVALID_ARGUMENT, "build_packed_row_ptr rejected its arguments")
    return out, int(total)


def build_uniform_block_row_ptr(rows: int, rows_per_block: int) -> np.ndarray:
    count = int(capi.lib().cb200_block_count_for_rows(rows, rows_per_block))
    out = np.zeros(count + 1, dtype=np.int64)
    rc = capi.lib().cb200_build_uniform_block_row_ptr(rows, rows_per_block, out.ctypes.data)
    if rc < 0:
        raise capi.Cb200Error(capi.INVALID_ARGUMENT, "build_uniform_block_row_ptr rejected its arguments")
    return out


def get_block(row_ptr, packed_row_ptr, block_row_ptr, block_index) -> dict:
    row_ptr = np.ascontiguousarray(row_ptr, dtype=np.int64)
    packed_row_ptr = np.ascontiguousarray(packed_row_ptr, dtype=np.int64)
    brp = None if block_row_ptr is None else np.ascontiguousarray(block_row_ptr, dtype=np.int64)
    out = capi.CsrBlock()
    capi.check(capi.lib().cb200_get_block(len(row_ptr) - 1, row_ptr.ctypes.data, packed_row_ptr.ctypes.data,
                                          None if brp is None else brp.ctypes.data,
                                          0 if brp is None else len(brp) - 1, block_index, C.byref(out)))
    return {n: getattr(out, n) for n, _ in capi.CsrBlock._fields_}


def partition_rows(rows: int, parts: int) -> np.ndarray:
    """Row range per shard: the reference's uniform rule with rows_per_block = ceil(rows/parts),
    padded with empty trailing shards so that there are exactly `parts` of them."""
    per = max(1, -(-rows // max(parts, 1)))
    brp = build_uniform_block_row_ptr(rows, per)
    if len(brp) - 1 < parts:
        brp = np.concatenate([brp, np.full(parts - (len(brp) - 1), rows, dtype=np.int64)])
    return brp


# ---- device containers -------------------------------------------------------------------

@dataclass
class QuantizedCsr:
    """Quantized CSR on one device (layout of cb200_qcsr)."""
    rows: int
    cols: int
    bits: int
    policy: int
    row_ptr: torch.Tensor            # int64 [rows+1]
    col_idx: torch.Tensor            # int32 [nnz]
    packed: torch.Tensor             # uint8
    scales: torch.Tensor | None      # float32 [cols]
    offsets: torch.Tensor | None     # float32 [cols] or [rows]
    packed_row_ptr: torch.Tensor | None = None   # int64 [rows+1]; None for 8-bit
    host_row_ptr: np.ndarray | None = None
    _desc: capi.QCsr | None = field(default=None, repr=False)

    @property
    def nnz(self) -> int:
        return int(self.col_idx.numel())

    @property
    def device(self):
        return self.row_ptr.device

    def desc(self) -> capi.QCsr:
        d = capi.header(capi.QCsr())
        d.rows, d.cols, d.nnz, d.bits, d.policy = self.rows, self.cols, self.nnz, self.bits, self.policy
        d.row_ptr = self.row_ptr.data_ptr()
        d.packed_row_ptr = None if self.packed_row_ptr is None else self.packed_row_ptr.data_ptr()
        d.col_idx = self.col_idx.data_ptr() if self.nnz else None
        d.packed_values = self.packed.data_ptr() if self.packed.numel() else None
        d.scales = None if self.scales is None else self.scales.data_ptr()
        d.offsets = None if self.offsets is None else self.offsets.data_ptr()
        self._desc = d
        return d

    @staticmethod
    def from_host(h: dict, device) -> "QuantizedCsr":
        def dev(a, dt):
            return None if a is None else torch.from_numpy(np.ascontiguousarray(a, dtype=dt)).to(device)
        return QuantizedCsr(rows=int(h["rows"]), cols=int(h["cols"]), bits=int(h["bits"]), policy=int(h["policy"]),
                            row_ptr=dev(h["row_ptr"], np.int64), col_idx=dev(h["col_idx"], np.int32),
                            packed=dev(h["packed"], np.uint8), scales=dev(h.get("scales"), np.float32),
                            offsets=dev(h.get("offsets"), np.float32),
                            packed_row_ptr=None if int(h["bits"]) == 8 and h.get("packed_row_ptr") is None
                            else dev(h["packed_row_ptr"], np.int64),
                            host_row_ptr=np.ascontiguousarray(h["row_ptr"], dtype=np.int64))

    def quantize_(self, values: torch.Tensor, row_begin=0, row_end=None) -> None:
        """Overwrite the packed codes of rows [row_begin,row_end) from one float per entry."""
        row_end = self.rows if row_end is None else row_end
        dev = self.device
        capi.check(capi.lib().cb200_quantize_rows(C.byref(self.desc()), row_begin, row_end, values.data_ptr(),
                                                  dev.index, _stream_handle(dev)))

    def dequantize(self, row_begin=0, row_end=None) -> torch.Tensor:
        row_end = self.rows if row_end is None else row_end
        dev = self.device
        lo, hi = (int(v) for v in self.row_ptr[[row_begin, row_end]].tolist())
        out = torch.empty(max(hi - lo, 1), dtype=torch.float32, device=dev)
        capi.check(capi.lib().cb200_dequantize_rows(C.byref(self.desc()), row_begin, row_end, out.data_ptr(),
                                                    dev.index, _stream_handle(dev)))
        return out[: hi - lo]


@dataclass
class QuantizedBell:
    """Quantized Blocked-ELL on one device (layout of cb200_qbell)."""
    rows: int
    cols: int
    block_size: int
    ell_cols: int
    row_stride_bytes: int
    bits: int
    policy: int
    block_col_idx: torch.Tensor      # uint32 stored as int32 bits [ceil(rows/bs) * ell_cols/bs]
    packed: torch.Tensor             # uint8 [rows * row_stride_bytes]
    scales: torch.Tensor | None
    offsets: torch.Tensor | None
    _desc: capi.QBell | None = field(default=None, repr=False)

    @property
    def device(self):
        return self.packed.device

    def desc(self) -> capi.QBell:
        d = capi.header(capi.QBell())
        d.rows, d.cols, d.block_size, d.ell_cols = self.rows, self.cols, self.block_size, self.ell_cols
        d.row_stride_bytes, d.bits, d.policy = self.row_stride_bytes, self.bits, self.policy
        d.block_col_idx = self.block_col_idx.data_ptr()
        d.packed_values = self.packed.data_ptr()
        d.scales = None if self.scales is None else self.scales.data_ptr()
        d.offsets = None if self.offsets is None else self.offsets.data_ptr()
        self._desc = d
        return d

    @staticmethod
    def from_host(h: dict, device) -> "QuantizedBell":
        def dev(a, dt):
            return None if a is None else torch.from_numpy(np.ascontiguousarray(a, dtype=dt)).to(device)
        bci = np.ascontiguousarray(h["block_col_idx"], dtype=np.uint32).view(np.int32)
        return QuantizedBell(rows=int(h["rows"]), cols=int(h["cols"]), block_size=int(h["block_size"]),
                             ell_cols=int(h["ell_cols"]), row_stride_bytes=int(h["row_stride_bytes"]),
                             bits=int(h["bits"]), policy=int(h["policy"]), block_col_idx=dev(bci, np.int32),
                             packed=dev(h["packed"], np.uint8), scales=dev(h.get("scales"), np.float32),
                             offsets=dev(h.get("offsets"), np.float32))


def quantize_bell_(x: QuantizedBell, values_by_slot: torch.Tensor, row_begin=0, row_end=None) -> None:
    row_end = x.rows if row_end is None else row_end
    dev = x.device
    capi.check(capi.lib().cb200_qbell_quantize_rows(C.byref(x.desc()), row_begin, row_end, values_by_slot.data_ptr(),
                                                    dev.index, _stream_handle(dev)))


def dequantize_bell(x: QuantizedBell, row_begin=0, row_end=None) -> torch.Tensor:
    row_end = x.rows if row_end is None else row_end
    dev = x.device
    out = torch.empty((row_end - row_begin, x.ell_cols), dtype=torch.float32, device=dev)
    capi.check(capi.lib().cb200_qbell_dequantize_rows(C.byref(x.desc()), row_begin, row_end, out.data_ptr(),
                                                      dev.index, _stream_handle(dev)))
    return out


def backend_query(projection: int, sparse=capi.DTYPE_U8, dense=capi.DTYPE_BF16, output=capi.DTYPE_F32,
                  multiply=capi.DTYPE_F32, accumulation=capi.DTYPE_F32, quantized=1) -> dict:
    pol = capi.header(capi.NumericPolicy())
    pol.sparse_storage, pol.dense_storage, pol.output_storage = sparse, dense, output
    pol.multiply, pol.accumulation, pol.quantized = multiply, accumulation, quantized
    cap = capi.Capability()
    capi.check(capi.lib().cb200_backend_query(projection, C.byref(pol), C.byref(cap)))
    return {"supported": bool(cap.supported), "flags": cap.flags, "persistent_bytes": cap.persistent_bytes,
            "transient_bytes": cap.transient_bytes, "name": (cap.name or b"").decode()}


# Schedule requested for every operation of a projection kind that names none itself (cb200_spmm_problem.
# schedule_hint): how a test pins one kernel for all the operations it prepares.  Empty by default.
SCHEDULE_REQUEST: dict[int, str | None] = {}


class PreparedSpmm:
    """prepare once, run many times (cb200_spmm_prepare / cb200_spmm_run)."""

    def __init__(self, projection: int, m: int, k: int, n: int, nnz: int, bits: int, policy: int, dense_dtype,
                 device, structure_epoch: int = 1, host_row_ptr: np.ndarray | None = None, deterministic=False,
                 multiply: int = 0, device_matrix=None, persistent_limit_bytes: int = 0, value_generation: int = 0,
                 schedule: str | None = None, persistent: torch.Tensor | None = None, prepare_stream: int | None = None):
        self.device = torch.device(device)
        pr = capi.header(capi.SpmmProblem())
        pr.projection, pr.m, pr.k, pr.n, pr.nnz, pr.bits, pr.policy = projection, m, k, n, nnz, bits, policy
        pr.dense_dtype = _TORCH_DENSE[dense_dtype] if isinstance(dense_dtype, torch.dtype) else dense_dtype
        pr.device = self.device.index if self.device.index is not None else torch.cuda.current_device()
        pr.structure_epoch = structure_epoch
        self._host_row_ptr = None
        if host_row_ptr is not None:
            self._host_row_ptr = np.ascontiguousarray(host_row_ptr, dtype=np.int64)
            pr.host_row_ptr = self._host_row_ptr.ctypes.data
        pr.deterministic = int(deterministic)
        pr.multiply = multiply  # 0 / DTYPE_F32: exact fp32 products; DTYPE_BF16: tensor-core products
        self._matrix_desc = None
        if device_matrix is not None:  # lets prepare build its persistent window-blocked copy
            self._matrix_desc = device_matrix.desc()
            pr.device_matrix = C.pointer(self._matrix_desc)
        pr.persistent_limit_bytes = persistent_limit_bytes  # 0: no limit on what prepare may keep on the device
        pr.value_generation = value_generation              # generation of the values device_matrix holds (0: not tracked)
        if schedule is None:
            schedule = SCHEDULE_REQUEST.get(projection)
        self._hint = schedule.encode() if schedule else None
        pr.schedule_hint = self._hint                       # one schedule by name; None lets prepare choose
        self._persistent = persistent                       # caller-owned block prepare builds its copies in
        if persistent is not None:
            pr.persistent, pr.persistent_bytes = persistent.data_ptr(), persistent.numel() * persistent.element_size()
        pr.prepare_stream = prepare_stream
        self.problem = pr
        self.handle = C.c_void_p()
        capi.check(capi.lib().cb200_spmm_prepare(C.byref(pr), C.byref(self.handle)))
        nbytes, align = C.c_uint64(), C.c_uint32()
        capi.check(capi.lib().cb200_prepared_workspace(self.handle, C.byref(nbytes), C.byref(align)))
        self.workspace_bytes, self.workspace_alignment = nbytes.value, align.value
        self.workspace = (torch.empty(self.workspace_bytes, dtype=torch.uint8, device=self.device)
                          if self.workspace_bytes else None)
        self.epoch = structure_epoch

    @property
    def schedule(self) -> str:
        return capi.lib().cb200_prepared_schedule(self.handle).decode()

    @property
    def persistent_bytes(self) -> int:
        """Device bytes the prepared operation owns (row order, window-blocked copy)."""
        return int(capi.lib().cb200_prepared_persistent_bytes(self.handle))

    def status(self, stream: int | None = None) -> int:
        """Status word of the launches that used this operation's workspace (cb200_prepared_status): 0, or
        raises Cb200Error(DEVICE_WAIT_TIMEOUT) when a kernel gave up a bounded wait.  Waits for the stream."""
        word = C.c_int32(-1)
        ws = None if self.workspace is None else C.c_void_p(self.workspace.data_ptr())
        capi.check(capi.lib().cb200_prepared_status(self.handle, ws, C.c_void_p(_stream_handle(self.device) if stream is None else stream),
                                                    C.byref(word)))
        return int(word.value)

    @staticmethod
    def persistent_requirement(projection, m, k, n, nnz, bits, policy, dense_dtype, device_index, multiply=0,
                               device_matrix=None, deterministic=False, persistent_limit_bytes=0, host_row_ptr=None,
                               schedule: str | None = None) -> int:
        """cb200_spmm_persistent_requirement: bytes a session reserves for the operation before sealing."""
        pr = capi.header(capi.SpmmProblem())
        pr.projection, pr.m, pr.k, pr.n, pr.nnz, pr.bits, pr.policy = projection, m, k, n, nnz, bits, policy
        pr.dense_dtype = _TORCH_DENSE[dense_dtype] if isinstance(dense_dtype, torch.dtype) else dense_dtype
        pr.device, pr.structure_epoch, pr.multiply, pr.deterministic = device_index, 1, multiply, int(deterministic)
        pr.persistent_limit_bytes = persistent_limit_bytes
        keep = None
        if device_matrix is not None:
            keep = device_matrix.desc()
            pr.device_matrix = C.pointer(keep)
        hrp = None
        if host_row_ptr is not None:
            hrp = np.ascontiguousarray(host_row_ptr, dtype=np.int64)
            pr.host_row_ptr = hrp.ctypes.data
        hint = schedule.encode() if schedule else None
        pr.schedule_hint = hint
        need = C.c_uint64()
        capi.check(capi.lib().cb200_spmm_persistent_requirement(C.byref(pr), C.byref(need)))
        del keep, hrp, hint
        return int(need.value)

    def make_launch(self, x, dense: torch.Tensor, out: torch.Tensor, alpha=1.0, beta=0.0, row_begin=0, row_end=capi.ALL_ROWS,
                    stream: int | None = None, epoch: int | None = None, epilogue: str | int = 0,
                    bias: torch.Tensor | None = None, value_generation: int = 0) -> capi.Launch:
        ln = capi.header(capi.Launch())
        desc = x.desc()
        if isinstance(x, QuantizedBell):
            ln.bell = C.pointer(desc)
        else:
            ln.csr = C.pointer(desc)
        ln.dense, ln.dense_ld = dense.data_ptr(), dense.stride(0)
        ln.out, ln.out_ld = out.data_ptr(), out.stride(0)
        ln.alpha, ln.beta = alpha, beta
        ln.structure_epoch = self.epoch if epoch is None else epoch
        ln.row_begin, ln.row_end = row_begin, row_end
        dev_index = self.problem.device
        ln.stream = _stream_handle(self.device) if stream is None else stream
        ln.device = dev_index
        ln.workspace_device = dev_index
        ln.workspace = None if self.workspace is None else self.workspace.data_ptr()
        ln.workspace_bytes = self.workspace_bytes
        ln.value_generation = value_generation
        ln.epilogue = capi.EPILOGUE[epilogue] if isinstance(epilogue, str) else int(epilogue)
        if bias is not None:
            if bias.dtype != torch.float32 or not bias.is_contiguous() or bias.numel() != self.problem.n:
                raise ValueError("bias must be a contiguous float32 vector with one value per output column")
            ln.bias = bias.data_ptr()
        ln._keep = (desc, x, dense, out, bias)
        return ln

    def run_launch(self, launch: capi.Launch) -> None:
        capi.check(capi.lib().cb200_spmm_run(self.handle, C.byref(launch)))

    def run(self, x, dense, out, **kw) -> torch.Tensor:
        self.run_launch(self.make_launch(x, dense, out, **kw))
        return out

    def close(self):
        if self.handle:
            capi.lib().cb200_prepared_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def spmm_forward(x: QuantizedCsr, w: torch.Tensor, out: torch.Tensor | None = None, alpha=1.0, beta=0.0,
                 multiply: int = 0, epilogue: str | int = 0, bias: torch.Tensor | None = None, schedule: str | None = None):
    """Y = act(alpha * deq(X) W + beta * Y + bias) (one-shot convenience: prepare + run).

    epilogue names one of capi.EPILOGUE ("none", "bias", "relu", "gelu_erf", "gelu_tanh", "bias_relu", ...).

    multiply=capi.DTYPE_BF16 with a bf16 W asks for tensor-core products (decoded values rounded to bf16)."""
    n = w.shape[1]
    if out is None:
        out = torch.empty(x.rows, n, dtype=torch.float32, device=x.device)
    op = PreparedSpmm(capi.PROJECTION_CSR, x.rows, x.cols, n, x.nnz, x.bits, x.policy, w.dtype, x.device,
                      host_row_ptr=x.host_row_ptr, multiply=multiply, schedule=schedule)
    op.run(x, w, out, alpha=alpha, beta=beta, epilogue=epilogue, bias=bias)
    op.close()
    return out


def spmm_transpose(x: QuantizedCsr, g: torch.Tensor, out: torch.Tensor | None = None, alpha=1.0, beta=0.0,
                   row_begin=0, row_end=capi.ALL_ROWS, multiply: int = 0, deterministic=False):
    """G' = alpha * deq(X)^T G + beta * G'.

    multiply=capi.DTYPE_BF16 asks for tensor-core products (decoded values and G rounded to bf16);
    deterministic=True for the gather schedule whose fp32 sums have a fixed order."""
    n = g.shape[1]
    if out is None:
        out = torch.empty(x.cols, n, dtype=torch.float32, device=x.device)
    op = PreparedSpmm(capi.PROJECTION_TRANSPOSE, x.rows, x.cols, n, x.nnz, x.bits, x.policy, g.dtype, x.device,
                      multiply=multiply, device_matrix=x if (multiply == capi.DTYPE_BF16 or deterministic) else None,
                      deterministic=deterministic)
    op.run(x, g, out, alpha=alpha, beta=beta, row_begin=row_begin, row_end=row_end)
    op.close()
    return out


def bell_forward(x: QuantizedBell, w: torch.Tensor, out: torch.Tensor | None = None, alpha=1.0, beta=0.0,
                 epilogue: str | int = 0, bias: torch.Tensor | None = None):
    n = w.shape[1]
    if out is None:
        out = torch.empty(x.rows, n, dtype=torch.float32, device=x.device)
    op = PreparedSpmm(capi.PROJECTION_BLOCKED_ELL, x.rows, x.cols, n, x.rows * x.ell_cols, x.bits, x.policy,
                      w.dtype, x.device)
    op.run(x, w, out, alpha=alpha, beta=beta, epilogue=epilogue, bias=bias)
    op.close()
    return out


# ---- CSR -> physical Blocked-ELL lowering on the device ---------------------------------------

class BellLowering:
    """cb200_bell_lowering_query / _materialize over device tensors.

    row_offsets / feature_ids: uint32 CSR with canonical feature ids (held as int32 tensors of the same
    bits); values: any dtype, one element (or one row of a 2-D tensor) per stored entry, copied bytewise;
    fb_offsets: host array of the semantic feature blocks in execution order; fperm[execution] =
    canonical feature, rperm[execution row] = canonical row."""

    def __init__(self, row_offsets, feature_ids, values, features: int, fb_offsets, fperm, rperm, device):
        self.device = torch.device(device)
        as_i32 = lambda a: torch.as_tensor(np.ascontiguousarray(a, dtype=np.uint32).view(np.int32)).to(self.device) \
            if not isinstance(a, torch.Tensor) else a.to(self.device)
        self.row_offsets, self.feature_ids = as_i32(row_offsets), as_i32(feature_ids)
        self.values = (values if isinstance(values, torch.Tensor) else torch.as_tensor(np.ascontiguousarray(values))).to(self.device).contiguous()
        self.fperm, self.rperm = as_i32(fperm), as_i32(rperm)
        self.rows, self.features, self.nnz = self.row_offsets.numel() - 1, int(features), self.feature_ids.numel()
        self.finv = torch.empty_like(self.fperm)
        self.finv[self.fperm.long()] = torch.arange(self.features, dtype=torch.int32, device=self.device)
        self.rinv = torch.empty_like(self.rperm)
        if self.rows:
            self.rinv[self.rperm.long()] = torch.arange(self.rows, dtype=torch.int32, device=self.device)
        self._fb = np.ascontiguousarray(fb_offsets, dtype=np.uint32)
        self.value_size = self.values.element_size() * (self.values.shape[1] if self.values.dim() == 2 else 1)
        inp = capi.header(capi.BellLoweringInput())
        inp.rows, inp.features, inp.nnz, inp.value_size_bytes = self.rows, self.features, self.nnz, self.value_size
        inp.row_offsets, inp.feature_ids = self.row_offsets.data_ptr(), self.feature_ids.data_ptr()
        inp.values = self.values.data_ptr() if self.nnz else None
        inp.feature_block_count = len(self._fb) - 1
        inp.feature_block_offsets = self._fb.ctypes.data
        inp.feature_permutation, inp.inverse_feature_permutation = self.fperm.data_ptr(), self.finv.data_ptr()
        inp.row_permutation, inp.inverse_row_permutation = self.rperm.data_ptr(), self.rinv.data_ptr()
        inp.device = self.device.index if self.device.index is not None else torch.cuda.current_device()
        self.input = inp
        need = C.c_uint64()
        capi.check(capi.lib().cb200_bell_lowering_workspace(C.byref(inp), C.byref(need)))
        self.workspace = torch.empty(need.value, dtype=torch.uint8, device=self.device)

    def query(self, block_size: int, max_value_expansion=64.0, max_storage_expansion=64.0,
              max_persistent=2 ** 63) -> capi.BellGeometry:
        policy = capi.BellLoweringPolicy(max_value_expansion, max_storage_expansion, max_persistent)
        geo = capi.BellGeometry()
        capi.check(capi.lib().cb200_bell_lowering_query(C.byref(self.input), C.c_uint32(block_size), C.byref(policy),
                                                        C.c_void_p(self.workspace.data_ptr()),
                                                        C.c_uint64(self.workspace.numel()),
                                                        C.c_void_p(_stream_handle(self.device)), C.byref(geo)))
        return geo

    def materialize(self, geo: capi.BellGeometry, layout=capi.BELL_VALUES_BLOCK_MAJOR, row_stride_bytes=0):
        """-> (padded feature-block offsets int32[blocks + 1], column indices int32, value bytes uint8)"""
        pfo = torch.empty(len(self._fb), dtype=torch.int32, device=self.device)
        cols = torch.empty(geo.column_index_count, dtype=torch.int32, device=self.device)
        nbytes = geo.padded_rows * row_stride_bytes if layout == capi.BELL_VALUES_ROW_MAJOR else geo.value_bytes
        vals = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
        capi.check(capi.lib().cb200_bell_lowering_materialize(
            C.byref(self.input), C.byref(geo), C.c_int32(layout), C.c_uint64(row_stride_bytes),
            C.c_void_p(pfo.data_ptr()), C.c_void_p(cols.data_ptr() if cols.numel() else None),
            C.c_void_p(vals.data_ptr() if vals.numel() else None), C.c_void_p(self.workspace.data_ptr()),
            C.c_uint64(self.workspace.numel()), C.c_void_p(_stream_handle(self.device))))
        return pfo, cols, vals


def build_execution_csr(row_offsets, block_ids, local_ids, canonical_ids, features: int, fb_offsets, fperm):
    """cb200_build_execution_csr over int32 device tensors (the bits of uint32 arrays).
    -> (flags, execution feature ids); flags 0 = ok, bit 0 invalid geometry, bit 1 incompatible identity."""
    device = row_offsets.device
    fbo = np.ascontiguousarray(fb_offsets, dtype=np.uint32)
    e = capi.header(capi.ExecutionCsr())
    e.rows, e.features, e.nnz = row_offsets.numel() - 1, int(features), block_ids.numel()
    e.row_offsets, e.block_ids = row_offsets.data_ptr(), block_ids.data_ptr()
    e.local_feature_ids, e.canonical_feature_ids = local_ids.data_ptr(), canonical_ids.data_ptr()
    e.feature_block_count, e.feature_block_offsets, e.feature_permutation = len(fbo) - 1, fbo.ctypes.data, fperm.data_ptr()
    out = torch.full((e.nnz,), -1, dtype=torch.int32, device=device)
    work = torch.empty(len(fbo), dtype=torch.int32, device=device)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    e.execution_feature_ids, e.workspace, e.workspace_bytes = out.data_ptr(), work.data_ptr(), work.numel() * 4
    e.status_word = status.data_ptr()
    e.device = device.index if device.index is not None else torch.cuda.current_device()
    capi.check(capi.lib().cb200_build_execution_csr(C.byref(e), C.c_void_p(_stream_handle(device))))
    return int(status.item()), out


def qcsr_gene_major(x: "QuantizedCsr"):
    """Gene-major copy (a CSC) of a device matrix (cb200_qcsr_gene_major): -> (col_ptr int64 [cols + 1],
    row_idx int32 [nnz], codes uint8 [nnz]), the cells ascending inside every gene, one code per byte."""
    lib = capi.lib()
    need = int(lib.cb200_qcsr_gene_major_workspace(x.rows, x.cols))
    device = x.device
    work = torch.empty(max(need, 256), dtype=torch.uint8, device=device)
    col_ptr = torch.empty(x.cols + 1, dtype=torch.int64, device=device)
    row_idx = torch.empty(max(x.nnz, 1), dtype=torch.int32, device=device)
    codes = torch.empty(max(x.nnz, 1), dtype=torch.uint8, device=device)
    desc = x.desc()
    index = device.index if device.index is not None else torch.cuda.current_device()
    capi.check(lib.cb200_qcsr_gene_major(C.byref(desc), col_ptr.data_ptr(), row_idx.data_ptr(), codes.data_ptr(),
                                         work.data_ptr(), work.numel(), index, _stream_handle(device)))
    if int(work[:4].view(torch.int32).item()) != 0:
        raise ValueError("a column index lies outside the matrix")
    return col_ptr, row_idx[:x.nnz], codes[:x.nnz]


def pack_dense_operand(source: torch.Tensor, fperm: torch.Tensor, col_major=False, fb_offsets=None,
                       padded_offsets=None) -> torch.Tensor:
    """packed[execution] = source[fperm[execution]] (cb200_pack_dense_operand).  source: 2-D, [features][columns]
    or, with col_major, [columns][features]; any stride along dim 0.  With fb_offsets / padded_offsets (host
    arrays) the rows follow the padded physical feature order of a Blocked-ELL lowering."""
    assert source.dim() == 2 and source.stride(1) == 1
    features, columns = (source.shape[1], source.shape[0]) if col_major else source.shape
    d = capi.header(capi.DensePack())
    d.feature_permutation, d.source = fperm.data_ptr(), source.data_ptr()
    d.features, d.columns, d.leading_dimension = features, columns, source.stride(0)
    d.source_col_major, d.value_size_bytes = int(col_major), source.element_size()
    rows = features
    keep = None
    if fb_offsets is not None:
        fbo = np.ascontiguousarray(fb_offsets, dtype=np.uint32)
        pfo = np.ascontiguousarray(padded_offsets, dtype=np.uint32)
        d.feature_block_count, d.feature_block_offsets, d.padded_feature_block_offsets = len(fbo) - 1, fbo.ctypes.data, pfo.ctypes.data
        rows, keep = int(pfo[-1]), (fbo, pfo)
    out = torch.empty(rows, columns, dtype=source.dtype, device=source.device)
    status = torch.zeros(1, dtype=torch.int32, device=source.device)
    d.packed, d.packed_capacity_bytes, d.status_word = out.data_ptr(), out.numel() * out.element_size(), status.data_ptr()
    d.device = source.device.index if source.device.index is not None else torch.cuda.current_device()
    capi.check(capi.lib().cb200_pack_dense_operand(C.byref(d), C.c_void_p(_stream_handle(source.device))))
    if int(status.item()) != 0:
        raise capi.Cb200Error(capi.STATUS_INVALID_SHAPE, "invalid geometry: feature permutation is out of range")
    del keep
    return out


# ---- the reference's public projection calls, routed ------------------------------------------

def public_layout(x) -> capi.PublicLayout:
    """cellerator_sparse_layout_desc fields of a quantized matrix: 32-bit row offsets for CSR (a uint32 copy
    of row_ptr is attached to the descriptor), the arrays of the matrix otherwise."""
    l = capi.header(capi.PublicLayout())
    l.rows, l.cols, l.bits, l.decode_policy = x.rows, x.cols, x.bits, x.policy
    l.packed_values = x.packed.data_ptr()
    l.column_scales = x.scales.data_ptr() if x.scales is not None else None
    off = x.offsets.data_ptr() if x.offsets is not None else None
    if x.policy == capi.DECODE_COLUMN_SCALE_ROW_OFFSET:
        l.row_offsets = off
    else:
        l.column_offsets = off
    if isinstance(x, QuantizedBell):
        l.layout = capi.PUBLIC_LAYOUT_QUANTIZED_BLOCKED_ELL
        l.block_size, l.ell_cols, l.row_stride_bytes = x.block_size, x.ell_cols, x.row_stride_bytes
        l.block_col_idx = x.block_col_idx.data_ptr()
        l._keep = (x,)
    else:
        l.layout = capi.PUBLIC_LAYOUT_QUANTIZED_CSR
        l.nnz = x.nnz
        narrow = x.row_ptr.to(torch.int32)                     # nnz < 2^32: the bits of a uint32
        l.major_ptr, l.minor_idx = narrow.data_ptr(), x.col_idx.data_ptr()
        l._keep = (x, narrow)
    return l


def public_projection(x, dense: torch.Tensor, backward=False) -> torch.Tensor:
    """cb200_public_projection_forward (out = deq(X) dense) or _backward_rhs (grad_rhs = deq(X)^T dense)."""
    l = public_layout(x)
    n = dense.shape[1]
    need = C.c_uint64()
    capi.check(capi.lib().cb200_public_projection_scratch(C.byref(l), C.c_int64(n), C.byref(need)))
    scratch = torch.empty(need.value, dtype=torch.uint8, device=dense.device)
    out = torch.empty(x.cols if backward else x.rows, n, dtype=torch.float32, device=dense.device)
    fn = capi.lib().cb200_public_projection_backward_rhs if backward else capi.lib().cb200_public_projection_forward
    dev = dense.device.index if dense.device.index is not None else torch.cuda.current_device()
    capi.check(fn(C.byref(l), C.c_void_p(dense.data_ptr()), C.c_int64(dense.stride(0)), C.c_int64(n), C.c_void_p(out.data_ptr()),
                  C.c_int64(out.stride(0)), C.c_int32(dev), C.c_void_p(_stream_handle(dense.device)),
                  C.c_void_p(scratch.data_ptr()), C.c_uint64(scratch.numel())))
    return out


# ---- host-buffer entry: what a caller with the matrix in host memory runs -------------------

@dataclass
class HostCsr:
    """Pinned host copy of a quantized CSR (same arrays as QuantizedCsr)."""
    rows: int
    cols: int
    bits: int
    policy: int
    row_ptr: torch.Tensor
    col_idx: torch.Tensor
    packed: torch.Tensor
    scales: torch.Tensor | None
    offsets: torch.Tensor | None
    packed_row_ptr: torch.Tensor | None

    @staticmethod
    def from_device(x: QuantizedCsr) -> "HostCsr":
        def pin(t):
            if t is None:
                return None
            h = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
            h.copy_(t)
            return h
        return HostCsr(x.rows, x.cols, x.bits, x.policy, pin(x.row_ptr), pin(x.col_idx), pin(x.packed), pin(x.scales),
                       pin(x.offsets), pin(x.packed_row_ptr))


class HostForward:
    """Y_host = deq(X_host) W_host with every byte crossing PCIe inside the call: the row range is
    cut into chunks; chunk i+1 is copied to the device while chunk i is multiplied and chunk
    i-1's rows of Y are copied back.  Device buffers are the ones of `x` / `dense` / `out`, which
    the call overwrites."""

    def __init__(self, op: PreparedSpmm, x: QuantizedCsr, dense: torch.Tensor, out: torch.Tensor, host: HostCsr,
                 w_host: torch.Tensor, y_host: torch.Tensor, chunks: int = 16):
        self.op, self.x, self.dense, self.out = op, x, dense, out
        self.host, self.w_host, self.y_host = host, w_host, y_host
        dev = x.device
        self.compute = torch.cuda.current_stream(dev)
        self.h2d = torch.cuda.Stream(device=dev)
        self.d2h = torch.cuda.Stream(device=dev)
        rp = host.row_ptr.numpy()
        prp = None if host.packed_row_ptr is None else host.packed_row_ptr.numpy()
        bounds = np.linspace(0, x.rows, max(1, chunks) + 1).astype(np.int64)
        self.parts = []
        for i in range(len(bounds) - 1):
            r0, r1 = int(bounds[i]), int(bounds[i + 1])
            if r0 == r1:
                continue
            n0, n1 = int(rp[r0]), int(rp[r1])
            p0, p1 = (n0, n1) if prp is None else (int(prp[r0]), int(prp[r1]))
            launch = op.make_launch(x, dense, out, row_begin=r0, row_end=r1, stream=self.compute.cuda_stream)
            self.parts.append((r0, r1, n0, n1, p0, p1, launch))
        small = [host.row_ptr, host.scales, host.offsets, host.packed_row_ptr, w_host]
        self.h2d_bytes = sum(t.numel() * t.element_size() for t in small if t is not None) \
            + host.col_idx.numel() * 4 + host.packed.numel()
        self.d2h_bytes = y_host.numel() * 4

    def run(self) -> None:
        x, h = self.x, self.host
        begin = torch.cuda.Event()
        begin.record(self.compute)
        self.h2d.wait_event(begin)
        self.d2h.wait_event(begin)
        with torch.cuda.stream(self.h2d):
            x.row_ptr.copy_(h.row_ptr, non_blocking=True)
            if h.scales is not None:
                x.scales.copy_(h.scales, non_blocking=True)
            if h.offsets is not None:
                x.offsets.copy_(h.offsets, non_blocking=True)
            if h.packed_row_ptr is not None:
                x.packed_row_ptr.copy_(h.packed_row_ptr, non_blocking=True)
            self.dense.copy_(self.w_host, non_blocking=True)
        for r0, r1, n0, n1, p0, p1, launch in self.parts:
            with torch.cuda.stream(self.h2d):
                x.col_idx[n0:n1].copy_(h.col_idx[n0:n1], non_blocking=True)
                x.packed[p0:p1].copy_(h.packed[p0:p1], non_blocking=True)
                ready = torch.cuda.Event()
                ready.record(self.h2d)
            self.compute.wait_event(ready)
            self.op.run_launch(launch)
            done = torch.cuda.Event()
            done.record(self.compute)
            self.d2h.wait_event(done)
            with torch.cuda.stream(self.d2h):
                self.y_host[r0:r1].copy_(self.out[r0:r1], non_blocking=True)
        end = torch.cuda.Event()
        end.record(self.d2h)
        self.compute.wait_event(end)
