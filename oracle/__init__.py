"""ctypes front end of the CPU oracle.  TEST INFRASTRUCTURE ONLY.

`Oracle()` loads ``oracle/liboracle.so`` (the C restatement in ``oracle.c``); `Reference()`
loads ``oracle/_ref/libcellerator_ref.so`` (the reference's own sources compiled in place)
when it has been built.  Both expose the same method names so that tests can run one
against the other.  Nothing in the product package imports this module; the test-suite, the
smoke check and the CPU-baseline leg of the benchmark do.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_LIB = os.path.join(_HERE, "liboracle.so")
REF_LIB = os.path.join(_HERE, "_ref", "libcellerator_ref.so")

POLICY_PER_GENE_AFFINE = 1
POLICY_COLUMN_SCALE_ROW_OFFSET = 2

EPILOGUE = {"none": 0, "bias": 1, "relu": 2, "gelu_erf": 3, "gelu_tanh": 4, "bias_relu": 5,
            "bias_gelu_erf": 6, "bias_gelu_tanh": 7}


def reference_root() -> str | None:
    """The Cellerator source tree to compile the reference from: the directory CELLERATOR_REFERENCE names, else
    a checkout called `reference` beside this repository.  None when neither holds the Cellerator headers."""
    beside = os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
    for root in (os.environ.get("CELLERATOR_REFERENCE", ""), beside):
        if root and os.path.isdir(os.path.join(root, "include", "Cellerator")):
            return os.path.abspath(root)
    return None


def build(ref: bool | None = None) -> None:
    """Compile liboracle.so, and the reference shim when the reference tree is present."""
    targets = ["all"]
    root = reference_root()
    if ref is None:
        ref = root is not None
    env = dict(os.environ)
    if ref:
        if root is None:
            raise FileNotFoundError("no Cellerator source tree: set CELLERATOR_REFERENCE")
        env["REFERENCE"] = root
        targets.append("ref")
        product = os.path.join(os.path.dirname(_HERE), "cellerator_b200", "lib", "libcellerator_b200.so")
        if os.path.exists(product):
            targets.append("conformance")   # the reference's operation core and planner driving the backend
    subprocess.run(["make", "-C", _HERE, *targets], check=True, capture_output=True, env=env)


def _p(a, ctype):
    if a is None:
        return None
    return a.ctypes.data_as(C.POINTER(ctype))


def _i64(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.int64)


def _f32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


class _Base:
    prefix = ""

    def __init__(self, path):
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        self.lib = C.CDLL(path)

    def _fn(self, name, restype=C.c_int):
        f = getattr(self.lib, self.prefix + name)
        f.restype = restype
        return f

    # ---- layout ---------------------------------------------------------
    def build_packed_row_ptr(self, bits, row_ptr):
        row_ptr = _i64(row_ptr)
        rows = len(row_ptr) - 1
        out = np.zeros(rows + 1, dtype=np.int64)
        total = self._fn("build_packed_row_ptr", C.c_int64)(
            C.c_int(bits), _p(row_ptr, C.c_int64), C.c_int64(rows), _p(out, C.c_int64))
        return out, int(total)

    def build_uniform_block_row_ptr(self, rows, rows_per_block):
        count = 0 if rows <= 0 or rows_per_block <= 0 else -(-rows // rows_per_block)
        out = np.zeros(count + 1, dtype=np.int64)
        rc = self._fn("build_uniform_block_row_ptr", C.c_int64)(
            C.c_int64(rows), C.c_int64(rows_per_block), _p(out, C.c_int64))
        return out, int(rc)

    def get_block(self, row_ptr, packed_row_ptr, block_row_ptr, block_index):
        row_ptr, packed_row_ptr = _i64(row_ptr), _i64(packed_row_ptr)
        brp = _i64(block_row_ptr)
        out = np.zeros(7, dtype=np.int64)
        self._fn("get_block", None)(
            C.c_int64(len(row_ptr) - 1), _p(row_ptr, C.c_int64), _p(packed_row_ptr, C.c_int64),
            _p(brp, C.c_int64), C.c_int64(0 if brp is None else len(brp) - 1), C.c_int64(block_index),
            _p(out, C.c_int64))
        return dict(zip(("block_index", "row_begin", "row_end", "nnz_begin", "nnz_end", "packed_begin",
                         "packed_end"), (int(v) for v in out)))

    # ---- scalar code rules ---------------------------------------------
    def quantize_code(self, bits, value, scale, offset):
        return int(self._fn("quantize_code", C.c_uint)(C.c_int(bits), C.c_float(value), C.c_float(scale),
                                                       C.c_float(offset)))

    def dequantize_code(self, code, scale, offset):
        return float(self._fn("dequantize_code", C.c_float)(C.c_uint(code), C.c_float(scale), C.c_float(offset)))

    # ---- BELL -----------------------------------------------------------
    def bell_pack(self, bits, policy, rows, cols, block_size, ell_cols, row_stride, block_col_idx, scales,
                  offsets, values_by_slot):
        bci = np.ascontiguousarray(block_col_idx, dtype=np.uint32)
        scales, offsets, vals = _f32(scales), _f32(offsets), _f32(values_by_slot)
        packed = np.full(rows * row_stride, 0xAA, dtype=np.uint8)
        rc = self._fn(self._bell_pack_name)(
            C.c_int(bits), C.c_int(policy), C.c_int64(rows), C.c_int64(cols), C.c_int(block_size),
            C.c_int64(ell_cols), C.c_int64(row_stride), _p(bci, C.c_uint32), _p(scales, C.c_float),
            _p(offsets, C.c_float), _p(vals, C.c_float), _p(packed, C.c_uint8))
        assert rc == 0, rc
        return packed

    def bell_unpack(self, bits, policy, rows, cols, block_size, ell_cols, row_stride, block_col_idx, scales,
                    offsets, packed):
        bci = np.ascontiguousarray(block_col_idx, dtype=np.uint32)
        scales, offsets = _f32(scales), _f32(offsets)
        packed = np.ascontiguousarray(packed, dtype=np.uint8)
        out = np.zeros(rows * ell_cols, dtype=np.float32)
        rc = self._fn(self._bell_unpack_name)(
            C.c_int(bits), C.c_int(policy), C.c_int64(rows), C.c_int64(cols), C.c_int(block_size),
            C.c_int64(ell_cols), C.c_int64(row_stride), _p(bci, C.c_uint32), _p(scales, C.c_float),
            _p(offsets, C.c_float), _p(packed, C.c_uint8), _p(out, C.c_float))
        assert rc == 0, rc
        return out.reshape(rows, ell_cols)

    # ---- referee ----------------------------------------------------------
    def spmm_reference(self, m, k, n, row_offsets, columns, values, rhs, *, transpose_sparse=False,
                       transpose_dense=False, rhs_col_major=False, rhs_ld=None, alpha=1.0, beta=0.0,
                       initial=None, initial_col_major=False, initial_ld=0, epilogue="none", bias=None):
        ro = np.ascontiguousarray(row_offsets, dtype=np.uint64)
        ci = np.ascontiguousarray(columns, dtype=np.uint32)
        vals, rhs, initial, bias = _f32(values), _f32(rhs), _f32(initial), _f32(bias)
        if rhs_ld is None:
            rr, rc_ = (n, k) if transpose_dense else (k, n)
            rhs_ld = rr if rhs_col_major else rc_
        ref = np.zeros(m * n, dtype=np.float64)
        rc = self._fn("spmm_reference")(
            C.c_uint64(m), C.c_uint64(k), C.c_uint64(n), C.c_int(int(transpose_sparse)),
            C.c_int(int(transpose_dense)), C.c_uint64(len(ci)), _p(ro, C.c_uint64), _p(ci, C.c_uint32),
            _p(vals, C.c_float), _p(rhs, C.c_float), C.c_int(int(rhs_col_major)), C.c_uint64(rhs_ld),
            C.c_double(alpha), C.c_double(beta), _p(initial, C.c_float), C.c_int(int(initial_col_major)),
            C.c_uint64(initial_ld), C.c_int(EPILOGUE[epilogue]), _p(bias, C.c_float), _p(ref, C.c_double),
            C.c_uint64(m * n))
        if rc != 0:
            raise RuntimeError(f"spmm_reference status {rc}")
        return ref.reshape(m, n)

    # ---- CSR -> physical Blocked-ELL lowering ------------------------------
    BELL_GEOMETRY = ("state", "padded_rows", "padded_features", "block_rows", "ell_blocks_per_row", "ell_columns",
                     "column_index_count", "value_bytes", "occupied_blocks", "stored_blocks", "dense_value_slots",
                     "persistent_bytes", "source_bytes")
    BELL_METRICS = ("scalar_occupancy", "ell_slot_utilization", "value_slot_expansion", "storage_expansion")

    def bell_lowering(self, row_offsets, feature_ids, values, features, fb_offsets, fperm, rperm, block_size, *,
                      materialize=True, max_value_expansion=64.0, max_storage_expansion=64.0,
                      max_persistent=2 ** 63, values_layout=0, row_stride_bytes=0):
        """query (+ materialize) for one block size.  Returns (status, geometry dict, padded feature-block
        offsets, column indices, value bytes); the arrays are None for a query or a rejected candidate."""
        u32 = lambda a: np.ascontiguousarray(a, dtype=np.uint32)
        ro, fid, fbo, fp, rp = u32(row_offsets), u32(feature_ids), u32(fb_offsets), u32(fperm), u32(rperm)
        vals = np.ascontiguousarray(values)
        rows, nnz = len(ro) - 1, len(fid)
        value_size = vals.dtype.itemsize if vals.ndim == 1 else vals.shape[1] * vals.dtype.itemsize
        finv = np.zeros(features, dtype=np.uint32)
        finv[fp % max(features, 1)] = np.arange(len(fp), dtype=np.uint32)
        rinv = np.zeros(rows, dtype=np.uint32)
        if rows:
            rinv[rp % rows] = np.arange(len(rp), dtype=np.uint32)
        geo, met = np.zeros(13, dtype=np.uint64), np.zeros(4, dtype=np.float64)
        fn = self._fn("bell_lowering")
        args = lambda pfo, ci, vo: (
            C.c_uint32(rows), C.c_uint32(features), C.c_uint32(nnz), C.c_uint32(value_size), _p(ro, C.c_uint32),
            _p(fid, C.c_uint32), vals.ctypes.data_as(C.c_void_p), C.c_uint32(len(fbo) - 1), _p(fbo, C.c_uint32),
            _p(fp, C.c_uint32), _p(finv, C.c_uint32), _p(rp, C.c_uint32), _p(rinv, C.c_uint32), C.c_uint32(block_size),
            C.c_double(max_value_expansion), C.c_double(max_storage_expansion), C.c_uint64(max_persistent),
            _p(geo, C.c_uint64), _p(met, C.c_double), _p(pfo, C.c_uint32), _p(ci, C.c_int32),
            None if vo is None else vo.ctypes.data_as(C.c_void_p), C.c_uint64(0 if ci is None else len(ci)),
            C.c_uint64(0 if vo is None else len(vo)), C.c_int(values_layout), C.c_uint64(row_stride_bytes))
        status = fn(*args(None, None, None))
        summary = lambda: {**dict(zip(self.BELL_GEOMETRY, (int(v) for v in geo))), **dict(zip(self.BELL_METRICS, met.tolist()))}
        if status != 0 or not materialize or int(geo[0]) != 0:
            return status, summary(), None, None, None
        pfo = np.zeros(len(fbo), dtype=np.uint32)
        ci = np.zeros(int(geo[6]), dtype=np.int32)
        nbytes = int(geo[1]) * row_stride_bytes if values_layout == 1 else int(geo[7])
        vo = np.full(nbytes, 0xCD, dtype=np.uint8)
        status = fn(*args(pfo, ci, vo))
        return status, summary(), pfo, ci, vo

    def pack_dense_operand(self, source, fperm, *, col_major=False, fb_offsets=None, padded_offsets=None):
        """packed[execution] = source[fperm[execution]] (2-D source [features][columns], or its transpose when
        col_major); with feature blocks, in the padded physical feature order of a Blocked-ELL lowering."""
        src = np.ascontiguousarray(source)
        features, columns = (src.shape[1], src.shape[0]) if col_major else src.shape
        fp = np.ascontiguousarray(fperm, dtype=np.uint32)
        fbo = None if fb_offsets is None else np.ascontiguousarray(fb_offsets, dtype=np.uint32)
        pfo = None if padded_offsets is None else np.ascontiguousarray(padded_offsets, dtype=np.uint32)
        rows = features if fbo is None else int(pfo[-1])
        out = np.full((rows, columns), 0, dtype=src.dtype)
        rc = self._fn("pack_dense_operand")(
            C.c_uint32(features), C.c_uint64(columns), C.c_uint64(src.shape[1]), C.c_int(int(col_major)),
            C.c_uint32(src.dtype.itemsize), _p(fp, C.c_uint32), src.ctypes.data_as(C.c_void_p),
            C.c_uint32(0 if fbo is None else len(fbo) - 1), _p(fbo, C.c_uint32), _p(pfo, C.c_uint32),
            out.ctypes.data_as(C.c_void_p))
        if rc != 0:
            raise RuntimeError(f"pack_dense_operand status {rc}")
        return out

    def build_execution_csr(self, row_offsets, block_ids, local_ids, canonical_ids, features, fb_offsets, fperm):
        """-> (status, execution feature ids) of an ordered plan partition (see oracle.c)."""
        u32 = lambda a: np.ascontiguousarray(a, dtype=np.uint32)
        ro, bi, li, ci, fbo, fp = u32(row_offsets), u32(block_ids), u32(local_ids), u32(canonical_ids), u32(fb_offsets), u32(fperm)
        out = np.full(len(bi), 0xFFFFFFFF, dtype=np.uint32)
        status = self._fn("build_execution_csr")(
            C.c_uint32(len(ro) - 1), C.c_uint32(len(bi)), C.c_uint32(features), C.c_uint32(len(fbo) - 1), _p(fbo, C.c_uint32),
            _p(fp, C.c_uint32), _p(ro, C.c_uint32), _p(bi, C.c_uint32), _p(li, C.c_uint32), _p(ci, C.c_uint32), _p(out, C.c_uint32))
        return status, out

    def digest_f32(self, values):
        v = _f32(values)
        out = np.zeros(2, dtype=np.uint64)
        self._digest(v, out)
        return int(out[0]), int(out[1])


class Oracle(_Base):
    """The C restatement (oracle.c)."""
    prefix = "orc_"
    _bell_pack_name = "bell_pack_row_major"
    _bell_unpack_name = "bell_unpack_row_major"

    def __init__(self):
        if not os.path.exists(ORACLE_LIB):
            build(ref=False)
        super().__init__(ORACLE_LIB)

    def request_contract(self, fields):
        """fields: the 48 values of a spmm_request in declaration order -> (validation code, trivial kind, low, high)"""
        f = np.ascontiguousarray(fields, dtype=np.uint64)
        assert f.size == 48
        out = np.zeros(4, dtype=np.uint64)
        self._fn("request_contract", None)(_p(f, C.c_uint64), _p(out, C.c_uint64))
        return tuple(int(v) for v in out)

    def _digest(self, v, out):
        self._fn("digest_f32", None)(_p(v, C.c_float), C.c_uint64(v.shape[0]), C.c_uint64(v.shape[1]),
                                     C.c_uint64(v.shape[1]), C.c_uint32(4), _p(out, C.c_uint64))

    # ---- gene-major copy and the order-fixed transpose (restatement only: the reference's CSC
    # transposer is device code, and its transpose kernel adds in atomic order) ----------------
    def qcsr_gene_major(self, bits, cols, row_ptr, packed_row_ptr, col_idx, packed):
        """-> (status, col_ptr, row_idx, codes): stable CSR -> CSC of the codes (see oracle.c)."""
        row_ptr, prp = _i64(row_ptr), _i64(packed_row_ptr)
        col_idx = np.ascontiguousarray(col_idx, dtype=np.int32)
        packed = np.ascontiguousarray(packed, dtype=np.uint8)
        rows, nnz = len(row_ptr) - 1, int(row_ptr[-1])
        col_ptr = np.zeros(cols + 1, dtype=np.int64)
        row_idx = np.zeros(max(nnz, 1), dtype=np.int32)
        codes = np.zeros(max(nnz, 1), dtype=np.uint8)
        rc = self._fn("qcsr_gene_major")(
            C.c_int(bits), C.c_int64(rows), C.c_int64(cols), _p(row_ptr, C.c_int64), _p(prp, C.c_int64),
            _p(col_idx, C.c_int32), _p(packed, C.c_uint8), _p(col_ptr, C.c_int64), _p(row_idx, C.c_int32), _p(codes, C.c_uint8))
        return rc, col_ptr, row_idx[:nnz], codes[:nnz]

    def qcsr_transpose_ordered(self, policy, col_ptr, row_idx, codes, scales, offsets, g, row_begin, row_end,
                               alpha=1.0, beta=0.0, out=None):
        """fp32 result of the deterministic transpose schedule, bit for bit (see oracle.c)."""
        col_ptr = _i64(col_ptr)
        row_idx = np.ascontiguousarray(row_idx, dtype=np.int32)
        codes = np.ascontiguousarray(codes, dtype=np.uint8)
        scales, offsets, g = _f32(scales), _f32(offsets), _f32(g)
        cols, n = len(col_ptr) - 1, g.shape[1]
        out = np.zeros((cols, n), dtype=np.float32) if out is None else np.ascontiguousarray(out, dtype=np.float32).copy()
        rc = self._fn("qcsr_transpose_ordered")(
            C.c_int(policy), C.c_int64(cols), C.c_int64(n), _p(col_ptr, C.c_int64), _p(row_idx, C.c_int32),
            _p(codes, C.c_uint8), _p(scales, C.c_float), _p(offsets, C.c_float), _p(g, C.c_float), C.c_int64(g.shape[1]),
            C.c_int64(row_begin), C.c_int64(row_end), C.c_float(alpha), C.c_float(beta), _p(out, C.c_float), C.c_int64(n))
        assert rc == 0, rc
        return out

    def pack_csr(self, bits, policy, row_ptr, packed_row_ptr, col_idx, scales, offsets, values,
                 row_begin=0, row_end=None, value_base=0, total_bytes=None):
        row_ptr, prp = _i64(row_ptr), _i64(packed_row_ptr)
        col_idx = np.ascontiguousarray(col_idx, dtype=np.int32)
        scales, offsets, values = _f32(scales), _f32(offsets), _f32(values)
        rows = len(row_ptr) - 1
        row_end = rows if row_end is None else row_end
        packed = np.zeros(int(prp[-1]) if total_bytes is None else total_bytes, dtype=np.uint8)
        rc = self._fn("pack_csr_rows")(
            C.c_int(bits), C.c_int(policy), C.c_int64(row_begin), C.c_int64(row_end), _p(row_ptr, C.c_int64),
            _p(prp, C.c_int64), _p(col_idx, C.c_int32), _p(scales, C.c_float), _p(offsets, C.c_float),
            C.c_int64(value_base), _p(values, C.c_float), _p(packed, C.c_uint8))
        assert rc == 0, rc
        return packed

    def unpack_csr(self, bits, policy, row_ptr, packed_row_ptr, col_idx, scales, offsets, packed,
                   row_begin=0, row_end=None, value_base=None):
        row_ptr, prp = _i64(row_ptr), _i64(packed_row_ptr)
        col_idx = np.ascontiguousarray(col_idx, dtype=np.int32)
        scales, offsets = _f32(scales), _f32(offsets)
        packed = np.ascontiguousarray(packed, dtype=np.uint8)
        rows = len(row_ptr) - 1
        row_end = rows if row_end is None else row_end
        base = int(row_ptr[row_begin]) if value_base is None else value_base
        out = np.zeros(int(row_ptr[row_end]) - base, dtype=np.float32)
        rc = self._fn("unpack_csr_rows")(
            C.c_int(bits), C.c_int(policy), C.c_int64(row_begin), C.c_int64(row_end), _p(row_ptr, C.c_int64),
            _p(prp, C.c_int64), _p(col_idx, C.c_int32), _p(scales, C.c_float), _p(offsets, C.c_float),
            _p(packed, C.c_uint8), C.c_int64(base), _p(out, C.c_float))
        assert rc == 0, rc
        return out

    def extract_codes(self, bits, row_ptr, packed_row_ptr, packed):
        row_ptr, prp = _i64(row_ptr), _i64(packed_row_ptr)
        packed = np.ascontiguousarray(packed, dtype=np.uint8)
        out = np.zeros(int(row_ptr[-1]), dtype=np.uint8)
        rc = self._fn("extract_csr_codes")(C.c_int(bits), C.c_int64(len(row_ptr) - 1), _p(row_ptr, C.c_int64),
                                           _p(prp, C.c_int64), _p(packed, C.c_uint8), _p(out, C.c_uint8))
        assert rc == 0, rc
        return out

    def bell_to_csr(self, bits, policy, rows, cols, block_size, ell_cols, row_stride, block_col_idx, scales,
                    offsets, packed):
        bci = np.ascontiguousarray(block_col_idx, dtype=np.uint32)
        scales, offsets = _f32(scales), _f32(offsets)
        packed = np.ascontiguousarray(packed, dtype=np.uint8)
        ro = np.zeros(rows + 1, dtype=np.uint64)
        f = self._fn("bell_to_csr", C.c_int64)
        args = [C.c_int(bits), C.c_int(policy), C.c_int64(rows), C.c_int64(cols), C.c_int(block_size),
                C.c_int64(ell_cols), C.c_int64(row_stride), _p(bci, C.c_uint32), _p(scales, C.c_float),
                _p(offsets, C.c_float), _p(packed, C.c_uint8), _p(ro, C.c_uint64)]
        count = f(*args, None, None)
        assert count >= 0
        cols_out = np.zeros(count, dtype=np.uint32)
        vals = np.zeros(count, dtype=np.float32)
        f(*args, _p(cols_out, C.c_uint32), _p(vals, C.c_float))
        return ro, cols_out, vals

    def _range_call(self, name, bits, policy, row_begin, row_end, cols, n, row_ptr, packed_row_ptr, col_idx,
                    packed, scales, offsets, dense, out_rows):
        row_ptr, prp = _i64(row_ptr), _i64(packed_row_ptr)
        col_idx = np.ascontiguousarray(col_idx, dtype=np.int32)
        packed = np.ascontiguousarray(packed, dtype=np.uint8)
        scales, offsets, dense = _f32(scales), _f32(offsets), _f32(dense)
        nnz = int(row_ptr[row_end] - row_ptr[row_begin])
        sv = np.zeros(max(nnz, 1), dtype=np.float32)
        so = np.zeros(row_end - row_begin + 1, dtype=np.uint64)
        ref = np.zeros(out_rows * n, dtype=np.float64)
        rc = self._fn(name)(
            C.c_int(bits), C.c_int(policy), C.c_int64(row_begin), C.c_int64(row_end), C.c_int64(cols),
            C.c_int64(n), _p(row_ptr, C.c_int64), _p(prp, C.c_int64), _p(col_idx, C.c_int32),
            _p(packed, C.c_uint8), _p(scales, C.c_float), _p(offsets, C.c_float), _p(dense, C.c_float),
            C.c_int64(dense.shape[1]), _p(sv, C.c_float), _p(so, C.c_uint64), _p(ref, C.c_double))
        if rc != 0:
            raise RuntimeError(f"{name} status {rc}")
        return ref.reshape(out_rows, n)

    def qcsr_forward(self, bits, policy, row_ptr, packed_row_ptr, col_idx, packed, scales, offsets, w,
                     cols, row_begin=0, row_end=None):
        """decode + referee over rows [row_begin, row_end): Y rows as float64."""
        row_end = len(row_ptr) - 1 if row_end is None else row_end
        return self._range_call("qcsr_forward_rows", bits, policy, row_begin, row_end, cols, w.shape[1],
                                row_ptr, packed_row_ptr, col_idx, packed, scales, offsets, w,
                                row_end - row_begin)

    def qcsr_transpose(self, bits, policy, row_ptr, packed_row_ptr, col_idx, packed, scales, offsets, g,
                       cols, row_begin=0, row_end=None):
        """decode + transposed referee over rows [row_begin, row_end): partial G' (cols x n) as float64."""
        row_end = len(row_ptr) - 1 if row_end is None else row_end
        return self._range_call("qcsr_transpose_rows", bits, policy, row_begin, row_end, cols, g.shape[1],
                                row_ptr, packed_row_ptr, col_idx, packed, scales, offsets, g, cols)

    def compare(self, reference, candidate, tol_abs=0.0, tol_rel=0.0, rel_floor=1e-30):
        ref = np.ascontiguousarray(reference, dtype=np.float64).ravel()
        cand = _f32(candidate).ravel()
        out = np.zeros(8, dtype=np.float64)
        rc = self._fn("compare")(_p(ref, C.c_double), _p(cand, C.c_float), C.c_uint64(ref.size),
                                 C.c_double(tol_abs), C.c_double(tol_rel), C.c_double(rel_floor),
                                 _p(out, C.c_double))
        keys = ("max_abs", "max_rel", "mean_abs", "rmse", "mismatch_count", "worst_index", "nonfinite_ref",
                "nonfinite_cand")
        d = dict(zip(keys, out.tolist()))
        d["status"] = rc
        return d


class Reference(_Base):
    """The reference's own sources (ref_shim.cc); whole-matrix calls only."""
    prefix = "ref_"
    _bell_pack_name = "bell_pack"
    _bell_unpack_name = "bell_unpack"

    def __init__(self):
        super().__init__(REF_LIB)

    @staticmethod
    def available():
        return os.path.exists(REF_LIB)

    def request_contract(self, fields):
        """fields: the 48 values of a spmm_request in declaration order -> (validation code, trivial kind, low, high)"""
        f = np.ascontiguousarray(fields, dtype=np.uint64)
        assert f.size == 48
        out = np.zeros(4, dtype=np.uint64)
        self._fn("request_contract", None)(_p(f, C.c_uint64), _p(out, C.c_uint64))
        return tuple(int(v) for v in out)

    def _digest(self, v, out):
        self._fn("digest_f32", None)(_p(v, C.c_float), C.c_uint64(v.shape[0]), C.c_uint64(v.shape[1]),
                                     C.c_uint64(v.shape[1]), _p(out, C.c_uint64))

    def pack_csr(self, bits, policy, row_ptr, packed_row_ptr, col_idx, scales, offsets, values, cols=None):
        row_ptr, prp = _i64(row_ptr), _i64(packed_row_ptr)
        col_idx = np.ascontiguousarray(col_idx, dtype=np.int32)
        scales, offsets, values = _f32(scales), _f32(offsets), _f32(values)
        cols = int(col_idx.max()) + 1 if cols is None else cols
        packed = np.zeros(int(prp[-1]), dtype=np.uint8)
        rc = self._fn("pack_csr")(
            C.c_int(bits), C.c_int(policy), C.c_int64(len(row_ptr) - 1), C.c_int64(cols), _p(row_ptr, C.c_int64),
            _p(prp, C.c_int64), _p(col_idx, C.c_int32), _p(scales, C.c_float), _p(offsets, C.c_float),
            _p(values, C.c_float), _p(packed, C.c_uint8))
        assert rc == 0, rc
        return packed

    def unpack_csr(self, bits, policy, row_ptr, packed_row_ptr, col_idx, scales, offsets, packed, cols=None):
        row_ptr, prp = _i64(row_ptr), _i64(packed_row_ptr)
        col_idx = np.ascontiguousarray(col_idx, dtype=np.int32)
        scales, offsets = _f32(scales), _f32(offsets)
        packed = np.ascontiguousarray(packed, dtype=np.uint8)
        cols = int(col_idx.max()) + 1 if cols is None else cols
        out = np.zeros(int(row_ptr[-1]), dtype=np.float32)
        rc = self._fn("unpack_csr")(
            C.c_int(bits), C.c_int(policy), C.c_int64(len(row_ptr) - 1), C.c_int64(cols), _p(row_ptr, C.c_int64),
            _p(prp, C.c_int64), _p(col_idx, C.c_int32), _p(scales, C.c_float), _p(offsets, C.c_float),
            _p(packed, C.c_uint8), _p(out, C.c_float))
        assert rc == 0, rc
        return out
