"""ctypes binding of libcellerator_b200.so (the C ABI of include/cellerator_b200.h).

This is a thin driver for tests and the benchmark: it passes raw device pointers (taken from
torch tensors, which only provide memory and streams) to the library.  There is no fallback:
if the library is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "lib", "libcellerator_b200.so")
SYNTH_PATH = os.path.join(HERE, "lib", "libcb200_synth.so")

ABI_VERSION = 2
ALL_ROWS = -1      # cb200_launch.row_end: up to the last row

SUCCESS, INVALID_ARGUMENT, INVALID_SHAPE, UNSUPPORTED, CUDA_ERROR, INTERNAL_ERROR, STALE_STRUCTURE, \
    INSUFFICIENT_WORKSPACE, INVALID_STREAM, SEALED = range(10)
STALE_VALUE, COMM_NOT_READY, DEVICE_WAIT_TIMEOUT = 10, 11, 12

DTYPE_U8, DTYPE_U4, DTYPE_F16, DTYPE_BF16, DTYPE_F32, DTYPE_F64 = 2, 32, 6, 7, 8, 9
DECODE_PER_GENE_AFFINE, DECODE_COLUMN_SCALE_ROW_OFFSET = 1, 2
PROJECTION_CSR, PROJECTION_BLOCKED_ELL, PROJECTION_TRANSPOSE = 5, 8, 10
CAP_DETERMINISTIC, CAP_GRAPH_CAPTURE, CAP_PERSISTENT_PREPROCESSING, CAP_COMPOSED_EPILOGUE = 1, 2, 4, 8


# cb200_status values the Python side names
STATUS_SUCCESS, STATUS_INVALID_ARGUMENT, STATUS_INVALID_SHAPE, STATUS_UNSUPPORTED = 0, 1, 2, 3


class Cb200Error(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"cb200 status {status}: {message}")
        self.status = status
        self.message = message


class QCsr(C.Structure):
    _fields_ = [("version", C.c_uint32), ("size", C.c_size_t), ("rows", C.c_int64), ("cols", C.c_int64),
                ("nnz", C.c_int64), ("bits", C.c_int32), ("policy", C.c_int32), ("row_ptr", C.c_void_p),
                ("packed_row_ptr", C.c_void_p), ("col_idx", C.c_void_p), ("packed_values", C.c_void_p),
                ("scales", C.c_void_p), ("offsets", C.c_void_p)]


class CsrBlock(C.Structure):
    _fields_ = [(n, C.c_int64) for n in ("block_index", "row_begin", "row_end", "nnz_begin", "nnz_end",
                                         "packed_begin", "packed_end")]


class QBell(C.Structure):
    _fields_ = [("version", C.c_uint32), ("size", C.c_size_t), ("rows", C.c_int64), ("cols", C.c_int64),
                ("block_size", C.c_int32), ("ell_cols", C.c_int32), ("row_stride_bytes", C.c_int64),
                ("bits", C.c_int32), ("policy", C.c_int32), ("block_col_idx", C.c_void_p),
                ("packed_values", C.c_void_p), ("scales", C.c_void_p), ("offsets", C.c_void_p)]


class NumericPolicy(C.Structure):
    _fields_ = [("version", C.c_uint32), ("size", C.c_size_t), ("sparse_storage", C.c_int32),
                ("dense_storage", C.c_int32), ("output_storage", C.c_int32), ("multiply", C.c_int32),
                ("accumulation", C.c_int32), ("quantized", C.c_int32)]


class Capability(C.Structure):
    _fields_ = [("version", C.c_uint32), ("size", C.c_size_t), ("supported", C.c_int32), ("flags", C.c_uint32),
                ("persistent_bytes", C.c_uint64), ("transient_bytes", C.c_uint64), ("name", C.c_char_p)]


class SpmmProblem(C.Structure):
    _fields_ = [("version", C.c_uint32), ("size", C.c_size_t), ("projection", C.c_int32), ("m", C.c_int64),
                ("k", C.c_int64), ("n", C.c_int64), ("nnz", C.c_int64), ("bits", C.c_int32), ("policy", C.c_int32),
                ("dense_dtype", C.c_int32), ("device", C.c_int32), ("structure_epoch", C.c_uint64),
                ("host_row_ptr", C.c_void_p), ("deterministic", C.c_int32), ("multiply", C.c_int32),
                ("device_matrix", C.POINTER(QCsr)), ("persistent_limit_bytes", C.c_uint64), ("value_generation", C.c_uint64),
                ("schedule_hint", C.c_char_p), ("persistent", C.c_void_p), ("persistent_bytes", C.c_uint64),
                ("prepare_stream", C.c_void_p)]


class Launch(C.Structure):
    _fields_ = [("version", C.c_uint32), ("size", C.c_size_t), ("csr", C.POINTER(QCsr)), ("bell", C.POINTER(QBell)),
                ("dense", C.c_void_p), ("dense_ld", C.c_int64), ("out", C.c_void_p), ("out_ld", C.c_int64),
                ("alpha", C.c_float), ("beta", C.c_float), ("structure_epoch", C.c_uint64), ("row_begin", C.c_int64),
                ("row_end", C.c_int64), ("stream", C.c_void_p), ("device", C.c_int32), ("workspace_device", C.c_int32),
                ("workspace", C.c_void_p), ("workspace_bytes", C.c_uint64), ("bias", C.c_void_p),
                ("epilogue", C.c_int32), ("value_generation", C.c_uint64)]


# cb200_epilogue: epilogue_kind of the request contract (operation.hh:49-61, same values)
EPILOGUE = {"none": 0, "bias": 1, "relu": 2, "gelu_erf": 3, "gelu_tanh": 4, "bias_relu": 5,
            "bias_gelu_erf": 6, "bias_gelu_tanh": 7}


class BellLoweringInput(C.Structure):
    _fields_ = [("version", C.c_uint32), ("size", C.c_size_t), ("rows", C.c_uint32), ("features", C.c_uint32),
                ("nnz", C.c_uint32), ("value_size_bytes", C.c_uint32), ("row_offsets", C.c_void_p),
                ("feature_ids", C.c_void_p), ("values", C.c_void_p), ("feature_block_count", C.c_uint32),
                ("feature_block_offsets", C.c_void_p), ("feature_permutation", C.c_void_p),
                ("inverse_feature_permutation", C.c_void_p), ("row_permutation", C.c_void_p),
                ("inverse_row_permutation", C.c_void_p), ("device", C.c_int32)]


class BellLoweringPolicy(C.Structure):
    _fields_ = [("maximum_value_slot_expansion", C.c_double), ("maximum_storage_expansion", C.c_double),
                ("maximum_persistent_bytes", C.c_uint64)]


class BellGeometry(C.Structure):
    _fields_ = [("version", C.c_uint32), ("size", C.c_size_t), ("state", C.c_int32), ("block_size", C.c_uint32),
                ("rows", C.c_uint32), ("features", C.c_uint32), ("padded_rows", C.c_uint32),
                ("padded_features", C.c_uint32), ("block_rows", C.c_uint32), ("ell_blocks_per_row", C.c_uint32),
                ("ell_columns", C.c_uint32), ("feature_block_offset_count", C.c_uint64),
                ("column_index_count", C.c_uint64), ("value_bytes", C.c_uint64), ("occupied_blocks", C.c_uint64),
                ("stored_blocks", C.c_uint64), ("dense_value_slots", C.c_uint64), ("persistent_bytes", C.c_uint64),
                ("source_bytes", C.c_uint64), ("scalar_occupancy", C.c_double), ("ell_slot_utilization", C.c_double),
                ("value_slot_expansion", C.c_double), ("storage_expansion", C.c_double)]


BELL_VALUES_BLOCK_MAJOR, BELL_VALUES_ROW_MAJOR = 0, 1


class PublicLayout(C.Structure):
    _fields_ = [("version", C.c_uint32), ("size", C.c_size_t), ("layout", C.c_int32), ("rows", C.c_uint32),
                ("cols", C.c_uint32), ("nnz", C.c_uint32), ("block_size", C.c_uint32), ("ell_cols", C.c_uint32),
                ("row_stride_bytes", C.c_uint32), ("bits", C.c_uint32), ("decode_policy", C.c_uint32),
                ("major_ptr", C.c_void_p), ("minor_idx", C.c_void_p), ("block_col_idx", C.c_void_p),
                ("packed_values", C.c_void_p), ("column_scales", C.c_void_p), ("column_offsets", C.c_void_p),
                ("row_offsets", C.c_void_p)]


PUBLIC_LAYOUT_QUANTIZED_BLOCKED_ELL, PUBLIC_LAYOUT_QUANTIZED_CSR = 4, 5


class ExecutionCsr(C.Structure):
    _fields_ = [("version", C.c_uint32), ("size", C.c_size_t), ("rows", C.c_uint32), ("features", C.c_uint32),
                ("nnz", C.c_uint32), ("row_offsets", C.c_void_p), ("block_ids", C.c_void_p),
                ("local_feature_ids", C.c_void_p), ("canonical_feature_ids", C.c_void_p),
                ("feature_block_count", C.c_uint32), ("feature_block_offsets", C.c_void_p),
                ("feature_permutation", C.c_void_p), ("execution_feature_ids", C.c_void_p), ("workspace", C.c_void_p),
                ("workspace_bytes", C.c_uint64), ("status_word", C.c_void_p), ("device", C.c_int32)]


class DensePack(C.Structure):
    _fields_ = [("version", C.c_uint32), ("size", C.c_size_t), ("feature_permutation", C.c_void_p),
                ("source", C.c_void_p), ("features", C.c_uint32), ("columns", C.c_uint64),
                ("leading_dimension", C.c_uint64), ("source_col_major", C.c_int32), ("value_size_bytes", C.c_uint32),
                ("feature_block_count", C.c_uint32), ("feature_block_offsets", C.c_void_p),
                ("padded_feature_block_offsets", C.c_void_p), ("packed", C.c_void_p),
                ("packed_capacity_bytes", C.c_uint64), ("status_word", C.c_void_p), ("device", C.c_int32)]


class FeatureOrderIdentity(C.Structure):
    _fields_ = [("schema_version", C.c_uint32), ("kind", C.c_uint32), ("feature_count", C.c_uint32),
                ("feature_axis_identity_version", C.c_uint32), ("feature_axis_identity", C.c_uint64),
                ("packing_geometry_identity", C.c_uint64)]


class ScalarValue(C.Structure):
    _fields_ = [("type_code", C.c_uint32), ("reserved", C.c_uint32), ("bits", C.c_uint64)]


class SpmmRequest(C.Structure):
    _fields_ = [("schema_version", C.c_uint32), ("operation", C.c_uint32), ("m", C.c_uint64), ("k", C.c_uint64),
                ("n", C.c_uint64), ("sparse_nnz", C.c_uint64), ("structure_schema_version", C.c_uint32),
                ("structure_identity_version", C.c_uint32), ("structure_value", C.c_uint64),
                ("transpose_sparse", C.c_uint32), ("transpose_dense", C.c_uint32), ("dense_rhs_layout", C.c_uint32),
                ("output_layout", C.c_uint32), ("dense_rhs_leading_dimension", C.c_uint64),
                ("output_leading_dimension", C.c_uint64), ("sparse_storage_type_code", C.c_uint32),
                ("dense_storage_type_code", C.c_uint32), ("output_storage_type_code", C.c_uint32),
                ("compute_type_code", C.c_uint32), ("accumulation_type_code", C.c_uint32), ("alpha", ScalarValue),
                ("beta", ScalarValue), ("determinism", C.c_uint32), ("workspace_kind", C.c_uint32),
                ("workspace_reserved", C.c_uint32), ("workspace_byte_limit", C.c_uint64), ("reuse_kind", C.c_uint32),
                ("reuse_reserved", C.c_uint32), ("reuse_expected_run_count", C.c_uint64), ("epilogue_kind", C.c_uint32),
                ("epilogue_bias_type_code", C.c_uint32), ("epilogue_bias_element_count", C.c_uint64),
                ("sparse_feature_order", FeatureOrderIdentity), ("dense_feature_order", FeatureOrderIdentity)]


# real::value_* type codes of the request contract (include/Cellerator/types.cuh:150-158)
TYPE_F16, TYPE_F32, TYPE_F64, TYPE_BF16 = 3, 4, 5, 6


class QBellHost(C.Structure):
    _fields_ = [("rows", C.c_uint32), ("cols", C.c_uint32), ("nnz", C.c_uint32), ("block_size", C.c_uint32),
                ("ell_cols", C.c_uint32), ("bits", C.c_uint32), ("row_stride_bytes", C.c_uint32),
                ("decode_policy", C.c_uint32), ("flags", C.c_uint32), ("storage", C.c_void_p),
                ("block_col_idx", C.c_void_p), ("packed_values", C.c_void_p), ("column_scales", C.c_void_p),
                ("column_offsets", C.c_void_p), ("row_offsets", C.c_void_p)]


class FleetOptions(C.Structure):
    _fields_ = [("version", C.c_uint32), ("size", C.c_size_t), ("device_count", C.c_int32),
                ("devices", C.POINTER(C.c_int32)), ("streams", C.POINTER(C.c_void_p)), ("enable_peer_access", C.c_int32),
                ("world_size", C.c_int32), ("world_rank", C.c_int32), ("nccl_unique_id", C.c_void_p),
                ("nccl_library", C.c_char_p)]


class HostStageOptions(C.Structure):
    _fields_ = [("version", C.c_uint32), ("size", C.c_size_t), ("device", C.c_int32), ("k", C.c_int64), ("n", C.c_int64),
                ("bits", C.c_int32), ("policy", C.c_int32), ("dense_dtype", C.c_int32), ("multiply", C.c_int32),
                ("max_chunk_rows", C.c_int64), ("max_chunk_nnz", C.c_int64), ("chunk_buffers", C.c_int32),
                ("narrow_indices", C.c_int32), ("host_threads", C.c_int32)]


class AllocationAccounting(C.Structure):
    _fields_ = [("current_bytes", C.c_uint64), ("high_water_bytes", C.c_uint64), ("allocation_count", C.c_uint64)]


class SessionAccounting(C.Structure):
    _fields_ = [("structure", AllocationAccounting), ("plan", AllocationAccounting), ("graph_stable", AllocationAccounting),
                ("transient", AllocationAccounting), ("device_query_count", C.c_uint64), ("handle_prepare_count", C.c_uint64),
                ("launch_bind_count", C.c_uint64), ("synchronization_count", C.c_uint64)]


class SessionCacheEntry(C.Structure):
    _fields_ = [("key_high", C.c_uint64), ("key_low", C.c_uint64), ("state", C.c_void_p), ("structure_epoch", C.c_uint64),
                ("generation", C.c_uint64)]


LIFETIME_STRUCTURE, LIFETIME_PLAN, LIFETIME_GRAPH_STABLE = 0, 1, 2


class SessionOptions(C.Structure):
    _fields_ = [("version", C.c_uint32), ("size", C.c_size_t), ("device", C.c_int32),
                ("owned_stream_count", C.c_uint32), ("external_stream_count", C.c_uint32),
                ("external_streams", C.POINTER(C.c_void_p))]


class LaunchBinding(C.Structure):
    _fields_ = [("status", C.c_int32), ("device", C.c_int32), ("stream", C.c_void_p), ("workspace", C.c_void_p),
                ("workspace_bytes", C.c_uint64)]


# every symbol that include/cellerator_b200.h declares
EXPORTED_SYMBOLS = [
    "cb200_status_string", "cb200_last_error", "cb200_abi_version", "cb200_build_packed_row_ptr",
    "cb200_block_count_for_rows", "cb200_build_uniform_block_row_ptr", "cb200_get_block", "cb200_quantize_rows",
    "cb200_dequantize_rows", "cb200_qbell_quantize_rows", "cb200_qbell_dequantize_rows",
    "cb200_backend_query", "cb200_spmm_prepare", "cb200_prepared_destroy",
    "cb200_prepared_workspace", "cb200_prepared_schedule", "cb200_prepared_persistent_bytes", "cb200_spmm_run", "cb200_kernel_launch_count",
    "cb200_qcsr_forward_static",
    "cb200_bell_lowering_workspace", "cb200_bell_lowering_query", "cb200_bell_lowering_materialize",
    "cb200_pack_dense_operand", "cb200_build_execution_csr",
    "cb200_qcsr_gene_major_workspace", "cb200_qcsr_gene_major",
    "cb200_public_projection_scratch", "cb200_public_projection_forward", "cb200_public_projection_backward_rhs",
    "cb200_session_create", "cb200_session_reserve_persistent", "cb200_session_reserve_transient",
    "cb200_session_seal", "cb200_session_bind", "cb200_session_synchronize", "cb200_session_destroy",
    "cb200_find_in_row", "cb200_get_code", "cb200_get_value", "cb200_get_values",
    "cb200_spmm_persistent_requirement", "cb200_prepared_output_shape", "cb200_prepared_status",
    "cb200_qcsr_forward_static_status", "cb200_public_projection_status",
    "cb200_spmm_request_validate", "cb200_spmm_request_classify", "cb200_spmm_request_signature",
    "cb200_spmm_request_from_problem",
    "cb200_qbell_pack_aux", "cb200_qbell_unpack_aux", "cb200_qbell_row_bytes", "cb200_qbell_aligned_row_bytes",
    "cb200_qbell_host_init", "cb200_qbell_host_bytes", "cb200_qbell_host_allocate", "cb200_qbell_host_pin",
    "cb200_qbell_host_unpin", "cb200_qbell_host_clear", "cb200_qbell_host_view", "cb200_qbell_host_upload",
    "cb200_fleet_unique_id", "cb200_fleet_create", "cb200_fleet_destroy", "cb200_fleet_slot_count",
    "cb200_fleet_world_size", "cb200_fleet_device", "cb200_fleet_stream", "cb200_fleet_communicator_ready",
    "cb200_fleet_request_scratch", "cb200_fleet_synchronize", "cb200_fleet_partition", "cb200_fleet_run_forward",
    "cb200_fleet_run_transpose", "cb200_fleet_allreduce_sum_f32",
    "cb200_host_stage_create", "cb200_host_stage_destroy", "cb200_host_stage_device_bytes", "cb200_host_forward",
    "cb200_host_encode_gene_gaps",
    "cb200_test_arm_wait_timeout", "cb200_test_disarm_wait_timeout",
    "cb200_session_reserve_persistent_as", "cb200_session_prepare_stream_libraries", "cb200_session_get_accounting",
    "cb200_session_graph_stable_address", "cb200_session_cache_insert", "cb200_session_cache_find",
]

_lib = None
_synth = None


def lib() -> C.CDLL:
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FileNotFoundError(
                f"{LIB_PATH} is missing: build it with `python -m cellerator_b200.build` (there is no CPU fallback)")
        L = C.CDLL(LIB_PATH)
        L.cb200_status_string.restype = C.c_char_p
        L.cb200_last_error.restype = C.c_char_p
        L.cb200_abi_version.restype = C.c_uint32
        L.cb200_kernel_launch_count.restype = C.c_uint64
        L.cb200_build_packed_row_ptr.restype = C.c_int64
        L.cb200_build_packed_row_ptr.argtypes = [C.c_int32, C.c_void_p, C.c_int64, C.c_void_p]
        L.cb200_block_count_for_rows.restype = C.c_int64
        L.cb200_block_count_for_rows.argtypes = [C.c_int64, C.c_int64]
        L.cb200_build_uniform_block_row_ptr.restype = C.c_int64
        L.cb200_build_uniform_block_row_ptr.argtypes = [C.c_int64, C.c_int64, C.c_void_p]
        L.cb200_get_block.argtypes = [C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64,
                                      C.POINTER(CsrBlock)]
        L.cb200_quantize_rows.argtypes = [C.POINTER(QCsr), C.c_int64, C.c_int64, C.c_void_p, C.c_int32, C.c_void_p]
        L.cb200_dequantize_rows.argtypes = [C.POINTER(QCsr), C.c_int64, C.c_int64, C.c_void_p, C.c_int32, C.c_void_p]
        L.cb200_qbell_quantize_rows.argtypes = [C.POINTER(QBell), C.c_int64, C.c_int64, C.c_void_p, C.c_int32, C.c_void_p]
        L.cb200_qbell_dequantize_rows.argtypes = [C.POINTER(QBell), C.c_int64, C.c_int64, C.c_void_p, C.c_int32, C.c_void_p]
        L.cb200_backend_query.argtypes = [C.c_int32, C.POINTER(NumericPolicy), C.POINTER(Capability)]
        L.cb200_qcsr_gene_major_workspace.restype = C.c_uint64
        L.cb200_qcsr_gene_major_workspace.argtypes = [C.c_int64, C.c_int64]
        L.cb200_qcsr_gene_major.argtypes = [C.POINTER(QCsr), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint64,
                                            C.c_int32, C.c_void_p]
        L.cb200_spmm_prepare.argtypes = [C.POINTER(SpmmProblem), C.POINTER(C.c_void_p)]
        L.cb200_prepared_destroy.argtypes = [C.c_void_p]
        L.cb200_prepared_destroy.restype = None
        L.cb200_prepared_workspace.argtypes = [C.c_void_p, C.POINTER(C.c_uint64), C.POINTER(C.c_uint32)]
        L.cb200_prepared_schedule.argtypes = [C.c_void_p]
        L.cb200_prepared_schedule.restype = C.c_char_p
        L.cb200_prepared_persistent_bytes.argtypes = [C.c_void_p]
        L.cb200_prepared_persistent_bytes.restype = C.c_uint64
        L.cb200_spmm_run.argtypes = [C.c_void_p, C.POINTER(Launch)]
        L.cb200_qcsr_forward_static.argtypes = [C.POINTER(QCsr), C.c_void_p, C.c_int32, C.c_int64, C.c_void_p,
                                                C.c_int64, C.c_float, C.c_float, C.c_int32, C.c_void_p]
        L.cb200_find_in_row.restype = C.c_int64
        L.cb200_find_in_row.argtypes = [C.POINTER(QCsr), C.c_int64, C.c_int64]
        L.cb200_get_code.restype = C.c_uint32
        L.cb200_get_code.argtypes = [C.POINTER(QCsr), C.c_int64, C.c_int64]
        L.cb200_get_value.restype = C.c_float
        L.cb200_get_value.argtypes = [C.POINTER(QCsr), C.c_int64, C.c_int64]
        L.cb200_get_values.argtypes = [C.POINTER(QCsr), C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p,
                                       C.c_int32, C.c_void_p]
        L.cb200_spmm_persistent_requirement.argtypes = [C.POINTER(SpmmProblem), C.POINTER(C.c_uint64)]
        L.cb200_prepared_output_shape.argtypes = [C.c_void_p, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]
        L.cb200_prepared_status.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(C.c_int32)]
        L.cb200_qcsr_forward_static_status.argtypes = [C.c_int32, C.c_void_p, C.POINTER(C.c_int32)]
        L.cb200_public_projection_status.argtypes = [C.c_void_p, C.c_int32, C.c_void_p, C.POINTER(C.c_int32)]
        L.cb200_spmm_request_validate.argtypes = [C.POINTER(SpmmRequest)]
        L.cb200_spmm_request_classify.argtypes = [C.POINTER(SpmmRequest)]
        L.cb200_spmm_request_signature.argtypes = [C.POINTER(SpmmRequest), C.POINTER(C.c_uint64 * 2)]
        L.cb200_spmm_request_from_problem.argtypes = [C.POINTER(SpmmProblem), C.POINTER(Launch), C.c_uint64, C.c_uint64,
                                                      C.POINTER(SpmmRequest)]
        L.cb200_qbell_pack_aux.restype = C.c_uint64
        L.cb200_qbell_pack_aux.argtypes = [C.c_uint32, C.c_uint32, C.c_uint64]
        L.cb200_qbell_unpack_aux.restype = None
        L.cb200_qbell_unpack_aux.argtypes = [C.c_uint64, C.POINTER(C.c_uint32), C.POINTER(C.c_uint32), C.POINTER(C.c_uint64),
                                             C.POINTER(C.c_uint32)]
        L.cb200_qbell_row_bytes.restype = C.c_uint32
        L.cb200_qbell_row_bytes.argtypes = [C.c_uint32, C.c_uint32]
        L.cb200_qbell_aligned_row_bytes.restype = C.c_uint32
        L.cb200_qbell_aligned_row_bytes.argtypes = [C.c_uint32, C.c_uint32, C.c_uint32]
        L.cb200_qbell_host_init.restype = None
        L.cb200_qbell_host_init.argtypes = [C.POINTER(QBellHost)] + [C.c_uint32] * 8
        L.cb200_qbell_host_bytes.restype = C.c_uint64
        L.cb200_qbell_host_bytes.argtypes = [C.POINTER(QBellHost)]
        L.cb200_qbell_host_allocate.argtypes = [C.POINTER(QBellHost)]
        L.cb200_qbell_host_pin.argtypes = [C.POINTER(QBellHost)]
        L.cb200_qbell_host_unpin.restype = None
        L.cb200_qbell_host_unpin.argtypes = [C.POINTER(QBellHost)]
        L.cb200_qbell_host_clear.restype = None
        L.cb200_qbell_host_clear.argtypes = [C.POINTER(QBellHost)]
        L.cb200_qbell_host_view.argtypes = [C.POINTER(QBellHost), C.POINTER(QBell)]
        L.cb200_qbell_host_upload.argtypes = [C.POINTER(QBellHost), C.c_void_p, C.c_uint64, C.c_int32, C.c_void_p,
                                              C.POINTER(QBell)]
        L.cb200_fleet_unique_id.argtypes = [C.c_char_p, C.c_void_p]
        L.cb200_fleet_create.argtypes = [C.POINTER(FleetOptions), C.POINTER(C.c_void_p)]
        L.cb200_fleet_destroy.restype = None
        L.cb200_fleet_destroy.argtypes = [C.c_void_p]
        for name in ("cb200_fleet_slot_count", "cb200_fleet_world_size", "cb200_fleet_communicator_ready"):
            getattr(L, name).argtypes = [C.c_void_p]
        L.cb200_fleet_device.argtypes = [C.c_void_p, C.c_uint32]
        L.cb200_fleet_stream.restype = C.c_void_p
        L.cb200_fleet_stream.argtypes = [C.c_void_p, C.c_uint32]
        L.cb200_fleet_request_scratch.argtypes = [C.c_void_p, C.c_uint32, C.c_uint64, C.POINTER(C.c_void_p)]
        L.cb200_fleet_synchronize.argtypes = [C.c_void_p, C.POINTER(C.c_uint32), C.c_uint32]
        L.cb200_fleet_partition.argtypes = [C.c_int64, C.c_int32, C.c_void_p, C.c_void_p, C.POINTER(CsrBlock)]
        L.cb200_fleet_run_forward.argtypes = [C.c_void_p, C.POINTER(C.c_uint32), C.c_uint32, C.POINTER(C.c_void_p),
                                              C.POINTER(Launch)]
        L.cb200_fleet_run_transpose.argtypes = [C.c_void_p, C.POINTER(C.c_uint32), C.c_uint32, C.POINTER(C.c_void_p),
                                                C.POINTER(Launch)]
        L.cb200_fleet_allreduce_sum_f32.argtypes = [C.c_void_p, C.POINTER(C.c_uint32), C.c_uint32, C.POINTER(C.c_void_p),
                                                    C.POINTER(C.c_void_p), C.c_uint64]
        L.cb200_host_stage_create.argtypes = [C.POINTER(HostStageOptions), C.POINTER(C.c_void_p)]
        L.cb200_host_stage_destroy.restype = None
        L.cb200_host_stage_destroy.argtypes = [C.c_void_p]
        L.cb200_host_stage_device_bytes.restype = C.c_uint64
        L.cb200_host_stage_device_bytes.argtypes = [C.c_void_p]
        L.cb200_host_encode_gene_gaps.restype = C.c_int64
        L.cb200_host_encode_gene_gaps.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32]
        L.cb200_host_forward.argtypes = [C.c_void_p, C.POINTER(QCsr), C.c_void_p, C.c_int64, C.c_void_p, C.c_int64,
                                         C.c_float, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]
        L.cb200_test_arm_wait_timeout.restype = None
        L.cb200_test_arm_wait_timeout.argtypes = [C.c_uint32]
        L.cb200_test_disarm_wait_timeout.restype = None
        L.cb200_session_create.argtypes = [C.POINTER(SessionOptions), C.POINTER(C.c_void_p)]
        L.cb200_session_reserve_persistent.argtypes = [C.c_void_p, C.c_uint64, C.POINTER(C.c_void_p)]
        L.cb200_session_reserve_persistent_as.argtypes = [C.c_void_p, C.c_int32, C.c_uint64, C.POINTER(C.c_void_p)]
        L.cb200_session_prepare_stream_libraries.argtypes = [C.c_void_p, C.c_uint32]
        L.cb200_session_get_accounting.argtypes = [C.c_void_p, C.POINTER(SessionAccounting)]
        L.cb200_session_graph_stable_address.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64]
        L.cb200_session_cache_insert.argtypes = [C.c_void_p, C.c_int32, C.POINTER(SessionCacheEntry)]
        L.cb200_session_cache_find.argtypes = [C.c_void_p, C.c_int32, C.c_uint64, C.c_uint64]
        L.cb200_session_cache_find.restype = C.POINTER(SessionCacheEntry)
        L.cb200_session_reserve_transient.argtypes = [C.c_void_p, C.c_uint32, C.c_uint64]
        L.cb200_session_seal.argtypes = [C.c_void_p]
        L.cb200_session_bind.argtypes = [C.c_void_p, C.c_uint32, C.c_uint64]
        L.cb200_session_bind.restype = LaunchBinding
        L.cb200_session_synchronize.argtypes = [C.c_void_p]
        L.cb200_session_destroy.argtypes = [C.c_void_p]
        L.cb200_session_destroy.restype = None
        _lib = L
    return _lib


def synth_lib() -> C.CDLL:
    global _synth
    if _synth is None:
        if not os.path.exists(SYNTH_PATH):
            raise FileNotFoundError(f"{SYNTH_PATH} is missing: build it with `python -m cellerator_b200.build`")
        _synth = C.CDLL(SYNTH_PATH)
    return _synth


def check(status: int) -> None:
    if status != SUCCESS:
        raise Cb200Error(status, lib().cb200_last_error().decode() or lib().cb200_status_string(status).decode())


def header(struct):
    struct.version = ABI_VERSION
    struct.size = C.sizeof(struct)
    return struct
