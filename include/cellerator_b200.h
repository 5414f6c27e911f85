/*
 * cellerator_b200 — C ABI of the B200 (sm_100a) backend for Cellerator's quantized
 * sparse-matrix path:  Y = dequant(X) * W  over a quantized CSR cells x genes matrix, its
 * gene-side transpose  G' = dequant(X)^T * G,  and the quantized Blocked-ELL projection.
 *
 * Everything here is plain C: pointers, sizes, integer status codes.  Device pointers are
 * CUDA device addresses on the device named by the call; `stream` is a cudaStream_t passed
 * as void*.  No entry point falls back to the CPU: without a usable CUDA device the compute
 * calls return CB200_STATUS_CUDA_ERROR.
 *
 * Each declaration cites the interface of the Cellerator reference that it stands in for
 * (paths relative to the Cellerator project root).
 *
 * Conventions (after include/Cellerator/abi.h:14-55,100-118): every descriptor starts with
 * {version, size}; functions return cb200_status; the text of the last failure on the calling
 * thread is available from cb200_last_error().
 */
#ifndef CELLERATOR_B200_H
#define CELLERATOR_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* every entry point below is exported even when the library is built with hidden visibility */
#if defined(__GNUC__)
#pragma GCC visibility push(default)
#endif

#define CB200_ABI_VERSION 1u

/* include/Cellerator/abi.h:14-21 (cellerator_status), extended with the operation-core
 * outcomes of operation_core.hh:118-131 that can cross this boundary. */
typedef enum cb200_status {
    CB200_STATUS_SUCCESS = 0,
    CB200_STATUS_INVALID_ARGUMENT = 1,
    CB200_STATUS_INVALID_SHAPE = 2,
    CB200_STATUS_UNSUPPORTED = 3,
    CB200_STATUS_CUDA_ERROR = 4,
    CB200_STATUS_INTERNAL_ERROR = 5,
    CB200_STATUS_STALE_STRUCTURE = 6,
    CB200_STATUS_INSUFFICIENT_WORKSPACE = 7,
    CB200_STATUS_INVALID_STREAM = 8,
    CB200_STATUS_SEALED = 9,
    CB200_STATUS_STALE_VALUE = 10 /* lifetime_validation_code::stale_value_generation, lifetimes.hh:88-94 */
} cb200_status;

/* execution::numeric_type, include/Cellerator/execution/operands.hh:9-20 (same values) */
typedef enum cb200_dtype {
    CB200_DTYPE_INVALID = 0,
    CB200_DTYPE_U8 = 2,
    CB200_DTYPE_U4 = 32, /* 4-bit nibble-packed codes; no counterpart enum value in the reference */
    CB200_DTYPE_F16 = 6,
    CB200_DTYPE_BF16 = 7,
    CB200_DTYPE_F32 = 8,
    CB200_DTYPE_F64 = 9
} cb200_dtype;

/* quantized::blocked_ell decode policies, include/Cellerator/quantized/blocked_ell.cuh:10-14;
 * metadata policies of include/Cellerator/quantized/metadata.cuh:7-56 */
typedef enum cb200_decode_policy {
    CB200_DECODE_PER_GENE_AFFINE = 1,        /* value = code*scales[gene] + offsets[gene] */
    CB200_DECODE_COLUMN_SCALE_ROW_OFFSET = 2 /* value = code*scales[gene] + offsets[row]  */
} cb200_decode_policy;

/* epilogue_kind of the SpMM request, include/Cellerator/compute/math/operation.hh:49-61 */
typedef enum cb200_epilogue {
    CB200_EPILOGUE_NONE = 0,
    CB200_EPILOGUE_BIAS = 1,
    CB200_EPILOGUE_RELU = 2,
    CB200_EPILOGUE_GELU_ERF = 3,
    CB200_EPILOGUE_GELU_TANH = 4,
    CB200_EPILOGUE_BIAS_RELU = 5,
    CB200_EPILOGUE_BIAS_GELU_ERF = 6,
    CB200_EPILOGUE_BIAS_GELU_TANH = 7
} cb200_epilogue;

/* core::projection_kind, operation_core.hh:25-37 (same values) */
typedef enum cb200_projection {
    CB200_PROJECTION_CSR = 5,
    CB200_PROJECTION_BLOCKED_ELL = 8,
    CB200_PROJECTION_TRANSPOSE = 10
} cb200_projection;

const char *cb200_status_string(cb200_status status); /* abi.h:100 */
const char *cb200_last_error(void);                   /* abi.h:101, thread-local */
uint32_t cb200_abi_version(void);

/* ------------------------------------------------------------------------------------ */
/* Quantized CSR layout.  quantized::csr_matrix, include/Cellerator/quantized/layout.cuh:12-38,
 * with the index widths of the referee's logical_csr_view (referee.hh:40-48): int64 row
 * pointers, int32 gene indices.  Code i of row r is byte packed_row_ptr[r] + i/cpb, bit shift
 * (i mod cpb)*bits, cpb = 8/bits (format.cuh:39-48).  For bits == 8 packed_row_ptr may be
 * NULL: it then equals row_ptr. `offsets` is per gene or per row according to `policy`;
 * NULL scales mean 1, NULL offsets mean 0 (metadata.cuh:17-27). */
typedef struct cb200_qcsr {
    uint32_t version;
    size_t size;
    int64_t rows;
    int64_t cols;
    int64_t nnz;
    int32_t bits;   /* 8 or 4 on the compute path; 1 and 2 on the codec path */
    int32_t policy; /* cb200_decode_policy */
    const int64_t *row_ptr;        /* rows+1 */
    const int64_t *packed_row_ptr; /* rows+1 byte offsets, or NULL when bits == 8 */
    const int32_t *col_idx;        /* nnz, ascending within a row */
    const uint8_t *packed_values;
    const float *scales;
    const float *offsets;
} cb200_qcsr;

/* quantized::csr_block, layout.cuh:41-49 */
typedef struct cb200_csr_block {
    int64_t block_index, row_begin, row_end, nnz_begin, nnz_end, packed_begin, packed_end;
} cb200_csr_block;

/* Host helpers (no CUDA call).
 * build_packed_row_ptr<Bits>, layout.cuh:111-129: returns total bytes, -1 on bad arguments. */
int64_t cb200_build_packed_row_ptr(int32_t bits, const int64_t *row_ptr, int64_t rows, int64_t *packed_row_ptr);
/* block_count_for_rows / build_uniform_block_row_ptr, layout.cuh:131-157: the row partition
 * used to shard cells over GPUs.  Returns the block count, -1 on bad arguments. */
int64_t cb200_block_count_for_rows(int64_t rows, int64_t rows_per_block);
int64_t cb200_build_uniform_block_row_ptr(int64_t rows, int64_t rows_per_block, int64_t *block_row_ptr);
/* get_block, access.cuh:7-44: host pointers. block_row_ptr NULL => one block over the matrix;
 * an out-of-range index yields an all-zero block. */
cb200_status cb200_get_block(int64_t rows, const int64_t *row_ptr, const int64_t *packed_row_ptr,
                             const int64_t *block_row_ptr, int64_t block_count, int64_t block_index,
                             cb200_csr_block *out);

/* Device codec over rows [row_begin,row_end) of a device-resident matrix.
 * launch_quantize_block / launch_dequantize_block, portable_backend.cuh:23-61 with
 * pack_row_values / unpack_row_values, packing.cuh:13-260.  `values` holds one float per nnz
 * of the range, values[0] belonging to nnz index row_ptr[row_begin] (block-local, rule of
 * packing.cuh:17-18).  Quantize writes m->packed_values (cast away const by the callee: the
 * caller owns the buffer), with the host rounding rule of access.cuh:104-131. */
cb200_status cb200_quantize_rows(const cb200_qcsr *m, int64_t row_begin, int64_t row_end, const float *values,
                                 int32_t device, void *stream);
cb200_status cb200_dequantize_rows(const cb200_qcsr *m, int64_t row_begin, int64_t row_end, float *values,
                                   int32_t device, void *stream);

/* ------------------------------------------------------------------------------------ */
/* Quantized Blocked-ELL layout.  quantized::blocked_ell::matrix, blocked_ell.cuh:18-36 and
 * sparse_ops::quantized_blocked_ell_view, src/compute/sparse/ops/ops.hh:28-42.  Row r, slot s
 * is code s of the row starting at packed_values + r*row_stride_bytes; block_col_idx has
 * ceil(rows/block_size) * (ell_cols/block_size) entries, 0xffffffff marks an empty block. */
typedef struct cb200_qbell {
    uint32_t version;
    size_t size;
    int64_t rows;
    int64_t cols;
    int32_t block_size;
    int32_t ell_cols;
    int64_t row_stride_bytes;
    int32_t bits;
    int32_t policy;
    const uint32_t *block_col_idx;
    const uint8_t *packed_values;
    const float *scales;
    const float *offsets;
} cb200_qbell;

/* Device codec of the Blocked-ELL layout over rows [row_begin,row_end): device-side form of
 * pack_row_major_values / unpack_row_major_values, blocked_ell.cuh:165-231.  `values_by_slot`
 * is row-major with ell_cols floats per row, values_by_slot[0] belonging to row_begin.
 * Quantize codes EVERY slot (a slot of an empty block uses gene 0's scale/offset, like the
 * reference) and zeroes the row padding; dequantize writes 0 for slots of empty blocks and
 * for genes >= cols. */
cb200_status cb200_qbell_quantize_rows(const cb200_qbell *m, int64_t row_begin, int64_t row_end,
                                       const float *values_by_slot, int32_t device, void *stream);
cb200_status cb200_qbell_dequantize_rows(const cb200_qbell *m, int64_t row_begin, int64_t row_end,
                                         float *values_by_slot, int32_t device, void *stream);

/* ------------------------------------------------------------------------------------ */
/* Capability query.  operation_candidate.supports_numeric + capability flags and byte
 * budgets, operation_core.hh:63-68,102-114,185,195-207.  Pure host; touches no device. */
typedef struct cb200_numeric_policy {
    uint32_t version;
    size_t size;
    int32_t sparse_storage; /* CB200_DTYPE_U8 | CB200_DTYPE_U4 */
    int32_t dense_storage;  /* CB200_DTYPE_F32 | CB200_DTYPE_BF16 */
    int32_t output_storage; /* CB200_DTYPE_F32 */
    int32_t multiply;       /* CB200_DTYPE_F32 (CSR, transpose) | CB200_DTYPE_BF16 (Blocked-ELL) */
    int32_t accumulation;   /* CB200_DTYPE_F32 */
    int32_t quantized;      /* non-zero: quantization_granularity != none */
} cb200_numeric_policy;

enum { /* candidate_capability_flag, operation_core.hh:63-68 (same bits) */
    CB200_CAP_DETERMINISTIC = 1u << 0,
    CB200_CAP_GRAPH_CAPTURE = 1u << 1,
    CB200_CAP_PERSISTENT_PREPROCESSING = 1u << 2,
    CB200_CAP_COMPOSED_EPILOGUE = 1u << 3
};

typedef struct cb200_capability {
    uint32_t version;
    size_t size;
    int32_t supported; /* 0 / 1 */
    uint32_t flags;    /* CB200_CAP_* */
    uint64_t persistent_bytes;
    uint64_t transient_bytes;
    const char *name;
} cb200_capability;

cb200_status cb200_backend_query(int32_t projection, const cb200_numeric_policy *numeric, cb200_capability *out);

/* ------------------------------------------------------------------------------------ */
/* Prepared-operation lifecycle.  operation_candidate.prepare -> prepared_operation ->
 * run_prepared_operation, operation_core.hh:159-193 and operation_core.cc:133-147,179-240.
 * Prepare does everything that may query the device, read row statistics or size scratch;
 * run validates the launch, enqueues on the caller's stream and returns without
 * synchronising or allocating (OPERATION_CORE.md:27-32). */
typedef struct cb200_spmm_problem {
    uint32_t version;
    size_t size;
    int32_t projection; /* cb200_projection */
    int64_t m;          /* cells (rows of X) */
    int64_t k;          /* genes (cols of X) */
    int64_t n;          /* dense columns */
    int64_t nnz;        /* CSR: stored entries; Blocked-ELL: rows*ell_cols */
    int32_t bits;
    int32_t policy;
    int32_t dense_dtype; /* W (forward, Blocked-ELL) or G (transpose) */
    int32_t device;
    uint64_t structure_epoch; /* non-zero; a launch with another epoch is stale (launch_bindings.hh:261-275) */
    /* Optional host copy of row_ptr (m+1) used to choose the row schedule; NULL = default. */
    const int64_t *host_row_ptr;
    int32_t deterministic; /* prepare_policy.deterministic, operation_core.hh:116-124; a transpose needs
                            * device_matrix for it (schedule "gene_gather"), else prepare is refused */
    /* numeric_policy.multiply of the request: 0 or CB200_DTYPE_F32 = exact fp32 products;
     * CB200_DTYPE_BF16 = decoded values may be rounded to bf16 and multiplied on the tensor cores
     * (CSR forward with bf16 W: schedules "tensor_windows" / "tensor_blocked"; transpose with the
     * matrix handed to prepare: "tensor_blocked", which rounds the fp32 G to bf16 as well;
     * Blocked-ELL with bf16 W always does).
     * fp32 products requested AND the matrix handed to prepare (dense enough): schedules
     * "tensor_blocked_x2" (forward, bf16 W) / "tensor_blocked_x3" (forward with fp32 W; transpose)
     * rebuild each fp32 product from bf16 tensor-core passes (value = hi + lo, fp32 dense operand =
     * hi + lo; hi*hi + hi*lo + lo*hi), relative error about 3 * 2^-17 per product: inside the 1e-4
     * bound of an fp32 operand, not bit-equal to an fp32 multiply.  Without device_matrix the fp32-FMA
     * kernels ("gene_tiled" / "warp_per_row", "vector_reductions") run. */
    int32_t multiply;
    /* Optional: the device-resident matrix itself (arrays on `device`, final contents).  With bf16
     * products allowed, prepare then builds a persistent window-blocked copy of it (one 32-bit
     * word per stored entry plus 8 bytes per 256-row x 128-gene segment; persistent_kernel_state,
     * operation_core.hh:126-129) and the schedule becomes "tensor_blocked".  Prepare launches
     * kernels on the device's default stream and synchronises.  Launches must then pass the same
     * arrays: other pointers are refused as a stale structure; changed codes need a new prepare.
     *
     * Forward with bf16 products on a matrix of 8 % density or more: prepare goes one step further
     * and keeps the decoded operand tiles themselves (schedule "tensor_dense": rows x genes x 2 bytes,
     * rounded up to 256 x 128 tiles; codes, scales and offsets are baked in, so a change of any of
     * them needs a new prepare).  A launch then streams the tiles into the tensor cores and does no
     * decoding.  Taken only when the tiles fit persistent_limit_bytes and half of the free device
     * memory; otherwise "tensor_blocked" stays. */
    const cb200_qcsr *device_matrix;
    /* prepare_policy.persistent_memory_limit (operation_core.hh:116-124): device bytes the prepared
     * operation may keep; 0 = no limit.  A copy that would exceed it is not built (the schedule
     * falls back to the next one that fits). */
    uint64_t persistent_limit_bytes;
    /* value_plane.generation (include/Cellerator/execution/lifetimes.hh:62-85) of the codes, scales and
     * offsets device_matrix points at; 0 = not tracked.  The reference's rule is that a prepared
     * operation does not freeze mutable values (lifetimes.hh:80-81); a copy built from device_matrix
     * does, so a launch that names another generation (cb200_launch.value_generation) is refused with
     * CB200_STATUS_STALE_VALUE instead of multiplying stale values. */
    uint64_t value_generation;
} cb200_spmm_problem;

typedef struct cb200_prepared cb200_prepared;

cb200_status cb200_spmm_prepare(const cb200_spmm_problem *problem, cb200_prepared **out);
void cb200_prepared_destroy(cb200_prepared *prepared);
/* workspace_requirement, launch_bindings.hh:67-71 */
cb200_status cb200_prepared_workspace(const cb200_prepared *prepared, uint64_t *minimum_bytes, uint32_t *alignment);
/* kernel choice made at prepare time, as text: "warp_per_row", "gene_tiled" (exact fp32 products);
 * "tensor_windows", "tensor_blocked", "tensor_dense" (CSR, bf16 products on tcgen05);
 * "tensor_blocked_x2" / "_x3" (fp32 products from bf16 passes); "tcgen05_block_rows" (Blocked-ELL);
 * transpose: "vector_reductions" (exact) or "tensor_blocked" */
const char *cb200_prepared_schedule(const cb200_prepared *prepared);
/* device bytes the prepared operation owns (row order, window-blocked copy): prepared_operation.persistent.bytes,
 * operation_core.hh:126-129,167-181; freed by cb200_prepared_destroy */
uint64_t cb200_prepared_persistent_bytes(const cb200_prepared *prepared);

/* launch_bindings, launch_bindings.hh:90-102: everything that changes per launch. */
typedef struct cb200_launch {
    uint32_t version;
    size_t size;
    const cb200_qcsr *csr;   /* CSR and transpose projections */
    const cb200_qbell *bell; /* Blocked-ELL projection */
    const void *dense;       /* W: k x n (forward, Blocked-ELL);  G: m x n (transpose); row-major */
    int64_t dense_ld;        /* elements */
    float *out;              /* Y: m x n (forward, Blocked-ELL);  G': k x n (transpose); row-major fp32 */
    int64_t out_ld;
    float alpha;             /* out = alpha * product + beta * out; beta == 0 never reads out */
    float beta;
    uint64_t structure_epoch;
    int64_t row_begin;       /* rows [row_begin,row_end) of X; out rows are indexed by absolute row */
    int64_t row_end;         /* 0,0 = all rows */
    void *stream;            /* stream_context, launch_bindings.hh:55-59 */
    int32_t device;
    int32_t workspace_device;
    void *workspace;         /* transient_workspace, launch_bindings.hh:61-65 */
    uint64_t workspace_bytes;
    /* Composed epilogue of the forward projections (CSR, Blocked-ELL), the request contract's
     * epilogue_kind with the referee's rule (operation.hh:49-61, referee.cc:81-97):
     *     out = act(alpha * product + beta * out + bias[column]).
     * bias has n floats on the device and is read only by the bias kinds; the transpose accepts
     * CB200_EPILOGUE_NONE only. */
    const float *bias;
    int32_t epilogue;        /* cb200_epilogue */
    /* value_binding.expected_generation of the launch's value plane (lifetimes.hh:82-85); 0 = not
     * tracked.  Compared with cb200_spmm_problem.value_generation when the prepared operation keeps a
     * copy of the values. */
    uint64_t value_generation;
} cb200_launch;

cb200_status cb200_spmm_run(const cb200_prepared *prepared, const cb200_launch *launch);

/* Number of kernel launches this library has enqueued since it was loaded (all threads). */
uint64_t cb200_kernel_launch_count(void);

/* Forward projection  Y = alpha * deq(X) * W + beta * Y  for callers that cannot allocate device
 * memory.  (No counterpart in the Cellerator reference, whose operations take their scratch from
 * the session or from request_scratch.)
 *
 * Who needs it: code that runs where cudaMalloc is off limits, e.g. a latency-critical region
 * that must stay free of allocator calls or a process whose device-memory budget is fixed and
 * policed, and language shims that can hand pointers through but have no device allocator of
 * their own.  Such callers cannot supply the workspace that cb200_spmm_run asks for.  Here the
 * kernel's scratch is a fixed 256-byte array that is part of the library's device image, so the
 * call needs only the inputs and the output; it performs no cudaMalloc / cudaFree and calls no
 * allocating library routine.
 *
 * Limits and rules:
 *  - the scratch the kernel needs must fit the 256-byte array (it does for every matrix size the
 *    kernel accepts; a larger need is refused with CB200_STATUS_INSUFFICIENT_WORKSPACE), and the
 *    shape must be one the gene-tiled kernel covers: 8- or 4-bit codes with per-gene scales,
 *    n in {32, 64, 128} for bf16 W ({32, 64} for fp32 W), W contiguous (leading dimension n) and
 *    16-byte aligned, Y rows 16-byte aligned; anything else returns CB200_STATUS_UNSUPPORTED;
 *  - every GPU that loads the library holds the array until the process exits;
 *  - all calls on a device share the array and it keeps the last call's contents: each call clears
 *    what must start at zero, in stream order, and calls that may overlap on the GPU (different
 *    streams without ordering) race on it, so serialise them;
 *  - the first call on each device looks up the array's device address (cudaGetSymbolAddress,
 *    with that device current) and caches it; make that first call before any stream capture.
 * w_dtype is CB200_DTYPE_BF16 or CB200_DTYPE_F32; x, w, y are device pointers on `device`. */
cb200_status cb200_qcsr_forward_static(const cb200_qcsr *x, const void *w, int32_t w_dtype, int64_t n, float *y,
                                       int64_t y_ld, float alpha, float beta, int32_t device, void *stream);

/* ------------------------------------------------------------------------------------ */
/* Runtime session.  runtime::execution_session, include/Cellerator/runtime/session.cuh:106-177:
 * init -> reserve persistent / transient -> seal -> bind per launch.  After sealing nothing
 * grows, and bind makes no CUDA call (SESSION.md:20-29). */
typedef struct cb200_session cb200_session;

typedef struct cb200_session_options {
    uint32_t version;
    size_t size;
    int32_t device;
    uint32_t owned_stream_count;
    uint32_t external_stream_count;
    void *const *external_streams;
} cb200_session_options;

typedef struct cb200_launch_binding { /* launch_runtime_binding, session.cuh:122-129 */
    cb200_status status;
    int32_t device;
    void *stream;
    void *workspace;
    uint64_t workspace_bytes;
} cb200_launch_binding;

cb200_status cb200_session_create(const cb200_session_options *options, cb200_session **out);
cb200_status cb200_session_reserve_persistent(cb200_session *s, uint64_t bytes, void **allocation);
cb200_status cb200_session_reserve_transient(cb200_session *s, uint32_t stream_index, uint64_t bytes);
cb200_status cb200_session_seal(cb200_session *s);
cb200_launch_binding cb200_session_bind(cb200_session *s, uint32_t stream_index, uint64_t required_workspace_bytes);
cb200_status cb200_session_synchronize(cb200_session *s);
void cb200_session_destroy(cb200_session *s);

/* ------------------------------------------------------------------------------------------
 * CSR -> physical Blocked-ELL lowering on the device: the reference's host loops
 * query_bell_candidates_host / materialize_bell_candidate_host
 * (include/Cellerator/compute/math/physical_bell.hh:48-192, src/compute/math/physical_bell.cc:98-200,
 * src/compute/math/physical_bell_candidates.cc:131-238) for one block size, with the same geometry,
 * metrics, column indices and value placement, bit for bit.  The reference's identity hashes
 * (FNV-1a chains over arrays the caller owns) are not computed here.
 * Conventions (physical_bell.cc:44-58): feature_permutation[execution] = canonical,
 * inverse_feature_permutation[canonical] = execution, row_permutation[execution row] = canonical row. */
typedef struct cb200_bell_lowering_input {
    uint32_t version;
    size_t size;
    /* bell_csr_source_view, physical_bell.hh:48-56: canonical feature ids, strictly increasing per row */
    uint32_t rows, features, nnz, value_size_bytes; /* value_size_bytes 1..16, copied bytewise */
    const uint32_t *row_offsets; /* device, rows + 1 */
    const uint32_t *feature_ids; /* device, nnz */
    const void *values;          /* device, nnz * value_size_bytes */
    /* bell_semantic_plan_view, physical_bell.hh:61-71 */
    uint32_t feature_block_count;
    const uint32_t *feature_block_offsets;       /* HOST, feature_block_count + 1, execution order */
    const uint32_t *feature_permutation;         /* device, features */
    const uint32_t *inverse_feature_permutation; /* device, features */
    /* cellpack::local_cell_order_view (CellPack/local_cell_ordering.hh:47-67), the two maps it carries */
    const uint32_t *row_permutation;         /* device, rows */
    const uint32_t *inverse_row_permutation; /* device, rows */
    int32_t device;
} cb200_bell_lowering_input;

typedef struct cb200_bell_lowering_policy { /* bell_lowering_policy, physical_bell.hh:90-94 (defaults 64, 64, no limit) */
    double maximum_value_slot_expansion;
    double maximum_storage_expansion;
    uint64_t maximum_persistent_bytes;
} cb200_bell_lowering_policy;

typedef enum cb200_bell_state { /* bell_candidate_state, physical_bell.hh:15-22 */
    CB200_BELL_STATE_LEGAL = 0,
    CB200_BELL_STATE_EMPTY_SOURCE = 1,
    CB200_BELL_STATE_VALUE_EXPANSION_EXCEEDED = 2,
    CB200_BELL_STATE_STORAGE_EXPANSION_EXCEEDED = 3,
    CB200_BELL_STATE_PERSISTENT_BYTES_EXCEEDED = 4,
    CB200_BELL_STATE_OVERFLOW = 5
} cb200_bell_state;

typedef struct cb200_bell_geometry { /* bell_candidate_requirements + bell_candidate_metrics, physical_bell.hh:96-123 */
    uint32_t version;
    size_t size;
    int32_t state; /* cb200_bell_state */
    uint32_t block_size, rows, features, padded_rows, padded_features, block_rows, ell_blocks_per_row, ell_columns;
    uint64_t feature_block_offset_count, column_index_count, value_bytes;
    uint64_t occupied_blocks, stored_blocks, dense_value_slots, persistent_bytes, source_bytes;
    double scalar_occupancy, ell_slot_utilization, value_slot_expansion, storage_expansion;
} cb200_bell_geometry;

typedef enum cb200_bell_values_layout {
    /* the reference's: values[((block_row * ell_blocks + slot) * bs + row_in_block) * bs + column_in_block]
     * (physical_bell.cc:183-189) */
    CB200_BELL_VALUES_BLOCK_MAJOR = 0,
    /* execution row r, slot s, column c at r * row_stride_bytes + (s * bs + c) * value_size_bytes: with
     * one-byte codes this is the packed_values array of a cb200_qbell, whose block_col_idx is the
     * column_indices array reinterpreted (-1 = 0xffffffff = empty) */
    CB200_BELL_VALUES_ROW_MAJOR = 1
} cb200_bell_values_layout;

/* workspace both calls need (device memory, 16-byte aligned) */
cb200_status cb200_bell_lowering_workspace(const cb200_bell_lowering_input *in, uint64_t *bytes);
/* Validates the input on the device (maps are inverses, CSR sorted and in range: the checks of
 * physical_bell.cc:27-80) and computes the geometry and metrics of one block size (8, 16 or 32).
 * Reads counters back: synchronises `stream`. */
cb200_status cb200_bell_lowering_query(const cb200_bell_lowering_input *in, uint32_t block_size,
                                       const cb200_bell_lowering_policy *policy, void *workspace,
                                       uint64_t workspace_bytes, void *stream, cb200_bell_geometry *out);
/* Writes padded_feature_block_offsets (feature_block_count + 1), column_indices (column_index_count,
 * -1 = empty, slots in ascending block column) and the values (zero where nothing is stored) into
 * device buffers, for a geometry that cb200_bell_lowering_query returned as legal for this input.
 * Enqueues on `stream`, does not synchronise. */
cb200_status cb200_bell_lowering_materialize(const cb200_bell_lowering_input *in, const cb200_bell_geometry *geometry,
                                             int32_t values_layout, uint64_t row_stride_bytes,
                                             uint32_t *padded_feature_block_offsets, int32_t *column_indices, void *values,
                                             void *workspace, uint64_t workspace_bytes, void *stream);

/* Feature-order pack of a dense operand on the device, pack_dense_operand_cuda
 * (include/Cellerator/compute/math/packed_dense_operand.hh:65-70,
 * src/compute/math/packed_dense_operand.cu:131-170,227-262):
 *     packed[execution][column] = source[feature_permutation[execution]][column],
 * contiguous row-major from a row- or column-major source, values copied bytewise.
 * With feature_block_count != 0 the rows follow the padded physical feature order of a Blocked-ELL
 * lowering instead (cb200_bell_lowering_materialize's padded_feature_block_offsets, here on the
 * HOST): semantic block b fills rows [padded[b], padded[b] + width_b), the rows of the padding are
 * zero, and the operand has padded[feature_block_count] rows -- the W the lowered matrix multiplies.
 * Enqueues on `stream`.  status_word (device, 4 bytes) is cleared first and holds 1 afterwards when a
 * permutation entry was out of range (those rows are left unwritten; the reference's
 * invalid_geometry). */
typedef struct cb200_dense_pack {
    uint32_t version;
    size_t size;
    const uint32_t *feature_permutation; /* device, features */
    const void *source;                  /* device */
    uint32_t features;
    uint64_t columns;
    uint64_t leading_dimension; /* of the source, in elements */
    int32_t source_col_major;   /* dense_layout_kind: 0 row-major [feature][column], 1 column-major */
    uint32_t value_size_bytes;  /* 1, 2, 4, 8 or 16 */
    uint32_t feature_block_count;                 /* 0: plain execution order */
    const uint32_t *feature_block_offsets;        /* HOST, feature_block_count + 1 */
    const uint32_t *padded_feature_block_offsets; /* HOST, feature_block_count + 1 */
    void *packed;                                 /* device */
    uint64_t packed_capacity_bytes;
    void *status_word; /* device, 4 bytes */
    int32_t device;
} cb200_dense_pack;

cb200_status cb200_pack_dense_operand(const cb200_dense_pack *pack, void *stream);

/* Execution-order feature ids of an ordered plan partition on the device: the loop of
 * build_execution_csr_view_host (include/Cellerator/compute/math/physical_csr.hh:172-177,
 * src/compute/math/physical_csr.cc:47-75; cellpack::ordered_plan_partition_view,
 * CellPack/apply_plan.hh:49-65): execution = feature_block_offsets[block] + local, which must map back
 * to the entry's canonical id through the plan's feature permutation and ascend strictly inside a
 * row.  The row offsets and values are used as they are (the reference's view aliases them too); the
 * FNV structure identity of the view stays with the caller.
 * Enqueues on `stream`.  status_word (device, 4 bytes): 0 = ok; bit 0 = invalid geometry (offsets do
 * not span nnz or are not monotone, block or local out of range), bit 1 = incompatible identity (an
 * entry does not map to packed order); with several violations both kinds are reported where the
 * reference returns the first in row-major order. */
typedef struct cb200_execution_csr {
    uint32_t version;
    size_t size;
    uint32_t rows, features, nnz;
    const uint32_t *row_offsets;           /* device, rows + 1 */
    const uint32_t *block_ids;             /* device, nnz */
    const uint32_t *local_feature_ids;     /* device, nnz */
    const uint32_t *canonical_feature_ids; /* device, nnz */
    uint32_t feature_block_count;
    const uint32_t *feature_block_offsets; /* HOST, feature_block_count + 1 */
    const uint32_t *feature_permutation;   /* device, features: execution -> canonical */
    uint32_t *execution_feature_ids;       /* device, nnz: the result */
    void *workspace;                       /* device, (feature_block_count + 1) * 4 bytes */
    uint64_t workspace_bytes;
    void *status_word;                     /* device, 4 bytes */
    int32_t device;
} cb200_execution_csr;

cb200_status cb200_build_execution_csr(const cb200_execution_csr *view, void *stream);

/* Gene-major copy (a CSC) of a quantized CSR matrix, built on the device: the CSR -> CSC transpose of
 * the reference (count_transpose_targets + scatter_transpose,
 * src/compute/matrix/convert/compressed.cu:146-178, reached through the compressed-matrix converters),
 * for the quantized format.  The reference places entries at atomicAdd(heads + minor, 1), which leaves
 * the order inside a gene to the scheduler; this build is a stable counting sort: inside every gene
 * the cells ascend, and every run produces the same arrays.
 *   col_ptr  device, cols + 1: first entry of each gene
 *   row_idx  device, nnz: the cell of each entry
 *   codes    device, nnz: one code per byte (4-bit sources are widened, the value is unchanged)
 * Scales and offsets are shared with the source.  Rows and genes below 2^31; column indices ascend
 * inside a row, as the format requires.  Enqueues on `stream`,
 * allocates nothing; `workspace` (device) needs cb200_qcsr_gene_major_workspace(rows, cols) bytes
 * (0 = shape outside the limits), and its first 32-bit word is 0 afterwards unless a column index lay
 * outside the matrix (bit 0).
 * cb200_spmm_prepare builds this copy itself for a transpose problem with deterministic = 1 and the
 * device matrix at hand (schedule "gene_gather"): the sums then have a fixed order -- per gene, eight
 * interleaved runs of 256-entry chunks added entry by entry with fp32 FMAs, the eight partial sums
 * added in order -- and the output is the same bits on every run. */
uint64_t cb200_qcsr_gene_major_workspace(int64_t rows, int64_t cols);
cb200_status cb200_qcsr_gene_major(const cb200_qcsr *x, int64_t *col_ptr, int32_t *row_idx, uint8_t *codes,
                                   void *workspace, uint64_t workspace_bytes, int32_t device, void *stream);

/* ------------------------------------------------------------------------------------------
 * Routing of the reference's public projection calls: cellerator_sparse_projection_forward /
 * _backward (include/Cellerator/abi.h:111-124, src/abi/abi.cu:278-396) for the quantized layouts,
 * which the reference declares (CELLERATOR_LAYOUT_QUANTIZED_BLOCKED_ELL, abi.h:31-36) and rejects
 * (abi.cu:325-326).  cb200_public_layout carries the fields of cellerator_sparse_layout_desc
 * (abi.h:68-89) these layouts use, with the same widths: 32-bit shapes and row offsets. */
typedef enum cb200_public_layout_kind {
    CB200_PUBLIC_LAYOUT_QUANTIZED_BLOCKED_ELL = 4, /* = CELLERATOR_LAYOUT_QUANTIZED_BLOCKED_ELL */
    CB200_PUBLIC_LAYOUT_QUANTIZED_CSR = 5          /* no counterpart yet: the next free value of cellerator_sparse_layout */
} cb200_public_layout_kind;

typedef struct cb200_public_layout {
    uint32_t version;
    size_t size;
    int32_t layout; /* cb200_public_layout_kind */
    uint32_t rows, cols, nnz;
    uint32_t block_size, ell_cols, row_stride_bytes; /* Blocked-ELL */
    uint32_t bits, decode_policy;                    /* cb200_decode_policy */
    const uint32_t *major_ptr;     /* CSR: rows + 1 */
    const uint32_t *minor_idx;     /* CSR: nnz gene indices */
    const uint32_t *block_col_idx; /* Blocked-ELL */
    const uint8_t *packed_values;
    const float *column_scales;
    const float *column_offsets; /* per-gene affine policy */
    const float *row_offsets;    /* column-scale / row-offset policy */
} cb200_public_layout;

/* scratch the calls below need for this layout (device memory, 256-byte aligned); they never allocate */
cb200_status cb200_public_projection_scratch(const cb200_public_layout *layout, int64_t out_cols, uint64_t *bytes);
/* out[rows, out_cols] = deq(X) * rhs[cols, out_cols]; fp32 row-major operands with leading dimensions
 * (matrix_ld_ of abi.cu), exact fp32 products; enqueues on `stream` */
cb200_status cb200_public_projection_forward(const cb200_public_layout *layout, const float *rhs, int64_t rhs_ld,
                                             int64_t out_cols, float *out, int64_t out_ld, int32_t device, void *stream,
                                             void *scratch, uint64_t scratch_bytes);
/* grad_rhs[cols, out_cols] = deq(X)^T * grad_out[rows, out_cols] (csr_spmm_bwd_rhs of abi.cu:376-389);
 * quantized CSR only.  grad_values has no meaning for integer codes and is not served. */
cb200_status cb200_public_projection_backward_rhs(const cb200_public_layout *layout, const float *grad_out,
                                                  int64_t grad_out_ld, int64_t out_cols, float *grad_rhs, int64_t grad_rhs_ld,
                                                  int32_t device, void *stream, void *scratch, uint64_t scratch_bytes);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif

#ifdef __cplusplus
}
#endif
#endif /* CELLERATOR_B200_H */
