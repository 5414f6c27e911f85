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

#define CB200_ABI_VERSION 2u

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
    CB200_STATUS_STALE_VALUE = 10, /* lifetime_validation_code::stale_value_generation, lifetimes.hh:88-94 */
    /* a collective was asked for and the fleet's NCCL communicator is not ready (nccl_communicator.ready,
     * include/Cellerator/dist/nccl_communicator.cuh:12-22); nothing falls back to another path */
    CB200_STATUS_COMM_NOT_READY = 11,
    /* a status query found the device status word of a launch set: a bounded wait inside a kernel ran out
     * and the launch's output is not valid */
    CB200_STATUS_DEVICE_WAIT_TIMEOUT = 12
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

/* Element look-up on a matrix whose arrays are HOST pointers: find_in_row / get_code / get_value,
 * include/Cellerator/quantized/access.cuh:47-79,133-153.  find_in_row scans the row from its start
 * and returns the index of the first entry of `column` in col_idx, -1 when the row holds none or an
 * argument is out of range.  get_code returns code `local_index` of the row's packed bytes.
 * get_value is the decoded value of (row, column), 0 where nothing is stored or the pair lies
 * outside the matrix (the reference's rule). */
int64_t cb200_find_in_row(const cb200_qcsr *m, int64_t row, int64_t column);
uint32_t cb200_get_code(const cb200_qcsr *m, int64_t row, int64_t local_index);
float cb200_get_value(const cb200_qcsr *m, int64_t row, int64_t column);
/* The same look-up for `count` (row, column) pairs of a DEVICE-resident matrix; rows, columns, values
 * and codes (optional, -1 where nothing is stored) are device arrays.  Enqueues on `stream`. */
cb200_status cb200_get_values(const cb200_qcsr *m, const int64_t *rows, const int32_t *columns, int64_t count,
                              float *values, int32_t *codes, int32_t device, void *stream);

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
                            * device_matrix for it, else prepare is refused: schedule "gene_gather" (fp32 FMAs
                            * entry by entry), or, with schedule_hint "tensor_blocked", the tensor-core schedules
                            * over the window-blocked copy, whose CTAs' sums are added in a fixed order too */
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
     * memory; otherwise "tensor_blocked" stays.
     *
     * The same with 4-bit codes and per-gene zero-points: prepare keeps dense tiles of CODES instead
     * (schedule "tensor_codes": rows x genes bytes, a byte per slot; 0 = nothing stored, code + 240 otherwise).
     * The matrix stays quantized: a launch decodes in registers with the scales and offsets it is given, so
     * only changed codes (a new structure or value generation) need a new prepare. */
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
    /* Optional request for one schedule by the name cb200_prepared_schedule reports ("gene_tiled",
     * "warp_per_row", "tensor_windows", "tensor_blocked", "tensor_dense", "tensor_codes"; transpose: "tensor_blocked",
     * "vector_reductions"; Blocked-ELL: "cuda_cores"); NULL or "" lets prepare choose from the shape and
     * the row statistics.  A request the shape or the policy cannot serve is not an error: prepare
     * keeps its own choice, and cb200_prepared_schedule tells which schedule runs.  This is the
     * planner's lever (one candidate per schedule); nothing in the library reads the environment. */
    const char *schedule_hint;
    /* Session-owned persistent memory (prepared_operation.persistent is borrowed, OPERATION_CORE.md:17-25;
     * the session reserves it before sealing, src/runtime/session_setup.cu.inc:111-140).  With
     * persistent != NULL prepare places everything it keeps on the device inside
     * [persistent, persistent + persistent_bytes), 256-byte aligned, and calls no cudaMalloc; the
     * block must hold cb200_spmm_persistent_requirement(problem) bytes and must outlive the prepared
     * operation, whose destroy call does not free it.  NULL: prepare allocates and destroy frees. */
    void *persistent;
    uint64_t persistent_bytes;
    /* Stream prepare enqueues its kernels and copies on (cudaStream_t; NULL = the device's default
     * stream).  Prepare waits for that stream before it returns, and for nothing else. */
    void *prepare_stream;
} cb200_spmm_problem;

typedef struct cb200_prepared cb200_prepared;

cb200_status cb200_spmm_prepare(const cb200_spmm_problem *problem, cb200_prepared **out);
/* Upper bound of the device bytes cb200_spmm_prepare would keep for this problem (0 when it keeps
 * nothing): what a session reserves as persistent memory before sealing and hands over in
 * cb200_spmm_problem.persistent.  Pure host arithmetic on the shape; the bound covers the padding of
 * the window-blocked copy, so prepare never needs more. */
cb200_status cb200_spmm_persistent_requirement(const cb200_spmm_problem *problem, uint64_t *bytes);
void cb200_prepared_destroy(cb200_prepared *prepared);
/* workspace_requirement, launch_bindings.hh:67-71 */
cb200_status cb200_prepared_workspace(const cb200_prepared *prepared, uint64_t *minimum_bytes, uint32_t *alignment);
/* kernel choice made at prepare time, as text: "warp_per_row", "gene_tiled" (exact fp32 products);
 * "tensor_windows", "tensor_blocked", "tensor_dense", "tensor_codes" (CSR, 16-bit products on tcgen05);
 * "tensor_blocked_x2" / "_x3" (fp32 products from bf16 passes); "tcgen05_block_rows" (Blocked-ELL);
 * transpose: "vector_reductions" (exact) or "tensor_blocked" */
const char *cb200_prepared_schedule(const cb200_prepared *prepared);
/* device bytes the prepared operation owns (row order, window-blocked copy): prepared_operation.persistent.bytes,
 * operation_core.hh:126-129,167-181; freed by cb200_prepared_destroy */
uint64_t cb200_prepared_persistent_bytes(const cb200_prepared *prepared);
/* rows x columns of the output a launch of this operation writes: m x n (forward, Blocked-ELL), k x n (transpose) */
cb200_status cb200_prepared_output_shape(const cb200_prepared *prepared, uint64_t *rows, uint64_t *columns);

#define CB200_ALL_ROWS (-1)

/* launch_bindings, launch_bindings.hh:90-102: everything that changes per launch.
 *
 * Status word.  The kernels wait on barriers with a bound; when a bound runs out the launch ends early,
 * its output is not valid, and the first 32-bit word of `workspace` is non-zero afterwards.  Every launch
 * clears that word on its stream first.  cb200_spmm_run cannot report it (it returns before the kernels
 * run): read it with cb200_prepared_status once the stream has passed the launch. */
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
    int64_t row_end;         /* CB200_ALL_ROWS (-1) = up to the last row; [r,r) is an empty shard: a forward
                              * launch then writes nothing, a transpose scales G' by beta */
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
/* Reads the status word of the launches that used `workspace` (the transient_workspace of
 * launch_bindings.hh:61-65): copies it to *host_word in stream order and waits for `stream`.  Returns
 * CB200_STATUS_SUCCESS when the word is 0, CB200_STATUS_DEVICE_WAIT_TIMEOUT when a kernel gave up a
 * bounded wait (the output of that launch is not valid; the context stays usable).  A binding calls
 * it where it would synchronise anyway: after the last launch of a step, before results are used.
 * A prepared operation whose schedule needs no workspace reports 0. */
cb200_status cb200_prepared_status(const cb200_prepared *prepared, const void *workspace, void *stream,
                                   int32_t *host_word);

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
/* Status word of the last cb200_qcsr_forward_static call on `device` (it lives in the library's own
 * array, which the caller cannot read): copied in stream order, then `stream` is waited for.  Same
 * return convention as cb200_prepared_status; allocates nothing.  Before the first static call on the
 * device there is nothing to read and the call returns CB200_STATUS_INVALID_ARGUMENT. */
cb200_status cb200_qcsr_forward_static_status(int32_t device, void *stream, int32_t *host_word);

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

/* persistent_lifetime, session.cuh:28-32: what a persistent reservation is tied to */
typedef enum cb200_persistent_lifetime {
    CB200_LIFETIME_STRUCTURE = 0,   /* lives as long as the structure (a window-blocked or gene-major copy) */
    CB200_LIFETIME_PLAN = 1,        /* lives as long as a prepared plan */
    CB200_LIFETIME_GRAPH_STABLE = 2 /* addresses that captured graphs hold */
} cb200_persistent_lifetime;

/* session_accounting, session.cuh:72-90: bytes and counts per class since the session was created */
typedef struct cb200_allocation_accounting {
    uint64_t current_bytes, high_water_bytes, allocation_count;
} cb200_allocation_accounting;
typedef struct cb200_session_accounting {
    cb200_allocation_accounting structure, plan, graph_stable, transient;
    uint64_t device_query_count, handle_prepare_count, launch_bind_count, synchronization_count;
} cb200_session_accounting;

/* session_cache_kind / session_cache_key / session_cache_entry, session.cuh:34-61: three fixed caches of 64 entries */
typedef enum cb200_session_cache_kind { CB200_CACHE_PLAN = 0, CB200_CACHE_PROJECTION = 1, CB200_CACHE_ORDER_TRANSFORM = 2 } cb200_session_cache_kind;
typedef struct cb200_session_cache_entry {
    uint64_t key_high, key_low;
    void *state;
    uint64_t structure_epoch, generation;
} cb200_session_cache_entry;

cb200_status cb200_session_create(const cb200_session_options *options, cb200_session **out);
/* reserve_persistent with lifetime CB200_LIFETIME_STRUCTURE */
cb200_status cb200_session_reserve_persistent(cb200_session *s, uint64_t bytes, void **allocation);
/* reserve_persistent, session_setup.cu.inc:111-140: one device allocation per call, at most 64, none after sealing */
cb200_status cb200_session_reserve_persistent_as(cb200_session *s, int32_t lifetime, uint64_t bytes, void **allocation);
/* prepare_stream_libraries: this backend uses no cuBLAS / cuSPARSE handle, so nothing is created; the call is
 * counted (handle_prepare_count) and refused after sealing, like the reference's */
cb200_status cb200_session_prepare_stream_libraries(cb200_session *s, uint32_t stream_index);
cb200_status cb200_session_get_accounting(const cb200_session *s, cb200_session_accounting *out);
/* graph_stable_address: 1 when [address, address + bytes) lies inside a graph-stable reservation */
int32_t cb200_session_graph_stable_address(const cb200_session *s, const void *address, uint64_t bytes);
/* insert_session_cache / find_session_cache: an entry with the same key is replaced; a full cache -> INSUFFICIENT_WORKSPACE;
 * find returns NULL when the key is absent */
cb200_status cb200_session_cache_insert(cb200_session *s, int32_t kind, const cb200_session_cache_entry *entry);
const cb200_session_cache_entry *cb200_session_cache_find(const cb200_session *s, int32_t kind, uint64_t key_high, uint64_t key_low);
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
    const uint8_t *packed_values;  /* CSR, 4-bit codes: a row's codes take ceil(entries / 2) bytes and the rows follow each other
                                    * (build_packed_row_ptr, quantized/layout.cuh:111-129); the calls derive the packed row
                                    * offsets from major_ptr on the stream, in the scratch */
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


/* Status word of the last routed projection call that used `scratch` (its first 32-bit word, see
 * cb200_launch): same convention as cb200_prepared_status. */
cb200_status cb200_public_projection_status(const void *scratch, int32_t device, void *stream, int32_t *host_word);

/* ------------------------------------------------------------------------------------------
 * The backend-neutral SpMM request and its 128-bit signature: spmm_request, validate_spmm_request,
 * classify_trivial_operation and make_operation_signature
 * (include/Cellerator/compute/math/operation.hh:136-221, src/compute/math/operation.cc:119-292,
 * src/compute/math/operation_signature.cc:30-68).  The signature is the key of the reference's plan
 * cache; it never depends on a live address.  Field meanings and enum values are the reference's:
 * type codes are real::value_* of include/Cellerator/types.cuh:150-158 (f16 3, f32 4, f64 5, bf16 6,
 * fp8 7 / 8), layouts 1 row-major / 2 column-major, workspace kinds 1..3, reuse kinds 1..3,
 * feature-order kinds 1 canonical / 2 packed, epilogue kinds as cb200_epilogue. */
typedef struct cb200_feature_order_identity { /* operation.hh:87-94 */
    uint32_t schema_version; /* 1 */
    uint32_t kind;
    uint32_t feature_count;
    uint32_t feature_axis_identity_version;
    uint64_t feature_axis_identity;
    uint64_t packing_geometry_identity;
} cb200_feature_order_identity;

typedef struct cb200_scalar_value { /* operation.hh:104-108 */
    uint32_t type_code;
    uint32_t reserved;
    uint64_t bits;
} cb200_scalar_value;

typedef struct cb200_spmm_request { /* operation.hh:136-164 */
    uint32_t schema_version; /* 1 */
    uint32_t operation;      /* 1 = spmm */
    uint64_t m, k, n, sparse_nnz;
    uint32_t structure_schema_version; /* sparse_structure_identity, operation.hh:98-102 */
    uint32_t structure_identity_version;
    uint64_t structure_value;
    uint32_t transpose_sparse, transpose_dense;   /* 0 none, 1 transpose */
    uint32_t dense_rhs_layout, output_layout;
    uint64_t dense_rhs_leading_dimension, output_leading_dimension;
    uint32_t sparse_storage_type_code, dense_storage_type_code, output_storage_type_code;
    uint32_t compute_type_code, accumulation_type_code;
    cb200_scalar_value alpha, beta;
    uint32_t determinism;    /* 0 allow non-deterministic, 1 deterministic */
    uint32_t workspace_kind, workspace_reserved;
    uint64_t workspace_byte_limit;
    uint32_t reuse_kind, reuse_reserved;
    uint64_t reuse_expected_run_count;
    uint32_t epilogue_kind, epilogue_bias_type_code;
    uint64_t epilogue_bias_element_count;
    cb200_feature_order_identity sparse_feature_order, dense_feature_order;
} cb200_spmm_request;

/* request_validation_code, operation.hh:63-80 (same values); 0 = ok */
int32_t cb200_spmm_request_validate(const cb200_spmm_request *request);
/* trivial_operation_kind, operation.hh:195-199: 0 none, 1 no output, 2 epilogue only */
int32_t cb200_spmm_request_classify(const cb200_spmm_request *request);
/* make_operation_signature: signature[0] = low, signature[1] = high */
cb200_status cb200_spmm_request_signature(const cb200_spmm_request *request, uint64_t signature[2]);
/* The request a prepared problem and one of its launches stand for (shapes, transposes, leading
 * dimensions, type codes, alpha / beta, determinism, epilogue), with the identities the caller owns
 * passed through: fills *request so that it validates and can be signed.  reuse: persistent. */
cb200_status cb200_spmm_request_from_problem(const cb200_spmm_problem *problem, const cb200_launch *launch,
                                             uint64_t structure_identity, uint64_t feature_axis_identity,
                                             cb200_spmm_request *request);

/* ------------------------------------------------------------------------------------------
 * Host container of a quantized Blocked-ELL matrix: matrix::quantized_blocked_ell,
 * include/Cellerator/matrix/quantized_blocked_ell.cuh:27-220.  One malloc slab holds, in this order,
 * block_col_idx, the packed codes, column scales, column offsets and row offsets; pin registers the
 * slab with the CUDA driver (cudaHostRegisterPortable) so that copies from it run asynchronously. */
enum { CB200_QBELL_HOST_REGISTERED = 1u << 0 };
typedef struct cb200_qbell_host {
    uint32_t rows, cols, nnz, block_size, ell_cols, bits, row_stride_bytes, decode_policy, flags;
    void *storage;
    uint32_t *block_col_idx;
    uint8_t *packed_values;
    float *column_scales;
    float *column_offsets;
    float *row_offsets;
} cb200_qbell_host;

/* aux word of the container's serialised header, quantized_blocked_ell.cuh:27-48:
 * (ell_width << 24) | (bits << 16) | block_size */
uint64_t cb200_qbell_pack_aux(uint32_t bits, uint32_t block_size, uint64_t ell_width);
void cb200_qbell_unpack_aux(uint64_t aux, uint32_t *bits, uint32_t *block_size, uint64_t *ell_width, uint32_t *ell_cols);
/* quantized_blocked_ell_row_bytes / _aligned_row_bytes (quantized_blocked_ell.cuh:50-66); alignment <= 1: no padding */
uint32_t cb200_qbell_row_bytes(uint32_t bits, uint32_t ell_cols);
uint32_t cb200_qbell_aligned_row_bytes(uint32_t bits, uint32_t ell_cols, uint32_t alignment);
/* init: row_stride_bytes 0 = aligned_row_bytes(bits, ell_cols, 16) */
void cb200_qbell_host_init(cb200_qbell_host *m, uint32_t rows, uint32_t cols, uint32_t nnz, uint32_t block_size,
                           uint32_t ell_cols, uint32_t bits, uint32_t decode_policy, uint32_t row_stride_bytes);
uint64_t cb200_qbell_host_bytes(const cb200_qbell_host *m); /* sizeof(*m) + the slab */
int32_t cb200_qbell_host_allocate(cb200_qbell_host *m);     /* 1 ok, 0 out of memory; frees what it held */
int32_t cb200_qbell_host_pin(cb200_qbell_host *m);          /* 1 registered (or nothing to register), 0 refused */
void cb200_qbell_host_unpin(cb200_qbell_host *m);
void cb200_qbell_host_clear(cb200_qbell_host *m);
/* the container as a cb200_qbell whose arrays are the slab's HOST pointers (offsets follow decode_policy) */
cb200_status cb200_qbell_host_view(const cb200_qbell_host *m, cb200_qbell *view);
/* Copies the slab to `device_storage` (device memory of cb200_qbell_host_bytes(m) - sizeof(*m) bytes, 256-byte
 * aligned) with one cudaMemcpyAsync on `stream` and fills *device_view with the device addresses of the
 * five arrays, which keep the slab's offsets. */
cb200_status cb200_qbell_host_upload(const cb200_qbell_host *m, void *device_storage, uint64_t device_bytes,
                                     int32_t device, void *stream, cb200_qbell *device_view);

/* ------------------------------------------------------------------------------------------
 * Multi-GPU layer.  fleet_context (src/compute/runtime/runtime.hh:47-87, runtime.cu:96-199): the
 * devices of one process as numbered slots, one stream per slot, peer access, grow-only scratch per
 * slot, and the NCCL communicator (nccl_communicator, init_local_nccl_communicator /
 * init_ranked_nccl_communicator, communicator_allreduce:
 * include/Cellerator/dist/nccl_communicator.cuh:12-22,109-156,290-315).  Two ways to build one:
 *   - one process, several GPUs (the reference's default): slots = devices[], communicator from
 *     ncclCommInitAll over them; world_size is the slot count;
 *   - one process per GPU: one slot, world_size / world_rank of the job and the 128-byte NCCL unique id
 *     that rank 0 made with cb200_fleet_unique_id and the launcher distributed (ncclCommInitRank).
 * NCCL is loaded at run time (dlopen of libnccl.so.2, or of options.nccl_library): a process that
 * already holds a copy shares it.  When the library or the communicator cannot be had the fleet is
 * still created, cb200_fleet_communicator_ready reports 0, and every call that needs a collective
 * returns CB200_STATUS_COMM_NOT_READY: nothing falls back to peer copies behind the caller's back
 * (the reference's reduce does, src/compute/runtime/reduce.cu:228-294).  No lock anywhere: one thread
 * drives a fleet, as in the reference. */
typedef struct cb200_fleet cb200_fleet;

typedef struct cb200_fleet_options {
    uint32_t version;
    size_t size;
    int32_t device_count;       /* local slots, 1..16 */
    const int32_t *devices;     /* CUDA ordinals; NULL = 0 .. device_count-1 */
    void *const *streams;       /* optional caller streams, one per slot; NULL = the fleet creates non-blocking ones */
    int32_t enable_peer_access; /* cudaDeviceEnablePeerAccess between the slots (discover_fleet's default) */
    int32_t world_size;         /* 0 = device_count (single process) */
    int32_t world_rank;         /* rank of slot 0; slot i has rank world_rank + i */
    const void *nccl_unique_id; /* 128 bytes; NULL with world_size == device_count: ncclCommInitAll */
    const char *nccl_library;   /* NULL = "libnccl.so.2" */
} cb200_fleet_options;

/* ncclGetUniqueId: 128 bytes for the launcher to hand to every rank */
cb200_status cb200_fleet_unique_id(const char *nccl_library, void *unique_id_128);
cb200_status cb200_fleet_create(const cb200_fleet_options *options, cb200_fleet **out);
void cb200_fleet_destroy(cb200_fleet *fleet);
int32_t cb200_fleet_slot_count(const cb200_fleet *fleet);
int32_t cb200_fleet_world_size(const cb200_fleet *fleet);
int32_t cb200_fleet_device(const cb200_fleet *fleet, uint32_t slot);           /* fleet_device_id; -1 = no such slot */
void *cb200_fleet_stream(const cb200_fleet *fleet, uint32_t slot);             /* fleet_stream */
int32_t cb200_fleet_communicator_ready(const cb200_fleet *fleet);              /* nccl_communicator.ready */
/* request_fleet_scratch, runtime.cu: device memory of the slot, at least `bytes`, kept until destroy; grows by
 * reallocation (contents are not kept), so ask for the largest size before the first launch */
cb200_status cb200_fleet_request_scratch(cb200_fleet *fleet, uint32_t slot, uint64_t bytes, void **scratch);
cb200_status cb200_fleet_synchronize(cb200_fleet *fleet, const uint32_t *slots, uint32_t slot_count); /* synchronize_slots */

/* Row ranges of `parts` shards: the reference's uniform rule (build_uniform_block_row_ptr with
 * rows_per_block = ceil(rows / parts), layout.cuh:131-157) read back through get_block
 * (access.cuh:7-44), padded with empty trailing shards when rows do not fill every part, so that
 * shard i belongs to rank i.  row_ptr / packed_row_ptr are HOST arrays (packed_row_ptr NULL: equal to
 * row_ptr, the 8-bit case).  blocks has `parts` entries. */
cb200_status cb200_fleet_partition(int64_t rows, int32_t parts, const int64_t *row_ptr, const int64_t *packed_row_ptr,
                                   cb200_csr_block *blocks);

/* dist::launch_csr_spmm_fwd_f16_f32 (src/compute/sparse/project/project.cu:321-341): the forward
 * projection of every listed slot, each on its slot's device and stream (launches[i].device and
 * .stream are overwritten with the slot's), no collective, no host synchronisation. */
cb200_status cb200_fleet_run_forward(cb200_fleet *fleet, const uint32_t *slots, uint32_t slot_count,
                                     cb200_prepared *const *prepared, cb200_launch *launches);
/* dist::launch_csr_spmm_bwd_rhs_f16_f32 + dist::reduce_sum_to_leader_f32
 * (src/compute/sparse/ops/kernels/dist_sparse.cu:24-32,177-197, src/compute/runtime/reduce.cu:147-294):
 * every listed slot computes its k x n partial of G' into launches[i].out, then ONE
 * ncclAllReduce(float32, sum) per slot over k*n floats (out_ld must equal n), in place, grouped, on the
 * slots' streams, so that every rank of the job ends with the sum.  Stream order carries the dependency:
 * no host synchronisation before the collective (the reference has one, reduce.cu:164).  A job of one
 * rank needs no communicator.  Otherwise a communicator that is not ready -> CB200_STATUS_COMM_NOT_READY
 * before any kernel is enqueued. */
cb200_status cb200_fleet_run_transpose(cb200_fleet *fleet, const uint32_t *slots, uint32_t slot_count,
                                       cb200_prepared *const *prepared, cb200_launch *launches);
/* reduce_sum_to_leader_f32 as an all-reduce: outs[i] = sum over the job's ranks of partials[i]
 * (count floats, device pointers of the slots; outs[i] may equal partials[i]). */
cb200_status cb200_fleet_allreduce_sum_f32(cb200_fleet *fleet, const uint32_t *slots, uint32_t slot_count,
                                           const float *const *partials, float *const *outs, uint64_t count);

/* ------------------------------------------------------------------------------------------
 * Forward projection from HOST buffers: the call of a caller whose matrix lives in host memory
 * (the reference's models and the public ABI copy their operands in before every projection,
 * src/abi/abi.cu:278-340).  The stage owns device buffers for `chunk_count` row chunks in flight and
 * three streams; a run cuts the row range into chunks of about rows / chunks_per_run rows, copies
 * chunk i+1 in (one cudaMemcpyAsync per array) while chunk i is multiplied and chunk i-1's rows of Y
 * are copied out.  Everything crosses PCIe inside the call; pinned host memory makes the copies
 * asynchronous.  The operation behind it is prepared without the matrix (CSR schedules that read the
 * arrays at launch), because the values arrive with the call. */
typedef struct cb200_host_stage cb200_host_stage;

typedef struct cb200_host_stage_options {
    uint32_t version;
    size_t size;
    int32_t device;
    int64_t k, n;
    int32_t bits, policy, dense_dtype, multiply;
    int64_t max_chunk_rows;   /* rows one device chunk buffer holds */
    int64_t max_chunk_nnz;    /* stored entries one device chunk buffer holds */
    int32_t chunk_buffers;    /* chunks in flight, 2..4 */
    /* A shorter form of the gene indices on the host -> device link (host threads rewrite a chunk's indices into a pinned
     * staging buffer, a kernel restores them on the device):
     *    0 = gap bytes (see 2) where at least four host threads are usable, for the share of each chunk's rows that
     *        keeps the host and the link busy for the same time (the first rewritten chunks of a call are timed and
     *        set the share; the other rows go as 32-bit indices; a call that found the host very slow, or genes that
     *        do not ascend, also keeps the next few calls on 32-bit indices);
     *    1 = 16-bit words (k <= 65,536 only; 32-bit elsewhere): 3 bytes per entry on the link instead of 5;
     *    2 = gap bytes, any k: one byte per entry (gene - previous gene of the row - 1), with a short list of
     *        {position, gene} for the entries whose gap does not fit: 2 bytes per entry on the link.  A chunk with more
     *        such entries than the list holds (one in 128; rows whose genes do not ascend) goes as 32-bit indices;
     *   -1 = 32-bit indices as they are. */
    int32_t narrow_indices;
    /* Host threads that narrow (the calling thread included): 0 = the cores this process may run on, at most 16.  A
     * process that shares its cores with other ranks passes its share. */
    int32_t host_threads;
} cb200_host_stage_options;

cb200_status cb200_host_stage_create(const cb200_host_stage_options *options, cb200_host_stage **out);
void cb200_host_stage_destroy(cb200_host_stage *stage);
uint64_t cb200_host_stage_device_bytes(const cb200_host_stage *stage);
/* The host half of the gap form, for callers that stage their own copies (and for tests): gaps[i] for the entries
 * [row_ptr[0], row_ptr[rows]) of col_idx, written from gaps[0] on -- gene - previous gene of the row - 1, the row's
 * first entry its gene; 255 marks an entry whose gene is listed instead ({position relative to row_ptr[0], gene},
 * ascending positions): a gap of 255 or more, or a gene that does not ascend.  `threads` host threads (1..64) share the
 * rows.  Returns the number of listed entries, -1 if there are more than `room`, -2 on bad arguments (no CUDA call). */
int64_t cb200_host_encode_gene_gaps(const int32_t *col_idx, const int64_t *row_ptr, int64_t rows, uint8_t *gaps, int32_t *exception_positions,
                                    int32_t *exception_genes, int64_t room, int32_t threads);
/* x: HOST arrays (row_ptr, col_idx, packed_values, packed_row_ptr for 4-bit codes, scales, offsets);
 * w: k x n HOST (dense_dtype), y: rows x n HOST fp32.  Returns after the last copy has landed in y
 * (it waits for its own streams).  h2d_bytes / d2h_bytes (optional) receive the bytes moved. */
cb200_status cb200_host_forward(cb200_host_stage *stage, const cb200_qcsr *x, const void *w, int64_t w_ld, float *y,
                                int64_t y_ld, float alpha, uint64_t *h2d_bytes, uint64_t *d2h_bytes);

/* ------------------------------------------------------------------------------------------
 * Test hook (no counterpart in the reference).  Makes the bounded waits of the tensor-core forward
 * kernel over the window-blocked copy observable: while armed, that kernel's W loader issues no
 * copies and every wait of the launch gives up after `poll_limit` polls, so the launch ends within
 * microseconds with the status word set, its TMEM freed and its output invalid.  The next launch after
 * cb200_test_disarm_wait_timeout is a normal one.  poll_limit is clamped to [64, 2^22]. */
void cb200_test_arm_wait_timeout(uint32_t poll_limit);
void cb200_test_disarm_wait_timeout(void);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif

#ifdef __cplusplus
}
#endif
#endif /* CELLERATOR_B200_H */
