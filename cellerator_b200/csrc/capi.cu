// extern "C" surface of libcellerator_b200.so (declared in include/cellerator_b200.h):
// status/error plumbing, host layout helpers, capability query, the prepared-operation
// lifecycle and the runtime session.  Kernels live in the other translation units.
#include "kernels.cuh"

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <new>
#include <vector>

namespace cb200 {

std::atomic<std::uint64_t> g_kernel_launches{0};

char *last_error_buffer() {
    thread_local char buffer[512] = "";
    return buffer;
}

cb200_status fail(cb200_status status, const char *fmt, ...) {
    va_list args;
    va_start(args, fmt);
    std::vsnprintf(last_error_buffer(), 512, fmt, args);
    va_end(args);
    return status;
}

void clear_error() { last_error_buffer()[0] = '\0'; }

namespace {

template<typename T>
bool valid_header(const T *desc) {
    return desc != nullptr && desc->version == CB200_ABI_VERSION && desc->size >= sizeof(T);
}

bool supported_bits(int bits) { return bits == 4 || bits == 8; }
bool supported_dense(int dtype) { return dtype == CB200_DTYPE_F32 || dtype == CB200_DTYPE_BF16; }

qcsr_view view_of(const cb200_qcsr &m) {
    return qcsr_view{m.rows, m.cols, m.nnz, m.bits, m.policy, m.row_ptr, m.packed_row_ptr,
                     m.col_idx, m.packed_values, m.scales, m.offsets};
}

qbell_view view_of(const cb200_qbell &m) {
    return qbell_view{m.rows, m.cols, m.block_size, m.ell_cols, m.row_stride_bytes, m.bits, m.policy,
                      m.block_col_idx, m.packed_values, m.scales, m.offsets};
}

} // namespace
} // namespace cb200

using namespace cb200;

// Prepared state: everything frozen at prepare time (operation_core.hh:167-181).  It owns no
// launch pointer.
struct cb200_prepared {
    cb200_spmm_problem problem;
    fwd_schedule schedule;
    const char *schedule_name;
    std::uint64_t workspace_bytes;
    std::uint32_t workspace_alignment;
    int sm_count;
    double mean_row_nnz, max_row_nnz;
    // persistent state built at prepare time (persistent_kernel_state, operation_core.hh:126-129):
    // the rows in descending order of length, on the device; null when no host row_ptr was given
    std::int32_t *row_order;
    // ... and, when prepare was given the device-resident matrix and bf16 products are allowed, the
    // window-blocked copy the tensor-core kernel streams
    blocked_layout blocked;
    // ... or, for a transpose that has to be deterministic, the gene-major copy the gather kernel reads
    gene_major_layout gene_major;
    std::uint64_t persistent_bytes;
    // the device memory all of the above lives in: the caller's block or this operation's own allocations
    device_arena arena;
    bool bell_cuda_cores; // Blocked-ELL: the caller asked for the CUDA-core kernel
};

struct cb200_session {
    int device;
    bool sealed;
    std::uint32_t stream_count;
    cudaStream_t streams[8];
    bool owned[8];
    void *transient[8];
    std::uint64_t transient_bytes[8];
    void *persistent[64];
    std::uint64_t persistent_bytes[64];
    int persistent_lifetime[64];
    std::uint32_t persistent_count;
    cb200_session_accounting accounting;
    cb200_session_cache_entry caches[3][64];
    std::uint32_t cache_size[3];
};

namespace {
void account(cb200_allocation_accounting *a, std::uint64_t bytes) {
    a->current_bytes += bytes;
    if (a->current_bytes > a->high_water_bytes) a->high_water_bytes = a->current_bytes;
    ++a->allocation_count;
}
} // namespace

extern "C" {

const char *cb200_status_string(cb200_status status) {
    switch (status) {
    case CB200_STATUS_SUCCESS: return "success";
    case CB200_STATUS_INVALID_ARGUMENT: return "invalid argument";
    case CB200_STATUS_INVALID_SHAPE: return "invalid shape";
    case CB200_STATUS_UNSUPPORTED: return "unsupported";
    case CB200_STATUS_CUDA_ERROR: return "CUDA error";
    case CB200_STATUS_INTERNAL_ERROR: return "internal error";
    case CB200_STATUS_STALE_STRUCTURE: return "stale structure";
    case CB200_STATUS_INSUFFICIENT_WORKSPACE: return "insufficient workspace";
    case CB200_STATUS_INVALID_STREAM: return "invalid stream";
    case CB200_STATUS_SEALED: return "session sealed";
    case CB200_STATUS_STALE_VALUE: return "stale value generation";
    case CB200_STATUS_COMM_NOT_READY: return "communicator not ready";
    case CB200_STATUS_DEVICE_WAIT_TIMEOUT: return "a bounded device wait ran out";
    }
    return "unknown status";
}

const char *cb200_last_error(void) { return last_error_buffer(); }
uint32_t cb200_abi_version(void) { return CB200_ABI_VERSION; }
uint64_t cb200_kernel_launch_count(void) { return g_kernel_launches.load(std::memory_order_relaxed); }

/* ---- host layout helpers ------------------------------------------------------------ */

int64_t cb200_build_packed_row_ptr(int32_t bits, const int64_t *row_ptr, int64_t rows, int64_t *packed_row_ptr) {
    if (row_ptr == nullptr || packed_row_ptr == nullptr || rows < 0 || !(bits == 1 || bits == 2 || bits == 4 || bits == 8))
        return -1;
    const int64_t per_byte = 8 / bits;
    int64_t total = 0;
    packed_row_ptr[0] = 0;
    for (int64_t r = 0; r < rows; ++r) {
        const int64_t count = row_ptr[r + 1] - row_ptr[r];
        total += count <= 0 ? 0 : (count + per_byte - 1) / per_byte;
        packed_row_ptr[r + 1] = total;
    }
    return total;
}

int64_t cb200_block_count_for_rows(int64_t rows, int64_t rows_per_block) {
    return (rows <= 0 || rows_per_block <= 0) ? 0 : (rows + rows_per_block - 1) / rows_per_block;
}

int64_t cb200_build_uniform_block_row_ptr(int64_t rows, int64_t rows_per_block, int64_t *block_row_ptr) {
    if (block_row_ptr == nullptr || rows < 0 || rows_per_block <= 0) return -1;
    const int64_t count = cb200_block_count_for_rows(rows, rows_per_block);
    for (int64_t b = 0; b < count; ++b) {
        const int64_t start = b * rows_per_block;
        block_row_ptr[b] = start < rows ? start : rows;
    }
    block_row_ptr[count] = rows;
    return count;
}

cb200_status cb200_get_block(int64_t rows, const int64_t *row_ptr, const int64_t *packed_row_ptr,
                             const int64_t *block_row_ptr, int64_t block_count, int64_t block_index,
                             cb200_csr_block *out) {
    clear_error();
    if (out == nullptr || row_ptr == nullptr || packed_row_ptr == nullptr)
        return fail(CB200_STATUS_INVALID_ARGUMENT, "get_block needs row_ptr, packed_row_ptr and an output");
    std::memset(out, 0, sizeof(*out));
    out->block_index = block_index;
    if (block_row_ptr == nullptr || block_count <= 0) {
        out->block_index = 0;
        out->row_end = rows;
    } else if (block_index < 0 || block_index >= block_count) {
        return CB200_STATUS_SUCCESS; /* all-zero block, like the reference */
    } else {
        out->row_begin = block_row_ptr[block_index];
        out->row_end = block_row_ptr[block_index + 1];
    }
    out->nnz_begin = row_ptr[out->row_begin];
    out->nnz_end = row_ptr[out->row_end];
    out->packed_begin = packed_row_ptr[out->row_begin];
    out->packed_end = packed_row_ptr[out->row_end];
    return CB200_STATUS_SUCCESS;
}

/* ---- device codec ------------------------------------------------------------------- */

cb200_status cb200_quantize_rows(const cb200_qcsr *m, int64_t row_begin, int64_t row_end, const float *values,
                                 int32_t device, void *stream) {
    clear_error();
    if (!valid_header(m)) return fail(CB200_STATUS_INVALID_ARGUMENT, "bad cb200_qcsr header");
    device_scope scope(device);
    CB200_CUDA_OK(scope.status);
    return launch_quantize_rows(view_of(*m), row_begin, row_end, values, static_cast<cudaStream_t>(stream));
}

cb200_status cb200_dequantize_rows(const cb200_qcsr *m, int64_t row_begin, int64_t row_end, float *values,
                                   int32_t device, void *stream) {
    clear_error();
    if (!valid_header(m)) return fail(CB200_STATUS_INVALID_ARGUMENT, "bad cb200_qcsr header");
    device_scope scope(device);
    CB200_CUDA_OK(scope.status);
    return launch_dequantize_rows(view_of(*m), row_begin, row_end, values, static_cast<cudaStream_t>(stream));
}

cb200_status cb200_qbell_quantize_rows(const cb200_qbell *m, int64_t row_begin, int64_t row_end,
                                       const float *values_by_slot, int32_t device, void *stream) {
    clear_error();
    if (!valid_header(m)) return fail(CB200_STATUS_INVALID_ARGUMENT, "bad cb200_qbell header");
    device_scope scope(device);
    CB200_CUDA_OK(scope.status);
    return launch_qbell_quantize_rows(view_of(*m), row_begin, row_end, values_by_slot, static_cast<cudaStream_t>(stream));
}

cb200_status cb200_qbell_dequantize_rows(const cb200_qbell *m, int64_t row_begin, int64_t row_end,
                                         float *values_by_slot, int32_t device, void *stream) {
    clear_error();
    if (!valid_header(m)) return fail(CB200_STATUS_INVALID_ARGUMENT, "bad cb200_qbell header");
    device_scope scope(device);
    CB200_CUDA_OK(scope.status);
    return launch_qbell_dequantize_rows(view_of(*m), row_begin, row_end, values_by_slot, static_cast<cudaStream_t>(stream));
}

/* ---- capability query ---------------------------------------------------------------- */

cb200_status cb200_backend_query(int32_t projection, const cb200_numeric_policy *numeric, cb200_capability *out) {
    clear_error();
    if (!valid_header(numeric) || out == nullptr) return fail(CB200_STATUS_INVALID_ARGUMENT, "bad query arguments");
    out->version = CB200_ABI_VERSION;
    out->size = sizeof(*out);
    out->supported = 0;
    out->flags = 0u;
    out->persistent_bytes = 0u;
    out->transient_bytes = 0u;
    out->name = "";
    const bool codes = numeric->sparse_storage == CB200_DTYPE_U8 || numeric->sparse_storage == CB200_DTYPE_U4;
    const bool common = codes && numeric->quantized != 0 && numeric->output_storage == CB200_DTYPE_F32 &&
                        numeric->accumulation == CB200_DTYPE_F32;
    switch (projection) {
    case CB200_PROJECTION_CSR:
        out->name = "cb200.qcsr.forward.sm100a";
        /* fp32 products for either W type; bf16 products (tensor cores) only with a bf16 W */
        out->supported = common && supported_dense(numeric->dense_storage) &&
                         (numeric->multiply == CB200_DTYPE_F32 ||
                          (numeric->multiply == CB200_DTYPE_BF16 && numeric->dense_storage == CB200_DTYPE_BF16));
        /* a row is summed by one owner in a fixed order: repeated runs are bitwise identical */
        out->flags = CB200_CAP_DETERMINISTIC | CB200_CAP_GRAPH_CAPTURE;
        break;
    case CB200_PROJECTION_TRANSPOSE:
        out->name = "cb200.qcsr.transpose.sm100a";
        /* G is fp32 storage either way; bf16 products round both factors (tensor-core schedule) */
        out->supported = common && numeric->dense_storage == CB200_DTYPE_F32 &&
                         (numeric->multiply == CB200_DTYPE_F32 || numeric->multiply == CB200_DTYPE_BF16);
        /* floating-point reductions, order not fixed -- unless prepare is asked for determinism and
         * handed the matrix, when it builds a gene-major copy and the sums have a fixed order */
        out->flags = CB200_CAP_GRAPH_CAPTURE;
        break;
    case CB200_PROJECTION_BLOCKED_ELL:
        out->name = "cb200.qbell.forward.sm100a";
        out->supported = common && supported_dense(numeric->dense_storage) &&
                         (numeric->multiply == CB200_DTYPE_F32 || numeric->multiply == CB200_DTYPE_BF16);
        out->flags = CB200_CAP_DETERMINISTIC | CB200_CAP_GRAPH_CAPTURE;
        break;
    default:
        return fail(CB200_STATUS_UNSUPPORTED, "unknown projection %d", projection);
    }
    return CB200_STATUS_SUCCESS;
}

} // extern "C"

/* ---- prepared operation --------------------------------------------------------------- */

namespace {

// What prepare will build for a problem, decided from the shape, the mean row length and the caller's
// request alone (no device query), so that the bytes it needs can be told before the session is sealed.
struct schedule_plan {
    cb200_status status = CB200_STATUS_SUCCESS;
    bool tiled = false;          // CSR forward: gene-tiled kernel (else warp per row)
    bool tensor_windows = false; // CSR forward: tensor cores fed from the CSR arrays
    bool blocked = false;        // window-blocked copy (forward or transpose)
    bool blocked_lo = false;     // ... with the second array of baked words (split products)
    bool split = false;          // fp32 products rebuilt from bf16 passes
    bool dense_wanted = false;   // forward: decoded operand tiles instead of entry words, when they fit
    bool dense_forced = false;   // ... asked for by name: the free-memory rule does not apply
    bool codes_wanted = false;   // forward, 4-bit codes: tiles of codes (a byte per slot) instead of decoded tiles
    bool gene_gather = false;    // transpose with a fixed order of the sums
    bool row_order = false;      // length-sorted row order for the tiled kernels
    bool bell_cuda_cores = false;
    double mean_row_nnz = 0.0;
};

bool hint_is(const char *hint, const char *name) { return hint != nullptr && std::strcmp(hint, name) == 0; }
bool hint_starts(const char *hint, const char *prefix) {
    return hint != nullptr && std::strncmp(hint, prefix, std::strlen(prefix)) == 0;
}

cb200_status validate_problem(const cb200_spmm_problem *problem) {
    if (!valid_header(problem)) return fail(CB200_STATUS_INVALID_ARGUMENT, "bad cb200_spmm_problem header");
    if (problem->m < 0 || problem->k < 0 || problem->n < 0 || problem->nnz < 0)
        return fail(CB200_STATUS_INVALID_SHAPE, "negative dimension");
    if (problem->structure_epoch == 0u) return fail(CB200_STATUS_STALE_STRUCTURE, "structure epoch must be non-zero");
    if (!supported_bits(problem->bits)) return fail(CB200_STATUS_UNSUPPORTED, "bits must be 4 or 8, got %d", problem->bits);
    if (problem->policy != CB200_DECODE_PER_GENE_AFFINE && problem->policy != CB200_DECODE_COLUMN_SCALE_ROW_OFFSET)
        return fail(CB200_STATUS_UNSUPPORTED, "unknown decode policy %d", problem->policy);
    if (problem->multiply != 0 && problem->multiply != CB200_DTYPE_F32 && problem->multiply != CB200_DTYPE_BF16)
        return fail(CB200_STATUS_UNSUPPORTED, "multiply must be fp32 or bf16, got %d", problem->multiply);
    if (problem->multiply == CB200_DTYPE_BF16 && problem->projection != CB200_PROJECTION_TRANSPOSE &&
        problem->dense_dtype != CB200_DTYPE_BF16)
        return fail(CB200_STATUS_UNSUPPORTED, "bf16 products on a forward projection need a bf16 dense operand");
    if (problem->persistent != nullptr && (reinterpret_cast<std::uintptr_t>(problem->persistent) & 255u) != 0u)
        return fail(CB200_STATUS_INVALID_ARGUMENT, "persistent memory must be 256-byte aligned");
    if (problem->projection == CB200_PROJECTION_TRANSPOSE) {
        if (problem->dense_dtype != CB200_DTYPE_F32) return fail(CB200_STATUS_UNSUPPORTED, "transpose takes fp32 G");
        // a fixed order of the sums needs the gene-major copy, which prepare builds from the matrix
        if (problem->deterministic &&
            (problem->device_matrix == nullptr || !qcsr_transpose_gather_shape_ok(problem->n) ||
             !qcsr_gene_major_shape_ok(problem->m, problem->k, problem->bits)))
            return fail(CB200_STATUS_UNSUPPORTED,
                        "a deterministic transpose needs the device matrix at prepare time and N in {32, 64, 128}; the other "
                        "transpose kernels add in atomic order");
    } else if (problem->projection == CB200_PROJECTION_CSR || problem->projection == CB200_PROJECTION_BLOCKED_ELL) {
        if (!supported_dense(problem->dense_dtype)) return fail(CB200_STATUS_UNSUPPORTED, "W must be fp32 or bf16");
    } else {
        return fail(CB200_STATUS_UNSUPPORTED, "unknown projection %d", problem->projection);
    }
    if (problem->device_matrix != nullptr && problem->projection != CB200_PROJECTION_BLOCKED_ELL) {
        const cb200_qcsr &dm = *problem->device_matrix;
        if (!valid_header(&dm) || dm.rows != problem->m || dm.cols != problem->k || dm.nnz != problem->nnz ||
            dm.bits != problem->bits || dm.policy != problem->policy)
            return fail(CB200_STATUS_INVALID_SHAPE, "the matrix handed to prepare disagrees with the problem");
    }
    return CB200_STATUS_SUCCESS;
}

schedule_plan plan_schedule(const cb200_spmm_problem &pr) {
    schedule_plan plan;
    const char *hint = (pr.schedule_hint != nullptr && pr.schedule_hint[0] != '\0') ? pr.schedule_hint : nullptr;
    const std::uint64_t limit = pr.persistent_limit_bytes;
    const std::uint64_t nnz = static_cast<std::uint64_t>(pr.nnz);
    plan.mean_row_nnz = pr.m > 0 ? static_cast<double>(pr.nnz) / static_cast<double>(pr.m) : 0.0;
    if (pr.projection == CB200_PROJECTION_BLOCKED_ELL) {
        plan.bell_cuda_cores = hint_is(hint, "cuda_cores");
        return plan;
    }
    if (pr.projection == CB200_PROJECTION_TRANSPOSE) {
        // With the matrix at hand: the tensor-core kernel over the window-blocked copy.  bf16 products
        // allowed: one pass (decoded values and G rounded to bf16).  fp32 products: three bf16 passes
        // (hi*hi + hi*lo + lo*hi) rebuild each product to ~3 * 2^-17 relative, inside the 1e-4 bound of
        // an fp32 G; that is not bit-equal to an fp32 multiply, and callers that need the fp32-FMA kernel
        // do not hand the matrix to prepare.  The cost follows the dense area, so it needs density.
        // Same bits on every run: the tensor-core kernel over the window-blocked copy gives that too (every CTA's sums go to
        // a slot of their own and are added in a fixed order), and a deterministic request that names it gets it; the
        // default stays the gather gene by gene from a gene-major copy, whose fp32 sums the oracle restates entry by entry.
        const bool named_blocked = hint != nullptr && hint_starts(hint, "tensor_blocked") && pr.device_matrix != nullptr &&
                                   qcsr_transpose_blocked_shape_ok(pr.m, pr.k, pr.n, pr.bits) && (limit == 0u || nnz * 4u <= limit);
        if (pr.deterministic && !named_blocked) {
            plan.gene_gather = true;
            if (limit != 0u && nnz * 5u + static_cast<std::uint64_t>(pr.k + 1) * 12u > limit) {
                plan.status = fail(CB200_STATUS_UNSUPPORTED, "the gene-major copy of a deterministic transpose exceeds the persistent memory limit");
            }
            return plan;
        }
        bool blocked = pr.device_matrix != nullptr && qcsr_transpose_blocked_shape_ok(pr.m, pr.k, pr.n, pr.bits);
        if (hint == nullptr) blocked = blocked && pr.m >= 16 * 256 && plan.mean_row_nnz >= 0.004 * static_cast<double>(pr.k);
        else blocked = blocked && hint_starts(hint, "tensor_blocked");
        if (blocked && limit != 0u && nnz * 4u > limit) blocked = false; // a word per entry has to fit under the caller's limit
        plan.blocked = blocked;
        plan.split = pr.multiply != CB200_DTYPE_BF16;
        // decoded values in the entry words, positions of this kernel's gene-major tile; a second array with the
        // next eight mantissa bits for the split passes when the limit has room
        plan.blocked_lo = blocked && plan.split && (limit == 0u || nnz * 8u <= limit);
        return plan;
    }
    // CSR forward.  Row schedule from the nnz/row distribution: the gene-tiled kernel pays a fixed cost per
    // (row, gene tile) visit, so it needs enough stored entries per visit and enough row groups to fill the
    // SMs; short or few rows go to the warp-per-row kernel.
    const std::int64_t row_bytes = pr.n * (pr.dense_dtype == CB200_DTYPE_BF16 ? 2 : 4);
    const bool shape_ok = (pr.n == 32 || pr.n == 64 || pr.n == 128) && row_bytes <= 256;
    const double tile_genes = row_bytes > 0 ? 98304.0 / static_cast<double>(row_bytes) : 0.0;
    const double per_visit = pr.k > 0 ? plan.mean_row_nnz * tile_genes / static_cast<double>(pr.k) : 0.0;
    bool tiled = shape_ok && pr.m >= 16 * 128 && (per_visit >= 6.0 || tile_genes >= pr.k);
    if (hint_is(hint, "warp_per_row")) tiled = false;
    if (hint_is(hint, "gene_tiled")) tiled = shape_ok;
    // bf16 products allowed: the tensor-core kernel, which treats 512-row x 64-gene windows as dense.  That
    // pays once a window holds enough stored entries (density) and there are row groups for every SM;
    // otherwise the exact kernels above run (they satisfy the policy too).
    const bool tensor_ok = pr.multiply == CB200_DTYPE_BF16 && pr.dense_dtype == CB200_DTYPE_BF16 &&
                           (pr.n == 32 || pr.n == 64 || pr.n == 128) && pr.k > 0;
    bool tensor = tensor_ok && pr.m >= 512 && plan.mean_row_nnz >= 0.10 * static_cast<double>(pr.k);
    if (hint != nullptr) tensor = tensor_ok && hint_is(hint, "tensor_windows");
    if (tensor) tiled = true; // same length-sorted row order
    // With the device-resident matrix at hand, prepare re-lays it once into the window-blocked copy
    // (persistent preprocessing) and the tensor-core kernel streams that instead of the CSR arrays.  Its
    // cost follows the dense area m x k, so it needs a minimum density to pay.  Two ways in: bf16 products
    // allowed (one pass), or fp32 products requested, which the kernel rebuilds from bf16 pieces in two
    // (bf16 W) or three (fp32 W) passes: not bit-equal to fp32 multiplies, but inside the 1e-4 bound;
    // callers that need the fp32-FMA kernel do not hand the matrix to prepare.  Split passes cost 2-3x, so
    // they need a denser matrix to beat the exact kernel.
    const bool split = pr.multiply != CB200_DTYPE_BF16;
    const bool blocked_ok = pr.device_matrix != nullptr && (tensor_ok || split) &&
                            qcsr_blocked_shape_ok(pr.m, pr.k, pr.n, pr.bits, pr.dense_dtype);
    const double min_density = !split ? 0.015 : (pr.dense_dtype == CB200_DTYPE_BF16 ? 0.04 : 0.06);
    bool blocked = blocked_ok && pr.m >= 16 * 256 && plan.mean_row_nnz >= min_density * static_cast<double>(pr.k);
    if (hint != nullptr)
        blocked = blocked_ok && (hint_starts(hint, "tensor_blocked") || (!split && (hint_is(hint, "tensor_dense") || hint_is(hint, "tensor_codes"))));
    if (blocked && limit != 0u && nnz * 4u > limit) blocked = false; // a word per entry
    plan.split = split;
    plan.blocked = blocked;
    // the entry words hold the decoded values (no look-up at launch); the split-product schedules get a
    // second array with the next eight mantissa bits when the limit has room for it
    plan.blocked_lo = blocked && split && (limit == 0u || nnz * 8u <= limit);
    if (blocked) {
        tiled = false; // no length-sorted row order: the copy works in natural row order, and the exact
        tensor = false; // kernel that serves unaligned row ranges runs in natural order too
        // Dense enough, bf16 products, and room for rows x genes x 2 bytes: keep the decoded operand tiles
        // instead of the entry words; a launch then streams them and decodes nothing.
        const std::uint64_t tile_bytes = qcsr_dense_tile_bytes(pr.m, pr.k);
        bool dense = !split && plan.mean_row_nnz >= 0.08 * static_cast<double>(pr.k);
        if (hint != nullptr) dense = !split && hint_is(hint, "tensor_dense");
        plan.dense_forced = dense && hint != nullptr;
        if (limit != 0u && tile_bytes > limit) dense = false;
        plan.dense_wanted = dense;
        // 4-bit codes with per-gene zero-points: keep tiles of CODES instead (one byte per slot, half the decoded
        // tiles; scale and zero-point applied at launch).  Preferred to the decoded tiles wherever both would be built.
        const bool codes_ok = !split && qcsr_codes_shape_ok(pr.m, pr.k, pr.n, pr.bits, pr.policy, pr.dense_dtype);
        bool codes = codes_ok && plan.mean_row_nnz >= 0.08 * static_cast<double>(pr.k);
        if (hint != nullptr) codes = codes_ok && hint_is(hint, "tensor_codes");
        if (limit != 0u && qcsr_code_tile_bytes(pr.m, pr.k) > limit) codes = false;
        if (codes) {
            plan.codes_wanted = true;
            plan.dense_wanted = false;
            plan.dense_forced = hint != nullptr;
        }
    }
    plan.tiled = tiled;
    plan.tensor_windows = tensor;
    // The tiled kernel gives each row to one lane group, so a CTA is as slow as its longest row.  With the
    // row lengths at hand, order the rows by length once: every CTA then works on rows of nearly equal length.
    plan.row_order = tiled && pr.host_row_ptr != nullptr && pr.m > 0 && pr.m <= 0x7fffffff;
    return plan;
}

std::uint64_t plan_persistent_bytes(const cb200_spmm_problem &pr, const schedule_plan &plan) {
    std::uint64_t bytes = 0;
    if (plan.gene_gather) bytes += qcsr_gene_major_layout_bytes_bound(pr.m, pr.k, pr.nnz);
    if (plan.blocked) bytes += qcsr_blocked_layout_bytes_bound(pr.m, pr.k, pr.nnz, plan.blocked_lo);
    if (plan.dense_wanted) bytes += device_arena::rounded(qcsr_dense_tile_bytes(pr.m, pr.k));
    if (plan.codes_wanted) bytes += device_arena::rounded(qcsr_code_tile_bytes(pr.m, pr.k));
    if (plan.row_order) bytes += device_arena::rounded(static_cast<std::uint64_t>(pr.m) * sizeof(std::int32_t));
    return bytes;
}

// cudaDeviceGetAttribute answers of a device, asked once (cudaGetDeviceProperties fills dozens of fields
// and costs milliseconds; the routed public calls prepare on every projection)
struct device_facts { int major = 0, sm_count = 0; };
cb200_status facts_of(int device, device_facts *out) {
    constexpr int kMax = 64;
    static std::atomic<int> cached_major[kMax], cached_sms[kMax];
    if (device >= 0 && device < kMax && cached_sms[device].load(std::memory_order_acquire) != 0) {
        out->major = cached_major[device].load(std::memory_order_relaxed);
        out->sm_count = cached_sms[device].load(std::memory_order_relaxed);
        return CB200_STATUS_SUCCESS;
    }
    int device_count = 0;
    CB200_CUDA_OK(cudaGetDeviceCount(&device_count));
    if (device < 0 || device >= device_count)
        return fail(CB200_STATUS_INVALID_STREAM, "device %d not present (%d visible)", device, device_count);
    CB200_CUDA_OK(cudaDeviceGetAttribute(&out->major, cudaDevAttrComputeCapabilityMajor, device));
    CB200_CUDA_OK(cudaDeviceGetAttribute(&out->sm_count, cudaDevAttrMultiProcessorCount, device));
    if (device < kMax) {
        cached_major[device].store(out->major, std::memory_order_relaxed);
        cached_sms[device].store(out->sm_count, std::memory_order_release);
    }
    return CB200_STATUS_SUCCESS;
}

} // namespace

extern "C" {

cb200_status cb200_spmm_persistent_requirement(const cb200_spmm_problem *problem, uint64_t *bytes) {
    clear_error();
    if (bytes == nullptr) return fail(CB200_STATUS_INVALID_ARGUMENT, "persistent_requirement needs an output");
    *bytes = 0u;
    const cb200_status valid = validate_problem(problem);
    if (valid != CB200_STATUS_SUCCESS) return valid;
    const schedule_plan plan = plan_schedule(*problem);
    if (plan.status != CB200_STATUS_SUCCESS) return plan.status;
    *bytes = plan_persistent_bytes(*problem, plan);
    return CB200_STATUS_SUCCESS;
}

cb200_status cb200_spmm_prepare(const cb200_spmm_problem *problem, cb200_prepared **out) {
    clear_error();
    if (out == nullptr) return fail(CB200_STATUS_INVALID_ARGUMENT, "prepare needs an output handle");
    *out = nullptr;
    const cb200_status valid = validate_problem(problem);
    if (valid != CB200_STATUS_SUCCESS) return valid;
    const schedule_plan plan = plan_schedule(*problem);
    if (plan.status != CB200_STATUS_SUCCESS) return plan.status;

    device_facts facts;
    const cb200_status found = facts_of(problem->device, &facts);
    if (found != CB200_STATUS_SUCCESS) return found;
    if (facts.major != 10)
        return fail(CB200_STATUS_UNSUPPORTED, "this library is built for sm_100a only; device %d has compute capability %d.x",
                    problem->device, facts.major);

    cb200_prepared *p = new (std::nothrow) cb200_prepared{};
    if (p == nullptr) return fail(CB200_STATUS_INTERNAL_ERROR, "out of host memory");
    p->problem = *problem;
    p->problem.host_row_ptr = nullptr; /* borrowed for the analysis below only */
    p->problem.device_matrix = nullptr;
    p->problem.schedule_hint = nullptr;
    p->sm_count = facts.sm_count;
    p->schedule = fwd_schedule::warp_per_row;
    p->schedule_name = "warp_per_row";
    p->workspace_alignment = 256u;
    p->workspace_bytes = 0u;
    p->mean_row_nnz = plan.mean_row_nnz;
    p->max_row_nnz = p->mean_row_nnz;
    p->bell_cuda_cores = plan.bell_cuda_cores;
    p->arena.borrowed = problem->persistent != nullptr;
    p->arena.base = static_cast<unsigned char *>(problem->persistent);
    p->arena.capacity = problem->persistent != nullptr ? problem->persistent_bytes : 0u;
    cudaStream_t stream = static_cast<cudaStream_t>(problem->prepare_stream);
    const auto abandon = [&](cb200_status st) {
        device_scope scope(problem->device);
        p->arena.release_all();
        delete p;
        return st;
    };
    if (p->arena.borrowed && plan_persistent_bytes(*problem, plan) - (plan.dense_wanted ? device_arena::rounded(qcsr_dense_tile_bytes(problem->m, problem->k)) : 0u) -
                                     (plan.codes_wanted ? device_arena::rounded(qcsr_code_tile_bytes(problem->m, problem->k)) : 0u) >
                                 p->arena.capacity)
        return abandon(fail(CB200_STATUS_INSUFFICIENT_WORKSPACE, "persistent memory of %llu bytes needed (cb200_spmm_persistent_requirement), %llu given",
                            (unsigned long long)plan_persistent_bytes(*problem, plan), (unsigned long long)p->arena.capacity));

    if (problem->host_row_ptr != nullptr && problem->projection != CB200_PROJECTION_BLOCKED_ELL) {
        int64_t longest = 0;
        for (int64_t r = 0; r < problem->m; ++r) {
            const int64_t c = problem->host_row_ptr[r + 1] - problem->host_row_ptr[r];
            if (c > longest) longest = c;
        }
        p->max_row_nnz = static_cast<double>(longest);
    }
    device_scope scope(problem->device);
    if (scope.status != cudaSuccess) return abandon(fail(CB200_STATUS_CUDA_ERROR, "%s", cudaGetErrorString(scope.status)));

    if (problem->projection == CB200_PROJECTION_TRANSPOSE) {
        p->workspace_bytes = qcsr_transpose_workspace_bytes(problem->k, problem->n, p->sm_count);
        p->schedule_name = "vector_reductions";
        if (plan.gene_gather) {
            const cb200_status st = build_gene_major_layout(view_of(*problem->device_matrix), p->arena, stream, &p->gene_major);
            if (st != CB200_STATUS_SUCCESS) return abandon(st);
            p->schedule_name = "gene_gather";
            p->workspace_bytes = qcsr_transpose_gather_workspace_bytes();
            p->persistent_bytes += p->gene_major.bytes;
        }
        if (plan.blocked) {
            const cb200_status st = build_blocked_layout(view_of(*problem->device_matrix), !plan.split || plan.blocked_lo, plan.blocked_lo,
                                                         true, p->arena, stream, &p->blocked);
            if (st != CB200_STATUS_SUCCESS) return abandon(st);
            p->schedule_name = problem->multiply == CB200_DTYPE_BF16 ? "tensor_blocked" : "tensor_blocked_x3";
            p->workspace_bytes = qcsr_transpose_blocked_workspace_bytes(problem->m, problem->k, problem->n);
            p->persistent_bytes += p->blocked.bytes;
        }
    }
    if (problem->projection == CB200_PROJECTION_BLOCKED_ELL && problem->dense_dtype == CB200_DTYPE_BF16 &&
        (problem->n == 128 || problem->n == 256) && !plan.bell_cuda_cores) {
        // the tensor-core kernel multiplies against W^T: room for that bf16 copy plus a status block
        p->workspace_bytes = qbell_tcgen05_workspace_bytes(problem->k, problem->n);
        p->schedule_name = "tcgen05_block_rows";
    } else if (problem->projection == CB200_PROJECTION_BLOCKED_ELL) {
        p->schedule_name = "cuda_cores";
    }
    if (problem->projection == CB200_PROJECTION_CSR) {
        if (plan.tiled) {
            p->schedule = fwd_schedule::gene_tiled;
            p->schedule_name = "gene_tiled";
        }
        p->workspace_bytes = qcsr_tiled_workspace_bytes(); // status word of the tiled kernel
        if (plan.tensor_windows) {
            p->schedule = fwd_schedule::tensor_windows;
            p->schedule_name = "tensor_windows";
            p->workspace_bytes = qcsr_mma_workspace_bytes(problem->k, problem->n);
        }
        if (plan.blocked) {
            const qcsr_view dm = view_of(*problem->device_matrix);
            // code tiles are made from code words; everything else from baked (decoded) words where it can be
            bool codes = plan.codes_wanted;
            if (codes && !plan.dense_forced && !p->arena.borrowed) {
                std::size_t free_bytes = 0, total_bytes = 0;
                codes = cudaMemGetInfo(&free_bytes, &total_bytes) == cudaSuccess &&
                        qcsr_code_tile_bytes(problem->m, problem->k) + static_cast<std::uint64_t>(problem->nnz) * 4u <= free_bytes / 2u;
            }
            cb200_status st = build_blocked_layout(dm, !codes && (!plan.split || plan.blocked_lo), !codes && plan.blocked_lo, false, p->arena,
                                                   stream, &p->blocked);
            if (st != CB200_STATUS_SUCCESS) return abandon(st);
            p->schedule = fwd_schedule::tensor_blocked;
            p->schedule_name = !plan.split ? "tensor_blocked"
                                           : (problem->dense_dtype == CB200_DTYPE_BF16 ? "tensor_blocked_x2" : "tensor_blocked_x3");
            p->workspace_bytes = std::max<std::uint64_t>(qcsr_blocked_workspace_bytes(problem->k, problem->n), 256u);
            if (codes) {
                bool built = false;
                st = bytify_blocked_layout(&p->blocked, p->arena, stream, &built);
                if (st != CB200_STATUS_SUCCESS) return abandon(st);
                if (built) {
                    p->schedule_name = "tensor_codes";
                    p->workspace_bytes = std::max<std::uint64_t>(p->workspace_bytes, qcsr_codes_workspace_bytes(problem->k, problem->n));
                }
            }
            bool dense = plan.dense_wanted;
            if (dense && !plan.dense_forced && !p->arena.borrowed) {
                // own allocations: the tiles may take half of what the device has free, no more
                std::size_t free_bytes = 0, total_bytes = 0;
                dense = cudaMemGetInfo(&free_bytes, &total_bytes) == cudaSuccess && qcsr_dense_tile_bytes(problem->m, problem->k) <= free_bytes / 2u;
            }
            if (dense) {
                bool built = false;
                st = densify_blocked_layout(dm, &p->blocked, p->arena, stream, &built);
                if (st != CB200_STATUS_SUCCESS) return abandon(st);
                if (built) p->schedule_name = "tensor_dense";
            }
            p->persistent_bytes += p->blocked.bytes;
        }
        if (plan.row_order) {
            std::vector<std::int32_t> order(static_cast<std::size_t>(problem->m));
            for (std::int64_t r = 0; r < problem->m; ++r) order[static_cast<std::size_t>(r)] = static_cast<std::int32_t>(r);
            const std::int64_t *rp = problem->host_row_ptr;
            std::stable_sort(order.begin(), order.end(), [rp](std::int32_t a, std::int32_t b) {
                return rp[a + 1] - rp[a] > rp[b + 1] - rp[b];
            });
            const std::size_t bytes = order.size() * sizeof(std::int32_t);
            p->row_order = static_cast<std::int32_t *>(p->arena.take(bytes));
            if (p->row_order == nullptr) return abandon(fail(CB200_STATUS_INSUFFICIENT_WORKSPACE, "no device memory for the row order"));
            cudaError_t err = cudaMemcpyAsync(p->row_order, order.data(), bytes, cudaMemcpyHostToDevice, stream);
            if (err == cudaSuccess) err = cudaStreamSynchronize(stream); // `order` leaves scope
            if (err != cudaSuccess) return abandon(fail(CB200_STATUS_CUDA_ERROR, "row order upload: %s", cudaGetErrorString(err)));
            p->persistent_bytes += bytes;
        }
    }
    *out = p;
    return CB200_STATUS_SUCCESS;
}

void cb200_prepared_destroy(cb200_prepared *prepared) {
    if (prepared == nullptr) return;
    if (prepared->arena.owned_count != 0) {
        device_scope scope(prepared->problem.device);
        prepared->arena.release_all();
    }
    delete prepared;
}

cb200_status cb200_prepared_workspace(const cb200_prepared *prepared, uint64_t *minimum_bytes, uint32_t *alignment) {
    clear_error();
    if (prepared == nullptr) return fail(CB200_STATUS_INVALID_ARGUMENT, "null prepared operation");
    if (minimum_bytes != nullptr) *minimum_bytes = prepared->workspace_bytes;
    if (alignment != nullptr) *alignment = prepared->workspace_alignment;
    return CB200_STATUS_SUCCESS;
}

const char *cb200_prepared_schedule(const cb200_prepared *prepared) {
    return prepared != nullptr ? prepared->schedule_name : "";
}

uint64_t cb200_prepared_persistent_bytes(const cb200_prepared *prepared) {
    return prepared != nullptr ? prepared->persistent_bytes : 0u;
}

cb200_status cb200_prepared_output_shape(const cb200_prepared *prepared, uint64_t *rows, uint64_t *columns) {
    clear_error();
    if (prepared == nullptr || rows == nullptr || columns == nullptr) return fail(CB200_STATUS_INVALID_ARGUMENT, "output_shape needs a prepared operation and outputs");
    const cb200_spmm_problem &pr = prepared->problem;
    *rows = static_cast<uint64_t>(pr.projection == CB200_PROJECTION_TRANSPOSE ? pr.k : pr.m);
    *columns = static_cast<uint64_t>(pr.n);
    return CB200_STATUS_SUCCESS;
}

cb200_status cb200_spmm_run(const cb200_prepared *prepared, const cb200_launch *launch) {
    clear_error();
    if (prepared == nullptr) return fail(CB200_STATUS_INVALID_ARGUMENT, "null prepared operation");
    if (!valid_header(launch)) return fail(CB200_STATUS_INVALID_ARGUMENT, "bad cb200_launch header");
    const cb200_spmm_problem &pr = prepared->problem;
    /* launch_bindings.hh:261-275,361-375: epoch, stream/device and workspace checks come first */
    if (launch->structure_epoch != pr.structure_epoch)
        return fail(CB200_STATUS_STALE_STRUCTURE, "launch epoch %llu != prepared epoch %llu",
                    (unsigned long long)launch->structure_epoch, (unsigned long long)pr.structure_epoch);
    if (launch->device != pr.device || launch->device < 0)
        return fail(CB200_STATUS_INVALID_STREAM, "launch device %d != prepared device %d", launch->device, pr.device);
    if (launch->workspace_device != launch->device)
        return fail(CB200_STATUS_INVALID_STREAM, "workspace lives on device %d, stream on device %d",
                    launch->workspace_device, launch->device);
    if (launch->workspace_bytes < prepared->workspace_bytes ||
        (prepared->workspace_bytes != 0u &&
         (launch->workspace == nullptr ||
          (reinterpret_cast<std::uintptr_t>(launch->workspace) & (prepared->workspace_alignment - 1u)) != 0u)))
        return fail(CB200_STATUS_INSUFFICIENT_WORKSPACE, "workspace of %llu bytes needed, %llu given",
                    (unsigned long long)prepared->workspace_bytes, (unsigned long long)launch->workspace_bytes);
    /* lifetimes.hh:160-172: the expected generation of a bound value plane must be the live one; here the
     * "live" values of a prepared copy are those it was built from */
    if ((prepared->blocked.seg_ptr != nullptr || prepared->blocked.dense_tiles != nullptr || prepared->blocked.code_tiles != nullptr ||
         prepared->gene_major.col_ptr != nullptr) &&
        pr.value_generation != 0u &&
        launch->value_generation != 0u && launch->value_generation != pr.value_generation)
        return fail(CB200_STATUS_STALE_VALUE, "the prepared operation keeps a copy of value generation %llu, the launch binds %llu",
                    (unsigned long long)pr.value_generation, (unsigned long long)launch->value_generation);
    if (launch->out == nullptr && pr.n != 0 && pr.m != 0)
        return fail(CB200_STATUS_INVALID_ARGUMENT, "null output");
    if (launch->dense == nullptr && pr.n != 0 && pr.k != 0) return fail(CB200_STATUS_INVALID_ARGUMENT, "null dense operand");
    if (launch->out == launch->dense && launch->out != nullptr)
        return fail(CB200_STATUS_INVALID_ARGUMENT, "output aliases the dense input");
    if (launch->dense_ld < pr.n || launch->out_ld < pr.n)
        return fail(CB200_STATUS_INVALID_SHAPE, "leading dimension smaller than n");

    /* operation.cc:45-64: the eight epilogue kinds; the bias kinds need a bias vector */
    if (launch->epilogue < CB200_EPILOGUE_NONE || launch->epilogue > CB200_EPILOGUE_BIAS_GELU_TANH)
        return fail(CB200_STATUS_UNSUPPORTED, "unknown epilogue kind %d", launch->epilogue);
    const bool bias_kind = launch->epilogue == CB200_EPILOGUE_BIAS || launch->epilogue >= CB200_EPILOGUE_BIAS_RELU;
    if (bias_kind && launch->bias == nullptr && pr.n != 0)
        return fail(CB200_STATUS_INVALID_ARGUMENT, "epilogue kind %d needs a bias vector", launch->epilogue);
    if (launch->epilogue != CB200_EPILOGUE_NONE && pr.projection == CB200_PROJECTION_TRANSPOSE)
        return fail(CB200_STATUS_UNSUPPORTED, "the transpose has no composed epilogue");

    dense_args d{launch->dense, launch->dense_ld, pr.dense_dtype, launch->out, launch->out_ld, pr.n,
                 launch->alpha, launch->beta, bias_kind ? launch->bias : nullptr, launch->epilogue};
    cudaStream_t stream = static_cast<cudaStream_t>(launch->stream);
    device_scope scope(launch->device);
    CB200_CUDA_OK(scope.status);

    int64_t row_begin = launch->row_begin, row_end = launch->row_end;
    if (row_end == CB200_ALL_ROWS) row_end = pr.m;
    if (row_begin < 0 || row_end > pr.m || row_begin > row_end)
        return fail(CB200_STATUS_INVALID_SHAPE, "row range [%lld,%lld) outside 0..%lld", (long long)row_begin,
                    (long long)row_end, (long long)pr.m);

    if (pr.projection == CB200_PROJECTION_BLOCKED_ELL) {
        if (!valid_header(launch->bell)) return fail(CB200_STATUS_INVALID_ARGUMENT, "bad cb200_qbell header");
        const cb200_qbell &b = *launch->bell;
        if (b.rows != pr.m || b.cols != pr.k || b.bits != pr.bits || b.policy != pr.policy)
            return fail(CB200_STATUS_INVALID_SHAPE, "Blocked-ELL matrix disagrees with the prepared problem");
        if (b.block_col_idx == nullptr || b.packed_values == nullptr)
            return fail(CB200_STATUS_INVALID_ARGUMENT, "Blocked-ELL matrix has null arrays");
        return launch_qbell_forward(view_of(b), d, row_begin, row_end, launch->workspace, launch->workspace_bytes,
                                    prepared->sm_count, prepared->bell_cuda_cores, stream);
    }
    if (!valid_header(launch->csr)) return fail(CB200_STATUS_INVALID_ARGUMENT, "bad cb200_qcsr header");
    const cb200_qcsr &x = *launch->csr;
    if (x.rows != pr.m || x.cols != pr.k || x.bits != pr.bits || x.policy != pr.policy || x.nnz != pr.nnz)
        return fail(CB200_STATUS_INVALID_SHAPE, "CSR matrix disagrees with the prepared problem");
    if (x.row_ptr == nullptr || (x.nnz != 0 && (x.col_idx == nullptr || x.packed_values == nullptr)))
        return fail(CB200_STATUS_INVALID_ARGUMENT, "CSR matrix has null arrays");
    if (pr.projection == CB200_PROJECTION_TRANSPOSE && prepared->gene_major.col_ptr != nullptr)
        return launch_qcsr_transpose_gather(view_of(x), d, row_begin, row_end, prepared->gene_major, launch->workspace,
                                            launch->workspace_bytes, prepared->sm_count, stream);
    if (pr.projection == CB200_PROJECTION_TRANSPOSE)
        return launch_qcsr_transpose(view_of(x), d, row_begin, row_end, &prepared->blocked, pr.multiply != CB200_DTYPE_BF16,
                                     launch->workspace, launch->workspace_bytes, prepared->sm_count, stream);
    return launch_qcsr_forward(view_of(x), d, row_begin, row_end, prepared->schedule, prepared->row_order, &prepared->blocked,
                               pr.multiply != CB200_DTYPE_BF16, launch->workspace, launch->workspace_bytes, prepared->sm_count,
                               stream);
}

cb200_status cb200_prepared_status(const cb200_prepared *prepared, const void *workspace, void *stream, int32_t *host_word) {
    clear_error();
    if (prepared == nullptr || host_word == nullptr) return fail(CB200_STATUS_INVALID_ARGUMENT, "status needs a prepared operation and an output");
    *host_word = 0;
    if (prepared->workspace_bytes == 0u) return CB200_STATUS_SUCCESS; // this schedule waits on nothing
    if (workspace == nullptr) return fail(CB200_STATUS_INVALID_ARGUMENT, "status needs the workspace of the launch");
    device_scope scope(prepared->problem.device);
    CB200_CUDA_OK(scope.status);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    CB200_CUDA_OK(cudaMemcpyAsync(host_word, workspace, sizeof(int32_t), cudaMemcpyDeviceToHost, s));
    CB200_CUDA_OK(cudaStreamSynchronize(s));
    if (*host_word != 0)
        return fail(CB200_STATUS_DEVICE_WAIT_TIMEOUT, "a kernel of the last launch gave up a bounded wait (status word %d): its output is not valid", *host_word);
    return CB200_STATUS_SUCCESS;
}

/* ---- session ------------------------------------------------------------------------------ */

cb200_status cb200_session_create(const cb200_session_options *options, cb200_session **out) {
    clear_error();
    if (out == nullptr) return fail(CB200_STATUS_INVALID_ARGUMENT, "session_create needs an output handle");
    *out = nullptr;
    if (!valid_header(options)) return fail(CB200_STATUS_INVALID_ARGUMENT, "bad cb200_session_options header");
    const std::uint32_t total = options->owned_stream_count + options->external_stream_count;
    if (total == 0u || total > 8u) return fail(CB200_STATUS_INVALID_ARGUMENT, "a session has 1..8 streams");
    if (options->external_stream_count != 0u && options->external_streams == nullptr)
        return fail(CB200_STATUS_INVALID_ARGUMENT, "external stream array is null");
    device_scope scope(options->device);
    CB200_CUDA_OK(scope.status);
    cb200_session *s = new (std::nothrow) cb200_session{};
    if (s == nullptr) return fail(CB200_STATUS_INTERNAL_ERROR, "out of host memory");
    s->device = options->device;
    for (std::uint32_t i = 0; i < options->external_stream_count; ++i) {
        s->streams[s->stream_count] = static_cast<cudaStream_t>(options->external_streams[i]);
        s->owned[s->stream_count++] = false;
    }
    for (std::uint32_t i = 0; i < options->owned_stream_count; ++i) {
        cudaStream_t stream = nullptr;
        const cudaError_t err = cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking);
        if (err != cudaSuccess) {
            cb200_session_destroy(s);
            return fail(CB200_STATUS_CUDA_ERROR, "cudaStreamCreateWithFlags: %s", cudaGetErrorString(err));
        }
        s->streams[s->stream_count] = stream;
        s->owned[s->stream_count++] = true;
    }
    *out = s;
    return CB200_STATUS_SUCCESS;
}

cb200_status cb200_session_reserve_persistent(cb200_session *s, uint64_t bytes, void **allocation) {
    return cb200_session_reserve_persistent_as(s, CB200_LIFETIME_STRUCTURE, bytes, allocation);
}

cb200_status cb200_session_reserve_persistent_as(cb200_session *s, int32_t lifetime, uint64_t bytes, void **allocation) {
    clear_error();
    if (s == nullptr || allocation == nullptr || bytes == 0u) return fail(CB200_STATUS_INVALID_ARGUMENT, "bad reserve arguments");
    if (lifetime < CB200_LIFETIME_STRUCTURE || lifetime > CB200_LIFETIME_GRAPH_STABLE)
        return fail(CB200_STATUS_INVALID_ARGUMENT, "unknown persistent lifetime %d", lifetime);
    if (s->sealed) return fail(CB200_STATUS_SEALED, "session is sealed; nothing can grow");
    if (s->persistent_count == 64u) return fail(CB200_STATUS_INSUFFICIENT_WORKSPACE, "64 persistent allocations at most");
    device_scope scope(s->device);
    CB200_CUDA_OK(scope.status);
    void *ptr = nullptr;
    CB200_CUDA_OK(cudaMalloc(&ptr, bytes));
    s->persistent[s->persistent_count] = ptr;
    s->persistent_bytes[s->persistent_count] = bytes;
    s->persistent_lifetime[s->persistent_count++] = lifetime;
    account(lifetime == CB200_LIFETIME_STRUCTURE ? &s->accounting.structure
                                                 : (lifetime == CB200_LIFETIME_PLAN ? &s->accounting.plan : &s->accounting.graph_stable),
            bytes);
    *allocation = ptr;
    return CB200_STATUS_SUCCESS;
}

cb200_status cb200_session_prepare_stream_libraries(cb200_session *s, uint32_t stream_index) {
    clear_error();
    if (s == nullptr || stream_index >= s->stream_count) return fail(CB200_STATUS_INVALID_ARGUMENT, "bad stream index");
    if (s->sealed) return fail(CB200_STATUS_SEALED, "session is sealed; nothing can grow");
    ++s->accounting.handle_prepare_count; // no library handle behind it: the kernels are this library's own
    return CB200_STATUS_SUCCESS;
}

cb200_status cb200_session_get_accounting(const cb200_session *s, cb200_session_accounting *out) {
    clear_error();
    if (s == nullptr || out == nullptr) return fail(CB200_STATUS_INVALID_ARGUMENT, "accounting needs a session and an output");
    *out = s->accounting;
    return CB200_STATUS_SUCCESS;
}

int32_t cb200_session_graph_stable_address(const cb200_session *s, const void *address, uint64_t bytes) {
    if (s == nullptr || address == nullptr) return 0;
    const std::uintptr_t lo = reinterpret_cast<std::uintptr_t>(address);
    for (std::uint32_t i = 0; i < s->persistent_count; ++i) {
        if (s->persistent_lifetime[i] != CB200_LIFETIME_GRAPH_STABLE) continue;
        const std::uintptr_t base = reinterpret_cast<std::uintptr_t>(s->persistent[i]);
        if (lo >= base && bytes <= s->persistent_bytes[i] && lo - base <= s->persistent_bytes[i] - bytes) return 1;
    }
    return 0;
}

cb200_status cb200_session_cache_insert(cb200_session *s, int32_t kind, const cb200_session_cache_entry *entry) {
    clear_error();
    if (s == nullptr || entry == nullptr || kind < CB200_CACHE_PLAN || kind > CB200_CACHE_ORDER_TRANSFORM || entry->state == nullptr ||
        (entry->key_high == 0u && entry->key_low == 0u))
        return fail(CB200_STATUS_INVALID_ARGUMENT, "bad cache entry");
    cb200_session_cache_entry *cache = s->caches[kind];
    for (std::uint32_t i = 0; i < s->cache_size[kind]; ++i) {
        if (cache[i].key_high == entry->key_high && cache[i].key_low == entry->key_low) {
            cache[i] = *entry;
            return CB200_STATUS_SUCCESS;
        }
    }
    if (s->cache_size[kind] == 64u) return fail(CB200_STATUS_INSUFFICIENT_WORKSPACE, "the session cache holds 64 entries");
    cache[s->cache_size[kind]++] = *entry;
    return CB200_STATUS_SUCCESS;
}

const cb200_session_cache_entry *cb200_session_cache_find(const cb200_session *s, int32_t kind, uint64_t key_high, uint64_t key_low) {
    if (s == nullptr || kind < CB200_CACHE_PLAN || kind > CB200_CACHE_ORDER_TRANSFORM) return nullptr;
    for (std::uint32_t i = 0; i < s->cache_size[kind]; ++i)
        if (s->caches[kind][i].key_high == key_high && s->caches[kind][i].key_low == key_low) return &s->caches[kind][i];
    return nullptr;
}

cb200_status cb200_session_reserve_transient(cb200_session *s, uint32_t stream_index, uint64_t bytes) {
    clear_error();
    if (s == nullptr || stream_index >= s->stream_count) return fail(CB200_STATUS_INVALID_ARGUMENT, "bad stream index");
    if (s->sealed) return fail(CB200_STATUS_SEALED, "session is sealed; nothing can grow");
    if (bytes <= s->transient_bytes[stream_index]) return CB200_STATUS_SUCCESS;
    device_scope scope(s->device);
    CB200_CUDA_OK(scope.status);
    void *ptr = nullptr;
    CB200_CUDA_OK(cudaMalloc(&ptr, bytes));
    if (s->transient[stream_index] != nullptr) {
        cudaFree(s->transient[stream_index]);
        s->accounting.transient.current_bytes -= s->transient_bytes[stream_index];
    }
    s->transient[stream_index] = ptr;
    s->transient_bytes[stream_index] = bytes;
    account(&s->accounting.transient, bytes);
    return CB200_STATUS_SUCCESS;
}

cb200_status cb200_session_seal(cb200_session *s) {
    clear_error();
    if (s == nullptr) return fail(CB200_STATUS_INVALID_ARGUMENT, "null session");
    s->sealed = true;
    return CB200_STATUS_SUCCESS;
}

cb200_launch_binding cb200_session_bind(cb200_session *s, uint32_t stream_index, uint64_t required_workspace_bytes) {
    cb200_launch_binding b{};
    b.status = CB200_STATUS_INVALID_ARGUMENT;
    b.device = -1;
    if (s == nullptr || stream_index >= s->stream_count) return b;
    if (!s->sealed) { b.status = CB200_STATUS_SEALED; return b; } /* bind only works on a sealed session */
    if (required_workspace_bytes > s->transient_bytes[stream_index]) { b.status = CB200_STATUS_INSUFFICIENT_WORKSPACE; return b; }
    ++s->accounting.launch_bind_count; // host bookkeeping only: no CUDA call, allocation or synchronisation here
    b.status = CB200_STATUS_SUCCESS;
    b.device = s->device;
    b.stream = s->streams[stream_index];
    b.workspace = s->transient[stream_index];
    b.workspace_bytes = s->transient_bytes[stream_index];
    return b;
}

cb200_status cb200_session_synchronize(cb200_session *s) {
    clear_error();
    if (s == nullptr) return fail(CB200_STATUS_INVALID_ARGUMENT, "null session");
    device_scope scope(s->device);
    CB200_CUDA_OK(scope.status);
    for (std::uint32_t i = 0; i < s->stream_count; ++i) CB200_CUDA_OK(cudaStreamSynchronize(s->streams[i]));
    ++s->accounting.synchronization_count;
    return CB200_STATUS_SUCCESS;
}

void cb200_session_destroy(cb200_session *s) {
    if (s == nullptr) return;
    device_scope scope(s->device);
    for (std::uint32_t i = 0; i < s->stream_count; ++i) {
        if (s->owned[i] && s->streams[i] != nullptr) cudaStreamDestroy(s->streams[i]);
        if (s->transient[i] != nullptr) cudaFree(s->transient[i]);
    }
    for (std::uint32_t i = 0; i < s->persistent_count; ++i) cudaFree(s->persistent[i]);
    delete s;
}

} // extern "C"
