// Host-side pieces of the C ABI that launch nothing (apart from one slab copy and the batched look-up):
// element look-up on a quantized CSR matrix, the backend-neutral SpMM request with its validation and
// 128-bit signature, and the host container of a quantized Blocked-ELL matrix.
#include "kernels.cuh"

#include <cstdlib>
#include <cstring>
#include <limits>

using namespace cb200;

namespace {

// format_traits<Bits>::unpack, include/Cellerator/quantized/format.cuh:39-48: code i of a row sits in
// byte i / cpb at bit shift (i mod cpb) * bits, low bits first.
__host__ __device__ inline unsigned unpack_code(const std::uint8_t *row_bytes, std::int64_t local, int bits) {
    if (bits == 8) return row_bytes[local];
    const int per_byte = 8 / bits;
    const unsigned byte = row_bytes[local / per_byte];
    return (byte >> ((local % per_byte) * bits)) & ((1u << bits) - 1u);
}

__host__ __device__ inline bool lookup_bits_ok(int bits) { return bits == 1 || bits == 2 || bits == 4 || bits == 8; }

// find_in_row + get_code + dequantize_code for one (row, column) pair; *code stays -1 when nothing is stored.
__host__ __device__ inline float lookup_value(const std::int64_t *row_ptr, const std::int64_t *packed_row_ptr,
                                              const std::int32_t *col_idx, const std::uint8_t *packed, const float *scales,
                                              const float *offsets, int bits, int policy, std::int64_t rows, std::int64_t cols,
                                              std::int64_t row, std::int64_t column, int *code) {
    *code = -1;
    if (row < 0 || row >= rows || column < 0 || column >= cols) return 0.0f;
    const std::int64_t begin = row_ptr[row], end = row_ptr[row + 1];
    for (std::int64_t i = begin; i < end; ++i) { // linear scan from the row's start, like the reference
        if (col_idx[i] != column) continue;
        const std::uint8_t *row_bytes = packed + (packed_row_ptr != nullptr ? packed_row_ptr[row] : begin);
        const unsigned c = unpack_code(row_bytes, i - begin, bits);
        *code = static_cast<int>(c);
        const float scale = scales != nullptr ? scales[column] : 1.0f;
        const float offset = offsets == nullptr ? 0.0f : offsets[policy == CB200_DECODE_COLUMN_SCALE_ROW_OFFSET ? row : column];
        // product and sum rounded separately on both sides (the device codec does the same), so that host and
        // device return the bits of the host reference built without fused multiply-add
#if defined(__CUDA_ARCH__)
        return __fadd_rn(__fmul_rn(static_cast<float>(c), scale), offset);
#else
        volatile float product = static_cast<float>(c) * scale;
        return product + offset;
#endif
    }
    return 0.0f;
}

__global__ void __launch_bounds__(256) lookup_values_kernel(const std::int64_t *row_ptr, const std::int64_t *packed_row_ptr,
                                                            const std::int32_t *col_idx, const std::uint8_t *packed,
                                                            const float *scales, const float *offsets, int bits, int policy,
                                                            std::int64_t rows, std::int64_t cols, const std::int64_t *want_rows,
                                                            const std::int32_t *want_cols, std::int64_t count, float *values,
                                                            std::int32_t *codes) {
    const std::int64_t i = static_cast<std::int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= count) return;
    int code = -1;
    const float v = lookup_value(row_ptr, packed_row_ptr, col_idx, packed, scales, offsets, bits, policy, rows, cols, want_rows[i],
                                 want_cols[i], &code);
    values[i] = v;
    if (codes != nullptr) codes[i] = code;
}

bool header_ok(const cb200_qcsr *m) { return m != nullptr && m->version == CB200_ABI_VERSION && m->size >= sizeof(cb200_qcsr); }

// ---- request contract -------------------------------------------------------------------------

constexpr std::uint32_t kTypeF16 = 3, kTypeF32 = 4, kTypeF64 = 5, kTypeBf16 = 6, kTypeFp8E4m3 = 7, kTypeFp8E5m2 = 8;

bool known_type(std::uint32_t code) { return code >= kTypeF16 && code <= kTypeFp8E5m2; }
bool bias_kind(std::uint32_t kind) { return kind == CB200_EPILOGUE_BIAS || (kind >= CB200_EPILOGUE_BIAS_RELU && kind <= CB200_EPILOGUE_BIAS_GELU_TANH); }
bool canonical_scalar(const cb200_scalar_value &v) {
    if (v.reserved != 0u) return false;
    if (v.type_code == kTypeF32) return (v.bits >> 32) == 0u;
    return v.type_code == kTypeF64;
}
bool scalar_zero(const cb200_scalar_value &v) {
    if (v.type_code == kTypeF32) {
        float f = 0.0f;
        std::memcpy(&f, &v.bits, sizeof(f));
        return f == 0.0f;
    }
    if (v.type_code == kTypeF64) {
        double d = 0.0;
        std::memcpy(&d, &v.bits, sizeof(d));
        return d == 0.0;
    }
    return false;
}
bool same_order(const cb200_feature_order_identity &a, const cb200_feature_order_identity &b) {
    return a.schema_version == b.schema_version && a.kind == b.kind && a.feature_count == b.feature_count &&
           a.feature_axis_identity_version == b.feature_axis_identity_version && a.feature_axis_identity == b.feature_axis_identity &&
           a.packing_geometry_identity == b.packing_geometry_identity;
}

std::uint64_t splitmix(std::uint64_t v) {
    v += 0x9e3779b97f4a7c15ull;
    v = (v ^ (v >> 30)) * 0xbf58476d1ce4e5b9ull;
    v = (v ^ (v >> 27)) * 0x94d049bb133111ebull;
    return v ^ (v >> 31);
}

} // namespace

extern "C" {

/* ---- element look-up ------------------------------------------------------------------------ */

int64_t cb200_find_in_row(const cb200_qcsr *m, int64_t row, int64_t column) {
    if (!header_ok(m) || m->row_ptr == nullptr || row < 0 || row >= m->rows) return -1;
    for (int64_t i = m->row_ptr[row]; i < m->row_ptr[row + 1]; ++i)
        if (m->col_idx[i] == column) return i;
    return -1;
}

uint32_t cb200_get_code(const cb200_qcsr *m, int64_t row, int64_t local_index) {
    if (!header_ok(m) || m->row_ptr == nullptr || m->packed_values == nullptr || !lookup_bits_ok(m->bits) || row < 0 ||
        row >= m->rows || local_index < 0 || local_index >= m->row_ptr[row + 1] - m->row_ptr[row])
        return 0u;
    const uint8_t *row_bytes = m->packed_values + (m->packed_row_ptr != nullptr ? m->packed_row_ptr[row] : m->row_ptr[row]);
    return unpack_code(row_bytes, local_index, m->bits);
}

float cb200_get_value(const cb200_qcsr *m, int64_t row, int64_t column) {
    if (!header_ok(m) || m->row_ptr == nullptr || !lookup_bits_ok(m->bits)) return 0.0f;
    if (m->bits != 8 && m->packed_row_ptr == nullptr) return 0.0f;
    int code = -1;
    return lookup_value(m->row_ptr, m->packed_row_ptr, m->col_idx, m->packed_values, m->scales, m->offsets, m->bits, m->policy,
                        m->rows, m->cols, row, column, &code);
}

cb200_status cb200_get_values(const cb200_qcsr *m, const int64_t *rows, const int32_t *columns, int64_t count, float *values,
                              int32_t *codes, int32_t device, void *stream) {
    clear_error();
    if (!header_ok(m)) return fail(CB200_STATUS_INVALID_ARGUMENT, "bad cb200_qcsr header");
    if (count < 0 || (count != 0 && (rows == nullptr || columns == nullptr || values == nullptr)))
        return fail(CB200_STATUS_INVALID_ARGUMENT, "look-up needs rows, columns and an output");
    if (!lookup_bits_ok(m->bits) || (m->bits != 8 && m->packed_row_ptr == nullptr))
        return fail(CB200_STATUS_UNSUPPORTED, "look-up takes 1/2/4/8-bit codes (sub-byte codes with packed_row_ptr)");
    if (count == 0) return CB200_STATUS_SUCCESS;
    if (m->row_ptr == nullptr || (m->nnz != 0 && (m->col_idx == nullptr || m->packed_values == nullptr)))
        return fail(CB200_STATUS_INVALID_ARGUMENT, "the matrix has null arrays");
    device_scope scope(device);
    CB200_CUDA_OK(scope.status);
    const unsigned grid = static_cast<unsigned>((count + 255) / 256);
    lookup_values_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(m->row_ptr, m->packed_row_ptr, m->col_idx,
                                                                              m->packed_values, m->scales, m->offsets, m->bits,
                                                                              m->policy, m->rows, m->cols, rows, columns, count,
                                                                              values, codes);
    count_launch();
    CB200_CUDA_OK(cudaGetLastError());
    return CB200_STATUS_SUCCESS;
}

/* ---- SpMM request: validation, trivial cases, signature ------------------------------------------ */

int32_t cb200_spmm_request_validate(const cb200_spmm_request *r) {
    enum { ok = 0, unsupported_version = 1, invalid_shape = 2, invalid_type = 3, invalid_scalar = 4, invalid_workspace_policy = 5,
           invalid_reuse = 6, invalid_feature_order = 7, feature_order_mismatch = 8, missing_bias = 9, unexpected_bias = 10,
           invalid_layout = 11, invalid_identity = 12, invalid_determinism = 14, invalid_epilogue = 15 };
    if (r == nullptr || r->schema_version != 1u || r->operation != 1u) return unsupported_version;
    constexpr std::uint64_t top = std::numeric_limits<std::uint64_t>::max();
    if (r->sparse_nnz != 0u && (r->m == 0u || r->k == 0u)) return invalid_shape;
    const bool sparse_over = r->m != 0u && r->k > top / r->m;
    const bool out_over = r->m != 0u && r->n > top / r->m;
    const bool dense_over = r->k != 0u && r->n > top / r->k;
    if (sparse_over || dense_over || out_over || r->sparse_nnz > r->m * r->k) return invalid_shape;
    if (r->transpose_sparse > 1u || r->transpose_dense > 1u) return invalid_layout;
    const auto layout_ok = [](std::uint32_t l) { return l == 1u || l == 2u; };
    if (!layout_ok(r->dense_rhs_layout) || !layout_ok(r->output_layout)) return invalid_layout;
    const std::uint64_t rhs_rows = r->transpose_dense == 0u ? r->k : r->n, rhs_cols = r->transpose_dense == 0u ? r->n : r->k;
    const std::uint64_t min_rhs_ld = r->dense_rhs_layout == 1u ? rhs_cols : rhs_rows;
    const std::uint64_t min_out_ld = r->output_layout == 1u ? r->n : r->m;
    if ((rhs_rows != 0u && rhs_cols != 0u && r->dense_rhs_leading_dimension < min_rhs_ld) ||
        (r->m != 0u && r->n != 0u && r->output_leading_dimension < min_out_ld))
        return invalid_layout;
    if (!known_type(r->sparse_storage_type_code) || !known_type(r->dense_storage_type_code) || !known_type(r->output_storage_type_code) ||
        !known_type(r->compute_type_code) || !known_type(r->accumulation_type_code))
        return invalid_type;
    if (r->alpha.type_code != r->compute_type_code || r->beta.type_code != r->compute_type_code || !canonical_scalar(r->alpha) ||
        !canonical_scalar(r->beta))
        return invalid_scalar;
    if (r->determinism > 1u) return invalid_determinism;
    if (r->workspace_kind < 1u || r->workspace_kind > 3u || r->workspace_reserved != 0u ||
        (r->workspace_kind == 2u) != (r->workspace_byte_limit != 0u))
        return invalid_workspace_policy;
    if (r->reuse_kind < 1u || r->reuse_kind > 3u || r->reuse_reserved != 0u ||
        (r->reuse_kind == 1u && r->reuse_expected_run_count != 1u) || (r->reuse_kind == 2u && r->reuse_expected_run_count == 0u) ||
        (r->reuse_kind == 3u && r->reuse_expected_run_count != 0u))
        return invalid_reuse;
    if (r->structure_schema_version != 1u || r->structure_identity_version == 0u || r->structure_value == 0u) return invalid_identity;
    const auto order_ok = [r](const cb200_feature_order_identity &o) {
        return o.schema_version == 1u && o.feature_count == r->k && o.feature_axis_identity != 0u &&
               o.feature_axis_identity_version != 0u &&
               ((o.kind == 1u && o.packing_geometry_identity == 0u) || (o.kind == 2u && o.packing_geometry_identity != 0u));
    };
    if (!order_ok(r->sparse_feature_order) || !order_ok(r->dense_feature_order)) return invalid_feature_order;
    if (!same_order(r->sparse_feature_order, r->dense_feature_order)) return feature_order_mismatch;
    if (r->epilogue_kind > CB200_EPILOGUE_BIAS_GELU_TANH) return invalid_epilogue;
    if (bias_kind(r->epilogue_kind)) {
        if (r->epilogue_bias_element_count != r->n || r->epilogue_bias_type_code != r->output_storage_type_code) return missing_bias;
    } else if (r->epilogue_bias_element_count != 0u || r->epilogue_bias_type_code != 0u) {
        return unexpected_bias;
    }
    return ok;
}

int32_t cb200_spmm_request_classify(const cb200_spmm_request *r) {
    if (r == nullptr || r->m == 0u || r->n == 0u) return 1;                           /* no output */
    if (r->k == 0u || r->sparse_nnz == 0u || scalar_zero(r->alpha)) return 2;         /* epilogue only */
    return 0;
}

cb200_status cb200_spmm_request_signature(const cb200_spmm_request *r, uint64_t signature[2]) {
    clear_error();
    if (r == nullptr || signature == nullptr) return fail(CB200_STATUS_INVALID_ARGUMENT, "signature needs a request and an output");
    /* the request's fields in declaration order (the reference's serialisation order), 32-bit ones widened */
    const std::uint64_t fields[] = {
        r->schema_version, r->operation, r->m, r->k, r->n, r->sparse_nnz, r->structure_schema_version,
        r->structure_identity_version, r->structure_value, r->transpose_sparse, r->transpose_dense, r->dense_rhs_layout,
        r->output_layout, r->dense_rhs_leading_dimension, r->output_leading_dimension, r->sparse_storage_type_code,
        r->dense_storage_type_code, r->output_storage_type_code, r->compute_type_code, r->accumulation_type_code,
        r->alpha.type_code, r->alpha.bits, r->beta.type_code, r->beta.bits, r->determinism, r->workspace_kind,
        r->workspace_byte_limit, r->reuse_kind, r->reuse_expected_run_count, r->epilogue_kind, r->epilogue_bias_type_code,
        r->epilogue_bias_element_count,
        r->sparse_feature_order.schema_version, r->sparse_feature_order.kind, r->sparse_feature_order.feature_count,
        r->sparse_feature_order.feature_axis_identity_version, r->sparse_feature_order.feature_axis_identity,
        r->sparse_feature_order.packing_geometry_identity,
        r->dense_feature_order.schema_version, r->dense_feature_order.kind, r->dense_feature_order.feature_count,
        r->dense_feature_order.feature_axis_identity_version, r->dense_feature_order.feature_axis_identity,
        r->dense_feature_order.packing_geometry_identity};
    std::uint64_t low = 0x43504d4154484f50ull, high = 0x53504d4d00000001ull; /* the two lane seeds of the schema */
    for (const std::uint64_t f : fields) {
        low = splitmix(low ^ f);
        high = splitmix(high + f + 0x9e3779b97f4a7c15ull);
    }
    signature[0] = low;
    signature[1] = high;
    return CB200_STATUS_SUCCESS;
}

cb200_status cb200_spmm_request_from_problem(const cb200_spmm_problem *problem, const cb200_launch *launch,
                                             uint64_t structure_identity, uint64_t feature_axis_identity,
                                             cb200_spmm_request *request) {
    clear_error();
    if (problem == nullptr || launch == nullptr || request == nullptr)
        return fail(CB200_STATUS_INVALID_ARGUMENT, "request_from_problem needs a problem, a launch and an output");
    if (problem->k < 0 || problem->k > 0xffffffffll) return fail(CB200_STATUS_INVALID_SHAPE, "feature count outside 32 bits");
    const auto type_code = [](int dtype) -> std::uint32_t {
        switch (dtype) {
        case CB200_DTYPE_F16: return kTypeF16;
        case CB200_DTYPE_BF16: return kTypeBf16;
        case CB200_DTYPE_F64: return kTypeF64;
        default: return kTypeF32;
        }
    };
    std::memset(request, 0, sizeof(*request));
    const bool transpose = problem->projection == CB200_PROJECTION_TRANSPOSE;
    request->schema_version = 1u;
    request->operation = 1u;
    /* logical dimensions after the declared transpose: the transpose multiplies X^T (k x m) with G (m x n) */
    request->m = static_cast<std::uint64_t>(transpose ? problem->k : problem->m);
    request->k = static_cast<std::uint64_t>(transpose ? problem->m : problem->k);
    request->n = static_cast<std::uint64_t>(problem->n);
    request->sparse_nnz = static_cast<std::uint64_t>(problem->nnz);
    request->structure_schema_version = 1u;
    request->structure_identity_version = 1u;
    request->structure_value = structure_identity;
    request->transpose_sparse = transpose ? 1u : 0u;
    request->dense_rhs_layout = request->output_layout = 1u;
    request->dense_rhs_leading_dimension = static_cast<std::uint64_t>(launch->dense_ld);
    request->output_leading_dimension = static_cast<std::uint64_t>(launch->out_ld);
    /* decoded values are fp32 (dequantize_code returns Real = float); the codes themselves have no real:: code */
    request->sparse_storage_type_code = kTypeF32;
    request->dense_storage_type_code = type_code(problem->dense_dtype);
    request->output_storage_type_code = kTypeF32;
    request->compute_type_code = kTypeF32;
    request->accumulation_type_code = kTypeF32;
    request->alpha.type_code = request->beta.type_code = kTypeF32;
    std::memcpy(&request->alpha.bits, &launch->alpha, sizeof(float));
    std::memcpy(&request->beta.bits, &launch->beta, sizeof(float));
    request->determinism = problem->deterministic ? 1u : 0u;
    request->workspace_kind = 1u;
    request->reuse_kind = 3u; /* persistent: a prepared operation is made to be run many times */
    request->reuse_expected_run_count = 0u;
    request->epilogue_kind = static_cast<std::uint32_t>(launch->epilogue);
    if (bias_kind(request->epilogue_kind)) {
        request->epilogue_bias_type_code = kTypeF32;
        request->epilogue_bias_element_count = request->n;
    }
    cb200_feature_order_identity order{};
    order.schema_version = 1u;
    order.kind = 1u;
    order.feature_count = static_cast<std::uint32_t>(request->k);
    order.feature_axis_identity_version = 1u;
    order.feature_axis_identity = feature_axis_identity;
    request->sparse_feature_order = request->dense_feature_order = order;
    return CB200_STATUS_SUCCESS;
}

/* ---- host container of a quantized Blocked-ELL matrix ------------------------------------------- */

uint64_t cb200_qbell_pack_aux(uint32_t bits, uint32_t block_size, uint64_t ell_width) {
    return (ell_width << 24) | (static_cast<uint64_t>(bits & 0xffu) << 16) | static_cast<uint64_t>(block_size);
}

void cb200_qbell_unpack_aux(uint64_t aux, uint32_t *bits, uint32_t *block_size, uint64_t *ell_width, uint32_t *ell_cols) {
    const uint32_t bs = static_cast<uint32_t>(aux & 0xffffull);
    const uint64_t width = aux >> 24;
    if (bits != nullptr) *bits = static_cast<uint32_t>((aux >> 16) & 0xffull);
    if (block_size != nullptr) *block_size = bs;
    if (ell_width != nullptr) *ell_width = width;
    if (ell_cols != nullptr) *ell_cols = static_cast<uint32_t>(width * bs);
}

uint32_t cb200_qbell_row_bytes(uint32_t bits, uint32_t ell_cols) {
    const uint32_t per_byte = bits == 0u ? 0u : 8u / bits;
    return per_byte == 0u ? 0u : (ell_cols + per_byte - 1u) / per_byte;
}

uint32_t cb200_qbell_aligned_row_bytes(uint32_t bits, uint32_t ell_cols, uint32_t alignment) {
    const uint32_t bytes = cb200_qbell_row_bytes(bits, ell_cols);
    return alignment <= 1u ? bytes : (bytes + alignment - 1u) / alignment * alignment;
}

void cb200_qbell_host_init(cb200_qbell_host *m, uint32_t rows, uint32_t cols, uint32_t nnz, uint32_t block_size, uint32_t ell_cols,
                           uint32_t bits, uint32_t decode_policy, uint32_t row_stride_bytes) {
    if (m == nullptr) return;
    std::memset(m, 0, sizeof(*m));
    m->rows = rows; m->cols = cols; m->nnz = nnz; m->block_size = block_size; m->ell_cols = ell_cols; m->bits = bits;
    m->row_stride_bytes = row_stride_bytes != 0u ? row_stride_bytes : cb200_qbell_aligned_row_bytes(bits, ell_cols, 16u);
    m->decode_policy = decode_policy;
}

} // extern "C"

namespace {

struct slab_layout {
    std::size_t idx_bytes, packed_offset, packed_bytes, scales_offset, offsets_offset, row_offsets_offset, total;
};

slab_layout layout_of(const cb200_qbell_host &m) {
    slab_layout l{};
    const std::size_t row_blocks = m.block_size == 0u ? 0u : (static_cast<std::size_t>(m.rows) + m.block_size - 1u) / m.block_size;
    const std::size_t width = (m.block_size == 0u || m.ell_cols == 0u) ? 0u : m.ell_cols / m.block_size;
    l.idx_bytes = row_blocks * width * sizeof(std::uint32_t);
    l.packed_offset = l.idx_bytes;
    l.packed_bytes = static_cast<std::size_t>(m.rows) * m.row_stride_bytes;
    l.scales_offset = (l.packed_offset + l.packed_bytes + sizeof(float) - 1u) / sizeof(float) * sizeof(float);
    l.offsets_offset = l.scales_offset + static_cast<std::size_t>(m.cols) * sizeof(float);
    l.row_offsets_offset = l.offsets_offset + static_cast<std::size_t>(m.cols) * sizeof(float);
    l.total = l.row_offsets_offset + static_cast<std::size_t>(m.rows) * sizeof(float);
    return l;
}

void release(cb200_qbell_host *m) {
    if ((m->flags & CB200_QBELL_HOST_REGISTERED) != 0u && m->storage != nullptr) cudaHostUnregister(m->storage);
    std::free(m->storage);
    m->flags = 0u;
    m->storage = nullptr;
    m->block_col_idx = nullptr;
    m->packed_values = nullptr;
    m->column_scales = m->column_offsets = m->row_offsets = nullptr;
}

void point_into(const cb200_qbell_host &m, const slab_layout &l, unsigned char *base, const std::uint32_t **idx,
                const std::uint8_t **packed, const float **scales, const float **col_offsets, const float **row_offsets) {
    *idx = l.idx_bytes != 0u ? reinterpret_cast<const std::uint32_t *>(base) : nullptr;
    *packed = l.packed_bytes != 0u ? base + l.packed_offset : nullptr;
    *scales = m.cols != 0u ? reinterpret_cast<const float *>(base + l.scales_offset) : nullptr;
    *col_offsets = m.cols != 0u ? reinterpret_cast<const float *>(base + l.offsets_offset) : nullptr;
    *row_offsets = m.rows != 0u ? reinterpret_cast<const float *>(base + l.row_offsets_offset) : nullptr;
}

void fill_view(const cb200_qbell_host &m, const std::uint32_t *idx, const std::uint8_t *packed, const float *scales,
               const float *col_offsets, const float *row_offsets, cb200_qbell *view) {
    std::memset(view, 0, sizeof(*view));
    view->version = CB200_ABI_VERSION;
    view->size = sizeof(*view);
    view->rows = m.rows; view->cols = m.cols; view->block_size = static_cast<int32_t>(m.block_size);
    view->ell_cols = static_cast<int32_t>(m.ell_cols); view->row_stride_bytes = m.row_stride_bytes;
    view->bits = static_cast<int32_t>(m.bits); view->policy = static_cast<int32_t>(m.decode_policy);
    view->block_col_idx = idx; view->packed_values = packed; view->scales = scales;
    view->offsets = m.decode_policy == CB200_DECODE_COLUMN_SCALE_ROW_OFFSET ? row_offsets : col_offsets;
}

} // namespace

extern "C" {

uint64_t cb200_qbell_host_bytes(const cb200_qbell_host *m) { return m == nullptr ? 0u : sizeof(*m) + layout_of(*m).total; }

int32_t cb200_qbell_host_allocate(cb200_qbell_host *m) {
    if (m == nullptr) return 0;
    release(m);
    const slab_layout l = layout_of(*m);
    if (l.total == 0u) return 1;
    unsigned char *base = static_cast<unsigned char *>(std::malloc(l.total));
    if (base == nullptr) return 0;
    m->storage = base;
    const std::uint32_t *idx; const std::uint8_t *packed; const float *scales, *col_offsets, *row_offsets;
    point_into(*m, l, base, &idx, &packed, &scales, &col_offsets, &row_offsets);
    m->block_col_idx = const_cast<std::uint32_t *>(idx);
    m->packed_values = const_cast<std::uint8_t *>(packed);
    m->column_scales = const_cast<float *>(scales);
    m->column_offsets = const_cast<float *>(col_offsets);
    m->row_offsets = const_cast<float *>(row_offsets);
    return 1;
}

int32_t cb200_qbell_host_pin(cb200_qbell_host *m) {
    if (m == nullptr) return 0;
    const std::size_t total = layout_of(*m).total;
    if (m->storage == nullptr || total == 0u || (m->flags & CB200_QBELL_HOST_REGISTERED) != 0u) return 1;
    const cudaError_t err = cudaHostRegister(m->storage, total, cudaHostRegisterPortable);
    if (err == cudaSuccess || err == cudaErrorHostMemoryAlreadyRegistered) {
        if (err != cudaSuccess) cudaGetLastError();
        m->flags |= CB200_QBELL_HOST_REGISTERED;
        return 1;
    }
    cudaGetLastError(); /* pinning is optional: the container stays usable, copies from it are just not asynchronous */
    return 0;
}

void cb200_qbell_host_unpin(cb200_qbell_host *m) {
    if (m == nullptr || (m->flags & CB200_QBELL_HOST_REGISTERED) == 0u || m->storage == nullptr) return;
    cudaHostUnregister(m->storage);
    m->flags &= ~static_cast<uint32_t>(CB200_QBELL_HOST_REGISTERED);
}

void cb200_qbell_host_clear(cb200_qbell_host *m) {
    if (m == nullptr) return;
    release(m);
    cb200_qbell_host_init(m, 0, 0, 0, 0, 0, 0, 0, 0);
    m->row_stride_bytes = 0u;
}

cb200_status cb200_qbell_host_view(const cb200_qbell_host *m, cb200_qbell *view) {
    clear_error();
    if (m == nullptr || view == nullptr) return fail(CB200_STATUS_INVALID_ARGUMENT, "view needs a container and an output");
    fill_view(*m, m->block_col_idx, m->packed_values, m->column_scales, m->column_offsets, m->row_offsets, view);
    return CB200_STATUS_SUCCESS;
}

cb200_status cb200_qbell_host_upload(const cb200_qbell_host *m, void *device_storage, uint64_t device_bytes, int32_t device,
                                     void *stream, cb200_qbell *device_view) {
    clear_error();
    if (m == nullptr || device_view == nullptr) return fail(CB200_STATUS_INVALID_ARGUMENT, "upload needs a container and an output view");
    const slab_layout l = layout_of(*m);
    if (l.total != 0u && (m->storage == nullptr || device_storage == nullptr))
        return fail(CB200_STATUS_INVALID_ARGUMENT, "upload needs an allocated container and device storage");
    if (device_bytes < l.total) return fail(CB200_STATUS_INSUFFICIENT_WORKSPACE, "device storage of %zu bytes needed, %llu given", l.total,
                                            static_cast<unsigned long long>(device_bytes));
    if (reinterpret_cast<std::uintptr_t>(device_storage) % 256u != 0u)
        return fail(CB200_STATUS_INVALID_ARGUMENT, "device storage must be 256-byte aligned");
    device_scope scope(device);
    CB200_CUDA_OK(scope.status);
    if (l.total != 0u)
        CB200_CUDA_OK(cudaMemcpyAsync(device_storage, m->storage, l.total, cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream)));
    const std::uint32_t *idx; const std::uint8_t *packed; const float *scales, *col_offsets, *row_offsets;
    point_into(*m, l, static_cast<unsigned char *>(device_storage), &idx, &packed, &scales, &col_offsets, &row_offsets);
    fill_view(*m, idx, packed, scales, col_offsets, row_offsets, device_view);
    return CB200_STATUS_SUCCESS;
}

} // extern "C"
