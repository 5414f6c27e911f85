// C entry points over the UNMODIFIED Cellerator reference sources, compiled in place.
//
// TEST INFRASTRUCTURE ONLY.  This translation unit includes the reference's own headers
// (found through -I at build time; nothing of the reference is copied into this
// repository) and is linked with the reference's referee.cc / operation.cc /
// operation_signature.cc / physical_bell.cc / physical_bell_candidates.cc / physical_csr.cc.  The resulting library, oracle/_ref/libcellerator_ref.so, is what
// the C restatement in oracle.c is validated against, and it can serve as the CPU baseline.
//
// The reference's quantized CSR uses `int` row pointers; the entry points here take the
// int64 arrays that the rest of this repository uses and narrow them (the caller keeps
// nnz below 2^31 on this path).
#include <Cellerator/compute/math/physical_bell.hh>
#include <Cellerator/compute/math/physical_csr.hh>
#include <Cellerator/compute/math/referee.hh>
#include <Cellerator/quantized/blocked_ell.cuh>
#include <Cellerator/quantized/packing.cuh>
#include <Cellerator/types.cuh>

#include <cstdint>
#include <cstring>
#include <vector>

namespace q = ::cellerator::quantized;
namespace cm = ::cellerator::compute::math;

namespace {

std::vector<int> narrow(const std::int64_t *src, std::int64_t count) {
    std::vector<int> out(static_cast<std::size_t>(count));
    for (std::int64_t i = 0; i < count; ++i) out[static_cast<std::size_t>(i)] = static_cast<int>(src[i]);
    return out;
}

template<int Bits, typename Meta>
int pack_impl(std::int64_t rows, std::int64_t cols, const std::vector<int> &rp, const std::vector<int> &prp,
              const int *col_idx, Meta meta, const float *values, unsigned char *packed) {
    auto m = q::make_matrix<Bits>(static_cast<int>(rows), static_cast<int>(cols), rp.back(), 0, rp.data(),
                                  prp.data(), col_idx, nullptr, packed, meta);
    return q::pack_nnz_values(&m, values);
}

template<int Bits, typename Meta>
int unpack_impl(std::int64_t rows, std::int64_t cols, const std::vector<int> &rp, const std::vector<int> &prp,
                const int *col_idx, Meta meta, const unsigned char *packed, float *values) {
    auto m = q::make_matrix<Bits>(static_cast<int>(rows), static_cast<int>(cols), rp.back(), 0, rp.data(),
                                  prp.data(), col_idx, nullptr, const_cast<unsigned char *>(packed), meta);
    return q::unpack_nnz_values(&m, values);
}

template<typename Fn>
int by_bits(int bits, Fn &&fn) {
    switch (bits) {
    case 1: return fn(std::integral_constant<int, 1>{});
    case 2: return fn(std::integral_constant<int, 2>{});
    case 4: return fn(std::integral_constant<int, 4>{});
    case 8: return fn(std::integral_constant<int, 8>{});
    default: return -2;
    }
}

cm::feature_order_identity order_for(cm::u64 k) {
    cm::feature_order_identity order;
    order.feature_count = static_cast<cm::u32>(k);
    order.feature_axis_identity_version = 1u;
    order.feature_axis_identity = 0xb200ull;
    return order;
}

} // namespace

extern "C" {

std::int64_t ref_build_packed_row_ptr(int bits, const std::int64_t *row_ptr, std::int64_t rows,
                                      std::int64_t *packed_row_ptr) {
    const std::vector<int> rp = narrow(row_ptr, rows + 1);
    std::vector<int> out(static_cast<std::size_t>(rows) + 1u, 0);
    const int total = by_bits(bits, [&](auto b) {
        return q::build_packed_row_ptr<decltype(b)::value>(rp.data(), static_cast<int>(rows), out.data());
    });
    for (std::int64_t i = 0; i <= rows; ++i) packed_row_ptr[i] = out[static_cast<std::size_t>(i)];
    return total;
}

std::int64_t ref_build_uniform_block_row_ptr(std::int64_t rows, std::int64_t rows_per_block,
                                             std::int64_t *block_row_ptr) {
    const int count = q::block_count_for_rows(static_cast<int>(rows), static_cast<int>(rows_per_block));
    std::vector<int> out(static_cast<std::size_t>(count) + 1u, 0);
    const int rc = q::build_uniform_block_row_ptr(static_cast<int>(rows), static_cast<int>(rows_per_block),
                                                  out.data());
    if (rc < 0) return rc;
    for (int i = 0; i <= count; ++i) block_row_ptr[i] = out[static_cast<std::size_t>(i)];
    return rc;
}

void ref_get_block(std::int64_t rows, const std::int64_t *row_ptr, const std::int64_t *packed_row_ptr,
                   const std::int64_t *block_row_ptr, std::int64_t block_count, std::int64_t block_index,
                   std::int64_t out[7]) {
    const std::vector<int> rp = narrow(row_ptr, rows + 1);
    const std::vector<int> prp = narrow(packed_row_ptr, rows + 1);
    std::vector<int> brp;
    if (block_row_ptr != nullptr && block_count > 0) brp = narrow(block_row_ptr, block_count + 1);
    auto m = q::make_matrix<8>(static_cast<int>(rows), 1, rp.back(), static_cast<int>(block_count), rp.data(),
                               prp.data(), nullptr, brp.empty() ? nullptr : brp.data(), nullptr,
                               q::make_per_gene_affine<float>(nullptr, nullptr));
    const q::csr_block b = q::get_block(&m, static_cast<int>(block_index));
    out[0] = b.block_index; out[1] = b.row_begin; out[2] = b.row_end; out[3] = b.nnz_begin;
    out[4] = b.nnz_end; out[5] = b.packed_begin; out[6] = b.packed_end;
}

unsigned ref_quantize_code(int bits, float value, float scale, float offset) {
    const auto meta = q::make_per_gene_affine<float>(&scale, &offset);
    unsigned out = 0u;
    by_bits(bits, [&](auto b) {
        out = q::quantize_code<decltype(b)::value, float>(value, meta, meta.prepare_row(0), 0);
        return 0;
    });
    return out;
}

float ref_dequantize_code(unsigned code, float scale, float offset) {
    const auto meta = q::make_per_gene_affine<float>(&scale, &offset);
    return q::dequantize_code<8, float>(code, meta, meta.prepare_row(0), 0);
}

// policy 1 = per_gene_affine (scales, offsets per gene); 2 = column_scale_row_offset
int ref_pack_csr(int bits, int policy, std::int64_t rows, std::int64_t cols, const std::int64_t *row_ptr,
                 const std::int64_t *packed_row_ptr, const std::int32_t *col_idx, const float *scales,
                 const float *offsets, const float *values, unsigned char *packed) {
    const std::vector<int> rp = narrow(row_ptr, rows + 1);
    const std::vector<int> prp = narrow(packed_row_ptr, rows + 1);
    return by_bits(bits, [&](auto b) {
        constexpr int B = decltype(b)::value;
        if (policy == 2)
            return pack_impl<B>(rows, cols, rp, prp, col_idx, q::make_column_scale_row_offset(scales, offsets),
                                values, packed);
        return pack_impl<B>(rows, cols, rp, prp, col_idx, q::make_per_gene_affine(scales, offsets), values,
                            packed);
    });
}

int ref_unpack_csr(int bits, int policy, std::int64_t rows, std::int64_t cols, const std::int64_t *row_ptr,
                   const std::int64_t *packed_row_ptr, const std::int32_t *col_idx, const float *scales,
                   const float *offsets, const unsigned char *packed, float *values) {
    const std::vector<int> rp = narrow(row_ptr, rows + 1);
    const std::vector<int> prp = narrow(packed_row_ptr, rows + 1);
    return by_bits(bits, [&](auto b) {
        constexpr int B = decltype(b)::value;
        if (policy == 2)
            return unpack_impl<B>(rows, cols, rp, prp, col_idx,
                                  q::make_column_scale_row_offset(scales, offsets), packed, values);
        return unpack_impl<B>(rows, cols, rp, prp, col_idx, q::make_per_gene_affine(scales, offsets), packed,
                              values);
    });
}

int ref_bell_pack(int bits, int policy, std::int64_t rows, std::int64_t cols, int block_size,
                  std::int64_t ell_cols, std::int64_t row_stride_bytes, const std::uint32_t *block_col_idx,
                  const float *scales, const float *offsets, const float *values_by_slot,
                  unsigned char *packed) {
    return by_bits(bits, [&](auto b) {
        constexpr int B = decltype(b)::value;
        if (policy == 2) {
            auto m = q::blocked_ell::make_matrix<B>(static_cast<int>(rows), static_cast<int>(cols), 0, block_size,
                                                    static_cast<int>(ell_cols), static_cast<int>(row_stride_bytes),
                                                    block_col_idx, packed,
                                                    q::make_column_scale_row_offset(scales, offsets));
            return q::blocked_ell::pack_row_major_values(&m, values_by_slot);
        }
        auto m = q::blocked_ell::make_matrix<B>(static_cast<int>(rows), static_cast<int>(cols), 0, block_size,
                                                static_cast<int>(ell_cols), static_cast<int>(row_stride_bytes),
                                                block_col_idx, packed, q::make_per_gene_affine(scales, offsets));
        return q::blocked_ell::pack_row_major_values(&m, values_by_slot);
    });
}

int ref_bell_unpack(int bits, int policy, std::int64_t rows, std::int64_t cols, int block_size,
                    std::int64_t ell_cols, std::int64_t row_stride_bytes, const std::uint32_t *block_col_idx,
                    const float *scales, const float *offsets, const unsigned char *packed,
                    float *values_by_slot) {
    unsigned char *p = const_cast<unsigned char *>(packed);
    return by_bits(bits, [&](auto b) {
        constexpr int B = decltype(b)::value;
        if (policy == 2) {
            auto m = q::blocked_ell::make_matrix<B>(static_cast<int>(rows), static_cast<int>(cols), 0, block_size,
                                                    static_cast<int>(ell_cols), static_cast<int>(row_stride_bytes),
                                                    block_col_idx, p,
                                                    q::make_column_scale_row_offset(scales, offsets));
            return q::blocked_ell::unpack_row_major_values(&m, values_by_slot);
        }
        auto m = q::blocked_ell::make_matrix<B>(static_cast<int>(rows), static_cast<int>(cols), 0, block_size,
                                                static_cast<int>(ell_cols), static_cast<int>(row_stride_bytes),
                                                block_col_idx, p, q::make_per_gene_affine(scales, offsets));
        return q::blocked_ell::unpack_row_major_values(&m, values_by_slot);
    });
}

// build_spmm_reference for f32 operands.  Layout flags: 0 row-major, 1 column-major.
int ref_spmm_reference(std::uint64_t m, std::uint64_t k, std::uint64_t n, int transpose_sparse,
                       int transpose_dense, std::uint64_t sparse_nnz, const std::uint64_t *row_offsets,
                       const std::uint32_t *column_indices, const float *sparse_values, const float *rhs,
                       int rhs_col_major, std::uint64_t rhs_ld, double alpha, double beta, const float *initial,
                       int initial_col_major, std::uint64_t initial_ld, int epilogue, const float *bias,
                       double *reference, std::uint64_t reference_capacity) {
    cm::spmm_request r;
    r.m = m; r.k = k; r.n = n; r.sparse_nnz = sparse_nnz;
    r.sparse_structure.identity_version = 1u;
    r.sparse_structure.value = 0xb200b200ull;
    r.transpose_sparse = transpose_sparse ? cm::transpose_kind::transpose : cm::transpose_kind::none;
    r.transpose_dense = transpose_dense ? cm::transpose_kind::transpose : cm::transpose_kind::none;
    r.dense_rhs_layout = rhs_col_major ? cm::dense_layout_kind::column_major : cm::dense_layout_kind::row_major;
    r.output_layout = initial_col_major ? cm::dense_layout_kind::column_major : cm::dense_layout_kind::row_major;
    r.dense_rhs_leading_dimension = rhs_ld;
    r.output_leading_dimension = initial_ld != 0u ? initial_ld : (initial_col_major ? m : n);
    r.sparse_storage_type_code = ::cellerator::real::value_f32;
    r.dense_storage_type_code = ::cellerator::real::value_f32;
    r.output_storage_type_code = ::cellerator::real::value_f32;
    r.compute_type_code = ::cellerator::real::value_f64;
    r.accumulation_type_code = ::cellerator::real::value_f64;
    r.alpha = cm::make_scalar(alpha);
    r.beta = cm::make_scalar(beta);
    r.epilogue.kind = static_cast<cm::epilogue_kind>(epilogue);
    const bool has_bias = epilogue == 1 || epilogue == 5 || epilogue == 6 || epilogue == 7;
    if (has_bias) {
        r.epilogue.bias_type_code = ::cellerator::real::value_f32;
        r.epilogue.bias_element_count = n;
    }
    r.sparse_feature_order = order_for(k);
    r.dense_feature_order = r.sparse_feature_order;

    const cm::u64 srows = transpose_sparse ? k : m;
    const cm::u64 scols = transpose_sparse ? m : k;
    const cm::logical_csr_view sparse{srows, scols, sparse_nnz, row_offsets, column_indices, sparse_values,
                                      static_cast<cm::u32>(::cellerator::real::value_f32)};
    const cm::logical_dense_view dense{rhs, transpose_dense ? n : k, transpose_dense ? k : n, rhs_ld,
                                       r.dense_rhs_layout, static_cast<cm::u32>(::cellerator::real::value_f32)};
    const cm::logical_dense_view prior{initial, m, n, r.output_leading_dimension, r.output_layout,
                                       static_cast<cm::u32>(::cellerator::real::value_f32)};
    const cm::referee_status status =
        cm::build_spmm_reference(r, sparse, dense, prior, bias, reference, reference_capacity);
    return static_cast<int>(status.code);
}

// The reference's request contract on a request handed over as 48 unsigned 64-bit fields in the
// declaration order of spmm_request (operation.hh:136-164; 32-bit fields widened, the two scalar and the
// two reserved words included as they lie): out[0] = validate_spmm_request code, out[1] =
// classify_trivial_operation kind, out[2], out[3] = make_operation_signature low, high.
void ref_request_contract(const std::uint64_t *f, std::uint64_t out[4]) {
    cm::spmm_request r;
    int i = 0;
    const auto u32 = [&]() { return static_cast<cm::u32>(f[i++]); };
    const auto u64 = [&]() { return f[i++]; };
    r.schema_version = u32(); r.operation = static_cast<cm::operation_kind>(u32());
    r.m = u64(); r.k = u64(); r.n = u64(); r.sparse_nnz = u64();
    r.sparse_structure.schema_version = u32(); r.sparse_structure.identity_version = u32(); r.sparse_structure.value = u64();
    r.transpose_sparse = static_cast<cm::transpose_kind>(u32()); r.transpose_dense = static_cast<cm::transpose_kind>(u32());
    r.dense_rhs_layout = static_cast<cm::dense_layout_kind>(u32()); r.output_layout = static_cast<cm::dense_layout_kind>(u32());
    r.dense_rhs_leading_dimension = u64(); r.output_leading_dimension = u64();
    r.sparse_storage_type_code = u32(); r.dense_storage_type_code = u32(); r.output_storage_type_code = u32();
    r.compute_type_code = u32(); r.accumulation_type_code = u32();
    r.alpha.type_code = u32(); r.alpha.reserved = u32(); r.alpha.bits = u64();
    r.beta.type_code = u32(); r.beta.reserved = u32(); r.beta.bits = u64();
    r.determinism = static_cast<cm::determinism_requirement>(u32());
    r.workspace.kind = static_cast<cm::workspace_policy_kind>(u32()); r.workspace.reserved = u32(); r.workspace.byte_limit = u64();
    r.reuse.kind = static_cast<cm::expected_reuse_kind>(u32()); r.reuse.reserved = u32(); r.reuse.expected_run_count = u64();
    r.epilogue.kind = static_cast<cm::epilogue_kind>(u32()); r.epilogue.bias_type_code = u32(); r.epilogue.bias_element_count = u64();
    for (cm::feature_order_identity *o : {&r.sparse_feature_order, &r.dense_feature_order}) {
        o->schema_version = u32(); o->kind = static_cast<cm::feature_order_kind>(u32()); o->feature_count = u32();
        o->feature_axis_identity_version = u32(); o->feature_axis_identity = u64(); o->packing_geometry_identity = u64();
    }
    const cm::operation_signature sig = cm::make_operation_signature(r);
    out[0] = static_cast<std::uint64_t>(cm::validate_spmm_request(r).code);
    out[1] = static_cast<std::uint64_t>(cm::classify_trivial_operation(r));
    out[2] = sig.low;
    out[3] = sig.high;
}

// digest helper of the referee
void ref_digest_f32(const float *values, std::uint64_t rows, std::uint64_t columns, std::uint64_t ld,
                    std::uint64_t out[2]) {
    const cm::logical_dense_view view{values, rows, columns, ld, cm::dense_layout_kind::row_major,
                                      static_cast<cm::u32>(::cellerator::real::value_f32)};
    cm::determinism_digest d;
    cm::digest_logical_dense(view, &d);
    out[0] = d.low;
    out[1] = d.high;
}

// query_bell_candidates_host + materialize_bell_candidate_host (physical_bell.hh:172-192) for one
// block size, same arguments and outputs as orc_bell_lowering in oracle.c.  The reference writes
// block-major values only (values_layout 0).
int ref_bell_lowering(std::uint32_t rows, std::uint32_t features, std::uint32_t nnz, std::uint32_t value_size,
                      const std::uint32_t *row_offsets, const std::uint32_t *feature_ids, const void *values,
                      std::uint32_t fb_count, const std::uint32_t *fb_offsets, const std::uint32_t *fperm,
                      const std::uint32_t *finv, const std::uint32_t *rperm, const std::uint32_t *rinv, std::uint32_t bs,
                      double max_value_expansion, double max_storage_expansion, std::uint64_t max_persistent,
                      std::uint64_t *geometry, double *metrics, std::uint32_t *padded_fb_offsets,
                      std::int32_t *column_indices, void *values_out, std::uint64_t column_capacity,
                      std::uint64_t value_capacity, int values_layout, std::uint64_t) {
    if (values_layout != 0) return -3;
    if (bs != 8u && bs != 16u && bs != 32u) return static_cast<int>(cm::bell_lowering_status_code::candidate_mismatch);
    cm::bell_csr_source_view source{rows, features, nnz, value_size, row_offsets, feature_ids, values};
    cm::bell_semantic_plan_view plan{};
    plan.semantic_schema_version = cellpack::packing_plan_semantic_schema_version;
    plan.full_row_count = rows == 0u ? 1u : rows;
    plan.feature_count = features;
    plan.feature_block_count = fb_count;
    plan.feature_block_geometry_identity = 0x12345678ull;
    plan.row_domain_identity = 0xabcddcbaull;
    plan.feature_block_offsets = fb_offsets;
    plan.feature_permutation = fperm;
    plan.inverse_feature_permutation = finv;
    cellpack::local_cell_order_view order{};
    order.order_schema_version = cellpack::local_cell_order_schema_version;
    order.signature_algorithm_version = cellpack::local_cell_signature_algorithm_version;
    order.window_size = 1024u;
    order.group_width = 32u;
    order.ordering_identity = 0xfedcba98ull;
    order.full_row_count = plan.full_row_count;
    order.row_count = rows;
    order.feature_block_count = fb_count;
    order.feature_block_geometry_identity = plan.feature_block_geometry_identity;
    order.row_domain_identity = plan.row_domain_identity;
    order.row_permutation = rperm;
    order.inverse_row_permutation = rinv;
    cm::bell_lowering_workspace_requirements need;
    cm::bell_lowering_status st = cm::query_bell_lowering_workspace_requirements(source, plan, order, &need);
    if (!st) return static_cast<int>(st.code);
    std::vector<std::uint32_t> markers(need.marker_count + 1u), block_offsets(need.feature_block_offset_count);
    const cm::bell_lowering_workspace ws{markers.size(), markers.data(), block_offsets.size(), block_offsets.data()};
    cm::bell_lowering_policy policy;
    policy.maximum_value_slot_expansion = max_value_expansion;
    policy.maximum_storage_expansion = max_storage_expansion;
    policy.maximum_persistent_bytes = static_cast<std::size_t>(max_persistent);
    cm::bell_candidate_set set;
    st = cm::query_bell_candidates_host(source, plan, order, policy, ws, &set);
    if (!st) return static_cast<int>(st.code);
    const cm::bell_candidate_requirements &c = set.candidates[bs == 8u ? 0 : (bs == 16u ? 1 : 2)];
    geometry[0] = static_cast<std::uint64_t>(c.state);
    geometry[1] = c.padded_row_count; geometry[2] = c.padded_feature_count; geometry[3] = c.block_row_count;
    geometry[4] = c.ell_blocks_per_row; geometry[5] = c.ell_columns; geometry[6] = c.column_index_count;
    geometry[7] = c.value_bytes; geometry[8] = c.metrics.occupied_blocks; geometry[9] = c.metrics.stored_blocks;
    geometry[10] = c.metrics.dense_value_slots; geometry[11] = c.metrics.persistent_bytes; geometry[12] = c.metrics.source_bytes;
    metrics[0] = c.metrics.scalar_occupancy; metrics[1] = c.metrics.ell_slot_utilization;
    metrics[2] = c.metrics.value_slot_expansion; metrics[3] = c.metrics.storage_expansion;
    if (column_indices == nullptr) return 0;
    const cm::bell_candidate_buffers buffers{padded_fb_offsets == nullptr ? 0u : static_cast<std::size_t>(fb_count) + 1u,
                                             padded_fb_offsets, static_cast<std::size_t>(column_capacity), column_indices,
                                             static_cast<std::size_t>(value_capacity), values_out};
    cm::physical_bell_view view;
    st = cm::materialize_bell_candidate_host(source, plan, order, policy, c, ws, buffers, &view);
    return static_cast<int>(st.code);
}

// build_execution_csr_view_host (physical_csr.hh:172-177), same arguments as orc_build_execution_csr.
int ref_build_execution_csr(std::uint32_t rows, std::uint32_t nnz, std::uint32_t features, std::uint32_t fb_count,
                            const std::uint32_t *fb_offsets, const std::uint32_t *fperm, const std::uint32_t *row_offsets,
                            const std::uint32_t *block_ids, const std::uint32_t *local_ids, const std::uint32_t *canonical_ids,
                            std::uint32_t *execution_ids) {
    cellpack::feature_weighted_row_reduction_plan_view plan;
    plan.semantic_plan_schema_version = cellpack::packing_plan_semantic_schema_version;
    plan.geometry_identity_version = cellpack::feature_block_geometry_identity_version;
    plan.feature_count = features;
    plan.feature_block_count = fb_count;
    plan.feature_block_geometry_identity = 0x03030303ull;
    plan.feature_block_offsets = fb_offsets;
    plan.feature_permutation = fperm;
    cellpack::ordered_plan_partition_view ordered;
    ordered.semantic_plan_schema_version = cellpack::packing_plan_semantic_schema_version;
    ordered.full_row_count = rows;
    ordered.row_count = rows;
    ordered.feature_count = features;
    ordered.nnz_count = nnz;
    ordered.value_size_bytes = 1u;
    ordered.feature_axis_fingerprint = 0x0303a11ull;
    ordered.feature_axis_fingerprint_version = 1u;
    ordered.row_domain_identity = 0x303ull;
    ordered.row_offsets = row_offsets;
    ordered.block_ids = block_ids;
    ordered.local_feature_ids = local_ids;
    ordered.canonical_feature_ids = canonical_ids;
    static const unsigned char nothing = 0;
    ordered.values = &nothing; // only its presence is checked; the view aliases it
    cm::execution_csr_view out;
    const cm::physical_view_status st = cm::build_execution_csr_view_host(plan, ordered, {nnz, execution_ids}, &out);
    return static_cast<int>(st.code);
}

} // extern "C"
