// C entry points over the UNMODIFIED Cellerator reference sources, compiled in place.
//
// TEST INFRASTRUCTURE ONLY.  This translation unit includes the reference's own headers
// (found through -I at build time; nothing of the reference is copied into this
// repository) and is linked with the reference's referee.cc / operation.cc /
// operation_signature.cc.  The resulting library, oracle/_ref/libcellerator_ref.so, is what
// the C restatement in oracle.c is validated against, and it can serve as the CPU baseline.
//
// The reference's quantized CSR uses `int` row pointers; the entry points here take the
// int64 arrays that the rest of this repository uses and narrow them (the caller keeps
// nnz below 2^31 on this path).
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

// make_operation_signature of the request used by tests/math_operation_contract_test.cc is
// checked by the reference's own test; here only the digest helper is exported.
void ref_digest_f32(const float *values, std::uint64_t rows, std::uint64_t columns, std::uint64_t ld,
                    std::uint64_t out[2]) {
    const cm::logical_dense_view view{values, rows, columns, ld, cm::dense_layout_kind::row_major,
                                      static_cast<cm::u32>(::cellerator::real::value_f32)};
    cm::determinism_digest d;
    cm::digest_logical_dense(view, &d);
    out[0] = d.low;
    out[1] = d.high;
}

} // extern "C"
