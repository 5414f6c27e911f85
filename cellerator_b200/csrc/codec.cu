// Device codec of the quantized CSR layout: quantise a float-per-entry array into packed
// codes and decode it back.
//
// Reference counterpart: portable_backend::launch_quantize_block / launch_dequantize_block
// (include/Cellerator/quantized/portable_backend.cuh:23-61), whose kernels give each THREAD a
// row (portable_quantize_kernel.cuh:7-19, portable_dequantize_kernel.cuh:7-19) and run
// pack_row_values / unpack_row_values (packing.cuh:13-260).  Here each WARP takes a row so
// that loads of genes, values and codes are coalesced; the byte layout is the same: code i of
// a row sits in byte i/cpb of the row at bit shift (i mod cpb)*bits, unused lanes of the last
// byte are 0.
//
// Rounding follows the reference's HOST rule (access.cuh:104-131): true IEEE division, round
// half away from zero, clamp.  The decode is a rounded product followed by a rounded sum
// (numeric.cuh:34-36 as compiled for a host without FMA contraction), so decoded floats are
// bit-identical to the host codec as well.
#include "kernels.cuh"

namespace cb200 {
namespace {

struct codec_params {
    const std::int64_t *row_ptr;
    const std::int64_t *packed_row_ptr;
    const std::int32_t *col_idx;
    std::uint8_t *packed;
    const float *scales;
    const float *offsets;
    float *values;
    std::int64_t row_begin, row_end;
    int policy;
};

template<int BITS>
__device__ __forceinline__ unsigned quantize_one(float value, float scale, float offset) {
    constexpr int max_code = (1 << BITS) - 1;
    if (scale == 0.0f) return 0u;
    const float q = __fdiv_rn(__fsub_rn(value, offset), scale);
    const float shifted = q >= 0.0f ? __fadd_rn(q, 0.5f) : __fsub_rn(q, 0.5f);
    // A float -> int conversion that overflows (or a NaN) is undefined in the host codec; on the
    // x86-64 hosts it runs on the conversion yields INT_MIN, which the rule then maps to code 0.
    // The device conversion would saturate to INT_MAX instead, so that case is decided here.
    if (!(shifted < 2147483648.0f)) return 0u;
    int rounded = static_cast<int>(shifted);
    if (rounded < 0) return 0u;
    if (rounded > max_code) rounded = max_code;
    return static_cast<unsigned>(rounded);
}

template<int BITS>
__global__ void __launch_bounds__(256) quantize_rows_kernel(const codec_params p) {
    constexpr int CPB = 8 / BITS;
    const int lane = threadIdx.x & 31;
    const std::int64_t row = p.row_begin + (static_cast<std::int64_t>(blockIdx.x) * (blockDim.x >> 5)) + (threadIdx.x >> 5);
    if (row >= p.row_end) return;
    const std::int64_t begin = __ldg(p.row_ptr + row);
    const std::int64_t end = __ldg(p.row_ptr + row + 1);
    const std::int64_t value_base = __ldg(p.row_ptr + p.row_begin);
    std::uint8_t *out = p.packed + (p.packed_row_ptr != nullptr ? __ldg(p.packed_row_ptr + row) : begin);
    const bool row_policy = p.policy == CB200_DECODE_COLUMN_SCALE_ROW_OFFSET;
    const float row_offset = (row_policy && p.offsets != nullptr) ? __ldg(p.offsets + row) : 0.0f;
    const std::int64_t nbytes = (end - begin + CPB - 1) / CPB;
    for (std::int64_t byte = lane; byte < nbytes; byte += 32) {
        unsigned packed = 0u;
#pragma unroll
        for (int slot = 0; slot < CPB; ++slot) {
            const std::int64_t idx = begin + byte * CPB + slot;
            if (idx < end) {
                const int gene = __ldg(p.col_idx + idx);
                const float scale = p.scales != nullptr ? __ldg(p.scales + gene) : 1.0f;
                const float offset = row_policy ? row_offset : (p.offsets != nullptr ? __ldg(p.offsets + gene) : 0.0f);
                packed |= quantize_one<BITS>(p.values[idx - value_base], scale, offset) << (slot * BITS);
            }
        }
        out[byte] = static_cast<std::uint8_t>(packed);
    }
}

template<int BITS>
__global__ void __launch_bounds__(256) dequantize_rows_kernel(const codec_params p) {
    constexpr int CPB = 8 / BITS;
    constexpr unsigned MASK = (1u << BITS) - 1u;
    const int lane = threadIdx.x & 31;
    const std::int64_t row = p.row_begin + (static_cast<std::int64_t>(blockIdx.x) * (blockDim.x >> 5)) + (threadIdx.x >> 5);
    if (row >= p.row_end) return;
    const std::int64_t begin = __ldg(p.row_ptr + row);
    const std::int64_t end = __ldg(p.row_ptr + row + 1);
    const std::int64_t value_base = __ldg(p.row_ptr + p.row_begin);
    const std::uint8_t *in = p.packed + (p.packed_row_ptr != nullptr ? __ldg(p.packed_row_ptr + row) : begin);
    const bool row_policy = p.policy == CB200_DECODE_COLUMN_SCALE_ROW_OFFSET;
    const float row_offset = (row_policy && p.offsets != nullptr) ? __ldg(p.offsets + row) : 0.0f;
    for (std::int64_t idx = begin + lane; idx < end; idx += 32) {
        const std::int64_t local = idx - begin;
        const unsigned byte = in[local / CPB];
        const unsigned code = (byte >> (static_cast<int>(local % CPB) * BITS)) & MASK;
        const int gene = __ldg(p.col_idx + idx);
        const float scale = p.scales != nullptr ? __ldg(p.scales + gene) : 1.0f;
        const float offset = row_policy ? row_offset : (p.offsets != nullptr ? __ldg(p.offsets + gene) : 0.0f);
        p.values[idx - value_base] = __fadd_rn(__fmul_rn(static_cast<float>(code), scale), offset);
    }
}

cb200_status check(const qcsr_view &x, std::int64_t row_begin, std::int64_t row_end, const void *values) {
    if (x.row_ptr == nullptr || x.col_idx == nullptr || x.packed == nullptr || values == nullptr)
        return fail(CB200_STATUS_INVALID_ARGUMENT, "codec needs row_ptr, col_idx, packed_values and values");
    if (row_begin < 0 || row_end > x.rows || row_begin > row_end)
        return fail(CB200_STATUS_INVALID_SHAPE, "row range [%lld,%lld) outside 0..%lld", (long long)row_begin,
                    (long long)row_end, (long long)x.rows);
    if (x.bits != 8 && x.packed_row_ptr == nullptr)
        return fail(CB200_STATUS_INVALID_ARGUMENT, "sub-byte codes need packed_row_ptr");
    return CB200_STATUS_SUCCESS;
}

codec_params make_params(const qcsr_view &x, std::int64_t row_begin, std::int64_t row_end, float *values) {
    codec_params p{};
    p.row_ptr = x.row_ptr; p.packed_row_ptr = x.packed_row_ptr; p.col_idx = x.col_idx;
    p.packed = const_cast<std::uint8_t *>(x.packed); p.scales = x.scales; p.offsets = x.offsets;
    p.values = values; p.row_begin = row_begin; p.row_end = row_end; p.policy = x.policy;
    return p;
}


// ---- Blocked-ELL codec (blocked_ell.cuh:120-231): one warp per row, lane = packed byte ------

struct bell_codec_params {
    std::int64_t rows, cols;
    int block_size, ell_cols, width;
    std::int64_t row_stride;
    const std::uint32_t *block_col_idx;
    std::uint8_t *packed;
    const float *scales;
    const float *offsets;
    float *values;
    std::int64_t row_begin, row_end;
    int policy;
};

// gene of slot `slot` of a row in block row `row_block`, -1 for an empty block
__device__ __forceinline__ std::int64_t bell_gene(const bell_codec_params &p, std::int64_t row_block, int slot) {
    const std::uint32_t bc = __ldg(p.block_col_idx + row_block * p.width + slot / p.block_size);
    if (bc == 0xffffffffu) return -1;
    return static_cast<std::int64_t>(bc) * p.block_size + slot % p.block_size;
}

template<int BITS>
__global__ void __launch_bounds__(256) bell_quantize_kernel(const bell_codec_params p) {
    constexpr int CPB = 8 / BITS;
    const int lane = threadIdx.x & 31;
    const std::int64_t row = p.row_begin + (static_cast<std::int64_t>(blockIdx.x) * (blockDim.x >> 5)) + (threadIdx.x >> 5);
    if (row >= p.row_end) return;
    std::uint8_t *out = p.packed + row * p.row_stride;
    const float *in = p.values + (row - p.row_begin) * p.ell_cols;
    const std::int64_t row_block = row / p.block_size;
    const bool row_policy = p.policy == CB200_DECODE_COLUMN_SCALE_ROW_OFFSET;
    const float row_offset = (row_policy && p.offsets != nullptr) ? __ldg(p.offsets + row) : 0.0f;
    const int used = (p.ell_cols + CPB - 1) / CPB;
    for (std::int64_t byte = lane; byte < p.row_stride; byte += 32) {
        unsigned packed = 0u;
        if (byte < used) {
#pragma unroll
            for (int slot_in = 0; slot_in < CPB; ++slot_in) {
                const int slot = static_cast<int>(byte) * CPB + slot_in;
                if (slot < p.ell_cols) {
                    const std::int64_t gene = bell_gene(p, row_block, slot);
                    const std::int64_t safe = (gene >= 0 && gene < p.cols) ? gene : 0; // never index past cols
                    const float scale = p.scales != nullptr ? __ldg(p.scales + safe) : 1.0f;
                    const float offset = row_policy ? row_offset : (p.offsets != nullptr ? __ldg(p.offsets + safe) : 0.0f);
                    packed |= quantize_one<BITS>(in[slot], scale, offset) << (slot_in * BITS);
                }
            }
        }
        out[byte] = static_cast<std::uint8_t>(packed);
    }
}

template<int BITS>
__global__ void __launch_bounds__(256) bell_dequantize_kernel(const bell_codec_params p) {
    constexpr int CPB = 8 / BITS;
    constexpr unsigned MASK = (1u << BITS) - 1u;
    const int lane = threadIdx.x & 31;
    const std::int64_t row = p.row_begin + (static_cast<std::int64_t>(blockIdx.x) * (blockDim.x >> 5)) + (threadIdx.x >> 5);
    if (row >= p.row_end) return;
    const std::uint8_t *in = p.packed + row * p.row_stride;
    float *out = p.values + (row - p.row_begin) * p.ell_cols;
    const std::int64_t row_block = row / p.block_size;
    const bool row_policy = p.policy == CB200_DECODE_COLUMN_SCALE_ROW_OFFSET;
    const float row_offset = (row_policy && p.offsets != nullptr) ? __ldg(p.offsets + row) : 0.0f;
    for (int slot = lane; slot < p.ell_cols; slot += 32) {
        const std::int64_t gene = bell_gene(p, row_block, slot);
        float v = 0.0f;
        if (gene >= 0 && gene < p.cols) {
            const unsigned code = (static_cast<unsigned>(in[slot / CPB]) >> ((slot % CPB) * BITS)) & MASK;
            const float scale = p.scales != nullptr ? __ldg(p.scales + gene) : 1.0f;
            const float offset = row_policy ? row_offset : (p.offsets != nullptr ? __ldg(p.offsets + gene) : 0.0f);
            v = __fadd_rn(__fmul_rn(static_cast<float>(code), scale), offset);
        }
        out[slot] = v;
    }
}

cb200_status bell_check(const qbell_view &x, std::int64_t row_begin, std::int64_t row_end, const void *values) {
    if (x.block_col_idx == nullptr || x.packed == nullptr || values == nullptr)
        return fail(CB200_STATUS_INVALID_ARGUMENT, "Blocked-ELL codec needs block_col_idx, packed_values and values");
    if (x.block_size <= 0 || x.ell_cols < 0 || x.ell_cols % x.block_size != 0)
        return fail(CB200_STATUS_INVALID_SHAPE, "ell_cols must be a multiple of block_size");
    if (row_begin < 0 || row_end > x.rows || row_begin > row_end)
        return fail(CB200_STATUS_INVALID_SHAPE, "row range outside the matrix");
    const std::int64_t need = (static_cast<std::int64_t>(x.ell_cols) * x.bits + 7) / 8;
    if (x.row_stride_bytes < need) return fail(CB200_STATUS_INVALID_SHAPE, "row_stride_bytes smaller than a packed row");
    return CB200_STATUS_SUCCESS;
}

bell_codec_params bell_params_of(const qbell_view &x, std::int64_t row_begin, std::int64_t row_end, float *values) {
    bell_codec_params p{};
    p.rows = x.rows; p.cols = x.cols; p.block_size = x.block_size; p.ell_cols = x.ell_cols;
    p.width = x.ell_cols / x.block_size; p.row_stride = x.row_stride_bytes; p.block_col_idx = x.block_col_idx;
    p.packed = const_cast<std::uint8_t *>(x.packed); p.scales = x.scales; p.offsets = x.offsets; p.values = values;
    p.row_begin = row_begin; p.row_end = row_end; p.policy = x.policy;
    return p;
}

} // namespace

cb200_status launch_qbell_quantize_rows(const qbell_view &x, std::int64_t row_begin, std::int64_t row_end,
                                        const float *values_by_slot, cudaStream_t stream) {
    const cb200_status ok = bell_check(x, row_begin, row_end, values_by_slot);
    if (ok != CB200_STATUS_SUCCESS) return ok;
    if (row_end == row_begin) return CB200_STATUS_SUCCESS;
    const bell_codec_params p = bell_params_of(x, row_begin, row_end, const_cast<float *>(values_by_slot));
    const unsigned grid = static_cast<unsigned>((row_end - row_begin + 7) / 8);
    switch (x.bits) {
    case 8: bell_quantize_kernel<8><<<grid, 256, 0, stream>>>(p); break;
    case 4: bell_quantize_kernel<4><<<grid, 256, 0, stream>>>(p); break;
    case 2: bell_quantize_kernel<2><<<grid, 256, 0, stream>>>(p); break;
    case 1: bell_quantize_kernel<1><<<grid, 256, 0, stream>>>(p); break;
    default: return fail(CB200_STATUS_UNSUPPORTED, "bits must be 1, 2, 4 or 8, got %d", x.bits);
    }
    count_launch();
    CB200_CUDA_OK(cudaGetLastError());
    return CB200_STATUS_SUCCESS;
}

cb200_status launch_qbell_dequantize_rows(const qbell_view &x, std::int64_t row_begin, std::int64_t row_end,
                                          float *values_by_slot, cudaStream_t stream) {
    const cb200_status ok = bell_check(x, row_begin, row_end, values_by_slot);
    if (ok != CB200_STATUS_SUCCESS) return ok;
    if (row_end == row_begin) return CB200_STATUS_SUCCESS;
    const bell_codec_params p = bell_params_of(x, row_begin, row_end, values_by_slot);
    const unsigned grid = static_cast<unsigned>((row_end - row_begin + 7) / 8);
    switch (x.bits) {
    case 8: bell_dequantize_kernel<8><<<grid, 256, 0, stream>>>(p); break;
    case 4: bell_dequantize_kernel<4><<<grid, 256, 0, stream>>>(p); break;
    case 2: bell_dequantize_kernel<2><<<grid, 256, 0, stream>>>(p); break;
    case 1: bell_dequantize_kernel<1><<<grid, 256, 0, stream>>>(p); break;
    default: return fail(CB200_STATUS_UNSUPPORTED, "bits must be 1, 2, 4 or 8, got %d", x.bits);
    }
    count_launch();
    CB200_CUDA_OK(cudaGetLastError());
    return CB200_STATUS_SUCCESS;
}

cb200_status launch_quantize_rows(const qcsr_view &x, std::int64_t row_begin, std::int64_t row_end,
                                  const float *values, cudaStream_t stream) {
    const cb200_status ok = check(x, row_begin, row_end, values);
    if (ok != CB200_STATUS_SUCCESS) return ok;
    if (row_end == row_begin) return CB200_STATUS_SUCCESS;
    const codec_params p = make_params(x, row_begin, row_end, const_cast<float *>(values));
    const unsigned grid = static_cast<unsigned>((row_end - row_begin + 7) / 8);
    switch (x.bits) {
    case 8: quantize_rows_kernel<8><<<grid, 256, 0, stream>>>(p); break;
    case 4: quantize_rows_kernel<4><<<grid, 256, 0, stream>>>(p); break;
    case 2: quantize_rows_kernel<2><<<grid, 256, 0, stream>>>(p); break;
    case 1: quantize_rows_kernel<1><<<grid, 256, 0, stream>>>(p); break;
    default: return fail(CB200_STATUS_UNSUPPORTED, "bits must be 1, 2, 4 or 8, got %d", x.bits);
    }
    count_launch();
    CB200_CUDA_OK(cudaGetLastError());
    return CB200_STATUS_SUCCESS;
}

cb200_status launch_dequantize_rows(const qcsr_view &x, std::int64_t row_begin, std::int64_t row_end,
                                    float *values, cudaStream_t stream) {
    const cb200_status ok = check(x, row_begin, row_end, values);
    if (ok != CB200_STATUS_SUCCESS) return ok;
    if (row_end == row_begin) return CB200_STATUS_SUCCESS;
    const codec_params p = make_params(x, row_begin, row_end, values);
    const unsigned grid = static_cast<unsigned>((row_end - row_begin + 7) / 8);
    switch (x.bits) {
    case 8: dequantize_rows_kernel<8><<<grid, 256, 0, stream>>>(p); break;
    case 4: dequantize_rows_kernel<4><<<grid, 256, 0, stream>>>(p); break;
    case 2: dequantize_rows_kernel<2><<<grid, 256, 0, stream>>>(p); break;
    case 1: dequantize_rows_kernel<1><<<grid, 256, 0, stream>>>(p); break;
    default: return fail(CB200_STATUS_UNSUPPORTED, "bits must be 1, 2, 4 or 8, got %d", x.bits);
    }
    count_launch();
    CB200_CUDA_OK(cudaGetLastError());
    return CB200_STATUS_SUCCESS;
}

} // namespace cb200
