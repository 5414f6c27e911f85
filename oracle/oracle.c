/*
 * CPU oracle for the quantized sparse-matrix path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the algorithms of the Cellerator reference
 * for: the quantized CSR codec, the uniform row partition, the quantized
 * Blocked-ELL codec, and the double-precision SpMM referee.  It exists so that
 * the CUDA kernels of this repository can be checked against something that
 * does not share any code with them.  Only the test-suite, the smoke check and
 * the CPU-baseline leg of the benchmark may call it; no product code path may
 * link or load it.
 *
 * Pinning: every function here is compared, on random and hand-written inputs,
 * with the reference's own sources compiled in place (see Makefile target `ref` and
 * ref_shim.cc) and with the known-answer vectors that the reference's tests
 * hold (tests/golden/).  Each function cites the reference file:line whose
 * behaviour it follows (paths are relative to the Cellerator project root).
 *
 * Index widths: row pointers are int64 and column indices int32 (the widths of
 * the referee's logical CSR view widened to signed), instead of the `int`
 * fields of quantized/layout.cuh; the arithmetic is otherwise the same.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_API __attribute__((visibility("default")))

enum { ORC_POLICY_PER_GENE_AFFINE = 1, ORC_POLICY_COLUMN_SCALE_ROW_OFFSET = 2 };

/* ------------------------------------------------------------------------ */
/* format: include/Cellerator/quantized/format.cuh:14-55                    */

static int orc_valid_bits(int bits) { return bits == 1 || bits == 2 || bits == 4 || bits == 8; }

/* format.cuh:25-27  bytes of one packed row = ceil(nnz / codes_per_byte) */
ORC_API int64_t orc_row_bytes(int bits, int64_t row_nnz) {
    const int64_t cpb = 8 / bits;
    return row_nnz <= 0 ? 0 : (row_nnz + cpb - 1) / cpb;
}

/* format.cuh:29-37  row bytes rounded up to `alignment` (BELL row stride) */
ORC_API int64_t orc_aligned_row_bytes(int bits, int64_t row_nnz, int64_t alignment) {
    const int64_t bytes = orc_row_bytes(bits, row_nnz);
    return alignment <= 1 ? bytes : ((bytes + alignment - 1) / alignment) * alignment;
}

/* format.cuh:39-48  code i lives in byte i / cpb at bit shift (i mod cpb) * bits */
static unsigned orc_unpack_code(int bits, const uint8_t *packed, int64_t local_index) {
    const int64_t cpb = 8 / bits;
    const int64_t slot = local_index / cpb;
    const int lane = (int)(local_index & (cpb - 1));
    return ((unsigned)packed[slot] >> (lane * bits)) & ((1u << bits) - 1u);
}

/* ------------------------------------------------------------------------ */
/* layout: include/Cellerator/quantized/layout.cuh:106-157                  */

/* layout.cuh:111-129  exclusive prefix sum of row_bytes; returns total or -1 */
ORC_API int64_t orc_build_packed_row_ptr(int bits, const int64_t *row_ptr, int64_t rows,
                                         int64_t *packed_row_ptr) {
    if (row_ptr == NULL || packed_row_ptr == NULL || rows < 0 || !orc_valid_bits(bits)) return -1;
    packed_row_ptr[0] = 0;
    for (int64_t r = 0; r < rows; ++r)
        packed_row_ptr[r + 1] = packed_row_ptr[r] + orc_row_bytes(bits, row_ptr[r + 1] - row_ptr[r]);
    return packed_row_ptr[rows];
}

/* layout.cuh:131-136 */
ORC_API int64_t orc_block_count_for_rows(int64_t rows, int64_t rows_per_block) {
    if (rows <= 0 || rows_per_block <= 0) return 0;
    return (rows + rows_per_block - 1) / rows_per_block;
}

/* layout.cuh:138-157  block b starts at min(b * rows_per_block, rows) */
ORC_API int64_t orc_build_uniform_block_row_ptr(int64_t rows, int64_t rows_per_block,
                                                int64_t *block_row_ptr) {
    const int64_t count = orc_block_count_for_rows(rows, rows_per_block);
    if (block_row_ptr == NULL || rows < 0 || rows_per_block <= 0) return -1;
    int64_t row = 0;
    for (int64_t b = 0; b < count; ++b) {
        block_row_ptr[b] = row;
        row += rows_per_block;
        if (row > rows) row = rows;
    }
    block_row_ptr[count] = rows;
    return count;
}

/* access.cuh:7-44  out = {block_index,row_begin,row_end,nnz_begin,nnz_end,packed_begin,packed_end};
 * no block metadata -> one block over the matrix; out-of-range index -> all-zero block. */
ORC_API void orc_get_block(int64_t rows, const int64_t *row_ptr, const int64_t *packed_row_ptr,
                           const int64_t *block_row_ptr, int64_t block_count, int64_t block_index,
                           int64_t out[7]) {
    out[0] = block_index;
    for (int i = 1; i < 7; ++i) out[i] = 0;
    if (row_ptr == NULL || packed_row_ptr == NULL) return;
    if (block_row_ptr == NULL || block_count <= 0) {
        out[0] = 0;
        out[1] = 0;
        out[2] = rows;
    } else {
        if (block_index < 0 || block_index >= block_count) return;
        out[1] = block_row_ptr[block_index];
        out[2] = block_row_ptr[block_index + 1];
    }
    out[3] = row_ptr[out[1]];
    out[4] = row_ptr[out[2]];
    out[5] = packed_row_ptr[out[1]];
    out[6] = packed_row_ptr[out[2]];
}

/* ------------------------------------------------------------------------ */
/* code <-> value: include/Cellerator/quantized/access.cuh:81-131           */

/* access.cuh:104-131  scale==0 -> 0; true division; round half away from zero; clamp.
 * When q +- 0.5 does not fit an int (or is NaN) the reference's conversion is undefined
 * behaviour; on the x86-64 hosts it runs on the result is INT_MIN, hence code 0, and that is
 * what this restatement, compiled for the same hosts, returns too. */
ORC_API unsigned orc_quantize_code(int bits, float value, float scale, float offset) {
    const int max_code = (1 << bits) - 1;
    const float centered = value - offset;
    if (scale == 0.0f) return 0u;
    const float q = centered / scale;
    const float shifted = q >= 0.0f ? q + 0.5f : q - 0.5f;
    if (!(shifted < 2147483648.0f)) return 0u; /* the INT_MIN case, made explicit */
    int rounded = (int)shifted;
    if (rounded < 0) return 0u;
    if (rounded > max_code) rounded = max_code;
    return (unsigned)rounded;
}

/* access.cuh:81-91 with numeric.cuh:34-36: float(code) * scale + offset, written as a
 * product then a sum.  Kept unfused here (volatile) so the result does not depend on
 * whether this file is built with FMA contraction; a fused device build may differ by
 * one ulp, the integer code never does. */
ORC_API float orc_dequantize_code(unsigned code, float scale, float offset) {
    volatile float product = (float)code * scale;
    return product + offset;
}

/* metadata.cuh:17-27,42-55  null scale array -> 1, null offset array -> 0; the row policy
 * reads its offset from row_offsets[row] */
static float orc_scale_for(const float *scales, int64_t column) {
    return scales != NULL ? scales[column] : 1.0f;
}
static float orc_offset_for(int policy, const float *offsets, int64_t row, int64_t column) {
    if (offsets == NULL) return 0.0f;
    return policy == ORC_POLICY_COLUMN_SCALE_ROW_OFFSET ? offsets[row] : offsets[column];
}

/* ------------------------------------------------------------------------ */
/* CSR pack / unpack: include/Cellerator/quantized/packing.cuh:13-328       */

/* packing.cuh:13-146,262-277  The reference's 8-bit path peels a head, writes 16 codes at a
 * time, then 4, then a tail; all of those store code i of the row at byte i, so the layout
 * is the single loop below.  Sub-byte rows fill each byte low lane first and leave the
 * lanes past the row end at 0.  `value_base` is the nnz index of values[0] (packing.cuh:17-18). */
ORC_API int orc_pack_csr_rows(int bits, int policy, int64_t row_begin, int64_t row_end,
                              const int64_t *row_ptr, const int64_t *packed_row_ptr,
                              const int32_t *col_idx, const float *scales, const float *offsets,
                              int64_t value_base, const float *values, uint8_t *packed_values) {
    if (!orc_valid_bits(bits) || row_ptr == NULL || packed_row_ptr == NULL || packed_values == NULL ||
        values == NULL)
        return -1;
    const int cpb = 8 / bits;
    const unsigned mask = (1u << bits) - 1u;
    for (int64_t row = row_begin; row < row_end; ++row) {
        int64_t index = row_ptr[row];
        const int64_t end = row_ptr[row + 1];
        uint8_t *out = packed_values + packed_row_ptr[row];
        while (index < end) {
            unsigned packed_byte = 0u;
            for (int lane = 0; lane < cpb; ++lane) {
                const int64_t current = index + lane;
                if (current < end) {
                    const int64_t column = col_idx[current];
                    const unsigned code = orc_quantize_code(
                        bits, values[current - value_base], orc_scale_for(scales, column),
                        orc_offset_for(policy, offsets, row, column));
                    packed_byte |= (code & mask) << (lane * bits);
                }
            }
            *out++ = (uint8_t)(packed_byte & 0xffu);
            index += cpb;
        }
    }
    return 0;
}

/* packing.cuh:148-260,279-292 */
ORC_API int orc_unpack_csr_rows(int bits, int policy, int64_t row_begin, int64_t row_end,
                                const int64_t *row_ptr, const int64_t *packed_row_ptr,
                                const int32_t *col_idx, const float *scales, const float *offsets,
                                const uint8_t *packed_values, int64_t value_base, float *values) {
    if (!orc_valid_bits(bits) || row_ptr == NULL || packed_row_ptr == NULL || values == NULL) return -1;
    for (int64_t row = row_begin; row < row_end; ++row) {
        const int64_t begin = row_ptr[row];
        const int64_t end = row_ptr[row + 1];
        const uint8_t *in = packed_values + packed_row_ptr[row];
        for (int64_t index = begin; index < end; ++index) {
            const int64_t column = col_idx[index];
            const unsigned code = orc_unpack_code(bits, in, index - begin);
            values[index - value_base] = orc_dequantize_code(
                code, orc_scale_for(scales, column), orc_offset_for(policy, offsets, row, column));
        }
    }
    return 0;
}

/* The integer half of unpack on its own: codes[i] for every nnz (format.cuh:39-48). */
ORC_API int orc_extract_csr_codes(int bits, int64_t rows, const int64_t *row_ptr,
                                  const int64_t *packed_row_ptr, const uint8_t *packed_values,
                                  uint8_t *codes) {
    if (!orc_valid_bits(bits) || row_ptr == NULL || packed_row_ptr == NULL || codes == NULL) return -1;
    for (int64_t row = 0; row < rows; ++row) {
        const int64_t begin = row_ptr[row];
        const int64_t end = row_ptr[row + 1];
        for (int64_t index = begin; index < end; ++index)
            codes[index] = (uint8_t)orc_unpack_code(bits, packed_values + packed_row_ptr[row], index - begin);
    }
    return 0;
}

/* ------------------------------------------------------------------------ */
/* Quantized Blocked-ELL: include/Cellerator/quantized/blocked_ell.cuh:99-231 */

#define ORC_INVALID_BLOCK_COL 0xffffffffu

/* blocked_ell.cuh:120-137  slot s of row r -> gene block_col_idx[(r/bs)*width + s/bs]*bs + s%bs,
 * -1 for an empty block or an out-of-range argument */
ORC_API int64_t orc_bell_column_for_slot(int64_t rows, int block_size, int64_t ell_cols,
                                         const uint32_t *block_col_idx, int64_t row, int64_t slot) {
    if (block_col_idx == NULL || row < 0 || row >= rows || slot < 0 || slot >= ell_cols || block_size <= 0)
        return -1;
    const int64_t width = ell_cols / block_size;
    const uint32_t block_col = block_col_idx[(row / block_size) * width + slot / block_size];
    if (block_col == ORC_INVALID_BLOCK_COL) return -1;
    return (int64_t)block_col * block_size + slot % block_size;
}

/* blocked_ell.cuh:165-213  every slot is quantized (an empty block uses column 0's
 * scale/offset); row padding bytes are 0.  One deliberate difference: for a slot of a present
 * block whose gene index is >= cols (ragged last block column) the reference indexes the
 * metadata arrays at that gene, i.e. past `cols`; here such a slot uses gene 0's metadata, so
 * the two agree whenever the caller's arrays repeat gene 0's entry in that padding. */
ORC_API int orc_bell_pack_row_major(int bits, int policy, int64_t rows, int64_t cols, int block_size,
                                    int64_t ell_cols, int64_t row_stride_bytes,
                                    const uint32_t *block_col_idx, const float *scales,
                                    const float *offsets, const float *values_by_slot,
                                    uint8_t *packed_values) {
    if (!orc_valid_bits(bits) || values_by_slot == NULL || packed_values == NULL || rows < 0 || ell_cols < 0 ||
        row_stride_bytes < orc_row_bytes(bits, ell_cols))
        return -1;
    const int cpb = 8 / bits;
    const unsigned mask = (1u << bits) - 1u;
    for (int64_t row = 0; row < rows; ++row) {
        uint8_t *out = packed_values + row * row_stride_bytes;
        int64_t out_byte = 0;
        for (int64_t slot = 0; slot < ell_cols; slot += cpb) {
            unsigned packed = 0u;
            for (int lane = 0; lane < cpb; ++lane) {
                const int64_t current = slot + lane;
                if (current < ell_cols) {
                    const int64_t column =
                        orc_bell_column_for_slot(rows, block_size, ell_cols, block_col_idx, row, current);
                    const int64_t safe_column = (column >= 0 && column < cols) ? column : 0;
                    const unsigned code = orc_quantize_code(
                        bits, values_by_slot[row * ell_cols + current], orc_scale_for(scales, safe_column),
                        orc_offset_for(policy, offsets, row, safe_column));
                    packed |= (code & mask) << (lane * bits);
                }
            }
            out[out_byte++] = (uint8_t)(packed & 0xffu);
        }
        while (out_byte < row_stride_bytes) out[out_byte++] = 0u;
    }
    return 0;
}

/* blocked_ell.cuh:139-163,215-231  a slot of an empty block, or one whose gene is >= cols,
 * decodes to exactly 0 */
ORC_API int orc_bell_unpack_row_major(int bits, int policy, int64_t rows, int64_t cols, int block_size,
                                      int64_t ell_cols, int64_t row_stride_bytes,
                                      const uint32_t *block_col_idx, const float *scales,
                                      const float *offsets, const uint8_t *packed_values,
                                      float *values_by_slot) {
    if (!orc_valid_bits(bits) || values_by_slot == NULL || packed_values == NULL || rows < 0 || ell_cols < 0)
        return -1;
    for (int64_t row = 0; row < rows; ++row) {
        const uint8_t *in = packed_values + row * row_stride_bytes;
        for (int64_t slot = 0; slot < ell_cols; ++slot) {
            const int64_t column = orc_bell_column_for_slot(rows, block_size, ell_cols, block_col_idx, row, slot);
            float v = 0.0f;
            if (column >= 0 && column < cols)
                v = orc_dequantize_code(orc_unpack_code(bits, in, slot), orc_scale_for(scales, column),
                                        orc_offset_for(policy, offsets, row, column));
            values_by_slot[row * ell_cols + slot] = v;
        }
    }
    return 0;
}

/* The slots that the reference's fused kernel multiplies
 * (src/compute/sparse/project/kernels/quantized_blocked_ell_spmm_fwd_kernel_.cuh:18-37): every
 * slot of a present block whose gene is < cols, structurally empty slots included.  Emits them
 * as a CSR (row_offsets uint64, columns uint32, values float) for the referee below.
 * Returns the number of entries, or -1.  Pass columns/values NULL to count only. */
ORC_API int64_t orc_bell_to_csr(int bits, int policy, int64_t rows, int64_t cols, int block_size,
                                int64_t ell_cols, int64_t row_stride_bytes, const uint32_t *block_col_idx,
                                const float *scales, const float *offsets, const uint8_t *packed_values,
                                uint64_t *row_offsets, uint32_t *columns, float *values) {
    if (!orc_valid_bits(bits) || block_col_idx == NULL || packed_values == NULL || row_offsets == NULL ||
        block_size <= 0)
        return -1;
    const int64_t width = ell_cols / block_size;
    uint64_t count = 0;
    row_offsets[0] = 0;
    for (int64_t row = 0; row < rows; ++row) {
        const uint8_t *in = packed_values + row * row_stride_bytes;
        for (int64_t sb = 0; sb < width; ++sb) {
            const uint32_t block_col = block_col_idx[(row / block_size) * width + sb];
            if (block_col == ORC_INVALID_BLOCK_COL) continue;
            for (int c = 0; c < block_size; ++c) {
                const int64_t gene = (int64_t)block_col * block_size + c;
                if (gene >= cols) break;
                if (columns != NULL && values != NULL) {
                    columns[count] = (uint32_t)gene;
                    values[count] = orc_dequantize_code(orc_unpack_code(bits, in, sb * block_size + c),
                                                        orc_scale_for(scales, gene),
                                                        orc_offset_for(policy, offsets, row, gene));
                }
                ++count;
            }
        }
        row_offsets[row + 1] = count;
    }
    return (int64_t)count;
}

/* ------------------------------------------------------------------------ */
/* SpMM referee: src/compute/math/referee.cc:101-253                        */

enum {
    ORC_EPI_NONE = 0, ORC_EPI_BIAS = 1, ORC_EPI_RELU = 2, ORC_EPI_GELU_ERF = 3, ORC_EPI_GELU_TANH = 4,
    ORC_EPI_BIAS_RELU = 5, ORC_EPI_BIAS_GELU_ERF = 6, ORC_EPI_BIAS_GELU_TANH = 7
};

static int orc_bias_epilogue(int kind) {
    return kind == ORC_EPI_BIAS || kind == ORC_EPI_BIAS_RELU || kind == ORC_EPI_BIAS_GELU_ERF ||
           kind == ORC_EPI_BIAS_GELU_TANH;
}

/* referee.cc:81-97 */
static double orc_apply_epilogue(double value, double bias, int kind) {
    if (orc_bias_epilogue(kind)) value += bias;
    if (kind == ORC_EPI_RELU || kind == ORC_EPI_BIAS_RELU) return fmax(value, 0.0);
    if (kind == ORC_EPI_GELU_ERF || kind == ORC_EPI_BIAS_GELU_ERF)
        return 0.5 * value * (1.0 + erf(value * 0.7071067811865475244));
    if (kind == ORC_EPI_GELU_TANH || kind == ORC_EPI_BIAS_GELU_TANH)
        return 0.5 * value * (1.0 + tanh(0.7978845608028653559 * (value + 0.044715 * value * value * value)));
    return value;
}

/* referee.cc:57-61  row-major: r*ld + c, column-major: c*ld + r */
static uint64_t orc_dense_index(int col_major, uint64_t ld, uint64_t r, uint64_t c) {
    return col_major ? c * ld + r : r * ld + c;
}

/*
 * referee.cc:101-253, for fp32 sparse values, fp32 dense operand and fp32 initial output.
 *   m,k,n         logical dims after the declared transposes (operation.hh:132-134)
 *   transpose_sparse  0: stored CSR is m x k;  1: stored CSR is k x m and Xt is applied
 *   transpose_dense   0: rhs is k x n;         1: rhs is n x k
 *   reference     m*n doubles, row-major
 * The accumulation order (stored row, entry, output column) and the product order
 * alpha * a * b, all in double, are the reference's.  Returns 0, or the referee_status_code
 * (referee.hh:16-27) of the first check that fails.
 */
ORC_API int orc_spmm_reference(uint64_t m, uint64_t k, uint64_t n, int transpose_sparse, int transpose_dense,
                               uint64_t sparse_nnz, const uint64_t *row_offsets, const uint32_t *column_indices,
                               const float *sparse_values, const float *rhs, int rhs_col_major, uint64_t rhs_ld,
                               double alpha, double beta, const float *initial, int initial_col_major,
                               uint64_t initial_ld, int epilogue, const float *bias, double *reference,
                               uint64_t reference_capacity) {
    const uint64_t out_count = m * n;
    if (out_count > reference_capacity || (out_count != 0 && reference == NULL)) return 4;
    const uint64_t sparse_rows = transpose_sparse ? k : m;
    const uint64_t sparse_cols = transpose_sparse ? m : k;
    if ((sparse_rows != 0 && row_offsets == NULL) ||
        (sparse_nnz != 0 && (column_indices == NULL || sparse_values == NULL)))
        return 2;
    if (sparse_rows != 0 && (row_offsets[0] != 0 || row_offsets[sparse_rows] != sparse_nnz)) return 2;
    if (beta != 0.0 && initial == NULL) return 2;
    if (orc_bias_epilogue(epilogue) && bias == NULL) return 1;

    for (uint64_t r = 0; r < m; ++r)
        for (uint64_t c = 0; c < n; ++c) {
            double init = 0.0;
            if (beta != 0.0) init = (double)initial[orc_dense_index(initial_col_major, initial_ld, r, c)];
            reference[r * n + c] = beta * init;
        }

    for (uint64_t prow = 0; prow < sparse_rows; ++prow) {
        const uint64_t begin = row_offsets[prow];
        const uint64_t end = row_offsets[prow + 1];
        if (begin > end || end > sparse_nnz) return 2;
        for (uint64_t e = begin; e < end; ++e) {
            const uint64_t pcol = column_indices[e];
            if (pcol >= sparse_cols) return 2;
            const uint64_t out_row = transpose_sparse ? pcol : prow;
            const uint64_t reduction = transpose_sparse ? prow : pcol;
            const double a = (double)sparse_values[e];
            for (uint64_t c = 0; c < n; ++c) {
                const uint64_t rr = transpose_dense ? c : reduction;
                const uint64_t rc = transpose_dense ? reduction : c;
                const double b = (double)rhs[orc_dense_index(rhs_col_major, rhs_ld, rr, rc)];
                reference[out_row * n + c] += alpha * a * b;
            }
        }
    }

    for (uint64_t r = 0; r < m; ++r)
        for (uint64_t c = 0; c < n; ++c) {
            const double b = orc_bias_epilogue(epilogue) ? (double)bias[c] : 0.0;
            double *v = &reference[r * n + c];
            *v = orc_apply_epilogue(*v, b, epilogue);
            if (!isfinite(*v)) return 5;
        }
    return 0;
}

/*
 * The composed CPU path the benchmark times as the CPU baseline: decode (packing.cuh:279-292) then the referee,
 * forward only, on the row range [row_begin, row_end) of a quantized CSR with int64 row
 * pointers.  Offsets are rebased so the referee sees row_offsets[0] == 0
 * (referee.cc:143-148).  `scratch_values` holds the decoded floats (nnz of the range),
 * `scratch_offsets` row_end-row_begin+1 uint64.  Y rows land in `reference` (double).
 */
ORC_API int orc_qcsr_forward_rows(int bits, int policy, int64_t row_begin, int64_t row_end, int64_t cols,
                                  int64_t n, const int64_t *row_ptr, const int64_t *packed_row_ptr,
                                  const int32_t *col_idx, const uint8_t *packed_values, const float *scales,
                                  const float *offsets, const float *w, int64_t w_ld, float *scratch_values,
                                  uint64_t *scratch_offsets, double *reference) {
    const int64_t rows = row_end - row_begin;
    const int64_t base = row_ptr[row_begin];
    int rc = orc_unpack_csr_rows(bits, policy, row_begin, row_end, row_ptr, packed_row_ptr, col_idx, scales,
                                 offsets, packed_values, base, scratch_values);
    if (rc != 0) return rc;
    for (int64_t r = 0; r <= rows; ++r) scratch_offsets[r] = (uint64_t)(row_ptr[row_begin + r] - base);
    return orc_spmm_reference((uint64_t)rows, (uint64_t)cols, (uint64_t)n, 0, 0, scratch_offsets[rows],
                              scratch_offsets, (const uint32_t *)(col_idx + base), scratch_values, w, 0,
                              (uint64_t)w_ld, 1.0, 0.0, NULL, 0, 0, ORC_EPI_NONE, NULL, reference,
                              (uint64_t)(rows * n));
}

/* Same for the gene-side transpose G' = deq(X)^T G over a row range: `reference` is cols*n
 * doubles and receives this range's partial sum (transpose_sparse, referee.cc:130-133,207-210). */
ORC_API int orc_qcsr_transpose_rows(int bits, int policy, int64_t row_begin, int64_t row_end, int64_t cols,
                                    int64_t n, const int64_t *row_ptr, const int64_t *packed_row_ptr,
                                    const int32_t *col_idx, const uint8_t *packed_values, const float *scales,
                                    const float *offsets, const float *g, int64_t g_ld, float *scratch_values,
                                    uint64_t *scratch_offsets, double *reference) {
    const int64_t rows = row_end - row_begin;
    const int64_t base = row_ptr[row_begin];
    int rc = orc_unpack_csr_rows(bits, policy, row_begin, row_end, row_ptr, packed_row_ptr, col_idx, scales,
                                 offsets, packed_values, base, scratch_values);
    if (rc != 0) return rc;
    for (int64_t r = 0; r <= rows; ++r) scratch_offsets[r] = (uint64_t)(row_ptr[row_begin + r] - base);
    /* stored CSR is rows x cols = k x m with m = cols, k = rows */
    return orc_spmm_reference((uint64_t)cols, (uint64_t)rows, (uint64_t)n, 1, 0, scratch_offsets[rows],
                              scratch_offsets, (const uint32_t *)(col_idx + base), scratch_values,
                              g + row_begin * g_ld, 0, (uint64_t)g_ld, 1.0, 0.0, NULL, 0, 0, ORC_EPI_NONE, NULL,
                              reference, (uint64_t)(cols * n));
}

/* ------------------------------------------------------------------------ */
/* comparison: include/Cellerator/compute/math/referee.hh:143-217           */

/* out = {max_abs, max_rel, mean_abs, rmse, mismatch_count, worst_index, nonfinite_ref, nonfinite_cand} */
ORC_API int orc_compare(const double *reference, const float *candidate, uint64_t count, double tol_abs,
                        double tol_rel, double rel_floor, double out[8]) {
    if ((count != 0 && (reference == NULL || candidate == NULL)) || tol_abs < 0.0 || tol_rel < 0.0 ||
        rel_floor <= 0.0)
        return 1;
    long double abs_sum = 0.0L, sq_sum = 0.0L;
    double max_abs = 0.0, max_rel = 0.0;
    uint64_t mismatch = 0, worst = 0, nf_ref = 0, nf_cand = 0;
    for (uint64_t i = 0; i < count; ++i) {
        const double expected = reference[i];
        const double actual = (double)candidate[i];
        if (!isfinite(expected)) { ++nf_ref; continue; }
        if (!isfinite(actual)) { ++nf_cand; continue; }
        const double a = fabs(actual - expected);
        const double r = a / fmax(fabs(expected), rel_floor);
        abs_sum += a;
        sq_sum += (long double)a * a;
        if (a > max_abs) { max_abs = a; worst = i; }
        max_rel = fmax(max_rel, r);
        if (a > tol_abs + tol_rel * fabs(expected)) ++mismatch;
    }
    out[0] = max_abs;
    out[1] = max_rel;
    out[2] = count ? (double)(abs_sum / count) : 0.0;
    out[3] = count ? sqrt((double)(sq_sum / count)) : 0.0;
    out[4] = (double)mismatch;
    out[5] = (double)worst;
    out[6] = (double)nf_ref;
    out[7] = (double)nf_cand;
    return nf_ref ? 5 : (nf_cand ? 6 : 0);
}

/* referee.hh:219-244 with :125-130  determinism digest of a row-major fp32 matrix:
 * FNV-style low word, boost-style high word, over rows, columns, type code, then the bit
 * pattern of every value widened to double. */
ORC_API void orc_digest_f32(const float *values, uint64_t rows, uint64_t columns, uint64_t ld,
                            uint32_t type_code, uint64_t out[2]) {
    uint64_t low = 1469598103934665603ull, high = 0x6a09e667f3bcc909ull;
#define ORC_MIX(v)                                                                  \
    do {                                                                            \
        const uint64_t x_ = (v);                                                    \
        low ^= x_;                                                                  \
        low *= 1099511628211ull;                                                    \
        high ^= x_ + 0x9e3779b97f4a7c15ull + (high << 6) + (high >> 2);             \
    } while (0)
    ORC_MIX(rows);
    ORC_MIX(columns);
    ORC_MIX((uint64_t)type_code);
    for (uint64_t r = 0; r < rows; ++r)
        for (uint64_t c = 0; c < columns; ++c) {
            const double d = (double)values[r * ld + c];
            uint64_t bits;
            memcpy(&bits, &d, sizeof bits);
            ORC_MIX(bits);
        }
#undef ORC_MIX
    out[0] = low;
    out[1] = high;
}

/* ---------------------------------------------------------------------------------------------
 * CSR -> physical Blocked-ELL lowering under a row order and a feature (gene) order.
 *
 * Follows query_bell_candidates_host / evaluate (src/compute/math/physical_bell_candidates.cc:131-238,
 * validation :13-52), validate (src/compute/math/physical_bell.cc:27-80) and
 * materialize_bell_candidate_host (physical_bell.cc:98-200) for ONE block size.  The identity hashes
 * of the reference (FNV-1a chains over the arrays) are not part of this restatement: they do not
 * influence geometry, column indices or values.
 *
 * Conventions (physical_bell.cc:44-58): feature_permutation[execution] = canonical,
 * inverse_feature_permutation[canonical] = execution, row_permutation[execution row] = canonical row.
 * Every semantic feature block [fb_offsets[b], fb_offsets[b+1]) of the execution order is padded on
 * its own to a multiple of the block size; a physical block column never spans two semantic blocks.
 *
 * geometry[13]: state, padded_rows, padded_features, block_rows, ell_blocks_per_row, ell_columns,
 *               column_index_count, value_bytes, occupied_blocks, stored_blocks, dense_value_slots,
 *               persistent_bytes, source_bytes.
 * metrics[4]:   scalar_occupancy, ell_slot_utilization, value_slot_expansion, storage_expansion.
 * column_indices == NULL: geometry only.  values_layout 0: block-major, as the reference
 * (values[(block_row * ell_blocks + slot) * bs^2 + row_in_block * bs + column_in_block]); 1: row-major
 * with row_stride_bytes per row (value of execution row r, slot s, column c at
 * r * row_stride_bytes + (s * bs + c) * value_size), the layout of the quantized Blocked-ELL
 * matrices (include/Cellerator/quantized/blocked_ell.cuh:29-47).
 * Returns the reference's bell_lowering_status_code (physical_bell.hh:24-34). */
static uint32_t orc_semantic_block(uint32_t fb_count, const uint32_t *fb_offsets, uint32_t execution) {
    uint32_t first = 0, last = fb_count;
    while (first + 1u < last) {
        const uint32_t middle = first + (last - first) / 2u;
        if (fb_offsets[middle] <= execution) first = middle;
        else last = middle;
    }
    return first;
}

ORC_API int orc_bell_lowering(uint32_t rows, uint32_t features, uint32_t nnz, uint32_t value_size,
                              const uint32_t *row_offsets, const uint32_t *feature_ids, const void *values,
                              uint32_t fb_count, const uint32_t *fb_offsets, const uint32_t *fperm,
                              const uint32_t *finv, const uint32_t *rperm, const uint32_t *rinv, uint32_t bs,
                              double max_value_expansion, double max_storage_expansion, uint64_t max_persistent,
                              uint64_t *geometry, double *metrics, uint32_t *padded_fb_offsets, int32_t *column_indices,
                              void *values_out, uint64_t column_capacity, uint64_t value_capacity, int values_layout,
                              uint64_t row_stride_bytes) {
    enum { OK = 0, INVALID_ARGUMENT = 1, INVALID_SOURCE = 2, INCOMPATIBLE_PLAN = 3, INCOMPATIBLE_ORDER = 4,
           INSUFFICIENT_CAPACITY = 5, CANDIDATE_REJECTED = 6, CANDIDATE_MISMATCH = 7, OVERFLOW_ = 8 };
    if (geometry == NULL || metrics == NULL || !(max_value_expansion > 0.0) || !(max_storage_expansion > 0.0) ||
        isinf(max_value_expansion) || isinf(max_storage_expansion))
        return INVALID_ARGUMENT;
    if (bs != 8u && bs != 16u && bs != 32u) return CANDIDATE_MISMATCH;
    if (features == 0u || fb_count == 0u || fb_offsets == NULL || fperm == NULL || finv == NULL) return INCOMPATIBLE_PLAN;
    if (value_size == 0u || value_size > 16u || row_offsets == NULL || (nnz != 0u && (feature_ids == NULL || values == NULL)))
        return INVALID_SOURCE;
    if (rperm == NULL || rinv == NULL) return INCOMPATIBLE_ORDER;
    if (fb_offsets[0] != 0u || fb_offsets[fb_count] != features) return INCOMPATIBLE_PLAN;
    for (uint32_t b = 0; b < fb_count; ++b)
        if (fb_offsets[b] >= fb_offsets[b + 1u]) return INCOMPATIBLE_PLAN;
    const uint64_t marker_count = rows > features ? rows : features;
    uint32_t *markers = (uint32_t *)calloc(marker_count + 1u, sizeof(uint32_t));
    uint32_t *block_offsets = (uint32_t *)calloc((size_t)fb_count + 1u, sizeof(uint32_t));
    if (markers == NULL || block_offsets == NULL) { free(markers); free(block_offsets); return INSUFFICIENT_CAPACITY; }
    int status = OK;
    for (uint32_t e = 0; e < features && status == OK; ++e) {
        const uint32_t c = fperm[e];
        if (c >= features || markers[c] != 0u || finv[c] != e) status = INCOMPATIBLE_PLAN;
        else markers[c] = 1u;
    }
    memset(markers, 0, (marker_count + 1u) * sizeof(uint32_t));
    for (uint32_t e = 0; e < rows && status == OK; ++e) {
        const uint32_t c = rperm[e];
        if (c >= rows || markers[c] != 0u || rinv[c] != e) status = INCOMPATIBLE_ORDER;
        else markers[c] = 1u;
    }
    if (status == OK && (row_offsets[0] != 0u || row_offsets[rows] != nnz)) status = INVALID_SOURCE;
    for (uint32_t r = 0; r < rows && status == OK; ++r) {
        const uint32_t begin = row_offsets[r], end = row_offsets[r + 1u];
        if (begin > end || end > nnz) { status = INVALID_SOURCE; break; }
        for (uint32_t i = begin; i < end; ++i)
            if (feature_ids[i] >= features || (i != begin && feature_ids[i] <= feature_ids[i - 1u])) { status = INVALID_SOURCE; break; }
    }
    if (status != OK) { free(markers); free(block_offsets); return status; }

    /* physical_bell_candidates.cc:96-110  every semantic block padded independently */
    uint64_t physical_blocks = 0;
    for (uint32_t b = 0; b < fb_count; ++b) {
        const uint64_t width = fb_offsets[b + 1u] - fb_offsets[b];
        physical_blocks += (width + bs - 1u) / bs;
        if (physical_blocks > 0x7fffffffull) { free(markers); free(block_offsets); return OVERFLOW_; }
        block_offsets[b + 1u] = (uint32_t)physical_blocks;
    }
    const uint64_t block_rows = ((uint64_t)rows + bs - 1u) / bs;
    const uint64_t padded_rows = block_rows * bs, padded_features = physical_blocks * bs;
    memset(geometry, 0, 13 * sizeof(uint64_t));
    memset(metrics, 0, 4 * sizeof(double));
    geometry[0] = 5; /* overflow until proven otherwise */
    if (padded_rows > 0xffffffffull || padded_features > 0xffffffffull) { free(markers); free(block_offsets); return OK; }
    uint32_t *epochs = (uint32_t *)calloc((size_t)physical_blocks + 1u, sizeof(uint32_t));
    if (epochs == NULL) { free(markers); free(block_offsets); return INSUFFICIENT_CAPACITY; }
#define ORC_PHYSICAL(execution, out_semantic)                                                        \
    (*(out_semantic) = orc_semantic_block(fb_count, fb_offsets, (execution)),                         \
     block_offsets[*(out_semantic)] + ((execution) - fb_offsets[*(out_semantic)]) / bs)
    /* :146-166  distinct physical blocks per block row; ELL width = their maximum */
    uint32_t maximum = 0;
    uint64_t occupied = 0;
    for (uint64_t br = 0; br < block_rows; ++br) {
        uint32_t active = 0;
        const uint32_t begin = (uint32_t)(br * bs), end = (uint32_t)(begin + bs < rows ? begin + bs : rows);
        for (uint32_t er = begin; er < end; ++er) {
            const uint32_t r = rperm[er];
            for (uint32_t i = row_offsets[r]; i < row_offsets[r + 1u]; ++i) {
                uint32_t semantic;
                const uint32_t p = ORC_PHYSICAL(finv[feature_ids[i]], &semantic);
                if (epochs[p] != (uint32_t)(br + 1u)) { epochs[p] = (uint32_t)(br + 1u); ++active; }
            }
        }
        occupied += active;
        if (active > maximum) maximum = active;
    }
    const uint64_t stored = block_rows * maximum;
    const uint64_t slots = stored * bs * bs;
    const uint64_t bytes = slots * value_size;
    const uint64_t persistent = stored * 4u + bytes + ((uint64_t)fb_count + 1u) * 4u;
    const uint64_t source_bytes = ((uint64_t)rows + 1u) * 4u + (uint64_t)nnz * (4u + value_size);
    geometry[1] = padded_rows; geometry[2] = padded_features; geometry[3] = block_rows; geometry[4] = maximum;
    geometry[5] = (uint64_t)maximum * bs; geometry[6] = stored; geometry[7] = bytes; geometry[8] = occupied;
    geometry[9] = stored; geometry[10] = slots; geometry[11] = persistent; geometry[12] = source_bytes;
    metrics[0] = slots == 0u ? 0.0 : (double)nnz / (double)slots;
    metrics[1] = stored == 0u ? 0.0 : (double)occupied / (double)stored;
    metrics[2] = nnz == 0u ? 0.0 : (double)slots / nnz;
    metrics[3] = source_bytes == 0u ? 0.0 : (double)persistent / (double)source_bytes;
    if (nnz == 0u) geometry[0] = 1;
    else if (metrics[2] > max_value_expansion) geometry[0] = 2;
    else if (metrics[3] > max_storage_expansion) geometry[0] = 3;
    else if (persistent > max_persistent) geometry[0] = 4;
    else geometry[0] = 0;

    if (column_indices != NULL) {
        /* physical_bell.cc:113-200 */
        if (geometry[0] != 0) status = CANDIDATE_REJECTED;
        else if (values_layout == 1 && row_stride_bytes < (uint64_t)maximum * bs * value_size) status = INSUFFICIENT_CAPACITY;
        else if (padded_fb_offsets == NULL || column_capacity < stored || (bytes != 0u && values_out == NULL) ||
                 value_capacity < (values_layout == 1 ? padded_rows * row_stride_bytes : bytes))
            status = INSUFFICIENT_CAPACITY;
        if (status == OK) {
            for (uint32_t b = 0; b <= fb_count; ++b) padded_fb_offsets[b] = block_offsets[b] * bs;
            for (uint64_t i = 0; i < stored; ++i) column_indices[i] = -1;
            memset(values_out, 0, values_layout == 1 ? padded_rows * row_stride_bytes : bytes);
            const unsigned char *src = (const unsigned char *)values;
            unsigned char *dst = (unsigned char *)values_out;
            for (uint64_t br = 0; br < block_rows; ++br) {
                memset(epochs, 0, ((size_t)physical_blocks + 1u) * sizeof(uint32_t));
                const uint32_t begin = (uint32_t)(br * bs), end = (uint32_t)(begin + bs < rows ? begin + bs : rows);
                for (uint32_t er = begin; er < end; ++er) {
                    const uint32_t r = rperm[er];
                    for (uint32_t i = row_offsets[r]; i < row_offsets[r + 1u]; ++i) {
                        uint32_t semantic;
                        epochs[ORC_PHYSICAL(finv[feature_ids[i]], &semantic)] = 1u;
                    }
                }
                uint32_t slot = 0; /* slots in ascending physical block column */
                for (uint64_t p = 0; p < physical_blocks; ++p) {
                    if (epochs[p] == 0u) continue;
                    epochs[p] = ++slot;
                    column_indices[br * maximum + slot - 1u] = (int32_t)p;
                }
                for (uint32_t er = begin; er < end; ++er) {
                    const uint32_t r = rperm[er];
                    for (uint32_t i = row_offsets[r]; i < row_offsets[r + 1u]; ++i) {
                        uint32_t semantic;
                        const uint32_t execution = finv[feature_ids[i]];
                        const uint32_t p = ORC_PHYSICAL(execution, &semantic);
                        const uint32_t local = (execution - fb_offsets[semantic]) % bs;
                        const uint64_t s = epochs[p] - 1u;
                        const uint64_t at = values_layout == 1
                                                ? (uint64_t)er * row_stride_bytes + (s * bs + local) * value_size
                                                : ((br * maximum + s) * bs * bs + (uint64_t)(er - begin) * bs + local) * value_size;
                        memcpy(dst + at, src + (uint64_t)i * value_size, value_size);
                    }
                }
            }
        }
    }
#undef ORC_PHYSICAL
    free(epochs); free(markers); free(block_offsets);
    return status;
}

/* ---------------------------------------------------------------------------------------------
 * Feature-order pack of a dense operand: packed[execution][column] = source[feature_permutation[execution]][column],
 * contiguous row-major, from a row- or column-major source.  Follows pack_dense_operand_host
 * (src/compute/math/packed_dense_operand.cu:186-226).  That file needs nvcc and the CUDA runtime to
 * build, so it is not part of oracle/_ref; this restatement is pinned on the expected vector of the
 * reference's own test (tests/math_execution_csr_test.cu:93-112).
 * With fb_count != 0 the rows are laid out in the padded physical feature order of a Blocked-ELL
 * lowering: semantic block b occupies rows [padded_offsets[b], padded_offsets[b] + width_b), the
 * rows of the padding are zero, and `packed` holds padded_offsets[fb_count] rows.
 * Returns 0, or 1 when a permutation entry is out of range (physical_view_status invalid_geometry). */
ORC_API int orc_pack_dense_operand(uint32_t features, uint64_t columns, uint64_t ld, int col_major, uint32_t value_size,
                                   const uint32_t *fperm, const void *source, uint32_t fb_count,
                                   const uint32_t *fb_offsets, const uint32_t *padded_offsets, void *packed) {
    const unsigned char *src = (const unsigned char *)source;
    unsigned char *dst = (unsigned char *)packed;
    if (fb_count != 0u) memset(dst, 0, (size_t)padded_offsets[fb_count] * columns * value_size);
    uint32_t block = 0;
    for (uint32_t execution = 0; execution < features; ++execution) {
        const uint32_t feature = fperm[execution];
        if (feature >= features) return 1;
        uint64_t row = execution;
        if (fb_count != 0u) {
            while (fb_offsets[block + 1u] <= execution) ++block;
            row = (uint64_t)padded_offsets[block] + (execution - fb_offsets[block]);
        }
        for (uint64_t column = 0; column < columns; ++column) {
            const uint64_t at = col_major ? column * ld + feature : (uint64_t)feature * ld + column;
            memcpy(dst + (row * columns + column) * value_size, src + at * value_size, value_size);
        }
    }
    return 0;
}

/* ---------------------------------------------------------------------------------------------
 * Execution-order feature ids of a partition-local CSR in packed feature order: entry i of an ordered
 * plan partition names its feature as (semantic block, position inside the block); its execution
 * feature id is fb_offsets[block] + local, which must map back to the entry's canonical id through
 * the plan's feature permutation and must ascend strictly inside a row.
 * Follows build_execution_csr_view_host (src/compute/math/physical_csr.cc:16-97), identities left out.
 * Returns physical_view_status_code (physical_csr.hh:17-26): 0 ok, 1 invalid argument, 2 incompatible
 * identity, 3 invalid geometry -- the first violation in row-major order, as the reference. */
ORC_API int orc_build_execution_csr(uint32_t rows, uint32_t nnz, uint32_t features, uint32_t fb_count,
                                    const uint32_t *fb_offsets, const uint32_t *fperm, const uint32_t *row_offsets,
                                    const uint32_t *block_ids, const uint32_t *local_ids, const uint32_t *canonical_ids,
                                    uint32_t *execution_ids) {
    if (fb_count == 0u || fb_offsets == NULL || (features != 0u && fperm == NULL) || fb_offsets[0] != 0u ||
        fb_offsets[fb_count] != features)
        return 1;
    if (row_offsets == NULL || (nnz != 0u && (block_ids == NULL || local_ids == NULL || canonical_ids == NULL))) return 2;
    if (nnz != 0u && execution_ids == NULL) return 4;
    if (row_offsets[0] != 0u || row_offsets[rows] != nnz) return 3;
    for (uint32_t r = 0; r < rows; ++r) {
        const uint32_t begin = row_offsets[r], end = row_offsets[r + 1u];
        if (end < begin || end > nnz) return 3;
        uint32_t previous = 0xffffffffu;
        for (uint32_t i = begin; i < end; ++i) {
            const uint32_t block = block_ids[i];
            if (block >= fb_count) return 3;
            const uint32_t block_begin = fb_offsets[block], block_end = fb_offsets[block + 1u];
            if (local_ids[i] >= block_end - block_begin) return 3;
            const uint32_t execution = block_begin + local_ids[i];
            if (fperm[execution] != canonical_ids[i] || (i != begin && execution <= previous)) return 2;
            execution_ids[i] = execution;
            previous = execution;
        }
    }
    return 0;
}

/* ------------------------------------------------------------------------ */
/* gene-major copy (CSC) and the order-fixed transpose                       */

/* CSR -> CSC of the codes as a stable counting sort: what count_transpose_targets +
 * scatter_transpose (src/compute/matrix/convert/compressed.cu:146-178) produce, with the one
 * freedom those kernels leave -- the order of the cells inside a gene, decided there by the order in
 * which atomicAdd(heads + minor, 1) happens to be served -- fixed to ascending cells.  Codes come out
 * one per byte.  Returns 0, or 1 when a column index lies outside the matrix. */
ORC_API int orc_qcsr_gene_major(int bits, int64_t rows, int64_t cols, const int64_t *row_ptr,
                                const int64_t *packed_row_ptr, const int32_t *col_idx, const uint8_t *packed,
                                int64_t *col_ptr, int32_t *row_idx, uint8_t *codes) {
    for (int64_t c = 0; c <= cols; ++c) col_ptr[c] = 0;
    for (int64_t i = row_ptr[0]; i < row_ptr[rows]; ++i) {
        if (col_idx[i] < 0 || col_idx[i] >= cols) return 1;
        col_ptr[col_idx[i] + 1] += 1; /* count_transpose_targets: ptr[minor + 1] += 1 */
    }
    for (int64_t c = 0; c < cols; ++c) col_ptr[c + 1] += col_ptr[c];
    int64_t *heads = (int64_t *)malloc((size_t)(cols > 0 ? cols : 1) * sizeof(int64_t));
    if (heads == NULL) return 2;
    for (int64_t c = 0; c < cols; ++c) heads[c] = col_ptr[c];
    for (int64_t r = 0; r < rows; ++r) {
        const uint8_t *row_bytes = packed + (packed_row_ptr != NULL ? packed_row_ptr[r] : row_ptr[r]);
        for (int64_t i = row_ptr[r]; i < row_ptr[r + 1]; ++i) {
            const int64_t dst = heads[col_idx[i]]++; /* scatter_transpose, rows taken in order */
            row_idx[dst] = (int32_t)r;
            codes[dst] = (uint8_t)orc_unpack_code(bits, row_bytes, i - row_ptr[r]);
        }
    }
    free(heads);
    return 0;
}

/* G' = alpha * deq(X)^T G + beta * G' from the gene-major copy, in the order the deterministic
 * device schedule defines (the reference's csr_spmm_bwd_rhs_kernel_ adds in atomic order and defines
 * none): the entries of a gene inside [row_begin, row_end) are cut into chunks of 256; run w of
 * eight takes the chunks w, w + 8, ... and adds them entry by entry with one fused multiply-add per
 * output column, the value decoded with a fused multiply-add as on the device; the eight partial sums
 * are added 0 + 1 + ... + 7; the output is alpha * sum, or fma(beta, old, alpha * sum). */
ORC_API int orc_qcsr_transpose_ordered(int policy, int64_t cols, int64_t n, const int64_t *col_ptr,
                                       const int32_t *row_idx, const uint8_t *codes, const float *scales,
                                       const float *offsets, const float *g, int64_t g_ld, int64_t row_begin,
                                       int64_t row_end, float alpha, float beta, float *out, int64_t out_ld) {
    float *part = (float *)malloc((size_t)(8 * (n > 0 ? n : 1)) * sizeof(float));
    if (part == NULL) return 2;
    for (int64_t c = 0; c < cols; ++c) {
        int64_t lo = col_ptr[c], hi = col_ptr[c + 1];
        while (lo < hi && row_idx[lo] < row_begin) ++lo;
        int64_t end = lo;
        while (end < hi && row_idx[end] < row_end) ++end;
        hi = end;
        for (int64_t i = 0; i < 8 * n; ++i) part[i] = 0.0f;
        const float scale = orc_scale_for(scales, c);
        for (int64_t e = lo; e < hi; ++e) {
            const int64_t run = ((e - lo) / 256) % 8;
            const int64_t r = row_idx[e];
            const float offset = policy == 2 ? (offsets != NULL ? offsets[r] : 0.0f) : (offsets != NULL ? offsets[c] : 0.0f);
            const float value = fmaf((float)codes[e], scale, offset);
            for (int64_t j = 0; j < n; ++j) part[run * n + j] = fmaf(value, g[r * g_ld + j], part[run * n + j]);
        }
        for (int64_t j = 0; j < n; ++j) {
            float sum = part[j];
            for (int w = 1; w < 8; ++w) sum = sum + part[w * n + j];
            float result = alpha * sum;
            if (beta != 0.0f) result = fmaf(beta, out[c * out_ld + j], result);
            out[c * out_ld + j] = result;
        }
    }
    free(part);
    return 0;
}
