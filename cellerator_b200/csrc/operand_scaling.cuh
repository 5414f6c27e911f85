// Power-of-two scaling of fp16 tensor-core operands and the small reductions that find the factors; shared by the
// window kernels (blocked_tile.cuh) and the Blocked-ELL kernel.  Everything here has internal linkage.
#pragma once

#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace cb200 {
namespace {

// fp16 operands.  The decoded values and W are rounded to 16 bits before the tensor cores multiply them.  bf16
// keeps 8 significant bits; fp16 keeps 11, which makes every product eight times more exact, but has a narrow
// exponent range.  So an fp16 operand is stored times a power of two that brings its largest magnitude into
// [2^14, 2^15), and the result is divided by the two factors again (exactly: they are powers of two).  Entries
// more than 2^-29 below the largest lose bits to fp16's subnormal range, an absolute error below 2^-40 of the
// largest magnitude.  The factor of W is found on the device at every launch (absmax_kernel), the factor of the
// decoded values at prepare time.
__host__ __device__ __forceinline__ float operand_scale(float absmax) {
    if (!(absmax > 0.0f) || !(absmax < 3.0e38f)) return 1.0f; // zero, infinite or NaN: leave the operand as it is
    int e = 0;
    frexpf(absmax, &e); // absmax = m * 2^e, m in [0.5, 1)
    e = e < -100 ? -100 : (e > 100 ? 100 : e);
    return ldexpf(1.0f, 15 - e);
}
// Largest magnitude of a dense operand as the bits of a float in *out_bits (zeroed by the caller before).
template<typename WT>
__device__ __forceinline__ void absmax_body(const WT *w, std::int64_t ld, std::int64_t rows, int n, unsigned *out_bits, unsigned block, unsigned blocks) {
    float m = 0.0f;
    const std::int64_t total = rows * n;
    // a contiguous, 16-byte aligned operand is read 16 bytes at a time (the usual case: a launch of the 8,192 x 256
    // Blocked-ELL configuration spent 12.6 us here reading element by element, with a 64-bit division each)
    if (ld == n && (reinterpret_cast<std::uintptr_t>(w) & 15u) == 0u && total % (16 / static_cast<std::int64_t>(sizeof(WT))) == 0) {
        const std::int64_t vectors = total / (16 / static_cast<std::int64_t>(sizeof(WT)));
        const uint4 *v4 = reinterpret_cast<const uint4 *>(w);
        for (std::int64_t i = static_cast<std::int64_t>(block) * blockDim.x + threadIdx.x; i < vectors; i += static_cast<std::int64_t>(blocks) * blockDim.x) {
            const uint4 q = __ldg(v4 + i);
            const std::uint32_t words[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                if constexpr (sizeof(WT) == 2) { // two bf16: their magnitudes are the words' halves without the sign bits, shifted up
                    m = fmaxf(m, __uint_as_float((words[k] & 0x7fffu) << 16));
                    m = fmaxf(m, __uint_as_float(words[k] & 0x7fff0000u));
                } else {
                    m = fmaxf(m, fabsf(__uint_as_float(words[k])));
                }
            }
        }
    } else
    for (std::int64_t i = static_cast<std::int64_t>(block) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<std::int64_t>(blocks) * blockDim.x) {
        const std::int64_t r = i / n;
        const int c = static_cast<int>(i - r * n);
        float v;
        if constexpr (sizeof(WT) == 2) v = __bfloat162float(w[r * ld + c]);
        else v = w[r * ld + c];
        m = fmaxf(m, fabsf(v)); // NaN entries are ignored here; they still reach the product
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31) == 0 && m > 0.0f) atomicMax(out_bits, __float_as_uint(m)); // non-negative floats order like their bits
}
template<typename WT>
__global__ void __launch_bounds__(256) absmax_kernel(const WT *w, std::int64_t ld, std::int64_t rows, int n, unsigned *out_bits) {
    absmax_body(w, ld, rows, n, out_bits, blockIdx.x, gridDim.x);
}

// Largest magnitude a decoded value can take, from the metadata alone: max over genes of |scale| * max code
// (+ |offset| of the gene) in bound[0], max over rows of |row offset| in bound[1] (row-offset policy), as the
// bits of non-negative floats.  The caller zeroes both words.
__device__ __forceinline__ void value_bound_body(const float *scales, const float *gene_offsets, std::int64_t genes, const float *row_offsets,
                                                 std::int64_t rows, float max_code, unsigned *bound, unsigned block) {
    const std::int64_t i = static_cast<std::int64_t>(block) * blockDim.x + threadIdx.x;
    float a = 0.0f, b = 0.0f;
    if (i < genes) a = fabsf(scales != nullptr ? scales[i] : 1.0f) * max_code + (gene_offsets != nullptr ? fabsf(gene_offsets[i]) : 0.0f);
    if (row_offsets != nullptr && i < rows) b = fabsf(row_offsets[i]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
        b = fmaxf(b, __shfl_xor_sync(0xffffffffu, b, o));
    }
    if ((threadIdx.x & 31) == 0) {
        if (a > 0.0f) atomicMax(bound, __float_as_uint(a));
        if (b > 0.0f) atomicMax(bound + 1, __float_as_uint(b));
    }
}
__global__ void __launch_bounds__(256) value_bound_kernel(const float *scales, const float *gene_offsets, std::int64_t genes,
                                                          const float *row_offsets, std::int64_t rows, float max_code, unsigned *bound) {
    value_bound_body(scales, gene_offsets, genes, row_offsets, rows, max_code, bound, blockIdx.x);
}

// One launch for the two reductions a launch starts with: blocks [0, w_blocks) find the largest |W| (the factor of the
// fp16 W operand), the others the bound of the decoded magnitudes from the scales and zero-points (the factor of
// the decoded operand).  The caller zeroes w_absmax[0] and value_bound[0..1].
__global__ void __launch_bounds__(256) operand_bounds_kernel(const __nv_bfloat16 *w, std::int64_t ld, std::int64_t genes, int n, unsigned w_blocks,
                                                             const float *scales, const float *gene_offsets, const float *row_offsets,
                                                             std::int64_t rows, float max_code, unsigned *w_absmax, unsigned *value_bound) {
    if (blockIdx.x < w_blocks) absmax_body(w, ld, genes, n, w_absmax, blockIdx.x, w_blocks);
    else value_bound_body(scales, gene_offsets, genes, row_offsets, rows, max_code, value_bound, blockIdx.x - w_blocks);
}

} // namespace
} // namespace cb200
