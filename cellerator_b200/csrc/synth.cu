// Seeded synthetic single-cell workloads, generated on the device so that the full-size
// benchmark matrices (10^9 stored entries) never have to exist on the host.
//
// This is workload synthesis for the benchmark and the tests, not part of the compute path:
// it is built into its own library (libcb200_synth.so).  The value model follows the
// benchmark configurations: gene indices uniform without replacement and sorted (selection
// sampling), counts from a negative binomial with a per-gene mean and dispersion 0.5 (a
// gamma(2)-Poisson mixture), forced >= 1 at stored positions, then log1p(count/rowsum*1e4);
// per-gene affine calibration offset = min, scale = max((max-min)/(2^bits-1), 1e-6), unseen
// genes scale 1 offset 0 (the recipe of bench/quantized_transfer_spmm_bench.cu:345-377 in the
// Cellerator tree).  All randomness is a counter-based hash of (seed, row, position), so a
// row's content does not depend on how the launch is shaped.
#include <cuda_runtime.h>

#include <cstdint>

#define SYNTH_API extern "C" __attribute__((visibility("default")))

namespace {

__host__ __device__ inline std::uint64_t mix64(std::uint64_t x) {
    x += 0x9e3779b97f4a7c15ull;
    x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ull;
    x = (x ^ (x >> 27)) * 0x94d049bb133111ebull;
    return x ^ (x >> 31);
}

__device__ inline std::uint32_t hash32(std::uint64_t seed, std::uint64_t a, std::uint64_t b, std::uint64_t c) {
    return static_cast<std::uint32_t>(mix64(mix64(mix64(seed ^ (a * 0xd1342543de82ef95ull)) + b) + c) >> 32);
}

__device__ inline float uniform01(std::uint32_t h) { return (static_cast<float>(h >> 8) + 0.5f) * (1.0f / 16777216.0f); }

// Negative-binomial count with mean `mu`, dispersion 0.5 (shape 2), at least 1.
__device__ inline float nb_count(std::uint64_t seed, std::uint64_t row, std::uint64_t gene, float mu) {
    const float u1 = uniform01(hash32(seed, row, gene, 1));
    const float u2 = uniform01(hash32(seed, row, gene, 2));
    const float lambda = -0.5f * mu * __logf(u1 * u2); // gamma(shape 2, scale mu/2)
    float count;
    if (lambda < 24.0f) {
        const float limit = __expf(-lambda);
        float prod = 1.0f;
        int k = 0;
        for (; k < 96; ++k) {
            prod *= uniform01(hash32(seed, row, gene, 8 + k));
            if (prod <= limit) break;
        }
        count = static_cast<float>(k);
    } else {
        const float a = uniform01(hash32(seed, row, gene, 3));
        const float b = uniform01(hash32(seed, row, gene, 4));
        const float z = sqrtf(-2.0f * __logf(a)) * __cosf(6.2831853f * b);
        count = rintf(lambda + sqrtf(lambda) * z);
    }
    return fmaxf(count, 1.0f);
}

// One thread per row: selection sampling of row_nnz sorted distinct genes out of `cols`.
__global__ void __launch_bounds__(128) columns_kernel(std::int64_t rows, std::int32_t cols, const std::int64_t *row_ptr,
                                                      std::int32_t *col_idx, std::uint64_t seed, std::int64_t row_base) {
    const std::int64_t row = static_cast<std::int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (row >= rows) return;
    std::int64_t out = row_ptr[row];
    std::uint64_t need = static_cast<std::uint64_t>(row_ptr[row + 1] - out);
    for (std::int32_t g = 0; g < cols && need != 0u; ++g) {
        const std::uint64_t remaining = static_cast<std::uint64_t>(cols - g);
        const std::uint64_t h = hash32(seed, static_cast<std::uint64_t>(row + row_base), static_cast<std::uint64_t>(g), 0);
        if (h * remaining < (need << 32)) {
            col_idx[out++] = g;
            --need;
        }
    }
}

// One warp per row: counts, row sum, log1p-normalised value per stored entry.
__global__ void __launch_bounds__(256) values_kernel(std::int64_t rows, const std::int64_t *row_ptr,
                                                     const std::int32_t *col_idx, const float *gene_mean, float *values,
                                                     std::uint64_t seed, std::int64_t row_base) {
    const int lane = threadIdx.x & 31;
    const std::int64_t row = static_cast<std::int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const std::int64_t begin = row_ptr[row], end = row_ptr[row + 1];
    float sum = 0.0f;
    for (std::int64_t i = begin + lane; i < end; i += 32) {
        const std::int32_t g = col_idx[i];
        const float c = nb_count(seed, static_cast<std::uint64_t>(row + row_base), static_cast<std::uint64_t>(g), gene_mean[g]);
        values[i] = c;
        sum += c;
    }
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
    const float inv = sum > 0.0f ? 1.0e4f / sum : 0.0f;
    for (std::int64_t i = begin + lane; i < end; i += 32) values[i] = log1pf(values[i] * inv);
}

// Per-gene min / max over stored entries (values are >= 0, so their bit patterns order like
// unsigned integers).
__global__ void __launch_bounds__(256) minmax_kernel(std::int64_t count, const std::int32_t *genes, const float *values,
                                                     std::uint32_t *gmin, std::uint32_t *gmax) {
    for (std::int64_t i = static_cast<std::int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count;
         i += static_cast<std::int64_t>(gridDim.x) * blockDim.x) {
        const std::uint32_t bits = __float_as_uint(values[i]);
        const std::int32_t g = genes[i];
        atomicMin(gmin + g, bits);
        atomicMax(gmax + g, bits);
    }
}

__global__ void init_minmax_kernel(std::int32_t cols, std::uint32_t *gmin, std::uint32_t *gmax) {
    const int g = blockIdx.x * blockDim.x + threadIdx.x;
    if (g < cols) {
        gmin[g] = 0xffffffffu;
        gmax[g] = 0u;
    }
}

__global__ void calibrate_kernel(std::int32_t cols, int bits, const std::uint32_t *gmin, const std::uint32_t *gmax,
                                 float *scales, float *offsets) {
    const int g = blockIdx.x * blockDim.x + threadIdx.x;
    if (g >= cols) return;
    if (gmin[g] == 0xffffffffu) {
        scales[g] = 1.0f;
        offsets[g] = 0.0f;
        return;
    }
    const float lo = __uint_as_float(gmin[g]);
    const float hi = __uint_as_float(gmax[g]);
    const float levels = static_cast<float>((1 << bits) - 1);
    scales[g] = fmaxf(__fdiv_rn(__fsub_rn(hi, lo), levels), 1.0e-6f);
    offsets[g] = lo;
}

// Blocked-ELL: per block row, `width` distinct ascending block columns out of `block_cols`.
__global__ void bell_blocks_kernel(std::int64_t block_rows, int width, int block_cols, std::uint32_t *block_col_idx,
                                   std::uint64_t seed, std::int64_t block_row_base) {
    const std::int64_t br = static_cast<std::int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (br >= block_rows) return;
    std::uint64_t need = static_cast<std::uint64_t>(width);
    int out = 0;
    for (int c = 0; c < block_cols && need != 0u; ++c) {
        const std::uint64_t remaining = static_cast<std::uint64_t>(block_cols - c);
        const std::uint64_t h = hash32(seed, static_cast<std::uint64_t>(br + block_row_base), static_cast<std::uint64_t>(c), 77);
        if (h * remaining < (need << 32)) {
            block_col_idx[br * width + out++] = static_cast<std::uint32_t>(c);
            --need;
        }
    }
}

// Blocked-ELL slot values (row-major, ell_cols per row): a slot is non-zero with probability
// `fill`; gene ids are written beside the values so that the per-gene calibration can reuse
// minmax_kernel over every slot of a present block.
__global__ void __launch_bounds__(256) bell_values_kernel(std::int64_t rows, int block_size, int ell_cols,
                                                          const std::uint32_t *block_col_idx, const float *gene_mean,
                                                          float fill, float *values_by_slot, std::int32_t *gene_by_slot,
                                                          std::uint64_t seed, std::int64_t row_base) {
    const int lane = threadIdx.x & 31;
    const std::int64_t row = static_cast<std::int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int width = ell_cols / block_size;
    const std::uint32_t *blocks = block_col_idx + (row / block_size) * width;
    float *out = values_by_slot + row * ell_cols;
    std::int32_t *gout = gene_by_slot + row * ell_cols;
    float sum = 0.0f;
    for (int s = lane; s < ell_cols; s += 32) {
        const std::int32_t g = static_cast<std::int32_t>(blocks[s / block_size]) * block_size + s % block_size;
        gout[s] = g;
        float c = 0.0f;
        if (uniform01(hash32(seed, static_cast<std::uint64_t>(row + row_base), static_cast<std::uint64_t>(g), 5)) < fill)
            c = nb_count(seed, static_cast<std::uint64_t>(row + row_base), static_cast<std::uint64_t>(g), gene_mean[g]);
        out[s] = c;
        sum += c;
    }
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
    const float inv = sum > 0.0f ? 1.0e4f / sum : 0.0f;
    for (int s = lane; s < ell_cols; s += 32) out[s] = log1pf(out[s] * inv);
}

int check(cudaError_t e) { return e == cudaSuccess ? 0 : static_cast<int>(e); }

} // namespace

// All pointers are device pointers on the current device; calls enqueue on `stream`.
// `row_base` offsets the hashed row id so that a shard generates the same rows that the whole
// matrix would hold at that position.

SYNTH_API int cb200_synth_columns(std::int64_t rows, std::int32_t cols, const std::int64_t *row_ptr,
                                  std::int32_t *col_idx, std::uint64_t seed, std::int64_t row_base, void *stream) {
    if (rows <= 0) return 0;
    columns_kernel<<<static_cast<unsigned>((rows + 127) / 128), 128, 0, static_cast<cudaStream_t>(stream)>>>(
        rows, cols, row_ptr, col_idx, seed, row_base);
    return check(cudaGetLastError());
}

SYNTH_API int cb200_synth_values(std::int64_t rows, const std::int64_t *row_ptr, const std::int32_t *col_idx,
                                 const float *gene_mean, float *values, std::uint64_t seed, std::int64_t row_base,
                                 void *stream) {
    if (rows <= 0) return 0;
    values_kernel<<<static_cast<unsigned>((rows + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        rows, row_ptr, col_idx, gene_mean, values, seed, row_base);
    return check(cudaGetLastError());
}

// gmin/gmax: caller-provided uint32[cols] scratch.  Call init once, accumulate over any number
// of (genes, values) arrays, then finish.
SYNTH_API int cb200_synth_calibrate_init(std::int32_t cols, std::uint32_t *gmin, std::uint32_t *gmax, void *stream) {
    init_minmax_kernel<<<(cols + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(cols, gmin, gmax);
    return check(cudaGetLastError());
}

SYNTH_API int cb200_synth_calibrate_accumulate(std::int64_t count, const std::int32_t *genes, const float *values,
                                               std::uint32_t *gmin, std::uint32_t *gmax, void *stream) {
    if (count <= 0) return 0;
    minmax_kernel<<<148 * 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(count, genes, values, gmin, gmax);
    return check(cudaGetLastError());
}

SYNTH_API int cb200_synth_calibrate_finish(std::int32_t cols, int bits, const std::uint32_t *gmin,
                                           const std::uint32_t *gmax, float *scales, float *offsets, void *stream) {
    calibrate_kernel<<<(cols + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(cols, bits, gmin, gmax, scales, offsets);
    return check(cudaGetLastError());
}

SYNTH_API int cb200_synth_bell_blocks(std::int64_t block_rows, int width, int block_cols, std::uint32_t *block_col_idx,
                                      std::uint64_t seed, std::int64_t block_row_base, void *stream) {
    if (block_rows <= 0) return 0;
    bell_blocks_kernel<<<static_cast<unsigned>((block_rows + 127) / 128), 128, 0, static_cast<cudaStream_t>(stream)>>>(
        block_rows, width, block_cols, block_col_idx, seed, block_row_base);
    return check(cudaGetLastError());
}

SYNTH_API int cb200_synth_bell_values(std::int64_t rows, int block_size, int ell_cols, const std::uint32_t *block_col_idx,
                                      const float *gene_mean, float fill, float *values_by_slot,
                                      std::int32_t *gene_by_slot, std::uint64_t seed, std::int64_t row_base, void *stream) {
    if (rows <= 0) return 0;
    bell_values_kernel<<<static_cast<unsigned>((rows + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        rows, block_size, ell_cols, block_col_idx, gene_mean, fill, values_by_slot, gene_by_slot, seed, row_base);
    return check(cudaGetLastError());
}
