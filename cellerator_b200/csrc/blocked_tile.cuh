// Geometry of the window tiles, the entry-word layout and the W records shared by the tensor-core
// kernels over the window-blocked copy (qcsr_forward_blocked.cu) and over the dense operand tiles
// (qcsr_forward_dense.cu).  Everything here has internal linkage: each translation unit that
// includes the header gets its own copy.
#pragma once

#include "kernels.cuh"
#include "operand_scaling.cuh"
#include "sm100_primitives.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace cb200 {
namespace {

// Geometry.  A (group, window) tile is 256 cells x 128 genes = 64 KB of bf16, double buffered.
// (512 cells x 64 genes halves the W bytes per unit of work but leaves 13 instead of 26 groups per
// SM on a 1M-cell shard; the coarser deal costs more than the W traffic saves: 8.0 ms against 7.5.)
constexpr int kWin = 128;                    // genes per window
constexpr int kWinShift = 7;
constexpr int kRows = 256;                   // cell rows per group
constexpr int kRowsShift = 8;
constexpr int kSubBlocks = kRows / 128;      // one M = 128 MMA each
constexpr int kProducerWarps = 16;           // zero + scatter; the first kEpilogueWarps of them also write Y
constexpr int kEpilogueWarps = kRows / 32;
constexpr int kProducerThreads = kProducerWarps * 32;
// Measured on the 1M x 33,538 matrix (ms per launch) for (chunk loader warps, chunk stages): (1, 2) 7.11,
// (2, 2) 7.13, (1, 3) 7.36, (2, 4) 7.38, (3, 3) 7.55, (1, 1) 8.96; W stages 4 / 3 / 2: 7.13 / 7.38 / 7.68.
constexpr int kChunkLoaders = 1;                // warps whose elected lane issues entry-chunk copies
constexpr int kThreads = kProducerThreads + 32 * (2 + kChunkLoaders); // + MMA warp + W loader warp + chunk loader warps
constexpr int kABufBytes = kRows * kWin * 2;    // 64 KB
constexpr int kSubBlockBytes = 128 * kWin * 2;  // 16 KB
constexpr int kRowGroupBytes = kWin * 16;       // W slice: 8 columns x kWin genes of bf16
constexpr int kChunkEntries = 2048;
constexpr int kChunkBytes = kChunkEntries * 4;
// chunk stages (template parameter CS of the kernel): 2 when a segment fits one chunk, 3 for denser matrices
constexpr int kMaxWStages = 6;
constexpr std::uint32_t kInvalidEntry = 0x80000000u; // padding of a segment
static_assert(kProducerWarps >= kEpilogueWarps && kABufBytes % (kProducerThreads * 16) == 0, "thread t < kRows owns row t in the epilogue");
static_assert(kABufBytes <= 65536, "an entry holds the byte position in the tile, halved, in 15 bits");

__host__ __device__ constexpr int record_bytes(int n) { return n * kWin * 2 + kWin * 8; }
__host__ __device__ constexpr int fixed_smem_bytes(int cs) { return 2 * kABufBytes + cs * kChunkBytes + kRows * 4 + 512; }
__host__ __device__ constexpr int w_stages(int n, int cs) {
    return (232448 - fixed_smem_bytes(cs)) / record_bytes(n) >= kMaxWStages ? kMaxWStages
                                                                            : (232448 - fixed_smem_bytes(cs)) / record_bytes(n);
}

// Byte position of (row within group, gene within window) in the A tile.  The tile is made of
// sub-blocks of 128 rows; a sub-block is K-major with the 128-byte swizzle: per 64 genes (a "half",
// kHalfBytes; one half when the window is 64 genes wide) 8-row atoms of 1,024 bytes in which row r
// holds its 64 genes in one 128-byte line whose 16-byte pieces are permuted by r mod 8.  The
// permutation spreads the scattered 2-byte stores of one row, and of neighbouring rows, over all
// shared-memory banks.
constexpr int kHalfBytes = 128 * 64 * 2; // 16 KB: 128 rows x 64 genes
__host__ __device__ constexpr std::uint32_t tile_offset(int rl, int gl) {
    return static_cast<std::uint32_t>((rl >> 7) * kSubBlockBytes + (gl >> 6) * kHalfBytes + ((rl & 127) >> 3) * 1024 +
                                      (rl & 7) * 128 + ((((gl & 63) >> 3) ^ (rl & 7)) * 16) + (gl & 7) * 2);
}
// The transpose kernel's tile of the same (group, window): M = gene, K = cell, K-major with the 128-byte
// swizzle: [cell quarter of 64][gene][64 cells], the 16-byte pieces of a gene's line permuted by gene mod 8.
__host__ __device__ constexpr std::uint32_t tile_offset_gene_major(int rl, int gl) {
    return static_cast<std::uint32_t>((rl >> 6) * (kWin * 128) + (gl >> 3) * 1024 + (gl & 7) * 128 + ((((rl & 63) >> 3) ^ (gl & 7)) << 4) +
                                      ((rl & 7) << 1));
}


// K-major operand, no swizzle: LBO = 128 B between the two core matrices one K = 16 step reads,
// SBO = kRowGroupBytes between groups of 8 rows.
__device__ __forceinline__ std::uint64_t smem_desc(std::uint32_t addr) {
    std::uint64_t d = 0;
    d |= static_cast<std::uint64_t>((addr & 0x3ffffu) >> 4);
    d |= static_cast<std::uint64_t>(128u >> 4) << 16;
    d |= static_cast<std::uint64_t>(static_cast<unsigned>(kRowGroupBytes) >> 4) << 32;
    d |= static_cast<std::uint64_t>(1) << 46; // descriptor version of this architecture
    return d;
}
// W [genes][n] (leading dimension ld) -> one record per window of 128 genes: the n x 128 slice of
// W^T in operand layout (byte offset of (column c, gene e) = (c/8)*2048 + (e/8)*128 + (c%8)*16 +
// (e%8)*2, zero for genes >= cols) followed by 128 x {scale, zero-point}.  part 0 writes
// hi = bf16(w) (w itself for a bf16 W); part 1 writes lo = bf16(w - hi), the next 8 mantissa bits.
// With absmax_bits != null the record holds fp16 instead: hi = fp16(w * s), lo = fp16(w * s - hi), s =
// operand_scale(largest |w|).  The grid is (windows, column groups): block (w, g) lays out columns [g, g + 1) * n /
// gridDim.y of window w; the blocks of group 0 also write the window's table.
constexpr int kPackColumns = 16; // columns of W per block of the packing kernel
template<typename WT>
__global__ void __launch_bounds__(256) pack_windows_kernel(const WT *w, std::int64_t ld, std::int64_t cols, int n, int part,
                                                           const float *scales, const float *offsets, int per_gene_offsets,
                                                           unsigned char *records, const unsigned *absmax_bits = nullptr) {
    const std::int64_t window = blockIdx.x;
    unsigned char *rec = records + window * record_bytes(n);
    __nv_bfloat16 *wt = reinterpret_cast<__nv_bfloat16 *>(rec);
    const bool fp16 = absmax_bits != nullptr;
    const float ws = fp16 ? operand_scale(__uint_as_float(*absmax_bits)) : 1.0f;
    const int group_cols = n / static_cast<int>(gridDim.y), c_first = static_cast<int>(blockIdx.y) * group_cols;
    for (int i = threadIdx.x; i < group_cols * kWin; i += blockDim.x) {
        const int e = i / group_cols, c = c_first + i % group_cols; // consecutive threads read consecutive columns of one gene
        const std::int64_t gene = window * kWin + e;
        float value = 0.0f;
        if (gene < cols) {
            if constexpr (sizeof(WT) == 2) value = __bfloat162float(w[gene * ld + c]);
            else value = w[gene * ld + c];
        }
        const int at = ((c >> 3) * kRowGroupBytes + (e >> 3) * 128 + (c & 7) * 16 + (e & 7) * 2) >> 1;
        if (fp16) {
            const float scaled = value * ws;
            __half h = __float2half_rn(scaled);
            if (part != 0) h = __float2half_rn(scaled - __half2float(h));
            reinterpret_cast<__half *>(rec)[at] = h;
            continue;
        }
        __nv_bfloat16 v = __float2bfloat16_rn(value);
        if (part != 0) v = __float2bfloat16_rn(value - __bfloat162float(v));
        wt[at] = v;
    }
    if (blockIdx.y != 0) return;
    float2 *table = reinterpret_cast<float2 *>(rec + n * kWin * 2);
    for (int e = threadIdx.x; e < kWin; e += blockDim.x) {
        const std::int64_t gene = window * kWin + e;
        float2 so = make_float2(0.0f, 0.0f);
        if (gene < cols) {
            so.x = scales != nullptr ? scales[gene] : 1.0f;
            so.y = (per_gene_offsets && offsets != nullptr) ? offsets[gene] : 0.0f;
        }
        table[e] = so;
    }
}

} // namespace
} // namespace cb200
