// Gene-major copy (a CSC) of a quantized CSR matrix, built on the device, and the order-fixed
// transpose  G' = alpha * deq(X)^T * G + beta * G'  that gathers from it.
//
// Reference counterpart of the build: the CSR -> CSC transpose kernels count_transpose_targets and
// scatter_transpose (src/compute/matrix/convert/compressed.cu:146-178): count the entries of each
// minor index with atomics, scan, then place every entry at atomicAdd(heads + minor, 1).  That leaves
// the order of the cells inside a gene to the scheduler.  Here the placement is a stable counting
// sort -- cells ascend inside every gene, the same arrays on every run -- in three steps:
//   1. one CTA per block of 1,024 rows counts its entries per gene in shared memory and writes the
//      counts row  counts[block][gene] (beyond 57,344 genes: one launch per range of that many);
//   2. per gene, the counts are scanned over the blocks (the offset of a block inside the gene's
//      segment) and the totals over the genes (col_ptr);
//   3. the CTA of a block walks its rows in order; the entries of one row go to different genes
//      (column indices ascend strictly inside a row), so a row is placed in parallel and a barrier
//      between rows keeps the cells of a gene in ascending order.  This pass runs once per range of
//      1,024 genes, so that the segments being written stay in L2.
// Codes are widened to one byte per entry in the copy (4-bit sources too): a gene's segment is
// written by many CTAs at once and bytes need no read-modify-write.
//
// Reference counterpart of the transpose: csr_spmm_bwd_rhs_kernel_
// (src/compute/sparse/ops/kernels/base_sparse/csr_spmm_bwd_rhs_kernel_.cuh:1-22), whose sums arrive
// in atomic order.  The gather kernel below fixes the order, so the result is the same bits on every
// run and the projection can serve a request that asks for determinism:
//   a CTA of 8 warps owns a gene; the gene's entries (restricted to the row range) are cut into
//   chunks of 256; warp w adds the chunks w, w + 8, ... entry after entry with one fp32 FMA per
//   (entry, output column); the eight partial sums are added 0 + 1 + ... + 7; the result is
//   alpha * sum, or fma(beta, old, alpha * sum) when beta != 0.
#include "kernels.cuh"

#include <algorithm>
#include <vector>

namespace cb200 {
namespace {

constexpr int kBlockRows = 1024;   // rows per CTA of the counting and the placing pass
constexpr int kBuildThreads = 1024;
constexpr int kGatherWarps = 8;
constexpr int kGatherChunk = 256;

struct gm_params {
    const std::int64_t *row_ptr;
    const std::int64_t *packed_row_ptr;
    const std::int32_t *col_idx;
    const std::uint8_t *packed;
    std::int64_t rows, cols;
    std::int64_t blocks;
    std::uint32_t *counts; // [blocks][cols]
    std::int64_t *col_ptr; // cols + 1
    std::int32_t *row_idx;
    std::uint8_t *codes;
    int *status;
};

template<int BITS>
__device__ __forceinline__ unsigned gm_load_code(const std::uint8_t *row_bytes, std::int64_t local) {
    if constexpr (BITS == 8) {
        return __ldg(row_bytes + local);
    } else {
        const unsigned byte = __ldg(row_bytes + (local >> 1));
        return (local & 1) ? (byte >> 4) : (byte & 0xfu);
    }
}

// step 1: counts[block][gene] for the genes [g0, g1): one launch per range of genes whose counters
// fit shared memory (one launch up to 57,344 genes)
__global__ void __launch_bounds__(kBuildThreads) gm_count_kernel(const gm_params p, int g0, int g1) {
    extern __shared__ std::uint32_t gm_hist[];
    const int span = g1 - g0;
    for (int c = threadIdx.x; c < span; c += kBuildThreads) gm_hist[c] = 0u;
    __syncthreads();
    const std::int64_t r0 = static_cast<std::int64_t>(blockIdx.x) * kBlockRows;
    const std::int64_t r1 = min(p.rows, r0 + kBlockRows);
    const std::int64_t begin = __ldg(p.row_ptr + r0), end = __ldg(p.row_ptr + r1);
    for (std::int64_t i = begin + threadIdx.x; i < end; i += kBuildThreads) {
        const int c = __ldg(p.col_idx + i);
        if (static_cast<unsigned>(c - g0) < static_cast<unsigned>(span)) atomicAdd(&gm_hist[c - g0], 1u);
        else if (static_cast<unsigned>(c) >= static_cast<unsigned>(p.cols)) atomicOr(p.status, 1); // outside the matrix: reported, left out
    }
    __syncthreads();
    std::uint32_t *row = p.counts + static_cast<std::int64_t>(blockIdx.x) * p.cols + g0;
    for (int c = threadIdx.x; c < span; c += kBuildThreads) row[c] = gm_hist[c];
}

// step 2a: per gene, exclusive scan of the counts over the blocks; the total goes to col_ptr[gene]
__global__ void __launch_bounds__(256) gm_block_scan_kernel(const gm_params p) {
    const std::int64_t c = static_cast<std::int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (c >= p.cols) return;
    std::uint32_t running = 0u;
    std::uint32_t *cell = p.counts + c;
    std::int64_t b = 0;
    for (; b + 4 <= p.blocks; b += 4) {
        const std::uint32_t t0 = cell[(b + 0) * p.cols], t1 = cell[(b + 1) * p.cols];
        const std::uint32_t t2 = cell[(b + 2) * p.cols], t3 = cell[(b + 3) * p.cols];
        cell[(b + 0) * p.cols] = running;
        cell[(b + 1) * p.cols] = running + t0;
        cell[(b + 2) * p.cols] = running + t0 + t1;
        cell[(b + 3) * p.cols] = running + t0 + t1 + t2;
        running += t0 + t1 + t2 + t3;
    }
    for (; b < p.blocks; ++b) {
        const std::uint32_t t = cell[b * p.cols];
        cell[b * p.cols] = running;
        running += t;
    }
    p.col_ptr[c] = static_cast<std::int64_t>(running);
}

// step 2b: col_ptr = exclusive scan of the totals, in place (one CTA; a thread owns a run of genes)
__global__ void __launch_bounds__(1024) gm_col_scan_kernel(std::int64_t *col_ptr, std::int64_t cols) {
    __shared__ std::int64_t sums[1024];
    const std::int64_t per = (cols + 1023) / 1024;
    const std::int64_t c0 = min(cols, per * threadIdx.x), c1 = min(cols, c0 + per);
    std::int64_t local = 0;
    for (std::int64_t c = c0; c < c1; ++c) local += col_ptr[c];
    sums[threadIdx.x] = local;
    __syncthreads();
    if (threadIdx.x == 0) {
        std::int64_t running = 0;
        for (int t = 0; t < 1024; ++t) {
            const std::int64_t s = sums[t];
            sums[t] = running;
            running += s;
        }
        col_ptr[cols] = running;
    }
    __syncthreads();
    std::int64_t running = sums[threadIdx.x];
    for (std::int64_t c = c0; c < c1; ++c) {
        const std::int64_t t = col_ptr[c];
        col_ptr[c] = running;
        running += t;
    }
}

// first index in [lo, hi) of an ascending run of column indices that is >= bound
__device__ __forceinline__ std::int64_t gm_lower_bound(const std::int32_t *col_idx, std::int64_t lo, std::int64_t hi, int bound) {
    while (lo < hi) {
        const std::int64_t mid = lo + ((hi - lo) >> 1);
        if (__ldg(col_idx + mid) < bound) lo = mid + 1;
        else hi = mid;
    }
    return lo;
}

constexpr int kFillGenes = 1024;   // genes per launch of the placing pass
constexpr int kStageEntries = 8192; // entries staged in shared memory per group of rows (>= kFillGenes: a row fits)

// step 3: place the entries of the genes [g0, g1), rows of a block in order.  One launch per gene
// range: all CTAs then write into the segments of the same few thousand genes, whose open sectors
// stay in L2 until they are full, and the per-gene state of a range fits shared memory twice per SM.
// The entries of a range are contiguous inside a row, because column indices ascend there.
// A CTA stages the entries of as many rows as fit (warp per row, coalesced, many loads in flight) as
// words (gene - g0) << 8 | code, then walks those rows in order out of shared memory with a barrier
// between rows: the ordered walk has no global load on its critical path.  Measured on 10^6 x 33,538
// with 1.8 G entries: 161 ms with every gene in one launch and the loads inside the walk, 99 ms with
// ranges of 4,096 genes, 66 ms with 1,024 (the sectors being filled by the 296 resident CTAs then
// fit L2: 19 MB), 110 ms with 512 (twice the launches, and a barrier per row in each).
template<int BITS>
__global__ void __launch_bounds__(kBuildThreads) gm_fill_kernel(const gm_params p, int g0, int g1) {
    extern __shared__ std::int64_t gm_fill_smem[];
    const int span = g1 - g0;
    std::int64_t *gene_base = gm_fill_smem;                  // [kFillGenes] first entry of the gene's segment
    std::int64_t *row_start = gene_base + kFillGenes;        // [kBlockRows + 1]
    std::int64_t *seg_lo = row_start + kBlockRows + 1;       // [kBlockRows] first entry of the row inside the range
    std::uint32_t *head = reinterpret_cast<std::uint32_t *>(seg_lo + kBlockRows); // [kFillGenes] next free slot of this block
    std::uint32_t *prefix = head + kFillGenes;               // [kBlockRows + 1] entries of the range before row r
    std::uint32_t *stage = prefix + kBlockRows + 1 + 1;      // [kStageEntries]
    const std::int64_t r0 = static_cast<std::int64_t>(blockIdx.x) * kBlockRows;
    const int block_rows = static_cast<int>(min(p.rows, r0 + kBlockRows) - r0);
    const std::uint32_t *mine = p.counts + static_cast<std::int64_t>(blockIdx.x) * p.cols + g0;
    for (int c = threadIdx.x; c < span; c += kBuildThreads) {
        head[c] = mine[c];
        gene_base[c] = __ldg(p.col_ptr + g0 + c);
    }
    for (int r = threadIdx.x; r <= block_rows; r += kBuildThreads) row_start[r] = __ldg(p.row_ptr + r0 + r);
    __syncthreads();
    for (int r = threadIdx.x; r < block_rows; r += kBuildThreads) {
        const std::int64_t lo = gm_lower_bound(p.col_idx, row_start[r], row_start[r + 1], g0);
        const std::int64_t hi = gm_lower_bound(p.col_idx, lo, row_start[r + 1], g1);
        seg_lo[r] = lo;
        prefix[r + 1] = static_cast<std::uint32_t>(min(hi - lo, static_cast<std::int64_t>(span))); // a row holds a gene once
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        std::uint32_t running = 0u;
        prefix[0] = 0u;
        for (int r = 1; r <= block_rows; ++r) {
            running += prefix[r];
            prefix[r] = running;
        }
    }
    __syncthreads();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int ra = 0;
    while (ra < block_rows) {
        // rows [ra, rb): as many as the stage holds (one row always fits)
        int rb = ra + 1;
        while (rb < block_rows && prefix[rb + 1] - prefix[ra] <= static_cast<std::uint32_t>(kStageEntries)) ++rb;
        const std::uint32_t first = prefix[ra];
        for (int r = ra + warp; r < rb; r += kBuildThreads / 32) {
            const std::int64_t lo = seg_lo[r], begin = row_start[r];
            const int count = static_cast<int>(prefix[r + 1] - prefix[r]);
            const std::uint8_t *row_bytes = p.packed + (p.packed_row_ptr != nullptr ? __ldg(p.packed_row_ptr + r0 + r) : begin);
            std::uint32_t *dst = stage + (prefix[r] - first);
            for (int q = lane; q < count; q += 32) {
                const unsigned c = static_cast<unsigned>(__ldg(p.col_idx + lo + q) - g0);
                const unsigned code = gm_load_code<BITS>(row_bytes, lo + q - begin);
                // a row that does not ascend can hold a gene of another range here: marked, left out below
                dst[q] = c < static_cast<unsigned>(span) ? ((c << 8) | code) : 0xffffffffu;
            }
        }
        __syncthreads();
        for (int r = ra; r < rb; ++r) {
            const int count = static_cast<int>(prefix[r + 1] - prefix[r]);
            const std::uint32_t *src = stage + (prefix[r] - first);
            const std::int32_t row = static_cast<std::int32_t>(r0 + r);
            for (int q = threadIdx.x; q < count; q += kBuildThreads) {
                const std::uint32_t word = src[q];
                if (word == 0xffffffffu) continue;
                const std::uint32_t c = word >> 8;
                const std::int64_t pos = gene_base[c] + atomicAdd(&head[c], 1u);
                p.row_idx[pos] = row;
                p.codes[pos] = static_cast<std::uint8_t>(word & 0xffu);
            }
            __syncthreads();
        }
        ra = rb;
    }
}


constexpr int kCountGenes = 56 * 1024; // genes per launch of the counting pass: a 32-bit counter each in shared memory
std::size_t fill_smem_bytes() {
    return static_cast<std::size_t>(kFillGenes + 2 * kBlockRows + 1) * 8u +
           static_cast<std::size_t>(kFillGenes + kBlockRows + 2 + kStageEntries) * 4u;
}

} // namespace

namespace {

struct gather_params {
    const std::int64_t *col_ptr;
    const std::int32_t *row_idx;
    const std::uint8_t *codes;
    const float *scales;
    const float *offsets;
    const float *g;
    float *out;
    std::int64_t g_ld, out_ld, cols;
    std::int64_t row_begin, row_end;
    int policy;
    int restrict_rows; // the launch covers a proper sub-range of the rows
    int aligned;       // G rows can be read with one vector load per lane
    float alpha, beta;
    unsigned *queue;   // next gene to hand out
    const std::int32_t *gene_order; // position in the queue -> gene (long genes first); null: natural order
};

// VEC consecutive floats of a row of G; ALIGNED: one vector load
template<int VEC, bool ALIGNED>
__device__ __forceinline__ void gather_load(const float *src, float (&v)[VEC]) {
    if constexpr (VEC == 2 && ALIGNED) {
        const float2 t = __ldg(reinterpret_cast<const float2 *>(src));
        v[0] = t.x; v[1] = t.y;
    } else if constexpr (VEC == 4 && ALIGNED) {
        const float4 t = __ldg(reinterpret_cast<const float4 *>(src));
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    } else {
#pragma unroll
        for (int k = 0; k < VEC; ++k) v[k] = __ldg(src + k);
    }
}

// float of the low byte of a word, one conversion instruction (a cvt from .u8 reads the low 8 bits
// of a wider source register)
__device__ __forceinline__ float low_byte_to_float(unsigned word) {
    float f;
    asm("cvt.rn.f32.u8 %0, %1;" : "=f"(f) : "r"(word));
    return f;
}

// first position in [lo, hi) whose row is >= bound
__device__ __forceinline__ std::int64_t gather_lower_bound(const std::int32_t *row_idx, std::int64_t lo, std::int64_t hi,
                                                           std::int64_t bound) {
    while (lo < hi) {
        const std::int64_t mid = lo + ((hi - lo) >> 1);
        if (static_cast<std::int64_t>(__ldg(row_idx + mid)) < bound) lo = mid + 1;
        else hi = mid;
    }
    return lo;
}

// N == 32 * VEC; lane l owns the output columns [l * VEC, l * VEC + VEC).  The inner loop is kept to
// two shuffles, one 32 x 32 -> 64-bit multiply-add for the address, one load and VEC FMAs per entry:
// the kernel issues an instruction in most cycles, so every instruction per entry counts.
// What bounds it then is the load/store unit's data pipe, which also carries the shuffles: 256 B of G
// and two 128 B shuffles per entry at N = 64.  PACKED (per-gene offsets, cells below 2^24) halves the
// shuffles: a lane hands out (cell << 8 | code) and every lane decodes the value itself -- the same
// fused multiply-add, so the same bits.
template<int VEC, bool ALIGNED, bool PACKED>
__global__ void __launch_bounds__(kGatherWarps * 32) qcsr_transpose_gather_kernel(const gather_params p) {
    __shared__ float part[kGatherWarps][32 * VEC];
    __shared__ unsigned next_gene;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool row_policy = p.policy == CB200_DECODE_COLUMN_SCALE_ROW_OFFSET;
    const std::uint32_t g_row_bytes = static_cast<std::uint32_t>(p.g_ld) * 4u; // the launcher checks it fits
    for (;;) {
        if (threadIdx.x == 0) next_gene = atomicAdd(p.queue, 1u);
        __syncthreads();
        if (next_gene >= p.cols) return;
        const std::int64_t gene = p.gene_order != nullptr ? __ldg(p.gene_order + next_gene) : static_cast<std::int64_t>(next_gene);
        std::int64_t lo = __ldg(p.col_ptr + gene), hi = __ldg(p.col_ptr + gene + 1);
        if (p.restrict_rows) {
            lo = gather_lower_bound(p.row_idx, lo, hi, p.row_begin);
            hi = gather_lower_bound(p.row_idx, lo, hi, p.row_end);
        }
        const float scale = p.scales != nullptr ? __ldg(p.scales + gene) : 1.0f;
        const float gene_offset = (!row_policy && p.offsets != nullptr) ? __ldg(p.offsets + gene) : 0.0f;
        float acc[VEC];
#pragma unroll
        for (int k = 0; k < VEC; ++k) acc[k] = 0.0f;
        const char *g_lane = reinterpret_cast<const char *>(p.g + lane * VEC);
        for (std::int64_t chunk = lo + static_cast<std::int64_t>(warp) * kGatherChunk; chunk < hi;
             chunk += static_cast<std::int64_t>(kGatherWarps) * kGatherChunk) {
            const std::int64_t chunk_end = min(hi, chunk + kGatherChunk);
            for (std::int64_t base = chunk; base < chunk_end; base += 32) {
                const int count = static_cast<int>(min(static_cast<std::int64_t>(32), chunk_end - base));
                int row = 0;
                float value = 0.0f;
                if (lane < count) {
                    row = __ldg(p.row_idx + base + lane);
                    const unsigned code = __ldg(p.codes + base + lane);
                    if constexpr (PACKED) {
                        row = static_cast<int>((static_cast<unsigned>(row) << 8) | code);
                    } else {
                        const float offset = row_policy ? (p.offsets != nullptr ? __ldg(p.offsets + row) : 0.0f) : gene_offset;
                        value = fmaf(static_cast<float>(code), scale, offset);
                    }
                }
                if (count == 32) {
#pragma unroll
                    for (int j0 = 0; j0 < 32; j0 += 8) { // eight rows of G in flight, then their FMAs in order
                        float gv[8][VEC], vv[8];
#pragma unroll
                        for (int u = 0; u < 8; ++u) {
                            unsigned r = static_cast<unsigned>(__shfl_sync(0xffffffffu, row, j0 + u));
                            if constexpr (PACKED) {
                                vv[u] = fmaf(low_byte_to_float(r), scale, gene_offset);
                                r >>= 8;
                            } else {
                                vv[u] = __shfl_sync(0xffffffffu, value, j0 + u);
                            }
                            gather_load<VEC, ALIGNED>(
                                reinterpret_cast<const float *>(g_lane + static_cast<std::uint64_t>(r) * g_row_bytes), gv[u]);
                        }
#pragma unroll
                        for (int u = 0; u < 8; ++u)
#pragma unroll
                            for (int k = 0; k < VEC; ++k) acc[k] = fmaf(vv[u], gv[u][k], acc[k]);
                    }
                } else {
                    for (int j = 0; j < count; ++j) {
                        unsigned r = static_cast<unsigned>(__shfl_sync(0xffffffffu, row, j));
                        float v;
                        if constexpr (PACKED) {
                            v = fmaf(low_byte_to_float(r), scale, gene_offset);
                            r >>= 8;
                        } else {
                            v = __shfl_sync(0xffffffffu, value, j);
                        }
                        float gv[VEC];
                        gather_load<VEC, ALIGNED>(
                            reinterpret_cast<const float *>(g_lane + static_cast<std::uint64_t>(r) * g_row_bytes), gv);
#pragma unroll
                        for (int k = 0; k < VEC; ++k) acc[k] = fmaf(v, gv[k], acc[k]);
                    }
                }
            }
        }
#pragma unroll
        for (int k = 0; k < VEC; ++k) part[warp][lane * VEC + k] = acc[k];
        __syncthreads();
        if (threadIdx.x < 32 * VEC) {
            float sum = part[0][threadIdx.x];
#pragma unroll
            for (int w = 1; w < kGatherWarps; ++w) sum = sum + part[w][threadIdx.x];
            float *dst = p.out + gene * p.out_ld + threadIdx.x;
            float result = p.alpha * sum;
            if (p.beta != 0.0f) result = fmaf(p.beta, *dst, result);
            *dst = result;
        }
    }
}

} // namespace

bool qcsr_gene_major_shape_ok(std::int64_t rows, std::int64_t cols, int bits) {
    return rows >= 0 && rows < (std::int64_t{1} << 31) && cols >= 1 && cols < (std::int64_t{1} << 31) && (bits == 8 || bits == 4);
}

std::uint64_t qcsr_gene_major_workspace_bytes(std::int64_t rows, std::int64_t cols) {
    const std::uint64_t blocks = static_cast<std::uint64_t>((rows + kBlockRows - 1) / kBlockRows);
    return 256u + blocks * static_cast<std::uint64_t>(cols) * 4u;
}

cb200_status launch_qcsr_gene_major(const qcsr_view &x, std::int64_t *col_ptr, std::int32_t *row_idx, std::uint8_t *codes,
                                    void *workspace, std::uint64_t workspace_bytes, cudaStream_t stream) {
    if (!qcsr_gene_major_shape_ok(x.rows, x.cols, x.bits))
        return fail(CB200_STATUS_UNSUPPORTED, "gene-major copy: up to 2^31 - 1 rows and genes, 8- or 4-bit codes");
    if (x.bits == 4 && x.packed_row_ptr == nullptr) return fail(CB200_STATUS_INVALID_ARGUMENT, "4-bit codes need packed_row_ptr");
    if (col_ptr == nullptr || (x.nnz > 0 && (row_idx == nullptr || codes == nullptr)) || x.row_ptr == nullptr)
        return fail(CB200_STATUS_INVALID_ARGUMENT, "null array");
    if (workspace == nullptr || workspace_bytes < qcsr_gene_major_workspace_bytes(x.rows, x.cols))
        return fail(CB200_STATUS_INSUFFICIENT_WORKSPACE, "gene-major copy needs %llu workspace bytes",
                    static_cast<unsigned long long>(qcsr_gene_major_workspace_bytes(x.rows, x.cols)));
    gm_params p{};
    p.row_ptr = x.row_ptr; p.packed_row_ptr = x.packed_row_ptr; p.col_idx = x.col_idx; p.packed = x.packed;
    p.rows = x.rows; p.cols = x.cols; p.blocks = (x.rows + kBlockRows - 1) / kBlockRows;
    p.status = static_cast<int *>(workspace);
    p.counts = reinterpret_cast<std::uint32_t *>(static_cast<unsigned char *>(workspace) + 256);
    p.col_ptr = col_ptr; p.row_idx = row_idx; p.codes = codes;
    CB200_CUDA_OK(cudaMemsetAsync(workspace, 0, 256, stream));
    if (p.blocks == 0) {
        CB200_CUDA_OK(cudaMemsetAsync(col_ptr, 0, static_cast<std::size_t>(x.cols + 1) * 8u, stream));
        return CB200_STATUS_SUCCESS;
    }
    const std::size_t count_smem = static_cast<std::size_t>(std::min<std::int64_t>(x.cols, kCountGenes)) * 4u;
    const std::size_t fill_smem = fill_smem_bytes();
    CB200_CUDA_OK(cudaFuncSetAttribute(gm_count_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(count_smem)));
    for (std::int64_t g0 = 0; g0 < x.cols; g0 += kCountGenes)
        gm_count_kernel<<<static_cast<unsigned>(p.blocks), kBuildThreads, count_smem, stream>>>(
            p, static_cast<int>(g0), static_cast<int>(std::min<std::int64_t>(x.cols, g0 + kCountGenes)));
    gm_block_scan_kernel<<<static_cast<unsigned>((x.cols + 255) / 256), 256, 0, stream>>>(p);
    gm_col_scan_kernel<<<1, 1024, 0, stream>>>(col_ptr, x.cols);
    if (x.bits == 8) {
        CB200_CUDA_OK(cudaFuncSetAttribute(gm_fill_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(fill_smem)));
        for (std::int64_t g0 = 0; g0 < x.cols; g0 += kFillGenes)
            gm_fill_kernel<8><<<static_cast<unsigned>(p.blocks), kBuildThreads, fill_smem, stream>>>(
                p, static_cast<int>(g0), static_cast<int>(std::min<std::int64_t>(x.cols, g0 + kFillGenes)));
    } else {
        CB200_CUDA_OK(cudaFuncSetAttribute(gm_fill_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(fill_smem)));
        for (std::int64_t g0 = 0; g0 < x.cols; g0 += kFillGenes)
            gm_fill_kernel<4><<<static_cast<unsigned>(p.blocks), kBuildThreads, fill_smem, stream>>>(
                p, static_cast<int>(g0), static_cast<int>(std::min<std::int64_t>(x.cols, g0 + kFillGenes)));
    }
    count_launch(2 + static_cast<std::uint64_t>((x.cols + kCountGenes - 1) / kCountGenes) +
                 static_cast<std::uint64_t>((x.cols + kFillGenes - 1) / kFillGenes));
    CB200_CUDA_OK(cudaGetLastError());
    return CB200_STATUS_SUCCESS;
}

std::uint64_t qcsr_gene_major_layout_bytes_bound(std::int64_t rows, std::int64_t cols, std::int64_t nnz) {
    const std::uint64_t entries = static_cast<std::uint64_t>(std::max<std::int64_t>(nnz, 1));
    return device_arena::rounded(qcsr_gene_major_workspace_bytes(rows, cols)) + device_arena::rounded(static_cast<std::uint64_t>(cols + 1) * 8u) +
           device_arena::rounded(entries * 4u) + device_arena::rounded(entries) + device_arena::rounded(static_cast<std::uint64_t>(cols) * 4u);
}

cb200_status build_gene_major_layout(const qcsr_view &x, device_arena &arena, cudaStream_t stream, gene_major_layout *out) {
    *out = gene_major_layout{};
    if (!qcsr_gene_major_shape_ok(x.rows, x.cols, x.bits)) return fail(CB200_STATUS_UNSUPPORTED, "shape outside the gene-major copy");
    const std::uint64_t ws_bytes = qcsr_gene_major_workspace_bytes(x.rows, x.cols);
    const std::size_t ptr_bytes = static_cast<std::size_t>(x.cols + 1) * 8u;
    const std::size_t idx_bytes = static_cast<std::size_t>(std::max<std::int64_t>(x.nnz, 1)) * 4u;
    const std::size_t code_bytes = static_cast<std::size_t>(std::max<std::int64_t>(x.nnz, 1));
    const std::size_t order_bytes = static_cast<std::size_t>(std::max<std::int64_t>(x.cols, 1)) * sizeof(std::int32_t);
    void *ws = arena.take(ws_bytes);
    out->col_ptr = static_cast<std::int64_t *>(arena.take(ptr_bytes));
    out->row_idx = static_cast<std::int32_t *>(arena.take(idx_bytes));
    out->codes = static_cast<std::uint8_t *>(arena.take(code_bytes));
    out->gene_order = static_cast<std::int32_t *>(arena.take(order_bytes));
    const auto give_up = [&](cb200_status st) {
        arena.give_back(out->gene_order, order_bytes);
        arena.give_back(out->codes, code_bytes);
        arena.give_back(out->row_idx, idx_bytes);
        arena.give_back(out->col_ptr, ptr_bytes);
        arena.give_back(ws, ws_bytes);
        *out = gene_major_layout{};
        return st;
    };
    if (ws == nullptr || out->col_ptr == nullptr || out->row_idx == nullptr || out->codes == nullptr || out->gene_order == nullptr)
        return give_up(fail(CB200_STATUS_INSUFFICIENT_WORKSPACE, "no device memory for the gene-major copy"));
    cb200_status st = launch_qcsr_gene_major(x, out->col_ptr, out->row_idx, out->codes, ws, ws_bytes, stream);
    if (st != CB200_STATUS_SUCCESS) return give_up(st);
    int status = 0;
    std::vector<std::int64_t> ptr(static_cast<std::size_t>(x.cols) + 1u);
    cudaError_t err = cudaMemcpyAsync(&status, ws, sizeof(int), cudaMemcpyDeviceToHost, stream);
    if (err == cudaSuccess) err = cudaMemcpyAsync(ptr.data(), out->col_ptr, ptr_bytes, cudaMemcpyDeviceToHost, stream);
    if (err == cudaSuccess) err = cudaStreamSynchronize(stream);
    if (err != cudaSuccess) return give_up(fail(CB200_STATUS_CUDA_ERROR, "gene-major copy: %s", cudaGetErrorString(err)));
    if (status != 0) return give_up(fail(CB200_STATUS_INVALID_SHAPE, "a column index lies outside the matrix"));
    // genes by descending entry count: a gene is one CTA's work, so the long ones have to start first
    std::vector<std::int32_t> order(static_cast<std::size_t>(x.cols));
    for (std::int64_t c = 0; c < x.cols; ++c) order[static_cast<std::size_t>(c)] = static_cast<std::int32_t>(c);
    std::stable_sort(order.begin(), order.end(), [&](std::int32_t a, std::int32_t b) {
        return ptr[static_cast<std::size_t>(a) + 1u] - ptr[static_cast<std::size_t>(a)] >
               ptr[static_cast<std::size_t>(b) + 1u] - ptr[static_cast<std::size_t>(b)];
    });
    err = cudaMemcpyAsync(out->gene_order, order.data(), order.size() * sizeof(std::int32_t), cudaMemcpyHostToDevice, stream);
    if (err == cudaSuccess) err = cudaStreamSynchronize(stream);
    if (err != cudaSuccess) return give_up(fail(CB200_STATUS_CUDA_ERROR, "gene-major copy: %s", cudaGetErrorString(err)));
    arena.give_back(ws, ws_bytes);
    out->bytes = ptr_bytes + idx_bytes + code_bytes + static_cast<std::size_t>(x.cols) * sizeof(std::int32_t);
    out->src_row_ptr = x.row_ptr; out->src_col_idx = x.col_idx; out->src_packed = x.packed;
    return CB200_STATUS_SUCCESS;
}

bool qcsr_transpose_gather_shape_ok(std::int64_t n) { return n == 32 || n == 64 || n == 128; }
std::uint64_t qcsr_transpose_gather_workspace_bytes() { return 256u; }

cb200_status launch_qcsr_transpose_gather(const qcsr_view &x, const dense_args &d, std::int64_t row_begin,
                                          std::int64_t row_end, const gene_major_layout &layout, void *workspace,
                                          std::uint64_t workspace_bytes, int sm_count, cudaStream_t stream) {
    if (d.n == 0 || x.cols == 0) return CB200_STATUS_SUCCESS;
    if (d.dense_dtype != CB200_DTYPE_F32) return fail(CB200_STATUS_UNSUPPORTED, "transpose takes an fp32 dense operand");
    if (!qcsr_transpose_gather_shape_ok(d.n)) return fail(CB200_STATUS_UNSUPPORTED, "the order-fixed transpose covers N in {32, 64, 128}");
    if (layout.col_ptr == nullptr) return fail(CB200_STATUS_INVALID_ARGUMENT, "no gene-major copy");
    if (layout.src_row_ptr != x.row_ptr || layout.src_col_idx != x.col_idx || layout.src_packed != x.packed)
        return fail(CB200_STATUS_STALE_STRUCTURE, "the gene-major copy was built from other arrays");
    if (workspace == nullptr || workspace_bytes < qcsr_transpose_gather_workspace_bytes())
        return fail(CB200_STATUS_INSUFFICIENT_WORKSPACE, "the order-fixed transpose needs 256 workspace bytes");
    gather_params p{};
    p.col_ptr = layout.col_ptr; p.row_idx = layout.row_idx; p.codes = layout.codes;
    p.scales = x.scales; p.offsets = x.offsets; p.g = static_cast<const float *>(d.dense); p.out = d.out;
    p.g_ld = d.dense_ld; p.out_ld = d.out_ld; p.cols = x.cols;
    p.row_begin = row_begin; p.row_end = std::max(row_begin, row_end);
    p.policy = x.policy; p.restrict_rows = (row_begin > 0 || row_end < x.rows) ? 1 : 0;
    const int vec = static_cast<int>(d.n / 32);
    p.aligned = (reinterpret_cast<std::uintptr_t>(d.dense) % (4u * vec) == 0u) && ((d.dense_ld * 4) % (4 * vec) == 0) ? 1 : 0;
    p.alpha = d.alpha; p.beta = d.beta;
    // word 0 of the workspace is the status word every schedule keeps there (this kernel waits on nothing, so it
    // stays 0); the gene queue is the word at byte 64
    p.queue = static_cast<unsigned *>(workspace) + 16;
    p.gene_order = layout.gene_order;
    CB200_CUDA_OK(cudaMemsetAsync(workspace, 0, 128, stream));
    const unsigned grid = static_cast<unsigned>(std::min<std::int64_t>(x.cols, static_cast<std::int64_t>(sm_count) * 8));
    if (d.dense_ld < 0 || d.dense_ld >= (std::int64_t{1} << 30))
        return fail(CB200_STATUS_UNSUPPORTED, "the order-fixed transpose takes rows of G below 4 GB");
    const bool packed = x.policy != CB200_DECODE_COLUMN_SCALE_ROW_OFFSET && x.rows <= (std::int64_t{1} << 24) && p.aligned;
    const unsigned threads = kGatherWarps * 32;
    if (packed) {
        if (vec == 1) qcsr_transpose_gather_kernel<1, true, true><<<grid, threads, 0, stream>>>(p);
        else if (vec == 2) qcsr_transpose_gather_kernel<2, true, true><<<grid, threads, 0, stream>>>(p);
        else qcsr_transpose_gather_kernel<4, true, true><<<grid, threads, 0, stream>>>(p);
    } else if (vec == 1) qcsr_transpose_gather_kernel<1, true, false><<<grid, threads, 0, stream>>>(p);
    else if (vec == 2 && p.aligned) qcsr_transpose_gather_kernel<2, true, false><<<grid, threads, 0, stream>>>(p);
    else if (vec == 2) qcsr_transpose_gather_kernel<2, false, false><<<grid, threads, 0, stream>>>(p);
    else if (p.aligned) qcsr_transpose_gather_kernel<4, true, false><<<grid, threads, 0, stream>>>(p);
    else qcsr_transpose_gather_kernel<4, false, false><<<grid, threads, 0, stream>>>(p);
    count_launch();
    CB200_CUDA_OK(cudaGetLastError());
    return CB200_STATUS_SUCCESS;
}

} // namespace cb200

extern "C" uint64_t cb200_qcsr_gene_major_workspace(int64_t rows, int64_t cols) {
    if (!cb200::qcsr_gene_major_shape_ok(rows, cols, 8)) return 0;
    return cb200::qcsr_gene_major_workspace_bytes(rows, cols);
}

extern "C" cb200_status cb200_qcsr_gene_major(const cb200_qcsr *x, int64_t *col_ptr, int32_t *row_idx, uint8_t *codes,
                                              void *workspace, uint64_t workspace_bytes, int32_t device, void *stream) {
    using namespace cb200;
    clear_error();
    if (x == nullptr || x->version != CB200_ABI_VERSION || x->size < sizeof(cb200_qcsr))
        return fail(CB200_STATUS_INVALID_ARGUMENT, "bad cb200_qcsr header");
    device_scope scope(device);
    CB200_CUDA_OK(scope.status);
    const qcsr_view view{x->rows, x->cols, x->nnz, x->bits, x->policy, x->row_ptr, x->packed_row_ptr,
                         x->col_idx, x->packed_values, x->scales, x->offsets};
    return launch_qcsr_gene_major(view, col_ptr, row_idx, codes, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}
