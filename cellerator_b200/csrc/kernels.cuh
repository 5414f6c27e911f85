// Launchers of the sm_100a kernels, called by the C-ABI layer (capi.cu).  Each takes device
// pointers and a stream, enqueues, and returns; none allocates or synchronises.
#pragma once

#include "common.cuh"

namespace cb200 {

struct qcsr_view {
    std::int64_t rows, cols, nnz;
    int bits, policy;
    const std::int64_t *row_ptr;
    const std::int64_t *packed_row_ptr; // may be null when bits == 8
    const std::int32_t *col_idx;
    const std::uint8_t *packed;
    const float *scales;
    const float *offsets;
};

struct dense_args {
    const void *dense; // W or G
    std::int64_t dense_ld;
    int dense_dtype; // CB200_DTYPE_F32 | CB200_DTYPE_BF16
    float *out;
    std::int64_t out_ld;
    std::int64_t n;
    float alpha, beta;
    const float *bias = nullptr;          // composed epilogue of the forward projections:
    int epilogue = CB200_EPILOGUE_NONE;   // out = act(alpha * product + beta * out + bias[column])
};

enum class fwd_schedule : int { warp_per_row = 0, gene_tiled = 1, tensor_windows = 2, tensor_blocked = 3 };

// Device memory a prepared operation keeps.  Two modes: pieces carved out of a block the caller owns (a
// session's persistent reservation: nothing is allocated or freed here), or pieces allocated one by one
// with cudaMalloc and freed when the operation is destroyed.  Pieces are 256-byte aligned.
struct device_arena {
    unsigned char *base = nullptr;
    std::uint64_t capacity = 0, used = 0;
    bool borrowed = false;
    static constexpr int kMaxOwned = 24;
    void *owned[kMaxOwned] = {};
    int owned_count = 0;

    static std::uint64_t rounded(std::uint64_t bytes) { return (bytes + 255u) & ~static_cast<std::uint64_t>(255u); }
    // nullptr: the borrowed block has no room left, or the allocation failed (the CUDA error is cleared)
    void *take(std::uint64_t bytes) {
        const std::uint64_t need = rounded(bytes == 0u ? 1u : bytes);
        if (borrowed) {
            if (need > capacity - used) return nullptr;
            void *p = base + used;
            used += need;
            return p;
        }
        if (owned_count == kMaxOwned) return nullptr;
        void *p = nullptr;
        if (cudaMalloc(&p, need) != cudaSuccess) {
            cudaGetLastError();
            return nullptr;
        }
        owned[owned_count++] = p;
        used += need;
        return p;
    }
    // A piece that is no longer needed: freed at once when owned; borrowed memory stays with its owner.
    void give_back(void *p, std::uint64_t bytes) {
        if (p == nullptr || borrowed) return;
        for (int i = 0; i < owned_count; ++i) {
            if (owned[i] != p) continue;
            cudaFree(p);
            owned[i] = owned[--owned_count];
            used -= rounded(bytes == 0u ? 1u : bytes);
            return;
        }
    }
    void release_all() {
        for (int i = 0; i < owned_count; ++i) cudaFree(owned[i]);
        owned_count = 0;
        used = 0;
    }
};

// Gene-tiled kernel (W staged through shared memory); *taken is false when the shape is outside
// what it covers, and the caller then runs the warp-per-row kernel.
bool qcsr_forward_tiled_supported(const qcsr_view &x, const dense_args &d);
// global scratch the tiled kernel needs, whatever the matrix: one status block (first word = status)
constexpr std::uint64_t qcsr_tiled_workspace_bytes() { return 256u; }
cb200_status launch_qcsr_forward_tiled(const qcsr_view &x, const dense_args &d, std::int64_t row_begin,
                                       std::int64_t row_end, int *status_word, const std::int32_t *row_order,
                                       int sm_count, cudaStream_t stream, bool *taken);

// Tensor-core kernel for bf16 products (decoded values rounded to bf16): entries are scattered
// into dense operand tiles in shared memory, window by window of 64 genes.  `workspace` holds the
// status word and W re-laid per window; *taken is false when the shape or workspace rules it out.
bool qcsr_forward_mma_supported(const qcsr_view &x, const dense_args &d);
std::uint64_t qcsr_mma_workspace_bytes(std::int64_t cols, std::int64_t n);
cb200_status launch_qcsr_forward_mma(const qcsr_view &x, const dense_args &d, std::int64_t row_begin,
                                     std::int64_t row_end, void *workspace, std::uint64_t workspace_bytes,
                                     const std::int32_t *row_order, int sm_count, cudaStream_t stream, bool *taken);

// Window-blocked copy of a matrix, built once at prepare time for the tensor-core kernel below:
// groups of 256 consecutive rows, inside a group the entries ordered by window of 128 genes, one
// 32-bit word per entry; seg_ptr[group * windows + window] is the first word of a segment.
struct blocked_layout {
    std::uint32_t *entries = nullptr;
    std::int64_t *seg_ptr = nullptr;
    std::int64_t groups = 0;
    int windows = 0;
    std::int64_t total_entries = 0;
    std::uint64_t bytes = 0;
    const void *src_row_ptr = nullptr, *src_col_idx = nullptr, *src_packed = nullptr; // arrays it was built from
    // Dense operand tiles (forward, bf16 products): per (group, window) the 64 KB tile of decoded bf16
    // values in the shared-memory image the MMA reads.  When set, entries / seg_ptr are gone.
    unsigned char *dense_tiles = nullptr;
    // baked: an entry word holds the decoded bf16 value (bits 0-15) and the byte position / 2 (bits
    // 16-30) instead of code and gene: the forward kernel stores it as it is, no table look-up.
    bool baked = false;
    // second array of baked words for the split-product schedules: bf16(value - hi) under the same
    // seg_ptr, so that the hi and the lo pass both run the look-up-free kernels
    std::uint32_t *entries_lo = nullptr;
    // the baked words hold byte positions in the transpose kernel's gene-major tile, not the forward one
    bool baked_gene_major = false;
    const void *src_scales = nullptr, *src_offsets = nullptr; // baked into the entries / the tiles
    // the baked words (and the dense tiles made from them) hold fp16(value * value_scale) instead of bf16(value):
    // 11 significant bits instead of 8; value_scale is a power of two chosen at prepare from the largest decoded
    // magnitude the scales and offsets allow (forward operations; the transpose keeps bf16)
    bool half_values = false;
    float value_scale = 1.0f;
    // Code tiles (forward, 4-bit codes, schedule "tensor_codes"): per (group, half window of 64 genes) a 16 KB stage
    // with one byte per (cell, gene), 0 = nothing stored, else code + 240.  When set, entries / seg_ptr are gone.
    // Scales and offsets are NOT in it: they are applied at launch.
    unsigned char *code_tiles = nullptr;
};
bool qcsr_blocked_shape_ok(std::int64_t rows, std::int64_t cols, std::int64_t n, int bits, int dense_dtype);
std::uint64_t qcsr_blocked_workspace_bytes(std::int64_t cols, std::int64_t n);
// Current device; memory from `arena`, kernels on `stream`, which is waited for.
// bake: decoded values in the entry words (forward, bf16 products only)
// bake_lo (needs bake): also the array of the next eight mantissa bits (split-product schedules)
// gene_major (needs bake): byte positions of the transpose kernel's tile in the baked words
cb200_status build_blocked_layout(const qcsr_view &x, bool bake, bool bake_lo, bool gene_major, device_arena &arena,
                                  cudaStream_t stream, blocked_layout *out);
// upper bound of what build_blocked_layout takes from the arena (scratch of the build included)
std::uint64_t qcsr_blocked_layout_bytes_bound(std::int64_t rows, std::int64_t cols, std::int64_t nnz, bool bake_lo);
// Dense operand tiles from the window-blocked copy (decoded values of `x` baked in; the entry words go
// back to the arena).  *built stays false, the copy untouched, when the arena has no room.  Waits for `stream`.
std::uint64_t qcsr_dense_tile_bytes(std::int64_t rows, std::int64_t cols);
cb200_status densify_blocked_layout(const qcsr_view &x, blocked_layout *layout, device_arena &arena, cudaStream_t stream,
                                    bool *built);
// Code tiles from the window-blocked copy built with code words (bake == false); the entry words go back to the arena.
bool qcsr_codes_shape_ok(std::int64_t rows, std::int64_t cols, std::int64_t n, int bits, int policy, int dense_dtype);
std::uint64_t qcsr_code_tile_bytes(std::int64_t rows, std::int64_t cols);
std::uint64_t qcsr_codes_workspace_bytes(std::int64_t cols, std::int64_t n);
cb200_status bytify_blocked_layout(blocked_layout *layout, device_arena &arena, cudaStream_t stream, bool *built);
cb200_status launch_qcsr_forward_codes(const qcsr_view &x, const dense_args &d, std::int64_t row_begin,
                                       std::int64_t row_end, void *workspace, std::uint64_t workspace_bytes,
                                       const blocked_layout &layout, int sm_count, cudaStream_t stream, bool *taken);
// *taken as for the blocked launch below; the tiles hold bf16(value): one pass of bf16 products only
cb200_status launch_qcsr_forward_dense(const qcsr_view &x, const dense_args &d, std::int64_t row_begin,
                                       std::int64_t row_end, void *workspace, std::uint64_t workspace_bytes,
                                       const blocked_layout &layout, int sm_count, cudaStream_t stream, bool *taken);
// *taken is false when the launch cannot use the copy (row range not starting on a group boundary,
// workspace too small, ...); a matrix other than the one the copy was built from is an error.
// split_products == false: one pass of bf16 products (bf16 W only); true: fp32 products rebuilt from
// bf16 pieces in two (bf16 W) or three (fp32 W) passes.
cb200_status launch_qcsr_forward_blocked(const qcsr_view &x, const dense_args &d, std::int64_t row_begin,
                                         std::int64_t row_end, void *workspace, std::uint64_t workspace_bytes,
                                         const blocked_layout &layout, bool split_products, int sm_count,
                                         cudaStream_t stream, bool *taken);

// Y[r,:] = alpha * sum_i deq(code_i) * W[col_i,:] + beta * Y[r,:]  for r in [row_begin,row_end)
cb200_status launch_qcsr_forward(const qcsr_view &x, const dense_args &d, std::int64_t row_begin,
                                 std::int64_t row_end, fwd_schedule schedule, const void *persistent,
                                 const blocked_layout *blocked, bool split_products, void *workspace,
                                 std::uint64_t workspace_bytes, int sm_count, cudaStream_t stream);

// Transpose on the tensor cores from the window-blocked copy (N in {32, 64}).  split_products == false:
// one pass of bf16 products; true: fp32 products rebuilt from three bf16 passes (hi*hi + hi*lo + lo*hi).
bool qcsr_transpose_blocked_shape_ok(std::int64_t rows, std::int64_t cols, std::int64_t n, int bits);
std::uint64_t qcsr_transpose_blocked_workspace_bytes(std::int64_t rows, std::int64_t cols, std::int64_t n);
cb200_status launch_qcsr_transpose_blocked(const qcsr_view &x, const dense_args &d, std::int64_t row_begin,
                                           std::int64_t row_end, void *workspace, std::uint64_t workspace_bytes,
                                           const blocked_layout &layout, bool split_products, int sm_count,
                                           cudaStream_t stream, bool *taken);

// G'[g,:] = alpha * sum_{r in range, col_i == g} deq(code_i) * G[r,:] + beta * G'[g,:]
// `blocked` (optional): the window-blocked copy of a prepared bf16-product operation.
cb200_status launch_qcsr_transpose(const qcsr_view &x, const dense_args &d, std::int64_t row_begin,
                                   std::int64_t row_end, const blocked_layout *blocked, bool split_products,
                                   void *workspace, std::uint64_t workspace_bytes, int sm_count, cudaStream_t stream);
std::uint64_t qcsr_transpose_workspace_bytes(std::int64_t cols, std::int64_t n, int sm_count);

// Gene-major copy (a CSC) of a matrix: cells ascend inside every gene; one code per byte (4-bit
// sources are widened).  Built once at prepare time for the order-fixed transpose below.
struct gene_major_layout {
    std::int64_t *col_ptr = nullptr;  // cols + 1
    std::int32_t *row_idx = nullptr;  // nnz
    std::uint8_t *codes = nullptr;    // nnz
    std::int32_t *gene_order = nullptr; // cols: genes by descending entry count (the gather kernel starts the long ones first)
    std::uint64_t bytes = 0;
    const void *src_row_ptr = nullptr, *src_col_idx = nullptr, *src_packed = nullptr; // arrays it was built from
};
bool qcsr_gene_major_shape_ok(std::int64_t rows, std::int64_t cols, int bits);
std::uint64_t qcsr_gene_major_workspace_bytes(std::int64_t rows, std::int64_t cols);
// Enqueues the stable counting sort into caller arrays; the first word of `workspace` ends up
// non-zero when a column index lies outside the matrix.
cb200_status launch_qcsr_gene_major(const qcsr_view &x, std::int64_t *col_ptr, std::int32_t *row_idx, std::uint8_t *codes,
                                    void *workspace, std::uint64_t workspace_bytes, cudaStream_t stream);
// current device; memory from `arena`, kernels and copies on `stream`, which is waited for
cb200_status build_gene_major_layout(const qcsr_view &x, device_arena &arena, cudaStream_t stream, gene_major_layout *out);
std::uint64_t qcsr_gene_major_layout_bytes_bound(std::int64_t rows, std::int64_t cols, std::int64_t nnz);
// Transpose with a fixed order of the fp32 sums (same bits on every run), N in {32, 64, 128}:
// gathers rows of G gene by gene from the gene-major copy.
bool qcsr_transpose_gather_shape_ok(std::int64_t n);
std::uint64_t qcsr_transpose_gather_workspace_bytes();
cb200_status launch_qcsr_transpose_gather(const qcsr_view &x, const dense_args &d, std::int64_t row_begin,
                                          std::int64_t row_end, const gene_major_layout &layout, void *workspace,
                                          std::uint64_t workspace_bytes, int sm_count, cudaStream_t stream);

struct qbell_view {
    std::int64_t rows, cols;
    int block_size, ell_cols;
    std::int64_t row_stride_bytes;
    int bits, policy;
    const std::uint32_t *block_col_idx;
    const std::uint8_t *packed;
    const float *scales;
    const float *offsets;
};

// `workspace` (optional) holds the transposed bf16 copy of W that the tensor-core kernel needs;
// without it (or for shapes that kernel does not cover) the CUDA-core kernel runs.
// cuda_cores_only: the caller asked for the CUDA-core kernel (schedule hint "cuda_cores")
cb200_status launch_qbell_forward(const qbell_view &x, const dense_args &d, std::int64_t row_begin,
                                  std::int64_t row_end, void *workspace, std::uint64_t workspace_bytes, int sm_count,
                                  bool cuda_cores_only, cudaStream_t stream);
std::uint64_t qbell_tcgen05_workspace_bytes(std::int64_t cols, std::int64_t n);

cb200_status launch_quantize_rows(const qcsr_view &x, std::int64_t row_begin, std::int64_t row_end,
                                  const float *values, cudaStream_t stream);
cb200_status launch_dequantize_rows(const qcsr_view &x, std::int64_t row_begin, std::int64_t row_end,
                                    float *values, cudaStream_t stream);

cb200_status launch_qbell_quantize_rows(const qbell_view &x, std::int64_t row_begin, std::int64_t row_end,
                                        const float *values_by_slot, cudaStream_t stream);
cb200_status launch_qbell_dequantize_rows(const qbell_view &x, std::int64_t row_begin, std::int64_t row_end,
                                          float *values_by_slot, cudaStream_t stream);

} // namespace cb200
