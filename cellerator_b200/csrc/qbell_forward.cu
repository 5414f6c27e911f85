// Quantized Blocked-ELL projection  Y = alpha * deq(X_bell) * W + beta * Y  on CUDA cores.
//
// Reference counterpart: quantized_blocked_ell_spmm_fwd_kernel_
// (src/compute/sparse/project/kernels/quantized_blocked_ell_spmm_fwd_kernel_.cuh:1-39, launcher
// src/compute/sparse/project/project.cu:72-168): one thread per (row, output column), each
// re-reading and re-decoding every slot of the row.  Semantics kept: every slot of a present
// block is decoded and multiplied (structurally empty slots included), a block whose index is
// 0xffffffff is skipped, and slots whose gene index is >= cols are skipped.
//
// This is the general kernel (any block size, bit width 4 or 8, fp32 or bf16 W): one warp
// per row, 32 slots per step decoded by the 32 lanes, then the same lane-group walk over W
// rows as the CSR kernel.  The tensor-core kernel for 32x32 blocks lives in
// qbell_tcgen05.cu and is selected by the launcher when its shape constraints hold.
#include "kernels.cuh"

#include <cstdlib>

namespace cb200 {

cb200_status launch_qbell_tcgen05(const qbell_view &x, const dense_args &d, std::int64_t row_begin,
                                  std::int64_t row_end, void *workspace, std::uint64_t workspace_bytes, int sm_count,
                                  cudaStream_t stream, bool *taken);

namespace {

struct bell_params {
    std::int64_t rows, cols;
    int block_size, ell_cols, width;
    std::int64_t row_stride;
    const std::uint32_t *block_col_idx;
    const std::uint8_t *packed;
    const float *scales;
    const float *offsets;
    const void *w;
    float *y;
    std::int64_t w_ld, y_ld;
    std::int64_t row_begin, row_end;
    int n, policy;
    float alpha, beta;
    const float *bias;
    int epilogue;
};

template<int BITS>
__device__ __forceinline__ void decode_slot(const bell_params &p, const std::uint8_t *row_bytes, std::int64_t row_block,
                                            float row_offset, bool row_policy, int slot, int &gene, float &value,
                                            bool &valid) {
    gene = 0;
    value = 0.0f;
    valid = false;
    if (slot >= p.ell_cols) return;
    const std::uint32_t bc = __ldg(p.block_col_idx + row_block * p.width + slot / p.block_size);
    if (bc == 0xffffffffu) return;
    const std::int64_t g = static_cast<std::int64_t>(bc) * p.block_size + slot % p.block_size;
    if (g >= p.cols) return;
    unsigned code;
    if constexpr (BITS == 8) {
        code = __ldg(row_bytes + slot);
    } else {
        const unsigned byte = __ldg(row_bytes + (slot >> 1));
        code = (slot & 1) ? (byte >> 4) : (byte & 0xfu);
    }
    const float scale = p.scales != nullptr ? __ldg(p.scales + g) : 1.0f;
    const float offset = row_policy ? row_offset : (p.offsets != nullptr ? __ldg(p.offsets + g) : 0.0f);
    gene = static_cast<int>(g);
    value = fmaf(static_cast<float>(code), scale, offset);
    valid = true;
}

template<int BITS, typename WT, int LPN>
__global__ void __launch_bounds__(256) qbell_fwd_warp_row_kernel(const bell_params p) {
    constexpr int NPS = 32 / LPN;
    const int lane = threadIdx.x & 31;
    const std::int64_t row = p.row_begin + (static_cast<std::int64_t>(blockIdx.x) * (blockDim.x >> 5)) + (threadIdx.x >> 5);
    if (row >= p.row_end) return;
    const std::uint8_t *row_bytes = p.packed + row * p.row_stride;
    const std::int64_t row_block = row / p.block_size;
    const bool row_policy = p.policy == CB200_DECODE_COLUMN_SCALE_ROW_OFFSET;
    const float row_offset = (row_policy && p.offsets != nullptr) ? __ldg(p.offsets + row) : 0.0f;
    const WT *w = static_cast<const WT *>(p.w);
    const int group = lane / LPN;
    const int col0 = (lane % LPN) * 8;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.0f;

    for (int base = 0; base < p.ell_cols; base += 32) {
        int gene;
        float value;
        bool valid;
        decode_slot<BITS>(p, row_bytes, row_block, row_offset, row_policy, base + lane, gene, value, valid);
        const unsigned mask = __ballot_sync(0xffffffffu, valid);
        if (mask == 0u) continue;
#pragma unroll
        for (int step = 0; step < LPN; ++step) {
            const int src = step * NPS + group;
            const int g = __shfl_sync(0xffffffffu, gene, src);
            const float v = __shfl_sync(0xffffffffu, value, src);
            if ((mask >> src) & 1u) {
                float wv[8];
                load8(w + static_cast<std::int64_t>(g) * p.w_ld + col0, wv);
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[i] = fmaf(v, wv[i], acc[i]);
            }
        }
    }
#pragma unroll
    for (int off = LPN; off < 32; off <<= 1) {
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], off);
    }
    if (lane < LPN) {
        float *out = p.y + row * p.y_ld + col0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float r = p.alpha * acc[i];
            if (p.beta != 0.0f) r = fmaf(p.beta, out[i], r);
            out[i] = finish_output(r, p.bias, col0 + i, p.epilogue);
        }
    }
}

template<int BITS, typename WT>
__global__ void __launch_bounds__(256) qbell_fwd_generic_kernel(const bell_params p) {
    const int lane = threadIdx.x & 31;
    const std::int64_t row = p.row_begin + (static_cast<std::int64_t>(blockIdx.x) * (blockDim.x >> 5)) + (threadIdx.x >> 5);
    if (row >= p.row_end) return;
    const std::uint8_t *row_bytes = p.packed + row * p.row_stride;
    const std::int64_t row_block = row / p.block_size;
    const bool row_policy = p.policy == CB200_DECODE_COLUMN_SCALE_ROW_OFFSET;
    const float row_offset = (row_policy && p.offsets != nullptr) ? __ldg(p.offsets + row) : 0.0f;
    const WT *w = static_cast<const WT *>(p.w);
    for (int tile = 0; tile < p.n; tile += 32) {
        const int col = tile + lane;
        float acc = 0.0f;
        for (int base = 0; base < p.ell_cols; base += 32) {
            int gene;
            float value;
            bool valid;
            decode_slot<BITS>(p, row_bytes, row_block, row_offset, row_policy, base + lane, gene, value, valid);
            const unsigned mask = __ballot_sync(0xffffffffu, valid);
            for (int j = 0; j < 32; ++j) {
                if (!((mask >> j) & 1u)) continue;
                const int g = __shfl_sync(0xffffffffu, gene, j);
                const float v = __shfl_sync(0xffffffffu, value, j);
                if (col < p.n) acc = fmaf(v, load1(w + static_cast<std::int64_t>(g) * p.w_ld + col), acc);
            }
        }
        if (col < p.n) {
            float *out = p.y + row * p.y_ld + col;
            float r = p.alpha * acc;
            if (p.beta != 0.0f) r = fmaf(p.beta, *out, r);
            *out = finish_output(r, p.bias, col, p.epilogue);
        }
    }
}

template<int BITS, typename WT>
cb200_status dispatch(const bell_params &p, bool vector_ok, cudaStream_t stream) {
    const unsigned grid = static_cast<unsigned>((p.row_end - p.row_begin + 7) / 8);
    bool done = false;
    if (vector_ok && p.n % 8 == 0) {
        done = true;
        switch (p.n / 8) {
        case 1: qbell_fwd_warp_row_kernel<BITS, WT, 1><<<grid, 256, 0, stream>>>(p); break;
        case 2: qbell_fwd_warp_row_kernel<BITS, WT, 2><<<grid, 256, 0, stream>>>(p); break;
        case 4: qbell_fwd_warp_row_kernel<BITS, WT, 4><<<grid, 256, 0, stream>>>(p); break;
        case 8: qbell_fwd_warp_row_kernel<BITS, WT, 8><<<grid, 256, 0, stream>>>(p); break;
        case 16: qbell_fwd_warp_row_kernel<BITS, WT, 16><<<grid, 256, 0, stream>>>(p); break;
        case 32: qbell_fwd_warp_row_kernel<BITS, WT, 32><<<grid, 256, 0, stream>>>(p); break;
        default: done = false; break;
        }
    }
    if (!done) qbell_fwd_generic_kernel<BITS, WT><<<grid, 256, 0, stream>>>(p);
    count_launch();
    CB200_CUDA_OK(cudaGetLastError());
    return CB200_STATUS_SUCCESS;
}

} // namespace

cb200_status launch_qbell_forward(const qbell_view &x, const dense_args &d, std::int64_t row_begin,
                                  std::int64_t row_end, void *workspace, std::uint64_t workspace_bytes, int sm_count,
                                  bool cuda_cores_only, cudaStream_t stream) {
    if (row_end <= row_begin || d.n == 0) return CB200_STATUS_SUCCESS;
    if (x.block_size <= 0 || x.ell_cols < 0 || x.ell_cols % x.block_size != 0)
        return fail(CB200_STATUS_INVALID_SHAPE, "ell_cols must be a multiple of block_size");
    if (x.bits != 8 && x.bits != 4) return fail(CB200_STATUS_UNSUPPORTED, "Blocked-ELL supports 8-bit and 4-bit codes");

    bool taken = false;
    const cb200_status tc = !cuda_cores_only ? launch_qbell_tcgen05(x, d, row_begin, row_end, workspace, workspace_bytes, sm_count,
                                                               stream, &taken)
                                        : CB200_STATUS_SUCCESS;
    if (tc != CB200_STATUS_SUCCESS || taken) return tc;

    bell_params p{};
    p.rows = x.rows; p.cols = x.cols; p.block_size = x.block_size; p.ell_cols = x.ell_cols;
    p.width = x.ell_cols / x.block_size; p.row_stride = x.row_stride_bytes; p.block_col_idx = x.block_col_idx;
    p.packed = x.packed; p.scales = x.scales; p.offsets = x.offsets; p.w = d.dense; p.y = d.out; p.w_ld = d.dense_ld;
    p.y_ld = d.out_ld; p.row_begin = row_begin; p.row_end = row_end; p.n = static_cast<int>(d.n); p.policy = x.policy;
    p.alpha = d.alpha; p.beta = d.beta; p.bias = d.bias; p.epilogue = d.epilogue;
    const std::size_t elem = d.dense_dtype == CB200_DTYPE_BF16 ? 2u : 4u;
    const bool vector_ok = (reinterpret_cast<std::uintptr_t>(d.dense) % 16u == 0u) && ((d.dense_ld * elem) % 16u == 0u);
    if (x.bits == 8) {
        if (d.dense_dtype == CB200_DTYPE_BF16) return dispatch<8, __nv_bfloat16>(p, vector_ok, stream);
        return dispatch<8, float>(p, vector_ok, stream);
    }
    if (d.dense_dtype == CB200_DTYPE_BF16) return dispatch<4, __nv_bfloat16>(p, vector_ok, stream);
    return dispatch<4, float>(p, vector_ok, stream);
}

} // namespace cb200
