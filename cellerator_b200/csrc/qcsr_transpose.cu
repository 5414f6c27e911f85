// Gene-side transpose of the fused path:  G' = alpha * deq(X)^T * G + beta * G'.
//
// Reference counterpart: csr_spmm_bwd_rhs_kernel_
// (src/compute/sparse/ops/kernels/base_sparse/csr_spmm_bwd_rhs_kernel_.cuh:1-22, launcher
// src/compute/sparse/ops/base_sparse.cu:373-393): zero the output, then one scalar atomicAdd
// per (stored entry, output column) over f16 values.  Here the codes are decoded in
// registers, one warp owns a cell row and keeps that row of G in registers, and each lane
// issues 128-bit vector reductions (red.global.add.v4.f32) into the gene row of G'.
// The order of the floating-point sums is not fixed: a problem that asks for determinism is
// served by the gather schedule over a gene-major copy instead (gene_major.cu).
#include "kernels.cuh"

#include <algorithm>

namespace cb200 {
namespace {

struct tr_params {
    const std::int64_t *row_ptr;
    const std::int64_t *packed_row_ptr;
    const std::int32_t *col_idx;
    const std::uint8_t *packed;
    const float *scales;
    const float *offsets;
    const float *g;
    float *out;
    std::int64_t g_ld, out_ld;
    std::int64_t row_begin, row_end;
    std::int64_t cols;
    int n;
    int policy;
    float alpha, beta;
};

template<int BITS>
__device__ __forceinline__ unsigned tr_load_code(const std::uint8_t *row_bytes, std::int64_t local) {
    if constexpr (BITS == 8) {
        return __ldg(row_bytes + local);
    } else {
        const unsigned byte = __ldg(row_bytes + (local >> 1));
        return (local & 1) ? (byte >> 4) : (byte & 0xfu);
    }
}

// out = beta * out (beta == 0 writes zeros without reading).
__global__ void __launch_bounds__(256) scale_output_kernel(float *out, std::int64_t rows, int n, std::int64_t ld, float beta) {
    const std::int64_t total = rows * n;
    for (std::int64_t i = static_cast<std::int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<std::int64_t>(gridDim.x) * blockDim.x) {
        float *p = out + (i / n) * ld + (i % n);
        *p = beta == 0.0f ? 0.0f : beta * *p;
    }
}

// One warp per cell row; N == 8 * LPN; G and G' rows 16-byte aligned.
template<int BITS, int LPN>
__global__ void __launch_bounds__(256) qcsr_transpose_atomic_kernel(const tr_params p) {
    constexpr int NPS = 32 / LPN;
    const int lane = threadIdx.x & 31;
    const std::int64_t row = p.row_begin + (static_cast<std::int64_t>(blockIdx.x) * (blockDim.x >> 5)) + (threadIdx.x >> 5);
    if (row >= p.row_end) return;
    const std::int64_t begin = __ldg(p.row_ptr + row);
    const std::int64_t end = __ldg(p.row_ptr + row + 1);
    const std::uint8_t *row_bytes = p.packed + (p.packed_row_ptr != nullptr ? __ldg(p.packed_row_ptr + row) : begin);
    const bool row_policy = p.policy == CB200_DECODE_COLUMN_SCALE_ROW_OFFSET;
    const float row_offset = (row_policy && p.offsets != nullptr) ? __ldg(p.offsets + row) : 0.0f;
    const int group = lane / LPN;
    const int col0 = (lane % LPN) * 8;

    float gr[8];
    load8(p.g + row * p.g_ld + col0, gr);
#pragma unroll
    for (int i = 0; i < 8; ++i) gr[i] *= p.alpha;

    for (std::int64_t base = begin; base < end; base += 32) {
        const int count = static_cast<int>(min(static_cast<std::int64_t>(32), end - base));
        int gene = 0;
        float value = 0.0f;
        if (lane < count) {
            const std::int64_t idx = base + lane;
            gene = __ldg(p.col_idx + idx);
            const unsigned code = tr_load_code<BITS>(row_bytes, idx - begin);
            const float scale = p.scales != nullptr ? __ldg(p.scales + gene) : 1.0f;
            const float offset = row_policy ? row_offset : (p.offsets != nullptr ? __ldg(p.offsets + gene) : 0.0f);
            value = fmaf(static_cast<float>(code), scale, offset);
        }
#pragma unroll
        for (int step = 0; step < LPN; ++step) {
            const int src = step * NPS + group;
            const int g = __shfl_sync(0xffffffffu, gene, src);
            const float v = __shfl_sync(0xffffffffu, value, src);
            if (src < count) {
                float *dst = p.out + static_cast<std::int64_t>(g) * p.out_ld + col0;
                atomicAdd(reinterpret_cast<float4 *>(dst), make_float4(v * gr[0], v * gr[1], v * gr[2], v * gr[3]));
                atomicAdd(reinterpret_cast<float4 *>(dst + 4), make_float4(v * gr[4], v * gr[5], v * gr[6], v * gr[7]));
            }
        }
    }
}

// Any N / leading dimension: scalar atomics, lane = output column within a 32-wide tile.
template<int BITS>
__global__ void __launch_bounds__(256) qcsr_transpose_generic_kernel(const tr_params p) {
    const int lane = threadIdx.x & 31;
    const std::int64_t row = p.row_begin + (static_cast<std::int64_t>(blockIdx.x) * (blockDim.x >> 5)) + (threadIdx.x >> 5);
    if (row >= p.row_end) return;
    const std::int64_t begin = __ldg(p.row_ptr + row);
    const std::int64_t end = __ldg(p.row_ptr + row + 1);
    const std::uint8_t *row_bytes = p.packed + (p.packed_row_ptr != nullptr ? __ldg(p.packed_row_ptr + row) : begin);
    const bool row_policy = p.policy == CB200_DECODE_COLUMN_SCALE_ROW_OFFSET;
    const float row_offset = (row_policy && p.offsets != nullptr) ? __ldg(p.offsets + row) : 0.0f;
    for (int tile = 0; tile < p.n; tile += 32) {
        const int col = tile + lane;
        const float gv = col < p.n ? p.alpha * __ldg(p.g + row * p.g_ld + col) : 0.0f;
        for (std::int64_t base = begin; base < end; base += 32) {
            const int count = static_cast<int>(min(static_cast<std::int64_t>(32), end - base));
            int gene = 0;
            float value = 0.0f;
            if (lane < count) {
                const std::int64_t idx = base + lane;
                gene = __ldg(p.col_idx + idx);
                const unsigned code = tr_load_code<BITS>(row_bytes, idx - begin);
                const float scale = p.scales != nullptr ? __ldg(p.scales + gene) : 1.0f;
                const float offset = row_policy ? row_offset : (p.offsets != nullptr ? __ldg(p.offsets + gene) : 0.0f);
                value = fmaf(static_cast<float>(code), scale, offset);
            }
            for (int j = 0; j < count; ++j) {
                const int g = __shfl_sync(0xffffffffu, gene, j);
                const float v = __shfl_sync(0xffffffffu, value, j);
                if (col < p.n) atomicAdd(p.out + static_cast<std::int64_t>(g) * p.out_ld + col, v * gv);
            }
        }
    }
}

template<int BITS>
cb200_status dispatch(const tr_params &p, bool vector_ok, cudaStream_t stream) {
    const std::int64_t rows = p.row_end - p.row_begin;
    constexpr int threads = 256;
    const unsigned grid = static_cast<unsigned>((rows + 7) / 8);
    if (vector_ok && p.n % 8 == 0 && p.n / 8 <= 32 && ((p.n / 8) & (p.n / 8 - 1)) == 0) {
        switch (p.n / 8) {
        case 1: qcsr_transpose_atomic_kernel<BITS, 1><<<grid, threads, 0, stream>>>(p); break;
        case 2: qcsr_transpose_atomic_kernel<BITS, 2><<<grid, threads, 0, stream>>>(p); break;
        case 4: qcsr_transpose_atomic_kernel<BITS, 4><<<grid, threads, 0, stream>>>(p); break;
        case 8: qcsr_transpose_atomic_kernel<BITS, 8><<<grid, threads, 0, stream>>>(p); break;
        case 16: qcsr_transpose_atomic_kernel<BITS, 16><<<grid, threads, 0, stream>>>(p); break;
        default: qcsr_transpose_atomic_kernel<BITS, 32><<<grid, threads, 0, stream>>>(p); break;
        }
    } else {
        qcsr_transpose_generic_kernel<BITS><<<grid, threads, 0, stream>>>(p);
    }
    count_launch();
    CB200_CUDA_OK(cudaGetLastError());
    return CB200_STATUS_SUCCESS;
}

} // namespace

std::uint64_t qcsr_transpose_workspace_bytes(std::int64_t, std::int64_t, int) { return 0; }

cb200_status launch_qcsr_transpose(const qcsr_view &x, const dense_args &d, std::int64_t row_begin,
                                   std::int64_t row_end, const blocked_layout *blocked, bool split_products,
                                   void *workspace, std::uint64_t workspace_bytes, int sm_count, cudaStream_t stream) {
    if (d.n == 0 || x.cols == 0) return CB200_STATUS_SUCCESS;
    if (d.dense_dtype != CB200_DTYPE_F32) return fail(CB200_STATUS_UNSUPPORTED, "transpose takes an fp32 dense operand");
    if (blocked != nullptr && blocked->seg_ptr != nullptr) {
        bool taken = false;
        const cb200_status st = launch_qcsr_transpose_blocked(x, d, row_begin, row_end, workspace, workspace_bytes, *blocked,
                                                              split_products, sm_count, stream, &taken);
        if (st != CB200_STATUS_SUCCESS || taken) return st;
    }
    // The output is initialised even for an empty row range: G' = beta * G'.
    {
        const std::int64_t total = x.cols * d.n;
        const unsigned grid = static_cast<unsigned>(std::min<std::int64_t>((total + 255) / 256, static_cast<std::int64_t>(sm_count) * 8));
        scale_output_kernel<<<grid, 256, 0, stream>>>(d.out, x.cols, static_cast<int>(d.n), d.out_ld, d.beta);
        count_launch();
        CB200_CUDA_OK(cudaGetLastError());
    }
    if (row_end <= row_begin) return CB200_STATUS_SUCCESS;
    tr_params p{};
    p.row_ptr = x.row_ptr; p.packed_row_ptr = x.packed_row_ptr; p.col_idx = x.col_idx; p.packed = x.packed;
    p.scales = x.scales; p.offsets = x.offsets; p.g = static_cast<const float *>(d.dense); p.out = d.out;
    p.g_ld = d.dense_ld; p.out_ld = d.out_ld; p.row_begin = row_begin; p.row_end = row_end; p.cols = x.cols;
    p.n = static_cast<int>(d.n); p.policy = x.policy; p.alpha = d.alpha; p.beta = d.beta;
    const bool vector_ok = (reinterpret_cast<std::uintptr_t>(d.dense) % 16u == 0u) && ((d.dense_ld * 4u) % 16u == 0u) &&
                           (reinterpret_cast<std::uintptr_t>(d.out) % 16u == 0u) && ((d.out_ld * 4u) % 16u == 0u);
    if (x.bits == 8) return dispatch<8>(p, vector_ok, stream);
    if (x.bits == 4) {
        if (x.packed_row_ptr == nullptr) return fail(CB200_STATUS_INVALID_ARGUMENT, "4-bit codes need packed_row_ptr");
        return dispatch<4>(p, vector_ok, stream);
    }
    return fail(CB200_STATUS_UNSUPPORTED, "transpose supports 8-bit and 4-bit codes, got %d", x.bits);
}

} // namespace cb200
