// Routing of the reference's public sparse-projection calls to this backend.
//
// cellerator_sparse_projection_forward / _backward (include/Cellerator/abi.h:111-124,
// src/abi/abi.cu:278-396) take a cellerator_sparse_layout_desc, fp32 row-major operands with explicit
// leading dimensions, and the context's device, stream and scratch.  The reference declares
// CELLERATOR_LAYOUT_QUANTIZED_BLOCKED_ELL (abi.h:31-36) and rejects it (abi.cu:325-326); these entry
// points are what its "unsupported layout" branch calls instead.  They take the descriptor's fields
// as plain values (cb200_public_layout mirrors them), prepare, run and destroy in one call, and never
// allocate: everything temporary lives in the caller's scratch.
//
// The public descriptor holds 32-bit row offsets; the kernels read 64-bit ones.  They are widened on
// the stream into the scratch, ahead of the launch.
#include "kernels.cuh"

namespace cb200 {
namespace {

__global__ void __launch_bounds__(256) widen_offsets_kernel(const std::uint32_t *src, std::int64_t count, std::int64_t *dst) {
    const std::int64_t i = static_cast<std::int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < count) dst[i] = static_cast<std::int64_t>(src[i]);
}

// 4-bit codes: the descriptor carries no packed row offsets, but the codec fixes them: a row's codes take
// ceil(entries / 2) bytes and rows follow each other without sharing a byte (include/Cellerator/quantized/layout.cuh:
// 111-129, build_packed_row_ptr), so packed[r] = sum of those over the rows before r.  One block walks the rows in tiles
// of 1,024 and carries the running total; `wide` holds the widened row offsets, rows + 1 of them.
__global__ void __launch_bounds__(1024) packed_offsets_kernel(const std::int64_t *wide, std::int64_t rows, std::int64_t *packed) {
    __shared__ long long warp_total[32];
    __shared__ long long carry;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    for (std::int64_t tile = 0; tile < rows; tile += 1024) {
        const std::int64_t r = tile + threadIdx.x;
        const long long mine = r < rows ? (wide[r + 1] - wide[r] + 1) / 2 : 0;
        long long sum = mine;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const long long up = __shfl_up_sync(0xffffffffu, sum, d);
            if (lane >= d) sum += up;
        }
        if (lane == 31) warp_total[warp] = sum;
        __syncthreads();
        if (warp == 0) {
            const long long total = warp_total[lane];
            long long run = total;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const long long up = __shfl_up_sync(0xffffffffu, run, d);
                if (lane >= d) run += up;
            }
            warp_total[lane] = run - total;
        }
        __syncthreads();
        const long long at = carry + warp_total[warp] + sum - mine;
        if (r < rows) packed[r] = at;
        __syncthreads();
        if (threadIdx.x == 1023) carry = at + mine;
        __syncthreads();
    }
    if (threadIdx.x == 0) packed[rows] = carry;
}

cb200_status check_layout(const cb200_public_layout *l) {
    if (l == nullptr || l->version != CB200_ABI_VERSION || l->size < sizeof(cb200_public_layout))
        return fail(CB200_STATUS_INVALID_ARGUMENT, "layout descriptor version or size mismatch");
    if (l->layout != CB200_PUBLIC_LAYOUT_QUANTIZED_BLOCKED_ELL && l->layout != CB200_PUBLIC_LAYOUT_QUANTIZED_CSR)
        return fail(CB200_STATUS_UNSUPPORTED, "layout %d is not one of the quantized layouts this backend serves", l->layout);
    if (l->decode_policy != CB200_DECODE_PER_GENE_AFFINE && l->decode_policy != CB200_DECODE_COLUMN_SCALE_ROW_OFFSET)
        return fail(CB200_STATUS_UNSUPPORTED, "unknown decode policy %u", l->decode_policy);
    if (l->packed_values == nullptr && l->rows != 0u) return fail(CB200_STATUS_INVALID_ARGUMENT, "quantized layout requires packed values");
    if (l->layout == CB200_PUBLIC_LAYOUT_QUANTIZED_BLOCKED_ELL) {
        if (l->bits != 8u && l->bits != 4u) return fail(CB200_STATUS_UNSUPPORTED, "Blocked-ELL codes must be 8 or 4 bits");
        if (l->block_size == 0u || l->ell_cols == 0u) return fail(CB200_STATUS_INVALID_SHAPE, "Blocked-ELL requires block_size and ell_cols");
        if (l->block_col_idx == nullptr) return fail(CB200_STATUS_INVALID_ARGUMENT, "Blocked-ELL requires block column indices");
    } else {
        if (l->bits != 8u && l->bits != 4u) return fail(CB200_STATUS_UNSUPPORTED, "quantized CSR codes must be 8 or 4 bits");
        if (l->major_ptr == nullptr || (l->nnz != 0u && l->minor_idx == nullptr))
            return fail(CB200_STATUS_INVALID_ARGUMENT, "CSR layout requires row offsets and column indices");
        if (l->cols > 0x7fffffffu) return fail(CB200_STATUS_INVALID_SHAPE, "gene indices must fit 31 bits");
    }
    return CB200_STATUS_SUCCESS;
}

const float *offsets_of(const cb200_public_layout &l) {
    return l.decode_policy == CB200_DECODE_COLUMN_SCALE_ROW_OFFSET ? l.row_offsets : l.column_offsets;
}

struct scratch_cursor {
    unsigned char *at;
    std::uint64_t left;
    void *take(std::uint64_t bytes) {
        const std::uint64_t need = (bytes + 255u) / 256u * 256u;
        if (at == nullptr || need > left) return nullptr;
        void *p = at;
        at += need;
        left -= need;
        return p;
    }
};

cb200_status route(const cb200_public_layout *l, int32_t projection, const float *dense, int64_t dense_ld, int64_t n, float *out,
                   int64_t out_ld, int32_t device, void *stream, void *scratch, uint64_t scratch_bytes) {
    cb200_status st = check_layout(l);
    if (st != CB200_STATUS_SUCCESS) return st;
    if (n <= 0 || n > 0x7fffffff) return fail(CB200_STATUS_INVALID_SHAPE, "projection output column count is out of range");
    if (dense == nullptr || out == nullptr) return fail(CB200_STATUS_INVALID_ARGUMENT, "operand data is null");
    if (dense_ld < n || out_ld < n) return fail(CB200_STATUS_INVALID_SHAPE, "leading dimension smaller than the column count");
    if (reinterpret_cast<std::uintptr_t>(scratch) % 256u != 0u) return fail(CB200_STATUS_INVALID_ARGUMENT, "scratch must be 256-byte aligned");
    scratch_cursor cur{static_cast<unsigned char *>(scratch), scratch_bytes};
    // the first 256 bytes of the scratch are the kernels' status block (first word = status), so that
    // cb200_public_projection_status finds it without knowing the layout; the widened offsets follow
    void *status_block = cur.take(256u);
    if (status_block == nullptr) return fail(CB200_STATUS_INSUFFICIENT_WORKSPACE, "scratch too small for the status block (256 bytes)");

    cb200_spmm_problem pr{};
    pr.version = CB200_ABI_VERSION;
    pr.size = sizeof pr;
    pr.projection = projection;
    pr.m = l->rows; pr.k = l->cols; pr.n = n;
    pr.bits = static_cast<int32_t>(l->bits);
    pr.policy = static_cast<int32_t>(l->decode_policy);
    pr.dense_dtype = CB200_DTYPE_F32;
    pr.device = device;
    pr.structure_epoch = 1u;
    pr.multiply = CB200_DTYPE_F32;
    cb200_launch ln{};
    ln.version = CB200_ABI_VERSION;
    ln.size = sizeof ln;
    cb200_qbell bell{};
    cb200_qcsr csr{};
    if (l->layout == CB200_PUBLIC_LAYOUT_QUANTIZED_BLOCKED_ELL) {
        if (projection != CB200_PROJECTION_BLOCKED_ELL) return fail(CB200_STATUS_UNSUPPORTED, "the backward pass of the Blocked-ELL layout is not served");
        pr.nnz = static_cast<int64_t>(l->rows) * l->ell_cols;
        bell.version = CB200_ABI_VERSION; bell.size = sizeof bell;
        bell.rows = l->rows; bell.cols = l->cols; bell.block_size = static_cast<int32_t>(l->block_size);
        bell.ell_cols = static_cast<int32_t>(l->ell_cols); bell.row_stride_bytes = l->row_stride_bytes;
        bell.bits = pr.bits; bell.policy = pr.policy; bell.block_col_idx = l->block_col_idx;
        bell.packed_values = l->packed_values; bell.scales = l->column_scales; bell.offsets = offsets_of(*l);
        ln.bell = &bell;
    } else {
        pr.nnz = l->nnz;
        std::int64_t *wide = static_cast<std::int64_t *>(cur.take((static_cast<std::uint64_t>(l->rows) + 1u) * 8u));
        if (wide == nullptr)
            return fail(CB200_STATUS_INSUFFICIENT_WORKSPACE, "scratch too small for the widened row offsets (%llu bytes)",
                        (static_cast<unsigned long long>(l->rows) + 1u) * 8u);
        device_scope scope(device);
        CB200_CUDA_OK(scope.status);
        const std::int64_t count = static_cast<std::int64_t>(l->rows) + 1;
        widen_offsets_kernel<<<static_cast<unsigned>((count + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(l->major_ptr, count, wide);
        count_launch();
        CB200_CUDA_OK(cudaGetLastError());
        csr.version = CB200_ABI_VERSION; csr.size = sizeof csr;
        csr.rows = l->rows; csr.cols = l->cols; csr.nnz = l->nnz; csr.bits = pr.bits; csr.policy = pr.policy;
        if (l->bits == 4u) { // the packed row offsets the descriptor does not carry
            std::int64_t *packed = static_cast<std::int64_t *>(cur.take((static_cast<std::uint64_t>(l->rows) + 1u) * 8u));
            if (packed == nullptr)
                return fail(CB200_STATUS_INSUFFICIENT_WORKSPACE, "scratch too small for the packed row offsets (%llu bytes)",
                            (static_cast<unsigned long long>(l->rows) + 1u) * 8u);
            packed_offsets_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(wide, static_cast<std::int64_t>(l->rows), packed);
            count_launch();
            CB200_CUDA_OK(cudaGetLastError());
            csr.packed_row_ptr = packed;
        }
        csr.row_ptr = wide; csr.col_idx = reinterpret_cast<const std::int32_t *>(l->minor_idx);
        csr.packed_values = l->packed_values; csr.scales = l->column_scales; csr.offsets = offsets_of(*l);
        ln.csr = &csr;
    }
    cb200_prepared *prepared = nullptr;
    st = cb200_spmm_prepare(&pr, &prepared);
    if (st != CB200_STATUS_SUCCESS) return st;
    std::uint64_t need = 0;
    std::uint32_t align = 256;
    cb200_prepared_workspace(prepared, &need, &align);
    // the exact fp32 schedules these calls select need the status block only
    void *ws = need == 0u ? nullptr : (need <= 256u ? status_block : cur.take(need));
    if (need != 0u && ws == nullptr) {
        cb200_prepared_destroy(prepared);
        return fail(CB200_STATUS_INSUFFICIENT_WORKSPACE, "scratch too small for the kernel workspace (%llu more bytes)",
                    static_cast<unsigned long long>(need));
    }
    ln.dense = dense; ln.dense_ld = dense_ld; ln.out = out; ln.out_ld = out_ld;
    ln.alpha = 1.0f; ln.beta = 0.0f; ln.structure_epoch = 1u; ln.stream = stream; ln.device = device;
    ln.row_begin = 0; ln.row_end = CB200_ALL_ROWS;
    ln.workspace_device = device; ln.workspace = ws; ln.workspace_bytes = need;
    if (need == 0u) { // a schedule without waits: the status block still reads 0 afterwards
        device_scope scope(device);
        CB200_CUDA_OK(scope.status);
        CB200_CUDA_OK(cudaMemsetAsync(status_block, 0, sizeof(int), static_cast<cudaStream_t>(stream)));
    }
    st = cb200_spmm_run(prepared, &ln);
    cb200_prepared_destroy(prepared);
    return st;
}

} // namespace
} // namespace cb200

extern "C" cb200_status cb200_public_projection_scratch(const cb200_public_layout *layout, int64_t, uint64_t *bytes) {
    using namespace cb200;
    clear_error();
    if (bytes == nullptr) return fail(CB200_STATUS_INVALID_ARGUMENT, "null argument");
    const cb200_status st = check_layout(layout);
    if (st != CB200_STATUS_SUCCESS) return st;
    // widened row offsets (CSR) + the status block of the fp32 schedules these calls select
    const std::uint64_t offsets = layout->layout == CB200_PUBLIC_LAYOUT_QUANTIZED_CSR ? (static_cast<std::uint64_t>(layout->rows) + 1u) * 8u : 0u;
    const std::uint64_t arrays = layout->layout == CB200_PUBLIC_LAYOUT_QUANTIZED_CSR && layout->bits == 4u ? 2u : 1u; // + packed row offsets
    *bytes = arrays * ((offsets + 255u) / 256u * 256u) + 512u;
    return CB200_STATUS_SUCCESS;
}

extern "C" cb200_status cb200_public_projection_forward(const cb200_public_layout *layout, const float *rhs, int64_t rhs_ld,
                                                        int64_t out_cols, float *out, int64_t out_ld, int32_t device, void *stream,
                                                        void *scratch, uint64_t scratch_bytes) {
    using namespace cb200;
    clear_error();
    const int32_t projection = layout != nullptr && layout->layout == CB200_PUBLIC_LAYOUT_QUANTIZED_BLOCKED_ELL
                                   ? CB200_PROJECTION_BLOCKED_ELL : CB200_PROJECTION_CSR;
    return route(layout, projection, rhs, rhs_ld, out_cols, out, out_ld, device, stream, scratch, scratch_bytes);
}

extern "C" cb200_status cb200_public_projection_backward_rhs(const cb200_public_layout *layout, const float *grad_out,
                                                             int64_t grad_out_ld, int64_t out_cols, float *grad_rhs,
                                                             int64_t grad_rhs_ld, int32_t device, void *stream, void *scratch,
                                                             uint64_t scratch_bytes) {
    using namespace cb200;
    clear_error();
    return route(layout, CB200_PROJECTION_TRANSPOSE, grad_out, grad_out_ld, out_cols, grad_rhs, grad_rhs_ld, device, stream,
                 scratch, scratch_bytes);
}

extern "C" cb200_status cb200_public_projection_status(const void *scratch, int32_t device, void *stream, int32_t *host_word) {
    using namespace cb200;
    clear_error();
    if (scratch == nullptr || host_word == nullptr) return fail(CB200_STATUS_INVALID_ARGUMENT, "status needs the scratch of the call and an output");
    *host_word = 0;
    device_scope scope(device);
    CB200_CUDA_OK(scope.status);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    CB200_CUDA_OK(cudaMemcpyAsync(host_word, scratch, sizeof(int32_t), cudaMemcpyDeviceToHost, s));
    CB200_CUDA_OK(cudaStreamSynchronize(s));
    if (*host_word != 0)
        return fail(CB200_STATUS_DEVICE_WAIT_TIMEOUT, "a kernel of the last routed projection gave up a bounded wait: its output is not valid");
    return CB200_STATUS_SUCCESS;
}
