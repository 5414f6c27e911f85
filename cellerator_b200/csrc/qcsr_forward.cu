// Fused dequantise + SpMM over a quantized CSR matrix:  Y = alpha * deq(X) * W + beta * Y.
//
// The Cellerator reference has no fused kernel for this layout; it decodes to a float array
// (include/Cellerator/quantized/portable_dequantize_kernel.cuh:7-19) and then runs
// csr_spmm_fwd_kernel_ (src/compute/sparse/project/kernels/csr_spmm_fwd_kernel_.cuh:1-22), one
// thread per (row, output column), every thread re-reading the row.  Here one warp owns a
// row: the 32 lanes read 32 consecutive (gene index, code) pairs with coalesced loads, apply
// the per-gene scale and zero-point in registers, and then the warp walks those 32 entries
// `NPS` at a time: a group of LPN lanes serves one entry, each lane holding 8 of the N output
// columns, so one 16-byte load per lane fetches a whole bf16 row of W across the group.
// Partial sums of the 32/LPN groups are combined with shuffles at the end of the row.
#include "kernels.cuh"

#include <cstdlib>
#include <cstring>

namespace cb200 {
namespace {

struct fwd_params {
    const std::int64_t *row_ptr;
    const std::int64_t *packed_row_ptr;
    const std::int32_t *col_idx;
    const std::uint8_t *packed;
    const float *scales;
    const float *offsets;
    const void *w;
    float *y;
    std::int64_t w_ld, y_ld;
    std::int64_t row_begin, row_end;
    int n;
    int policy;
    float alpha, beta;
    const float *bias;
    int epilogue;
};

// Code of entry `local` (index within its row) for a row whose packed bytes start at `row_bytes`.
template<int BITS>
__device__ __forceinline__ unsigned load_code(const std::uint8_t *row_bytes, std::int64_t local) {
    if constexpr (BITS == 8) {
        return __ldg(row_bytes + local);
    } else {
        const unsigned byte = __ldg(row_bytes + (local >> 1));
        return (local & 1) ? (byte >> 4) : (byte & 0xfu);
    }
}

// acc[0..7] += v * w[0..7] with packed two-wide fp32 FMAs (fma.rn.f32x2, sm_100): half the
// issue slots of eight scalar FMAs.
__device__ __forceinline__ void fma8(float (&acc)[8], float v, const float (&w)[8]) {
    const float2 vv = make_float2(v, v);
    unsigned long long vp;
    memcpy(&vp, &vv, 8);
#pragma unroll
    for (int i = 0; i < 8; i += 2) {
        float2 a = make_float2(acc[i], acc[i + 1]);
        const float2 b = make_float2(w[i], w[i + 1]);
        unsigned long long ap, bp;
        memcpy(&ap, &a, 8);
        memcpy(&bp, &b, 8);
        asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(ap) : "l"(vp), "l"(bp));
        memcpy(&a, &ap, 8);
        acc[i] = a.x;
        acc[i + 1] = a.y;
    }
}

// One warp per row, N == 8 * LPN, dense rows 16-byte aligned.  The (gene, code, scale, offset)
// loads of the next 32 entries are issued before the current 32 are multiplied.
template<int BITS, typename WT, int LPN>
__global__ void __launch_bounds__(256) qcsr_fwd_warp_row_kernel(const fwd_params p) {
    constexpr int NPS = 32 / LPN; // entries served per step
    const int lane = threadIdx.x & 31;
    const std::int64_t row = p.row_begin + (static_cast<std::int64_t>(blockIdx.x) * (blockDim.x >> 5)) + (threadIdx.x >> 5);
    if (row >= p.row_end) return;

    const std::int64_t begin = __ldg(p.row_ptr + row);
    const std::int64_t end = __ldg(p.row_ptr + row + 1);
    const std::uint8_t *row_bytes = p.packed + (p.packed_row_ptr != nullptr ? __ldg(p.packed_row_ptr + row) : begin);
    const bool row_policy = p.policy == CB200_DECODE_COLUMN_SCALE_ROW_OFFSET;
    const float row_offset = (row_policy && p.offsets != nullptr) ? __ldg(p.offsets + row) : 0.0f;
    const WT *w = static_cast<const WT *>(p.w);
    const int group = lane / LPN;           // which entry of a step this lane serves
    const WT *wcol = w + (lane % LPN) * 8;  // first output column held by this lane

    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.0f;

    // entry `idx` decoded by this lane: gene index and dequantised value (0 past the row end)
    auto fetch = [&](std::int64_t idx, int &gene, float &value) {
        gene = 0;
        value = 0.0f;
        if (idx < end) {
            gene = __ldg(p.col_idx + idx);
            const unsigned code = load_code<BITS>(row_bytes, idx - begin);
            const float scale = p.scales != nullptr ? __ldg(p.scales + gene) : 1.0f;
            const float offset = row_policy ? row_offset : (p.offsets != nullptr ? __ldg(p.offsets + gene) : 0.0f);
            value = fmaf(static_cast<float>(code), scale, offset);
        }
    };

    int gene, next_gene;
    float value, next_value;
    fetch(begin + lane, gene, value);
    for (std::int64_t base = begin; base < end; base += 32) {
        fetch(base + 32 + lane, next_gene, next_value);
        const int count = static_cast<int>(min(static_cast<std::int64_t>(32), end - base));
        if (count == 32) {
#pragma unroll
            for (int step = 0; step < LPN; ++step) {
                const int src = step * NPS + group;
                const int g = __shfl_sync(0xffffffffu, gene, src);
                const float v = __shfl_sync(0xffffffffu, value, src);
                float wv[8];
                load8(wcol + static_cast<std::int64_t>(g) * p.w_ld, wv);
                fma8(acc, v, wv);
            }
        } else {
#pragma unroll
            for (int step = 0; step < LPN; ++step) {
                const int src = step * NPS + group;
                const int g = __shfl_sync(0xffffffffu, gene, src);
                const float v = __shfl_sync(0xffffffffu, value, src);
                if (src < count) {
                    float wv[8];
                    load8(wcol + static_cast<std::int64_t>(g) * p.w_ld, wv);
                    fma8(acc, v, wv);
                }
            }
        }
        gene = next_gene;
        value = next_value;
    }

#pragma unroll
    for (int off = LPN; off < 32; off <<= 1) {
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], off);
    }
    if (lane < LPN) {
        float *out = p.y + row * p.y_ld + (lane % LPN) * 8;
        float4 lo = make_float4(p.alpha * acc[0], p.alpha * acc[1], p.alpha * acc[2], p.alpha * acc[3]);
        float4 hi = make_float4(p.alpha * acc[4], p.alpha * acc[5], p.alpha * acc[6], p.alpha * acc[7]);
        if (p.beta != 0.0f) {
            const float4 a = *reinterpret_cast<const float4 *>(out);
            const float4 b = *reinterpret_cast<const float4 *>(out + 4);
            lo.x = fmaf(p.beta, a.x, lo.x); lo.y = fmaf(p.beta, a.y, lo.y);
            lo.z = fmaf(p.beta, a.z, lo.z); lo.w = fmaf(p.beta, a.w, lo.w);
            hi.x = fmaf(p.beta, b.x, hi.x); hi.y = fmaf(p.beta, b.y, hi.y);
            hi.z = fmaf(p.beta, b.z, hi.z); hi.w = fmaf(p.beta, b.w, hi.w);
        }
        if (p.epilogue != CB200_EPILOGUE_NONE) {
            const int c = (lane % LPN) * 8;
            lo.x = finish_output(lo.x, p.bias, c + 0, p.epilogue); lo.y = finish_output(lo.y, p.bias, c + 1, p.epilogue);
            lo.z = finish_output(lo.z, p.bias, c + 2, p.epilogue); lo.w = finish_output(lo.w, p.bias, c + 3, p.epilogue);
            hi.x = finish_output(hi.x, p.bias, c + 4, p.epilogue); hi.y = finish_output(hi.y, p.bias, c + 5, p.epilogue);
            hi.z = finish_output(hi.z, p.bias, c + 6, p.epilogue); hi.w = finish_output(hi.w, p.bias, c + 7, p.epilogue);
        }
        *reinterpret_cast<float4 *>(out) = lo;
        *reinterpret_cast<float4 *>(out + 4) = hi;
    }
}

// Any N, any leading dimension: one warp per row, lane = output column within a 32-wide tile.
template<int BITS, typename WT>
__global__ void __launch_bounds__(256) qcsr_fwd_generic_kernel(const fwd_params p) {
    const int lane = threadIdx.x & 31;
    const std::int64_t row = p.row_begin + (static_cast<std::int64_t>(blockIdx.x) * (blockDim.x >> 5)) + (threadIdx.x >> 5);
    if (row >= p.row_end) return;
    const std::int64_t begin = __ldg(p.row_ptr + row);
    const std::int64_t end = __ldg(p.row_ptr + row + 1);
    const std::uint8_t *row_bytes = p.packed + (p.packed_row_ptr != nullptr ? __ldg(p.packed_row_ptr + row) : begin);
    const bool row_policy = p.policy == CB200_DECODE_COLUMN_SCALE_ROW_OFFSET;
    const float row_offset = (row_policy && p.offsets != nullptr) ? __ldg(p.offsets + row) : 0.0f;
    const WT *w = static_cast<const WT *>(p.w);

    for (int tile = 0; tile < p.n; tile += 32) {
        const int col = tile + lane;
        float acc = 0.0f;
        for (std::int64_t base = begin; base < end; base += 32) {
            const int count = static_cast<int>(min(static_cast<std::int64_t>(32), end - base));
            int gene = 0;
            float value = 0.0f;
            if (lane < count) {
                const std::int64_t idx = base + lane;
                gene = __ldg(p.col_idx + idx);
                const unsigned code = load_code<BITS>(row_bytes, idx - begin);
                const float scale = p.scales != nullptr ? __ldg(p.scales + gene) : 1.0f;
                const float offset = row_policy ? row_offset : (p.offsets != nullptr ? __ldg(p.offsets + gene) : 0.0f);
                value = fmaf(static_cast<float>(code), scale, offset);
            }
            for (int j = 0; j < count; ++j) {
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
cb200_status dispatch_n(const fwd_params &p, bool vector_ok, cudaStream_t stream) {
    const std::int64_t rows = p.row_end - p.row_begin;
    constexpr int threads = 128; // four rows per CTA (64 to 256 threads measured within 2 % of each other)
    const unsigned grid = static_cast<unsigned>((rows + (threads / 32) - 1) / (threads / 32));
    if (vector_ok && p.n % 8 == 0) {
        switch (p.n / 8) {
        case 1: qcsr_fwd_warp_row_kernel<BITS, WT, 1><<<grid, threads, 0, stream>>>(p); break;
        case 2: qcsr_fwd_warp_row_kernel<BITS, WT, 2><<<grid, threads, 0, stream>>>(p); break;
        case 4: qcsr_fwd_warp_row_kernel<BITS, WT, 4><<<grid, threads, 0, stream>>>(p); break;
        case 8: qcsr_fwd_warp_row_kernel<BITS, WT, 8><<<grid, threads, 0, stream>>>(p); break;
        case 16: qcsr_fwd_warp_row_kernel<BITS, WT, 16><<<grid, threads, 0, stream>>>(p); break;
        case 32: qcsr_fwd_warp_row_kernel<BITS, WT, 32><<<grid, threads, 0, stream>>>(p); break;
        default: qcsr_fwd_generic_kernel<BITS, WT><<<grid, threads, 0, stream>>>(p); break;
        }
    } else {
        qcsr_fwd_generic_kernel<BITS, WT><<<grid, threads, 0, stream>>>(p);
    }
    count_launch();
    CB200_CUDA_OK(cudaGetLastError());
    return CB200_STATUS_SUCCESS;
}

} // namespace

cb200_status launch_qcsr_forward(const qcsr_view &x, const dense_args &d, std::int64_t row_begin,
                                 std::int64_t row_end, fwd_schedule schedule, const void *persistent,
                                 const blocked_layout *blocked, bool split_products, void *workspace,
                                 std::uint64_t workspace_bytes, int sm_count, cudaStream_t stream) {
    if (row_end <= row_begin || d.n == 0) return CB200_STATUS_SUCCESS;
    if (row_end - row_begin > 0x7fffffffll) return fail(CB200_STATUS_INVALID_SHAPE, "row range too large for one launch");
    if (schedule == fwd_schedule::tensor_blocked && blocked != nullptr) {
        // a row range that does not start on a group boundary runs the exact gene-tiled kernel below
        bool taken = false;
        const cb200_status st = launch_qcsr_forward_blocked(x, d, row_begin, row_end, workspace, workspace_bytes, *blocked,
                                                            split_products, sm_count, stream, &taken);
        if (st != CB200_STATUS_SUCCESS || taken) return st;
    }
    if (schedule == fwd_schedule::tensor_windows) {
        bool taken = false;
        const cb200_status st = launch_qcsr_forward_mma(x, d, row_begin, row_end, workspace, workspace_bytes,
                                                        static_cast<const std::int32_t *>(persistent), sm_count, stream,
                                                        &taken);
        if (st != CB200_STATUS_SUCCESS || taken) return st;
    }
    if (schedule != fwd_schedule::warp_per_row) {
        bool taken = false;
        const cb200_status st = launch_qcsr_forward_tiled(x, d, row_begin, row_end, static_cast<int *>(workspace),
                                                          static_cast<const std::int32_t *>(persistent), sm_count,
                                                          stream, &taken);
        if (st != CB200_STATUS_SUCCESS || taken) return st;
    }
    fwd_params p{};
    p.row_ptr = x.row_ptr; p.packed_row_ptr = x.packed_row_ptr; p.col_idx = x.col_idx; p.packed = x.packed;
    p.scales = x.scales; p.offsets = x.offsets; p.w = d.dense; p.y = d.out; p.w_ld = d.dense_ld; p.y_ld = d.out_ld;
    p.row_begin = row_begin; p.row_end = row_end; p.n = static_cast<int>(d.n); p.policy = x.policy;
    p.alpha = d.alpha; p.beta = d.beta; p.bias = d.bias; p.epilogue = d.epilogue;

    const std::size_t elem = d.dense_dtype == CB200_DTYPE_BF16 ? 2u : 4u;
    const bool vector_ok = (reinterpret_cast<std::uintptr_t>(d.dense) % 16u == 0u) && ((d.dense_ld * elem) % 16u == 0u) &&
                           (reinterpret_cast<std::uintptr_t>(d.out) % 16u == 0u) && ((d.out_ld * 4u) % 16u == 0u);
    if (x.bits == 8) {
        if (d.dense_dtype == CB200_DTYPE_BF16) return dispatch_n<8, __nv_bfloat16>(p, vector_ok, stream);
        return dispatch_n<8, float>(p, vector_ok, stream);
    }
    if (x.bits == 4) {
        if (x.packed_row_ptr == nullptr) return fail(CB200_STATUS_INVALID_ARGUMENT, "4-bit codes need packed_row_ptr");
        if (d.dense_dtype == CB200_DTYPE_BF16) return dispatch_n<4, __nv_bfloat16>(p, vector_ok, stream);
        return dispatch_n<4, float>(p, vector_ok, stream);
    }
    return fail(CB200_STATUS_UNSUPPORTED, "forward SpMM supports 8-bit and 4-bit codes, got %d", x.bits);
}

} // namespace cb200
