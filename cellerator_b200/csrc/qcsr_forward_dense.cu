// Quantized CSR forward projection on the tensor cores from dense operand tiles kept at prepare
// (schedule "tensor_dense"):
//     Y[cells, N] = alpha * deq(X)[cells, genes] * W[genes, N] + beta * Y,   N in {32, 64, 128}.
// The tiles are built from the window-blocked copy (qcsr_forward_blocked.cu), whose geometry and W
// records they share (blocked_tile.cuh).  Reference counterpart: csr_spmm_fwd over dequantised values
// (src/compute/sparse/ops/base_sparse.cu); the reference keeps no such copy, its prepared_operation only
// has room for one (persistent_kernel_state, operation_core.hh:126-129).
#include "blocked_tile.cuh"

#include <algorithm>

namespace cb200 {
namespace {

// Dense operand tiles (schedule "tensor_dense").
//
// Above a few per cent of density the scatter is the whole cost of a window, and it repeats the
// same work on every launch: the matrix does not change between launches.  So prepare can run the
// scatter once and keep its result: for every (group, window) the 64 KB operand tile, in exactly the
// shared-memory image the MMA reads (K-major, 128-byte swizzle), stored as two 32 KB half-stages
// (64 genes each; inside a half-stage the two 128-row sub-blocks follow each other).  A launch then
// only streams: the copy engine brings half-stages into a ring, one thread issues the MMAs, the
// accumulators of a group are double buffered in TMEM so that writing Y overlaps the next group.
// The kernel moves 2 bytes per matrix element (decoded bf16) instead of ~5 per stored entry, which
// is more HBM traffic above ~40 % density only in theory: below it the tile build, not HBM, bounds
// the blocked kernel.  Cost: rows x genes x 2 bytes of device memory per prepared operation.

constexpr int kDenseStageBytes = kSubBlocks * kHalfBytes; // 32 KB: 256 rows x 64 genes
constexpr int kDenseBStages = 3;
constexpr int kDenseALoaders = 2;                          // warps whose elected lane issues half-stage copies, in turn
constexpr int kDenseThreads = kRows + 32 * (2 + kDenseALoaders); // 8 epilogue warps, MMA warp, W loader warp, A loader warps
__host__ __device__ constexpr int dense_a_stages(int n) {
    return (232448 - 1024 - kDenseBStages * n * kWin * 2) / kDenseStageBytes > 6
               ? 6
               : (232448 - 1024 - kDenseBStages * n * kWin * 2) / kDenseStageBytes;
}

// One CTA per (group, window) segment of the window-blocked copy: zero a tile in shared memory,
// decode and scatter the segment's entries exactly as the blocked kernel does, write the tile out.
__global__ void __launch_bounds__(512) densify_kernel(const std::uint32_t *entries, const std::int64_t *seg_ptr,
                                                      const float *scales, const float *gene_offsets,
                                                      const float *row_offsets, std::int64_t rows, std::int64_t cols,
                                                      int windows, int baked, unsigned char *tiles) {
    extern __shared__ __align__(16) unsigned char tile[];
    const std::int64_t seg = blockIdx.x;
    const std::int64_t group = seg / windows;
    const std::int64_t gene0 = (seg % windows) * kWin;
    const int tid = threadIdx.x;
#pragma unroll
    for (int k = 0; k < kABufBytes / (512 * 16); ++k)
        *reinterpret_cast<uint4 *>(tile + k * (512 * 16) + tid * 16) = make_uint4(0u, 0u, 0u, 0u);
    __syncthreads();
    const std::int64_t lo = seg_ptr[seg], hi = seg_ptr[seg + 1];
    for (std::int64_t i = lo + tid; i < hi; i += 512) {
        const std::uint32_t e = entries[i];
        if (static_cast<int>(e) < 0) continue; // padding
        if (baked != 0) {
            *reinterpret_cast<unsigned short *>(tile + (((e >> 16) & 0x7fffu) << 1)) = static_cast<unsigned short>(e & 0xffffu);
            continue;
        }
        const std::int64_t gene = gene0 + ((e >> 8) & (kWin - 1));
        const std::uint32_t off = ((e >> 15) & 0x7fffu) << 1;
        if (gene >= cols) continue;
        const float scale = scales != nullptr ? __ldg(scales + gene) : 1.0f;
        float add = gene_offsets != nullptr ? __ldg(gene_offsets + gene) : 0.0f;
        if (row_offsets != nullptr) {
            const std::int64_t row = group * kRows + (((off / kSubBlockBytes) << 7) | (((off >> 10) & 15u) << 3) | ((off >> 7) & 7u));
            add = row < rows ? __ldg(row_offsets + row) : 0.0f;
        }
        *reinterpret_cast<__nv_bfloat16 *>(tile + off) = __float2bfloat16_rn(fmaf(static_cast<float>(e & 0xffu), scale, add));
    }
    __syncthreads();
    unsigned char *out = tiles + static_cast<std::size_t>(seg) * kABufBytes;
#pragma unroll
    for (int k = 0; k < kABufBytes / (512 * 16); ++k) {
        const int o = k * (512 * 16) + tid * 16; // tile image: [sub-block][half][16 KB]; stored: [half][sub-block][16 KB]
        const int sb = o / kSubBlockBytes, half = (o / kHalfBytes) % (kWin / 64);
        *reinterpret_cast<uint4 *>(out + half * kDenseStageBytes + sb * kHalfBytes + (o % kHalfBytes)) =
            *reinterpret_cast<const uint4 *>(tile + o);
    }
}

struct dense_params {
    const unsigned char *tiles;   // [group][window][half][sub-block][16 KB]
    const unsigned char *records; // W windows in operand layout, record_bytes(N) apart
    float *y;
    std::int64_t y_ld;
    std::int64_t row_end; // rows >= row_end are computed but not written
    std::int64_t group_begin, group_end;
    int windows;
    float alpha, beta;
    const float *bias;
    int epilogue;
    int *status;
    std::uint32_t idesc;       // bf16 or fp16 operands
    float result_scale;        // fp16 tiles: 1 / (the power of two the values were stored times)
    const unsigned *w_absmax;  // fp16 operands: largest |W| of this launch as float bits; else null
};

template<int NC>
__global__ void __launch_bounds__(kDenseThreads, 1) qcsr_fwd_dense_kernel(const dense_params p) {
    constexpr int SA = dense_a_stages(NC);
    constexpr int SB = kDenseBStages;
    constexpr int WREC = NC * kWin * 2;       // bytes of one W window in operand layout
    constexpr int REC = record_bytes(NC);     // distance of the windows' records in global memory
    constexpr int kAccCols = kSubBlocks * NC; // one accumulator set: a group's rows x N
    constexpr int kTmemCols = 2 * kAccCols < 32 ? 32 : 2 * kAccCols;
    const std::uint32_t IDESC = p.idesc;
    static_assert(SA >= 2, "the half-stage ring needs two stages");
    extern __shared__ __align__(1024) unsigned char smem[];
    // [SA][half-stage] | [SB][W window] | barriers | tmem slot | abort
    std::uint64_t *bars = reinterpret_cast<std::uint64_t *>(smem + SA * kDenseStageBytes + SB * WREC);
    std::uint64_t *a_full = bars;              // [SA] copy engine -> MMA
    std::uint64_t *a_empty = a_full + SA;      // [SA] MMA commit -> A loaders
    std::uint64_t *b_full = a_empty + SA;      // [SB] copy engine -> MMA
    std::uint64_t *b_empty = b_full + SB;      // [SB] MMA commit -> W loader
    std::uint64_t *acc_full = b_empty + SB;    // [2]  MMA commit -> epilogue warps
    std::uint64_t *acc_empty = acc_full + 2;   // [2]  epilogue warps -> MMA (one arrival per warp)
    std::uint32_t *tmem_slot = reinterpret_cast<std::uint32_t *>(acc_empty + 2);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const std::uint32_t smem0 = smem_addr(smem);
    const std::uint32_t bstage0 = smem0 + SA * kDenseStageBytes;

    if (tid == 0) {
        for (int s = 0; s < SA; ++s) {
            bar_init(smem_addr(a_full + s), 1);
            bar_init(smem_addr(a_empty + s), 1);
        }
        for (int s = 0; s < SB; ++s) {
            bar_init(smem_addr(b_full + s), 1);
            bar_init(smem_addr(b_empty + s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            bar_init(smem_addr(acc_full + b), 1);
            bar_init(smem_addr(acc_empty + b), kEpilogueWarps);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)), "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const std::uint32_t tmem_base = *tmem_slot;

    const std::int64_t first_group = p.group_begin + blockIdx.x;
    const std::int64_t my_groups = first_group < p.group_end ? (p.group_end - first_group + gridDim.x - 1) / gridDim.x : 0;

    if (warp < kEpilogueWarps) {
        // ================= thread t writes row t of the group: TMEM lane = row within the sub-block =================
        const int sub = tid >> 7;
        for (std::int64_t gi = 0; gi < my_groups; ++gi) {
            const std::uint32_t ab = static_cast<std::uint32_t>(gi & 1);
            const std::int64_t row = (first_group + gi * gridDim.x) * kRows + tid;
            bar_wait(smem_addr(acc_full + ab), static_cast<std::uint32_t>((gi >> 1) & 1), abort_flag);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int h = 0; h < NC / 32; ++h) {
                float v[32];
                tmem_ld32(tmem_base + (static_cast<std::uint32_t>((warp & 3) * 32) << 16) + ab * kAccCols + sub * NC + h * 32, v);
                if (row < p.row_end) {
                    float *out = p.y + row * p.y_ld + h * 32;
                    store_row32(out, v, p.alpha * p.result_scale / (p.w_absmax != nullptr ? operand_scale(__uint_as_float(__ldg(p.w_absmax))) : 1.0f), p.beta, p.bias, h * 32, p.epilogue);
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) bar_arrive(smem_addr(acc_empty + ab));
        }
    } else if (warp == kEpilogueWarps) {
        // ================= MMA issuer =================
        long long qa = 0, qb = 0;
        for (std::int64_t g = 0; g < my_groups; ++g) {
            const std::uint32_t ab = static_cast<std::uint32_t>(g & 1);
            bar_wait(smem_addr(acc_empty + ab), static_cast<std::uint32_t>(((g >> 1) & 1) ^ 1), abort_flag);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            for (int w = 0; w < p.windows; ++w, ++qb) {
                const int s = static_cast<int>(qb % SB);
                bar_wait(smem_addr(b_full + s), static_cast<std::uint32_t>((qb / SB) & 1), abort_flag);
                const std::uint32_t b_tile = bstage0 + s * WREC;
                for (int half = 0; half < kWin / 64; ++half, ++qa) {
                    const int sa = static_cast<int>(qa % SA);
                    bar_wait(smem_addr(a_full + sa), static_cast<std::uint32_t>((qa / SA) & 1), abort_flag);
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    if (lane == 0) {
                        const std::uint32_t a_stage = smem0 + sa * kDenseStageBytes;
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk) {
                            const std::uint64_t db = smem_desc(b_tile + (half * 4 + kk) * 256);
#pragma unroll
                            for (int sb = 0; sb < kSubBlocks; ++sb)
                                mma_bf16(tmem_base + ab * kAccCols + sb * NC, smem_desc_sw128(a_stage + sb * kHalfBytes + kk * 32), db,
                                         IDESC, w > 0 || half > 0 || kk > 0);
                        }
                        mma_commit(smem_addr(a_empty + sa));
                        if (half == kWin / 64 - 1) {
                            mma_commit(smem_addr(b_empty + s));
                            if (w == p.windows - 1) mma_commit(smem_addr(acc_full + ab));
                        }
                    }
                    __syncwarp();
                }
            }
        }
    } else if (warp == kEpilogueWarps + 1) {
        // ================= W loader =================
        if (lane == 0) {
            const long long total = my_groups * p.windows;
            for (long long q = 0; q < total; ++q) {
                const int s = static_cast<int>(q % SB);
                bar_wait(smem_addr(b_empty + s), static_cast<std::uint32_t>(((q / SB) & 1) ^ 1), abort_flag);
                bar_arrive_expect_tx(smem_addr(b_full + s), WREC);
                bulk_copy_g2s(bstage0 + s * WREC, p.records + static_cast<std::size_t>(q % p.windows) * REC, WREC, smem_addr(b_full + s));
            }
        }
    } else {
        // ================= A loaders: half-stages in turn =================
        if (lane == 0) {
            const long long per_group = static_cast<long long>(p.windows) * (kWin / 64);
            const long long total = my_groups * per_group;
            for (long long q = warp - kEpilogueWarps - 2; q < total; q += kDenseALoaders) {
                const int s = static_cast<int>(q % SA);
                const std::int64_t group = first_group + (q / per_group) * gridDim.x;
                const unsigned char *src = p.tiles + (static_cast<std::size_t>(group) * per_group + static_cast<std::size_t>(q % per_group)) * kDenseStageBytes;
                bar_wait(smem_addr(a_empty + s), static_cast<std::uint32_t>(((q / SA) & 1) ^ 1), abort_flag);
                bar_arrive_expect_tx(smem_addr(a_full + s), kDenseStageBytes);
                bulk_copy_g2s(smem0 + s * kDenseStageBytes, src, kDenseStageBytes, smem_addr(a_full + s));
            }
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
    if (tid == 0 && *abort_flag != 0 && p.status != nullptr) atomicExch(p.status, 1);
}

template<int NC>
cb200_status launch_dense(const dense_params &p, int sm_count, cudaStream_t stream) {
    constexpr std::size_t smem = dense_a_stages(NC) * kDenseStageBytes + kDenseBStages * NC * kWin * 2 +
                                 (2 * dense_a_stages(NC) + 2 * kDenseBStages + 4) * sizeof(std::uint64_t) + 16;
    static_assert(smem <= 232448, "shared memory budget");
    CB200_CUDA_OK(cudaFuncSetAttribute(qcsr_fwd_dense_kernel<NC>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    const std::int64_t groups = p.group_end - p.group_begin;
    const unsigned grid = static_cast<unsigned>(groups < sm_count ? groups : sm_count);
    qcsr_fwd_dense_kernel<NC><<<grid, kDenseThreads, smem, stream>>>(p);
    count_launch();
    CB200_CUDA_OK(cudaGetLastError());
    return CB200_STATUS_SUCCESS;
}

} // namespace

std::uint64_t qcsr_dense_tile_bytes(std::int64_t rows, std::int64_t cols) {
    const std::uint64_t groups = static_cast<std::uint64_t>((rows + kRows - 1) / kRows);
    const std::uint64_t windows = static_cast<std::uint64_t>((cols + kWin - 1) / kWin);
    return groups * windows * static_cast<std::uint64_t>(kABufBytes);
}

// Turns the window-blocked copy into dense operand tiles (decoded bf16 values, scales and offsets of
// `x` baked in); the entry words go back to the arena.  *built is false, with the copy left as it was,
// when the arena has no room for the tiles.  Waits for `stream`.
cb200_status densify_blocked_layout(const qcsr_view &x, blocked_layout *layout, device_arena &arena, cudaStream_t stream,
                                    bool *built) {
    *built = false;
    if (layout == nullptr || layout->seg_ptr == nullptr) return CB200_STATUS_SUCCESS;
    const std::int64_t segments = layout->groups * layout->windows;
    const std::uint64_t bytes = static_cast<std::uint64_t>(segments) * kABufBytes;
    unsigned char *tiles = static_cast<unsigned char *>(arena.take(bytes));
    if (tiles == nullptr) return CB200_STATUS_SUCCESS; // out of memory is not an error of the prepare: the blocked copy stays
    const bool row_policy = x.policy == CB200_DECODE_COLUMN_SCALE_ROW_OFFSET;
    cudaError_t err = cudaFuncSetAttribute(densify_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kABufBytes);
    if (err == cudaSuccess && segments > 0) {
        densify_kernel<<<static_cast<unsigned>(segments), 512, kABufBytes, stream>>>(layout->entries, layout->seg_ptr, x.scales,
                                                                                     row_policy ? nullptr : x.offsets,
                                                                                     row_policy ? x.offsets : nullptr, x.rows, x.cols,
                                                                                     layout->windows, layout->baked ? 1 : 0, tiles);
        count_launch();
        err = cudaGetLastError();
    }
    if (err == cudaSuccess) err = cudaStreamSynchronize(stream);
    if (err != cudaSuccess) {
        arena.give_back(tiles, bytes);
        return fail(CB200_STATUS_CUDA_ERROR, "building the dense operand tiles: %s", cudaGetErrorString(err));
    }
    arena.give_back(layout->entries, static_cast<std::uint64_t>(layout->total_entries) * 4u);
    arena.give_back(layout->seg_ptr, static_cast<std::uint64_t>(segments + 1) * 8u);
    layout->entries = nullptr;
    layout->seg_ptr = nullptr;
    layout->total_entries = 0;
    layout->dense_tiles = tiles;
    layout->bytes = bytes;
    layout->baked = false; // half_values / value_scale stay: the tiles hold what the baked words held
    layout->src_scales = x.scales;
    layout->src_offsets = x.offsets;
    *built = true;
    return CB200_STATUS_SUCCESS;
}

cb200_status launch_qcsr_forward_dense(const qcsr_view &x, const dense_args &d, std::int64_t row_begin,
                                              std::int64_t row_end, void *workspace, std::uint64_t workspace_bytes,
                                              const blocked_layout &layout, int sm_count, cudaStream_t stream, bool *taken) {
    if (d.dense_dtype != CB200_DTYPE_BF16) return CB200_STATUS_SUCCESS;
    if (d.n != 32 && d.n != 64 && d.n != 128) return CB200_STATUS_SUCCESS;
    if (row_begin % kRows != 0) return CB200_STATUS_SUCCESS; // a launch starts on a group boundary, else another kernel runs
    if (reinterpret_cast<std::uintptr_t>(d.out) % 16u != 0u || (d.out_ld * 4u) % 16u != 0u) return CB200_STATUS_SUCCESS;
    if (workspace == nullptr || workspace_bytes < qcsr_blocked_workspace_bytes(x.cols, d.n)) return CB200_STATUS_SUCCESS;
    if (reinterpret_cast<std::uintptr_t>(workspace) % 256u != 0u) return CB200_STATUS_SUCCESS;
    if (x.row_ptr != layout.src_row_ptr || x.col_idx != layout.src_col_idx || x.packed != layout.src_packed ||
        x.scales != layout.src_scales || x.offsets != layout.src_offsets)
        return fail(CB200_STATUS_STALE_STRUCTURE, "the launch's matrix is not the one the dense operand tiles were built from");
    int *status = static_cast<int *>(workspace);
    unsigned *w_absmax = reinterpret_cast<unsigned *>(workspace) + 1; // fp16 operands: float bits of the largest |W|
    unsigned char *records = static_cast<unsigned char *>(workspace) + 256;
    const bool half = layout.half_values;
    CB200_CUDA_OK(cudaMemsetAsync(status, 0, 2 * sizeof(int), stream));
    if (half) {
        const std::int64_t elements = x.cols * d.n;
        const unsigned blocks = static_cast<unsigned>(std::min<std::int64_t>((elements + 1023) / 1024, 4 * static_cast<std::int64_t>(sm_count)));
        absmax_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16 *>(d.dense), d.dense_ld, x.cols, static_cast<int>(d.n), w_absmax);
        count_launch();
        CB200_CUDA_OK(cudaGetLastError());
    }
    pack_windows_kernel<__nv_bfloat16><<<dim3(static_cast<unsigned>(layout.windows), static_cast<unsigned>(d.n / kPackColumns)), 256, 0, stream>>>(
        static_cast<const __nv_bfloat16 *>(d.dense), d.dense_ld, x.cols, static_cast<int>(d.n), 0, nullptr, nullptr, 0, records,
        half ? w_absmax : nullptr);
    count_launch();
    CB200_CUDA_OK(cudaGetLastError());
    dense_params p{};
    p.tiles = layout.dense_tiles; p.records = records; p.y = d.out; p.y_ld = d.out_ld; p.row_end = row_end;
    p.group_begin = row_begin / kRows; p.group_end = (row_end + kRows - 1) / kRows; p.windows = layout.windows;
    p.alpha = d.alpha; p.beta = d.beta; p.bias = d.bias; p.epilogue = d.epilogue; p.status = status;
    p.idesc = instr_desc(static_cast<int>(d.n), half);
    p.result_scale = half ? 1.0f / layout.value_scale : 1.0f;
    p.w_absmax = half ? w_absmax : nullptr;
    *taken = true;
    switch (d.n) {
    case 32: return launch_dense<32>(p, sm_count, stream);
    case 64: return launch_dense<64>(p, sm_count, stream);
    default: return launch_dense<128>(p, sm_count, stream);
    }
}

} // namespace cb200
