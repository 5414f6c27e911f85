// Tensor-core kernel of the quantized Blocked-ELL projection for 32x32 blocks:
//     Y[cells, N] = alpha * deq(X_bell)[cells, genes] * W[genes, N] + beta * Y,   N in {128, 256}.
//
// Reference counterpart: quantized_blocked_ell_spmm_fwd_kernel_ (scalar, one thread per output
// element, src/compute/sparse/project/kernels/quantized_blocked_ell_spmm_fwd_kernel_.cuh:1-39) and
// the cuSPARSE f16 Blocked-ELL route (src/compute/sparse/project/project.cu:258-298).
//
// Formulation.  A block row is 32 cells and ell_cols/32 present blocks, each naming 32 genes.  A
// block row therefore is a dense contraction over K = 32 * blocks genes, but with only 32 rows --
// too few for the M side of a tcgen05 MMA.  The product is computed transposed:
//     D^T[N, 32 cells] += W^T[N, 32 genes of the block] * deq(X)^T[32 genes, 32 cells]
// i.e. M = 128 output columns per MMA (two MMAs side by side for N = 256), N_mma = 32 cells,
// K = 16 genes per instruction, fp32 accumulators in TMEM (lane = output column, TMEM column =
// cell).  Both operands are K-major in shared memory in the no-swizzle core-matrix layout
// (8 rows x 16 bytes per core matrix): that needs W^T, so a small kernel first writes, into the
// caller's workspace, W^T per gene block of 32 (genes padded with zeros) already in that operand
// layout; a block's N x 32 slice is then one contiguous 16 KB range.
//
// Operands are fp16 (eleven significant bits against bf16's eight), each stored times a power of two that brings
// its largest magnitude into [2^14, 2^15) so that fp16's exponent range cannot overflow; the factors (found on the
// device at every launch: largest |W|, and the bound of the decoded magnitudes from scales and offsets) are divided
// out of the result.  The decode runs on pairs: a byte permute (code -> fp16 1024 + code), a subtraction, a fused
// multiply-add with the pair's {scale, offset} from a table of fp16 pairs written beside W^T at launch.
//
// One CTA (288 threads, two CTAs per SM) streams the present blocks of its block rows, two at a time, through a
// 2-stage ring (two blocks share a stage's waits, proxy fence and hand-over: 0.273 ms against 0.296 with one
// block per stage and four stages, on 250k cells x 8,192 genes):
//   warps 4-7  producers: one thread fetches the block's slice of W^T with a single bulk async copy
//              (cp.async.bulk, byte-counted on the stage's mbarrier; fetching it as 1,024 separate
//              16-byte cp.async chunks doubled the L2 sector traffic and ran at half the speed);
//              all 128 decode the block's 32 x 32 codes to fp16 (per-gene scale / zero-point
//              applied in registers) straight into the operand layout.  Codes and metadata of a
//              whole block row are staged in shared memory one block row ahead, so decoding never
//              waits on DRAM;
//   warp  8    one elected thread issues the MMAs, commits them to the stage's "empty" barrier
//              and, after the last block of a block row, to the accumulator's "full" barrier;
//   warps 0-3  epilogue: tcgen05.ld the accumulators (double buffered in TMEM so the next block
//              row's MMAs overlap), apply alpha / beta, store Y rows coalesced.
// Empty blocks (index 0xffffffff) are skipped; genes >= cols and cells past the last row decode
// to 0.  Every barrier wait is bounded; on a time-out a status word is set, the waits stop
// blocking, and the kernel still runs to completion and frees its TMEM.
#include "kernels.cuh"
#include "operand_scaling.cuh"
#include "sm100_primitives.cuh"

#include <cuda_bf16.h>

namespace cb200 {

std::uint64_t qbell_tcgen05_workspace_bytes(std::int64_t cols, std::int64_t n) {
    const std::int64_t kpad = (cols + 31) / 32 * 32;
    return static_cast<std::uint64_t>(n * kpad * 2 + 256 + kpad * 4); // status block | W^T (fp16) | {scale, offset} pairs
}

namespace {

constexpr int kStages = 2;          // ring stages; a stage holds up to kStageBlocks present blocks of one block row
constexpr int kStageBlocks = 2;     // two blocks share the stage's waits, proxy fence and hand-over
constexpr int kMaxWidth = 16;                      // blocks per block row the staging area holds
constexpr int kCodesStageBytes = 32 * 512;         // one block row of codes: 32 cells x up to 512 bytes
constexpr int kMetaStageBytes = kMaxWidth * 128;   // per block: 16 gene pairs x {scale pair, offset pair} as fp16
constexpr int kEpilogueThreads = 128; // warps 0-3
constexpr int kProducerThreads = 128; // warps 4-7
constexpr int kThreads = 288;         // + MMA warp 8
constexpr int kATileBytes = 256 * 64; // 256 output columns x 32 genes fp16
constexpr int kBTileBytes = 32 * 64;  // 32 cells x 32 genes fp16
constexpr int kBlockBytes = kATileBytes + kBTileBytes; // one block's operands: [A 16 KB | B 2 KB]
constexpr int kStageBytes = kStageBlocks * kBlockBytes;

struct tc_params {
    std::int64_t rows, cols;
    int width; // blocks per block row
    std::int64_t row_stride;
    const std::uint32_t *block_col_idx;
    const std::uint8_t *packed;
    const float *scales;
    const float *offsets;
    const __half *wt;        // [kpad/32 gene blocks][n x 32 slice of W^T in operand layout], fp16 times a power of two
    const uint2 *pairs;      // per pair of genes {scale pair, offset pair} as fp16, times the decoded operand's power of two;
                             // row-offset policy: the offset pair holds 1 for a gene of the matrix, 0 for padding
    const unsigned *w_absmax;    // largest |W| of this launch as float bits
    const unsigned *value_bound; // [2] bounds of the decoded magnitudes as float bits
    std::int64_t kpad;
    float *y;
    std::int64_t y_ld;
    std::int64_t block_row_begin, block_row_end; // block rows of this launch
    std::int64_t row_begin, row_end;             // cell rows of this launch
    int n;
    int policy;
    float alpha, beta;
    const float *bias;
    int epilogue;
    int *status;
};

__device__ __forceinline__ void bar_expect_tx(std::uint32_t bar, std::uint32_t bytes) {
    asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_16(std::uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template<int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
// K-major, no swizzle: core matrices of 8 rows x 16 bytes; LBO (between the two core matrices a
// K = 16 instruction reads) = 128 B, SBO (between groups of 8 rows) = 512 B.
__device__ __forceinline__ std::uint64_t smem_desc(std::uint32_t addr) {
    std::uint64_t d = 0;
    d |= static_cast<std::uint64_t>((addr & 0x3ffffu) >> 4);
    d |= static_cast<std::uint64_t>(128u >> 4) << 16;
    d |= static_cast<std::uint64_t>(512u >> 4) << 32;
    d |= static_cast<std::uint64_t>(1) << 46; // descriptor version of this architecture
    return d;
}
// kind::f16 instruction descriptor: D fp32, A and B fp16 (format 0), both K-major, N = 32, M = 128.
constexpr std::uint32_t kInstrDesc = (1u << 4) | ((32u >> 3) << 17) | ((128u >> 4) << 24);

__device__ __forceinline__ void mma_f16(std::uint32_t tmem_d, std::uint64_t desc_a, std::uint64_t desc_b, bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        :
        : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(kInstrDesc), "r"(accumulate ? 1u : 0u), "r"(0u)
        : "memory");
}
// W [genes][n] (leading dimension ld) -> per gene block of 32, the n x 32 slice of W^T already in
// the shared-memory operand layout (core matrices of 8 output columns x 8 genes, 128 bytes each:
// byte offset of (column m, gene e) = (m/8)*512 + (e/8)*128 + (m%8)*16 + (e%8)*2), zero for
// genes >= cols, as fp16(w * ws), ws = operand_scale(largest |w|) (eleven significant bits instead of bf16's
// eight; the exponent range is kept by the power of two).  A block's slice is one contiguous n*64-byte range, so
// the main kernel fetches it with a single bulk copy.  The block's 16 gene pairs of {scale pair, offset pair}
// (fp16, times vs = operand_scale(bound of the decoded magnitudes)) are written beside it.
__global__ void __launch_bounds__(256) pack_w_kernel(const __nv_bfloat16 *w, std::int64_t ld, std::int64_t cols, int n, __half *packed_wt,
                                                     const float *scales, const float *offsets, int row_policy, const unsigned *w_absmax,
                                                     const unsigned *value_bound, uint2 *pairs) {
    const std::int64_t block = blockIdx.x;                     // gene block
    const float ws = operand_scale(__uint_as_float(*w_absmax));
    __half *dst = packed_wt + block * static_cast<std::int64_t>(n) * 32;
    // a thread makes one 16-byte piece: a column's values of eight consecutive genes; consecutive threads take consecutive
    // columns, so that their loads of a gene's row and their pieces are contiguous
    for (int item = threadIdx.x; item < n * 4; item += blockDim.x) {
        const int m = item % n, e8 = item / n;
        std::uint32_t packed[4];
#pragma unroll
        for (int j = 0; j < 8; j += 2) {
            float v[2];
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                const std::int64_t gene = block * 32 + e8 * 8 + j + k;
                v[k] = gene < cols ? __bfloat162float(w[gene * ld + m]) : 0.0f;
            }
            const __half2 h = __floats2half2_rn(v[0] * ws, v[1] * ws);
            packed[j >> 1] = *reinterpret_cast<const std::uint32_t *>(&h);
        }
        *reinterpret_cast<uint4 *>(reinterpret_cast<unsigned char *>(dst) + (m >> 3) * 512 + e8 * 128 + (m & 7) * 16) =
            make_uint4(packed[0], packed[1], packed[2], packed[3]);
    }
    if (threadIdx.x < 16) {
        const float vs = operand_scale(__uint_as_float(value_bound[0]) + __uint_as_float(value_bound[1]));
        float sc[2], of[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const std::int64_t g = block * 32 + threadIdx.x * 2 + i;
            sc[i] = g < cols ? (scales != nullptr ? scales[g] : 1.0f) * vs : 0.0f;
            if (row_policy) of[i] = g < cols ? 1.0f : 0.0f;
            else of[i] = g < cols && offsets != nullptr ? offsets[g] * vs : 0.0f;
        }
        const __half2 s2 = __floats2half2_rn(sc[0], sc[1]), o2 = __floats2half2_rn(of[0], of[1]);
        pairs[block * 16 + threadIdx.x] = make_uint2(*reinterpret_cast<const unsigned *>(&s2), *reinterpret_cast<const unsigned *>(&o2));
    }
}

template<int BITS, int H /* N / 128 */>
__global__ void __launch_bounds__(kThreads, 2) qbell_tcgen05_kernel(const tc_params p) {
    extern __shared__ __align__(1024) unsigned char smem[];
    // [kStages][kStageBlocks][A 16 KB | B 2 KB] | staged codes [2] | staged scales/offsets [2] | barriers | tmem base | flags
    std::uint64_t *bars = reinterpret_cast<std::uint64_t *>(smem + kStages * kStageBytes + 2 * kCodesStageBytes + 2 * kMetaStageBytes);
    std::uint64_t *full_bar = bars;                  // [kStages]  producers -> MMA      (one arrival per warp)
    std::uint64_t *empty_bar = bars + kStages;       // [kStages]  MMA commit -> producers (1 arrival)
    std::uint64_t *acc_full = bars + 2 * kStages;    // [2]        MMA commit -> epilogue  (1 arrival)
    std::uint64_t *acc_empty = bars + 2 * kStages + 2; // [2]      epilogue -> MMA        (128 arrivals)
    std::uint32_t *tmem_slot = reinterpret_cast<std::uint32_t *>(bars + 2 * kStages + 4);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    int *row_has_blocks = const_cast<int *>(reinterpret_cast<volatile int *>(tmem_slot + 2)); // [2] per accumulator buffer

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const std::uint32_t smem0 = smem_addr(smem);
    constexpr int kTmemCols = 2 * H * 32; // two accumulator buffers

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            bar_init(smem_addr(full_bar + s), kProducerThreads / 32); // one arrival per producer warp
            bar_init(smem_addr(empty_bar + s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            bar_init(smem_addr(acc_full + b), 1);
            bar_init(smem_addr(acc_empty + b), kEpilogueThreads);
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

    const std::int64_t first = p.block_row_begin + blockIdx.x;
    const std::int64_t step = gridDim.x;
    const bool row_policy = p.policy == CB200_DECODE_COLUMN_SCALE_ROW_OFFSET;

    if (warp >= 4 && warp < 8) {
        // ================= producers =================
        const int pt = tid - 128;          // 0..127
        // B tile: cell within the block row, 8-gene chunk.  A warp takes 16 cells x 2 neighbouring chunks.  The two lanes
        // of a pair READ the two halves of one 16-byte piece of a cell's staged codes (the pieces of a row are permuted by
        // cell mod 8 when they are staged, so the eight cells of a half warp read eight different bank groups).  The odd
        // lanes then swap their codes with the odd lane eight further on, so that a quarter warp DECODES AND STORES cells
        // c .. c + 3 of one chunk and cells c + 4 .. c + 7 of the next: eight different bank groups of the B tile.
        const int pair = (pt & 31) >> 1, parity = pt & 1, cell_base = ((pt >> 5) & 1) * 16;
        const int load_cell = cell_base + pair;
        const int cell = cell_base + (parity != 0 ? (pair ^ 4) : pair), chunk = (pt >> 6) * 2 + parity;
        const std::uint32_t codes_stage = smem0 + kStages * kStageBytes;          // [2][32 cells][512 B]
        const std::uint32_t meta_stage = codes_stage + 2 * kCodesStageBytes;       // [2][16 slots][32 scales | 32 offsets]
        const int row_bytes = p.width * 32 * BITS / 8;
        const int chunks_per_row = row_bytes / 16;
        const float vs = operand_scale(__uint_as_float(__ldg(p.value_bound)) + __uint_as_float(__ldg(p.value_bound + 1)));
        const __half2 magic = __half2half2(__ushort_as_half(static_cast<unsigned short>(0x6400u))); // 1024: fp16(0x6400 | code) = 1024 + code

        // Codes and per-gene metadata of a whole block row are brought into shared memory one block
        // row ahead of their use, so that decoding an item never waits on DRAM.
        auto prefetch_block_row = [&](std::int64_t br, int buf) {
            for (int i = pt; i < 32 * chunks_per_row; i += kProducerThreads) {
                const int c_cell = i / chunks_per_row, c = i % chunks_per_row;
                const std::int64_t row = br * 32 + c_cell;
                if (row >= p.row_begin && row < p.row_end)
                    cp_async_16(codes_stage + buf * kCodesStageBytes + c_cell * 512 + ((c ^ (c_cell & 7)) << 4), p.packed + row * p.row_stride + c * 16);
            }
            for (int i = pt; i < p.width * 8; i += kProducerThreads) { // a block's 16 pairs: eight 16-byte pieces
                const int slot = i >> 3, q = i & 7;
                const std::uint32_t bc = __ldg(p.block_col_idx + br * p.width + slot);
                if (bc == 0xffffffffu) continue;
                cp_async_16(meta_stage + buf * kMetaStageBytes + slot * 128 + q * 16, p.pairs + static_cast<std::int64_t>(bc) * 16 + q * 2);
            }
        };

        long long item = 0;                // items issued by this thread
        int iteration = 0;
        if (first < p.block_row_end) prefetch_block_row(first, 0);
        cp_async_commit();
        for (std::int64_t br = first; br < p.block_row_end; br += step, ++iteration) {
            const int buf = iteration & 1;
            const std::int64_t row = br * 32 + cell;
            const bool cell_valid = row >= p.row_begin && row < p.row_end;
            // row-offset policy: the cell's offset, times the operand's power of two, for both genes of a pair
            const __half2 row_offset2 = __float2half2_rn((row_policy && p.offsets != nullptr && cell_valid) ? __ldg(p.offsets + row) * vs : 0.0f);
            // this block row's staged data is complete for every producer thread, and everyone has
            // finished decoding the previous block row (whose buffer the next prefetch overwrites)
            cp_async_wait<0>();
            asm volatile("bar.sync 1, %0;" ::"n"(kProducerThreads) : "memory");
            if (br + step < p.block_row_end) prefetch_block_row(br + step, buf ^ 1);
            cp_async_commit();
            const std::uint32_t my_codes = codes_stage + buf * kCodesStageBytes + load_cell * 512;
            const std::uint32_t my_meta = meta_stage + buf * kMetaStageBytes + chunk * 32; // the chunk's four gene pairs
            // the block columns of the block row: one load per lane, handed round by shuffles (a load per block put a
            // global-memory latency at the head of every item)
            const std::uint32_t bc_lane = lane < p.width ? __ldg(p.block_col_idx + br * p.width + lane) : 0xffffffffu;
            // present blocks of the block row, taken two at a time
            unsigned todo = __ballot_sync(0xffffffffu, bc_lane != 0xffffffffu);
            while (todo != 0u) {
                int slots[kStageBlocks];
                int blocks = 0;
#pragma unroll
                for (int j = 0; j < kStageBlocks; ++j) {
                    slots[j] = todo != 0u ? __ffs(static_cast<int>(todo)) - 1 : -1;
                    if (todo != 0u) {
                        todo &= todo - 1u;
                        ++blocks;
                    }
                }
                const int stage = static_cast<int>(item % kStages);
                bar_wait(smem_addr(empty_bar + stage), static_cast<std::uint32_t>(((item / kStages) & 1) ^ 1), abort_flag);
                const std::uint32_t stage_base = smem0 + stage * kStageBytes;
                // ---- A: the blocks' slices of W^T, already in operand layout: one bulk copy each
                if (pt == 0) bar_expect_tx(smem_addr(full_bar + stage), static_cast<std::uint32_t>(blocks) * (H * 128 * 64));
#pragma unroll
                for (int j = 0; j < kStageBlocks; ++j) {
                if (slots[j] < 0) break;
                const int slot = slots[j];
                const std::uint32_t bc = __shfl_sync(0xffffffffu, bc_lane, slot);
                const std::uint32_t a_tile = stage_base + j * kBlockBytes;
                const std::uint32_t b_tile = a_tile + kATileBytes;
                if (pt == 0)
                    bulk_copy_g2s(a_tile, p.wt + static_cast<std::int64_t>(bc) * (H * 128 * 32), H * 128 * 64, smem_addr(full_bar + stage));
                // ---- B: decode 8 codes of (cell, genes chunk) to fp16, from the staged copies: per pair of codes a byte
                //      permute (code -> fp16 1024 + code), a subtraction (exact), a fused multiply-add with the pair's
                //      {scale, offset}; genes past the matrix have scale and offset 0
                std::uint32_t out[4];
                // every lane reads and swaps (rows outside the launch hold stale bytes that are never decoded)
                std::uint32_t lo = 0, hi = 0;
                if constexpr (BITS == 8)
                    asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];" : "=r"(lo), "=r"(hi) : "r"(my_codes + (((slot * 2 + (chunk >> 1)) ^ (load_cell & 7)) << 4) + (chunk & 1) * 8));
                else
                    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(lo) : "r"(my_codes + ((slot ^ (load_cell & 7)) << 4) + chunk * 4));
                {
                    const std::uint32_t lo_far = __shfl_xor_sync(0xffffffffu, lo, 8), hi_far = __shfl_xor_sync(0xffffffffu, hi, 8);
                    if (parity != 0) {
                        lo = lo_far;
                        hi = hi_far;
                    }
                }
                if (cell_valid) {
                    std::uint32_t raw[4];
                    if constexpr (BITS == 8) {
                        raw[0] = __byte_perm(lo, 0x64646464u, 0x4140u);
                        raw[1] = __byte_perm(lo, 0x64646464u, 0x4342u);
                        raw[2] = __byte_perm(hi, 0x64646464u, 0x4140u);
                        raw[3] = __byte_perm(hi, 0x64646464u, 0x4342u);
                    } else {
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const std::uint32_t two = lo >> (8 * e); // the byte that holds the pair's two 4-bit codes
                            raw[e] = 0x64006400u | (two & 0xfu) | ((two & 0xf0u) << 12);
                        }
                    }
                    uint4 m0, m1; // {scale pair, offset pair} of the chunk's pairs 0-1 and 2-3
                    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(m0.x), "=r"(m0.y), "=r"(m0.z), "=r"(m0.w) : "r"(my_meta + slot * 128));
                    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(m1.x), "=r"(m1.y), "=r"(m1.z), "=r"(m1.w) : "r"(my_meta + slot * 128 + 16));
                    const std::uint32_t sc[4] = {m0.x, m0.z, m1.x, m1.z}, of[4] = {m0.y, m0.w, m1.y, m1.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const __half2 code2 = __hsub2(*reinterpret_cast<const __half2 *>(&raw[e]), magic);
                        __half2 o2 = *reinterpret_cast<const __half2 *>(&of[e]);
                        if (row_policy) o2 = __hmul2(o2, row_offset2); // the pair's {1 | 0} times the cell's offset
                        const __half2 v = __hfma2(code2, *reinterpret_cast<const __half2 *>(&sc[e]), o2);
                        out[e] = *reinterpret_cast<const std::uint32_t *>(&v);
                    }
                } else {
#pragma unroll
                    for (int e = 0; e < 4; ++e) out[e] = 0u;
                }
                {
                    const std::uint32_t dst = b_tile + (cell >> 3) * 512 + chunk * 128 + (cell & 7) * 16;
                    const std::uint32_t *w32 = out;
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(w32[0]), "r"(w32[1]), "r"(w32[2]), "r"(w32[3])
                                 : "memory");
                }
                } // blocks of the stage
                fence_async_proxy();                      // the B tiles were written with ordinary stores
                __syncwarp();
                if (lane == 0) bar_arrive(smem_addr(full_bar + stage));
                ++item;
            }
        }
        cp_async_wait<0>();
    } else if (warp == 8) {
        // ================= MMA issuer =================
        long long item = 0;
        long long use = 0; // block rows handled (accumulator buffer uses)
        for (std::int64_t br = first; br < p.block_row_end; br += step, ++use) {
            const int buf = static_cast<int>(use & 1);
            bar_wait(smem_addr(acc_empty + buf), static_cast<std::uint32_t>(((use >> 1) & 1) ^ 1), abort_flag);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            bool any = false;
            const std::uint32_t bc_lane = lane < p.width ? __ldg(p.block_col_idx + br * p.width + lane) : 0xffffffffu;
            unsigned todo = __ballot_sync(0xffffffffu, bc_lane != 0xffffffffu);
            while (todo != 0u) {
                int blocks = 0;
#pragma unroll
                for (int j = 0; j < kStageBlocks; ++j)
                    if (todo != 0u) {
                        todo &= todo - 1u;
                        ++blocks;
                    }
                const int stage = static_cast<int>(item % kStages);
                bar_wait(smem_addr(full_bar + stage), static_cast<std::uint32_t>((item / kStages) & 1), abort_flag);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (lane == 0) {
#pragma unroll
                    for (int j = 0; j < kStageBlocks; ++j) {
                        if (j >= blocks) break;
                        const std::uint32_t a_tile = smem0 + stage * kStageBytes + j * kBlockBytes;
                        const std::uint32_t b_tile = a_tile + kATileBytes;
#pragma unroll
                        for (int h = 0; h < H; ++h) {
#pragma unroll
                            for (int kk = 0; kk < 2; ++kk) {
                                mma_f16(tmem_base + buf * (H * 32) + h * 32, smem_desc(a_tile + h * 8192 + kk * 256),
                                         smem_desc(b_tile + kk * 256), any || j > 0 || kk > 0);
                            }
                        }
                    }
                    mma_commit(smem_addr(empty_bar + stage)); // the stage is free once these MMAs have read it
                }
                __syncwarp();
                any = true;
                ++item;
            }
            if (lane == 0) {
                row_has_blocks[buf] = any ? 1 : 0;
                mma_commit(smem_addr(acc_full + buf));        // accumulators complete (or nothing was issued)
            }
            __syncwarp();
        }
    } else if (warp < 4) {
        // ================= epilogue =================
        // both operands were stored times powers of two (fp16 range): the result is divided by them again
        const float alpha = p.alpha / (operand_scale(__uint_as_float(__ldg(p.w_absmax))) *
                                       operand_scale(__uint_as_float(__ldg(p.value_bound)) + __uint_as_float(__ldg(p.value_bound + 1))));
        long long use = 0;
        for (std::int64_t br = first; br < p.block_row_end; br += step, ++use) {
            const int buf = static_cast<int>(use & 1);
            bar_wait(smem_addr(acc_full + buf), static_cast<std::uint32_t>((use >> 1) & 1), abort_flag);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const bool any = *reinterpret_cast<volatile int *>(row_has_blocks + buf) != 0;
            const std::int64_t row0 = br * 32;
#pragma unroll
            for (int h = 0; h < H; ++h) {
                float v[32];
                if (any) {
                    tmem_ld32(tmem_base + (static_cast<std::uint32_t>(warp * 32) << 16) + buf * (H * 32) + h * 32, v);
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = 0.0f;
                }
                const int col = h * 128 + warp * 32 + lane;
                // this thread writes one output column of 32 rows: its bias is loaded once
                const bool composed = p.epilogue != CB200_EPILOGUE_NONE;
                const float bias = composed && epilogue_has_bias(p.epilogue) ? __ldg(p.bias + col) : 0.0f;
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    const std::int64_t row = row0 + c;
                    if (row >= p.row_begin && row < p.row_end) {
                        float *out = p.y + row * p.y_ld + col;
                        float r = alpha * v[c];
                        if (p.beta != 0.0f) r = fmaf(p.beta, *out, r);
                        if (composed) r = apply_epilogue(r, bias, p.epilogue);
                        *out = r;
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            bar_arrive(smem_addr(acc_empty + buf));
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

constexpr std::size_t kSmemBytes = kStages * kStageBytes + 2 * kCodesStageBytes + 2 * kMetaStageBytes + (2 * kStages + 4) * sizeof(std::uint64_t) + 32;

template<int BITS, int H>
cb200_status launch(const tc_params &p, int sm_count, cudaStream_t stream) {
    CB200_CUDA_OK(cudaFuncSetAttribute(qbell_tcgen05_kernel<BITS, H>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(kSmemBytes)));
    const std::int64_t block_rows = p.block_row_end - p.block_row_begin;
    const unsigned grid = static_cast<unsigned>(block_rows < 2ll * sm_count ? block_rows : 2ll * sm_count);
    qbell_tcgen05_kernel<BITS, H><<<grid, kThreads, kSmemBytes, stream>>>(p);
    count_launch();
    CB200_CUDA_OK(cudaGetLastError());
    return CB200_STATUS_SUCCESS;
}

} // namespace

cb200_status launch_qbell_tcgen05(const qbell_view &x, const dense_args &d, std::int64_t row_begin,
                                  std::int64_t row_end, void *workspace, std::uint64_t workspace_bytes, int sm_count,
                                  cudaStream_t stream, bool *taken) {
    *taken = false;
    if (x.block_size != 32 || (d.n != 128 && d.n != 256) || d.dense_dtype != CB200_DTYPE_BF16) return CB200_STATUS_SUCCESS;
    if (x.bits != 8 && x.bits != 4) return CB200_STATUS_SUCCESS;
    if (x.ell_cols <= 0 || x.ell_cols % 32 != 0 || x.ell_cols / 32 > kMaxWidth) return CB200_STATUS_SUCCESS;
    // staging copies move 16 bytes at a time
    if (x.row_stride_bytes % 16 != 0 || reinterpret_cast<std::uintptr_t>(x.packed) % 16u != 0u) return CB200_STATUS_SUCCESS;
    if (reinterpret_cast<std::uintptr_t>(x.scales) % 16u != 0u || reinterpret_cast<std::uintptr_t>(x.offsets) % 16u != 0u) return CB200_STATUS_SUCCESS;
    if (workspace == nullptr || workspace_bytes < qbell_tcgen05_workspace_bytes(x.cols, d.n)) return CB200_STATUS_SUCCESS;
    if (reinterpret_cast<std::uintptr_t>(workspace) % 256u != 0u) return CB200_STATUS_SUCCESS;
    if (row_end <= row_begin) return CB200_STATUS_SUCCESS;

    const std::int64_t kpad = (x.cols + 31) / 32 * 32;
    int *status = static_cast<int *>(workspace);
    unsigned *w_absmax = reinterpret_cast<unsigned *>(workspace) + 1;    // float bits of the largest |W|
    unsigned *value_bound = reinterpret_cast<unsigned *>(workspace) + 2; // [2], [3]: bounds of the decoded magnitudes
    __half *wt = reinterpret_cast<__half *>(static_cast<unsigned char *>(workspace) + 256);
    uint2 *pairs = reinterpret_cast<uint2 *>(static_cast<unsigned char *>(workspace) + 256 + d.n * kpad * 2);
    const bool row_policy = x.policy == CB200_DECODE_COLUMN_SCALE_ROW_OFFSET;
    CB200_CUDA_OK(cudaMemsetAsync(status, 0, 4 * sizeof(int), stream));
    const std::int64_t elements = x.cols * d.n;
    const unsigned w_blocks = static_cast<unsigned>(std::min<std::int64_t>((elements + 1023) / 1024, 4 * static_cast<std::int64_t>(sm_count)));
    const std::int64_t span = std::max<std::int64_t>(x.cols, row_policy ? x.rows : 0);
    operand_bounds_kernel<<<w_blocks + static_cast<unsigned>((span + 255) / 256), 256, 0, stream>>>(
        static_cast<const __nv_bfloat16 *>(d.dense), d.dense_ld, x.cols, static_cast<int>(d.n), w_blocks, x.scales,
        row_policy ? nullptr : x.offsets, row_policy ? x.offsets : nullptr, x.rows, static_cast<float>((1 << x.bits) - 1), w_absmax, value_bound);
    pack_w_kernel<<<static_cast<unsigned>(kpad / 32), 256, 0, stream>>>(static_cast<const __nv_bfloat16 *>(d.dense), d.dense_ld, x.cols,
                                                                        static_cast<int>(d.n), wt, x.scales, x.offsets, row_policy ? 1 : 0,
                                                                        w_absmax, value_bound, pairs);
    count_launch(2);
    CB200_CUDA_OK(cudaGetLastError());
    tc_params p{};
    p.rows = x.rows; p.cols = x.cols; p.width = x.ell_cols / 32; p.row_stride = x.row_stride_bytes;
    p.block_col_idx = x.block_col_idx; p.packed = x.packed; p.scales = x.scales; p.offsets = x.offsets;
    p.wt = wt; p.pairs = pairs; p.w_absmax = w_absmax; p.value_bound = value_bound; p.kpad = kpad; p.y = d.out; p.y_ld = d.out_ld;
    p.block_row_begin = row_begin / 32; p.block_row_end = (row_end + 31) / 32;
    p.row_begin = row_begin; p.row_end = row_end;
    p.n = static_cast<int>(d.n); p.policy = x.policy; p.alpha = d.alpha; p.beta = d.beta; p.bias = d.bias; p.epilogue = d.epilogue; p.status = status;
    *taken = true;
    if (x.bits == 8) return d.n == 256 ? launch<8, 2>(p, sm_count, stream) : launch<8, 1>(p, sm_count, stream);
    return d.n == 256 ? launch<4, 2>(p, sm_count, stream) : launch<4, 1>(p, sm_count, stream);
}

} // namespace cb200
