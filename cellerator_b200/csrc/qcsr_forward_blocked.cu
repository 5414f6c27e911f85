// Quantized CSR forward projection on the tensor cores from a window-blocked copy of the matrix
// (schedule "tensor_blocked"), for callers whose numeric policy allows bf16 products and who hand
// the device-resident matrix to prepare:
//     Y[cells, N] = alpha * deq(X)[cells, genes] * W[genes, N] + beta * Y,   N in {32, 64, 128}.
//
// Reference counterpart: csr_spmm_fwd over dequantised values (src/compute/sparse/ops/base_sparse.cu)
// behind the CP-Math sparse_dense_multiply operation; the reference has no persistent re-layout,
// its prepared_operation only carries one (persistent_kernel_state, operation_core.hh:126-129).
//
// Idea.  At N = 64 a stored entry costs 64 multiply-adds; the CUDA cores cannot do that at the
// rate HBM delivers entries, the tensor cores can, even if a 256-cell x 128-gene window of the
// matrix (1,750 stored entries on the 1M x 33,538 matrix) is multiplied as a dense tile.  So the
// kernel densifies window by window: the window's entries are decoded to bf16 and scattered into
// a zeroed operand tile in shared memory, and sixteen 128 x N x 16 tcgen05 MMAs multiply the tile
// with the window's slice of W.  Feeding that from CSR needs one thread per row, which diverges
// and issues one uncoalesced load per four entries.  Instead prepare re-lays the matrix once:
// groups of 256 consecutive cell rows, and inside a group the entries ordered by gene window.
// An entry of the copy is one 32-bit word {code, gene within window, byte position in the tile};
// a (group, window) segment is contiguous, so the copy engine streams it into shared memory and
// every lane of the CTA decodes entries, four at a time, with no divergence.  When the operation
// multiplies in one bf16 pass, prepare decodes as well ("baked" words {bf16 value, byte position}):
// a launch then stores the words' low halves where their high halves say, with no table look-up and
// no wait for the W stage (6.93 ms against 7.11 on the 1M x 33,538 matrix).  The split-product
// schedules need the next eight mantissa bits too: prepare writes a second array of baked words,
// bf16(value - hi), under the same segment table (12.7 ms against 14.4 for the two passes), or keeps
// the code words when the caller's memory limit has no room for it.
//
// Two kernels live in this file, a third in qcsr_forward_dense.cu; all persistent with one CTA per SM
// and row groups dealt round-robin:
//   qcsr_fwd_blocked_kernel   one scatter group: code words (split-product schedules under a memory
//                             limit), and baked words whose segments span several chunks;
//   qcsr_fwd_blocked2_kernel  baked words, two scatter groups on alternate windows, an MMA-issuing warp per row
//                             sub-block: every pass of the default schedules (5.04 ms per pass on the
//                             1M x 33,538 matrix; 640 threads);
//   qcsr_fwd_dense_kernel     no scatter at all: prepare kept the operand tiles ("tensor_dense").
//
// Structure of a CTA of the first kernel (608 threads):
//   warps 0-15  zero the A tile (128-byte swizzled K-major layout), wait for the segment's chunks
//               (8 KB each, 2-stage ring), decode and scatter; later thread t < 256 owns TMEM lane t:
//               row t of the group, and writes that row of Y;
//   warp 16     one thread issues the MMAs (2 row sub-blocks x 8 K-steps per window), commits the
//               window to the "A tile free" and "W stage free" barriers, the last window of a group
//               to "accumulators complete";
//   warp 17     one thread feeds the W ring with bulk async copies: W slices, re-laid per window
//               into the K-major core-matrix operand layout by a small kernel before the main one,
//               each followed by the window's {scale, zero-point} table;
//   warp 18     one thread feeds the entry-chunk ring (the code deals chunks to kChunkLoaders such warps
//               in turn; one measured best).
// Every barrier wait is bounded; on a time-out a status word is raised, waits stop blocking, and
// the kernel runs to completion and frees its TMEM.  A non-zero status means Y is not valid.
//
// What bounds it.  Per window the shared memory moves ~64 KB of zeroes, ~20 KB of entries, tables and
// scattered values, ~24 KB of copies coming in and 96 KB of MMA operand reads (the A tile once, the
// W slice once per row sub-block): the kernel runs at the shared-memory bandwidth of the SM, not at
// the tensor pipe's nor at HBM's: the MMAs are held to the rate at which they read their operands (one
// 128 x 64 x 16 MMA per 43-47 cycles), which fills 55 % of a window's time in the two-group kernel.
#include "blocked_tile.cuh"

#include <algorithm>
#include <cstring>

namespace cb200 {
namespace {

// (geometry, entry-word layout and W records: blocked_tile.cuh)

// ---------------------------------------------------------------------------------------------
// prepare time: the window-blocked copy

template<int BITS>
__device__ __forceinline__ unsigned load_code(const std::uint8_t *row_bytes, std::int64_t local) {
    if constexpr (BITS == 8) {
        return row_bytes[local];
    } else {
        const unsigned byte = row_bytes[local >> 1];
        return (local & 1) ? (byte >> 4) : (byte & 0xfu);
    }
}

// One warp per row; the lanes read 32 consecutive entries at a time (coalesced).  A run is a
// maximal stretch of consecutive entries, within those 32, in one gene window (rows with ascending
// genes have one run per window they touch, plus one where a window straddles two reads).  The first
// lane of a run speaks for it: FILL == false adds the run length to counts[group * windows + window];
// FILL == true reserves the run's place in the segment with one atomic, and every lane of the run
// writes its entry there.  Entries with a gene outside [0, cols) are left out by both passes.
// bake != 0: the entry holds bf16(code * scale + offset) and the byte position instead of code and gene
// (bake == 2: the offset is the row's, not the gene's).
template<int BITS, bool FILL>
__global__ void __launch_bounds__(256) blocked_pass_kernel(const std::int64_t *row_ptr, const std::int64_t *packed_row_ptr,
                                                           const std::int32_t *col_idx, const std::uint8_t *packed,
                                                           std::int64_t rows, std::int64_t cols, int windows,
                                                           unsigned *counts, unsigned long long *cursor, std::uint32_t *entries,
                                                           int bake, const float *scales, const float *offsets,
                                                           std::uint32_t *entries_lo, int gene_major, float half_scale) {
    const int lane = threadIdx.x & 31;
    const std::int64_t r = static_cast<std::int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= rows) return; // warp-uniform
    const std::int64_t group = r >> kRowsShift;
    const int rl = static_cast<int>(r & (kRows - 1));
    const std::int64_t begin = row_ptr[r], end = row_ptr[r + 1];
    const std::uint8_t *row_bytes = packed + (packed_row_ptr != nullptr ? packed_row_ptr[r] : begin);
    // the genes of the next 32 entries are requested before this read's are worked on: two loads of a row in flight
    std::int32_t ahead = begin + lane < end ? col_idx[begin + lane] : 0;
    for (std::int64_t base = begin; base < end; base += 32) {
        const std::int64_t i = base + lane;
        const std::int32_t now = ahead;
        if (i + 32 < end) ahead = col_idx[i + 32];
        int window = -2; // past the row's end
        int gl = 0;
        if (i < end) {
            const std::int64_t gene = now;
            window = (gene >= 0 && gene < cols) ? static_cast<int>(gene >> kWinShift) : -1;
            gl = static_cast<int>(gene & (kWin - 1));
        }
        const int before = __shfl_up_sync(0xffffffffu, window, 1);
        const bool head = lane == 0 || window != before;
        const unsigned heads = __ballot_sync(0xffffffffu, head);
        const int start = 31 - __clz(static_cast<int>(heads & (0xffffffffu >> (31 - lane)))); // first lane of this lane's run
        const unsigned later = lane == 31 ? 0u : (heads >> (lane + 1)) << (lane + 1);         // run heads after this lane
        const int next = later != 0u ? __ffs(static_cast<int>(later)) - 1 : 32;
        unsigned long long place = 0;
        if (head && window >= 0) {
            const std::int64_t seg = group * windows + window;
            if constexpr (!FILL) atomicAdd(counts + seg, static_cast<unsigned>(next - lane));
            else place = atomicAdd(cursor + seg, static_cast<unsigned long long>(next - lane));
        }
        if constexpr (FILL) {
            place = __shfl_sync(0xffffffffu, place, start);
            if (window >= 0) {
                const std::uint32_t code = load_code<BITS>(row_bytes, i - begin);
                std::uint32_t word;
                if (bake != 0) {
                    const std::int64_t gene = now;
                    const float scale = scales != nullptr ? scales[gene] : 1.0f;
                    const float add = offsets != nullptr ? offsets[bake == 2 ? r : gene] : 0.0f;
                    const float value = fmaf(static_cast<float>(code), scale, add);
                    const std::uint32_t position = ((gene_major != 0 ? tile_offset_gene_major(rl, gl) : tile_offset(rl, gl)) >> 1) << 16;
                    if (half_scale != 0.0f) { // fp16(value * 2^k): 11 significant bits; the launch divides the result by 2^k again
                        const float scaled = value * half_scale;
                        const __half h = __float2half_rn(scaled);
                        word = static_cast<std::uint32_t>(__half_as_ushort(h)) | position;
                        if (entries_lo != nullptr) // the next eleven bits, for the split-product passes
                            entries_lo[place + static_cast<unsigned>(lane - start)] =
                                static_cast<std::uint32_t>(__half_as_ushort(__float2half_rn(scaled - __half2float(h)))) | position;
                    } else {
                        const __nv_bfloat16 v = __float2bfloat16_rn(value);
                        word = static_cast<std::uint32_t>(__bfloat16_as_ushort(v)) | position;
                        if (entries_lo != nullptr) // the next eight mantissa bits, for the split-product passes
                            entries_lo[place + static_cast<unsigned>(lane - start)] =
                                static_cast<std::uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(value - __bfloat162float(v)))) | position;
                    }
                } else {
                    word = code | (static_cast<std::uint32_t>(gl) << 8) | ((tile_offset(rl, gl) >> 1) << 15);
                }
                entries[place + static_cast<unsigned>(lane - start)] = word;
            }
        }
    }
}

// seg_ptr[i] = sum of counts[0..i) rounded up to multiples of 4 (16-byte segments for the copy engine), cursor =
// seg_ptr, in three steps over tiles of kScanTile segments: every block scans its tile and leaves the tile's total;
// one block scans the totals; every block adds its tile's base.  Consecutive threads take consecutive segments.
constexpr int kScanTile = 1024;
__device__ __forceinline__ long long block_exclusive_scan(long long mine, long long *total) {
    __shared__ long long warp_total[32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    long long sum = mine;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const long long up = __shfl_up_sync(0xffffffffu, sum, d);
        if (lane >= d) sum += up;
    }
    if (lane == 31) warp_total[warp] = sum;
    __syncthreads();
    if (warp == 0) {
        const long long t = warp_total[lane];
        long long run = t;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const long long up = __shfl_up_sync(0xffffffffu, run, d);
            if (lane >= d) run += up;
        }
        warp_total[lane] = run - t;
    }
    __syncthreads();
    const long long before = warp_total[warp] + sum - mine;
    if (total != nullptr && threadIdx.x == kScanTile - 1) *total = before + mine;
    __syncthreads(); // the shared array may be used again
    return before;
}
__global__ void __launch_bounds__(kScanTile) segment_tile_scan_kernel(const unsigned *counts, std::int64_t segments, std::int64_t *seg_ptr,
                                                                      long long *tile_totals) {
    const std::int64_t i = static_cast<std::int64_t>(blockIdx.x) * kScanTile + threadIdx.x;
    const long long mine = i < segments ? static_cast<long long>((counts[i] + 3u) & ~3u) : 0;
    const long long before = block_exclusive_scan(mine, tile_totals + blockIdx.x);
    if (i < segments) seg_ptr[i] = before;
}
__global__ void __launch_bounds__(kScanTile) tile_totals_scan_kernel(long long *tile_totals, std::int64_t tiles, std::int64_t *grand_total) {
    __shared__ long long carry, step_total;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    for (std::int64_t base = 0; base < tiles; base += kScanTile) {
        const std::int64_t t = base + threadIdx.x;
        const long long mine = t < tiles ? tile_totals[t] : 0;
        const long long before = block_exclusive_scan(mine, &step_total);
        if (t < tiles) tile_totals[t] = carry + before;
        __syncthreads();
        if (threadIdx.x == 0) carry += step_total;
        __syncthreads();
    }
    if (threadIdx.x == 0) *grand_total = carry;
}
__global__ void __launch_bounds__(kScanTile) segment_add_base_kernel(const long long *tile_bases, std::int64_t segments, std::int64_t *seg_ptr,
                                                                     unsigned long long *cursor) {
    const std::int64_t i = static_cast<std::int64_t>(blockIdx.x) * kScanTile + threadIdx.x;
    if (i >= segments) return;
    const long long at = seg_ptr[i] + tile_bases[blockIdx.x];
    seg_ptr[i] = at;
    cursor[i] = static_cast<unsigned long long>(at);
}

// ---------------------------------------------------------------------------------------------
// run time

struct blocked_params {
    const std::uint32_t *entries;
    const std::int64_t *seg_ptr;
    const float *row_offsets; // per cell row, row-offset policy only
    const unsigned char *records;
    float *y;
    std::int64_t y_ld;
    std::int64_t row_end;     // rows >= row_end are computed but not written
    std::int64_t group_begin, group_end;
    int windows;
    float alpha, beta;
    const float *bias;   // composed epilogue, applied by the last pass only
    int epilogue;
    int *status;
    int value_part; // 0: the tile holds hi = bf16(value); 1: lo = bf16(value - hi)
    std::uint32_t idesc;       // instruction descriptor: bf16 or fp16 operands
    float result_scale;        // 1 / (the power of two fp16 values were stored times); 1 for bf16 words
    const unsigned *w_absmax;  // fp16 operands: largest |W| of this launch as float bits (its factor is undone too); else null
    int poll_limit; // polls a bounded wait makes before it gives up (kPollLimit; less under the test hook)
    int withhold_w; // test hook: the W loader issues no copies, so the waits for W run out
};

// Test hook (cb200_test_arm_wait_timeout): read at launch time by the two-group kernel's launcher.
std::atomic<int> g_test_poll_limit{0}; // 0 = not armed

template<int NC, int CS, bool BAKED>
__global__ void __launch_bounds__(kThreads, 1) qcsr_fwd_blocked_kernel(const blocked_params p) {
    constexpr int REC = record_bytes(NC);
    constexpr int STAGES = w_stages(NC, CS);
    constexpr int kTmemCols = kSubBlocks * NC < 32 ? 32 : kSubBlocks * NC; // one accumulator per row sub-block
    const std::uint32_t IDESC = p.idesc;
    extern __shared__ __align__(1024) unsigned char smem[];
    // [2][A tile] | [STAGES][W record] | [CS][entry chunk] | row offsets | barriers | chunk meta | tmem | abort
    unsigned char *chunk_base = smem + 2 * kABufBytes + STAGES * REC;
    float *row_offset_s = reinterpret_cast<float *>(chunk_base + CS * kChunkBytes);
    std::uint64_t *bars = reinterpret_cast<std::uint64_t *>(row_offset_s + kRows);
    std::uint64_t *a_full = bars;                      // [2]            scatter warps -> MMA (one arrival per warp)
    std::uint64_t *a_empty = bars + 2;                 // [2]            MMA commit -> scatter warps
    std::uint64_t *w_full = bars + 4;                  // [STAGES]       copy engine -> MMA, scatter warps
    std::uint64_t *w_empty = w_full + STAGES;          // [STAGES]       MMA commit -> loader
    std::uint64_t *c_full = w_empty + STAGES;          // [CS] copy engine -> scatter warps
    std::uint64_t *c_empty = c_full + CS;    // [CS] scatter warps -> loader (one arrival per warp)
    std::uint64_t *acc_full = c_empty + CS;  // MMA commit -> scatter warps
    std::uint64_t *acc_empty = acc_full + 1;           // scatter warps -> MMA (one arrival per warp)
    volatile int *chunk_meta = reinterpret_cast<volatile int *>(acc_empty + 1); // [CS] (entries << 1) | last chunk of its window
    std::uint32_t *tmem_slot = reinterpret_cast<std::uint32_t *>(const_cast<int *>(chunk_meta) + CS + 1);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    unsigned char *scratch_slot = reinterpret_cast<unsigned char *>(tmem_slot + 2);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const std::uint32_t smem0 = smem_addr(smem);
    const std::uint32_t wstage0 = smem0 + 2 * kABufBytes;
    const std::uint32_t chunk0 = wstage0 + STAGES * REC;

    if (tid == 0) {
        for (int b = 0; b < 2; ++b) {
            bar_init(smem_addr(a_full + b), kProducerWarps);
            bar_init(smem_addr(a_empty + b), 1);
        }
        for (int s = 0; s < STAGES; ++s) {
            bar_init(smem_addr(w_full + s), 1);
            bar_init(smem_addr(w_empty + s), 1);
        }
        for (int s = 0; s < CS; ++s) {
            bar_init(smem_addr(c_full + s), 1);
            bar_init(smem_addr(c_empty + s), kProducerWarps);
        }
        bar_init(smem_addr(acc_full), 1);
        bar_init(smem_addr(acc_empty), kEpilogueWarps);
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

    // this CTA's row groups: group_begin + blockIdx.x, + gridDim.x, ...
    const std::int64_t first_group = p.group_begin + blockIdx.x;
    const std::int64_t my_groups = first_group < p.group_end ? (p.group_end - first_group + gridDim.x - 1) / gridDim.x : 0;

    if (warp < kProducerWarps) {
        // ================= zero, scatter, epilogue =================
        const int sub = tid >> 7;
        // fp16 operands were stored times powers of two: the result is divided by both again
        const float alpha = p.alpha * p.result_scale / (p.w_absmax != nullptr ? operand_scale(__uint_as_float(__ldg(p.w_absmax))) : 1.0f);
        const bool use_row_offset = p.row_offsets != nullptr;
        long long q = 0;  // windows done by this CTA
        long long qc = 0; // chunks done by this CTA
        for (std::int64_t gi = 0; gi < my_groups; ++gi) {
            const std::int64_t group = first_group + gi * gridDim.x;
            const std::int64_t row = group * kRows + tid;
            if (use_row_offset) {
                asm volatile("bar.sync 1, %0;" ::"n"(kProducerThreads) : "memory"); // the previous group's scatter is over
                if (tid < kRows) row_offset_s[tid] = row < p.row_end ? __ldg(p.row_offsets + row) : 0.0f;
                asm volatile("bar.sync 1, %0;" ::"n"(kProducerThreads) : "memory");
            }
            for (int w = 0; w < p.windows; ++w, ++q) {
                const std::uint32_t b = static_cast<std::uint32_t>(q & 1);
                const int s = static_cast<int>(q % STAGES);
                bar_wait(smem_addr(a_empty + b), static_cast<std::uint32_t>(((q >> 1) & 1) ^ 1), abort_flag);
                unsigned char *tile = smem + b * kABufBytes;
#pragma unroll
                for (int k = 0; k < kABufBytes / (kProducerThreads * 8); ++k) // 8-byte stores: see the two-group kernel
                    *reinterpret_cast<uint2 *>(tile + k * (kProducerThreads * 8) + tid * 8) = make_uint2(0u, 0u);
                asm volatile("bar.sync 1, %0;" ::"n"(kProducerThreads) : "memory"); // the whole tile is zero before anyone scatters
                // the W stage carries the decode table; baked entries do not need it, only the MMA waits for W
                if constexpr (!BAKED) bar_wait(smem_addr(w_full + s), static_cast<std::uint32_t>((q / STAGES) & 1), abort_flag);
                const float2 *table = reinterpret_cast<const float2 *>(smem + 2 * kABufBytes + s * REC + NC * kWin * 2);
                bool last = false;
                int guard = 0;
                while (!last && ++guard < (1 << 20)) {
                    const int cs = static_cast<int>(qc % CS);
                    bar_wait(smem_addr(c_full + cs), static_cast<std::uint32_t>((qc / CS) & 1), abort_flag);
                    const int meta = chunk_meta[cs];
                    const int count = *abort_flag != 0 ? 0 : (meta >> 1);
                    last = (meta & 1) != 0 || *abort_flag != 0;
                    const uint4 *chunk = reinterpret_cast<const uint4 *>(chunk_base + cs * kChunkBytes);
                    for (int i = tid * 4; i < count; i += kProducerThreads * 4) { // segments are padded to multiples of 4
                        const uint4 e4 = chunk[i >> 2];
                        const std::uint32_t e[4] = {e4.x, e4.y, e4.z, e4.w};
                        if constexpr (BAKED) {
                            // decoded at prepare time: the word is {bf16 value, byte position / 2}
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                unsigned char *dst = static_cast<int>(e[k]) >= 0 ? tile + (((e[k] >> 16) & 0x7fffu) << 1) : scratch_slot;
                                *reinterpret_cast<unsigned short *>(dst) = static_cast<unsigned short>(e[k] & 0xffffu);
                            }
                            continue;
                        }
                        float2 t[4];
#pragma unroll
                        for (int k = 0; k < 4; ++k) t[k] = table[(e[k] >> 8) & (kWin - 1)];
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const std::uint32_t off = ((e[k] >> 15) & 0x7fffu) << 1;
                            float add = t[k].y;
                            if (use_row_offset) // row within the group, back from the byte position in the tile
                                add = row_offset_s[((off / kSubBlockBytes) << 7) | (((off >> 10) & 15u) << 3) | ((off >> 7) & 7u)];
                            const float value = fmaf(static_cast<float>(e[k] & 0xffu), t[k].x, add);
                            // padding words (top bit set) are stored to a scratch slot instead of branching
                            unsigned char *dst = static_cast<int>(e[k]) >= 0 ? tile + off : scratch_slot;
                            __nv_bfloat16 bv = __float2bfloat16_rn(value);
                            if (p.value_part != 0) bv = __float2bfloat16_rn(value - __bfloat162float(bv)); // the next 8 mantissa bits
                            *reinterpret_cast<__nv_bfloat16 *>(dst) = bv;
                        }
                    }
                    __syncwarp();
                    if (lane == 0) bar_arrive(smem_addr(c_empty + cs));
                    ++qc;
                }
                fence_async_proxy(); // the tile was written with ordinary stores, the MMA reads it through the async proxy
                __syncwarp();
                if (lane == 0) bar_arrive(smem_addr(a_full + b));
            }

            // ---- thread t < 256 writes row t of the group: TMEM lane = row within the sub-block
            if (warp >= kEpilogueWarps) continue;
            bar_wait(smem_addr(acc_full), static_cast<std::uint32_t>(gi & 1), abort_flag);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int h = 0; h < NC / 32; ++h) {
                float v[32];
                tmem_ld32(tmem_base + (static_cast<std::uint32_t>((warp & 3) * 32) << 16) + sub * NC + h * 32, v);
                if (row < p.row_end) {
                    float *out = p.y + row * p.y_ld + h * 32;
                    store_row32(out, v, alpha, p.beta, p.bias, h * 32, p.epilogue);
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) bar_arrive(smem_addr(acc_empty));
        }
    } else if (warp == kProducerWarps) {
        // ================= MMA issuer =================
        long long q = 0;
        for (std::int64_t g = 0; g < my_groups; ++g) {
            bar_wait(smem_addr(acc_empty), static_cast<std::uint32_t>((g & 1) ^ 1), abort_flag);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            for (int w = 0; w < p.windows; ++w, ++q) {
                const std::uint32_t b = static_cast<std::uint32_t>(q & 1);
                const int s = static_cast<int>(q % STAGES);
                bar_wait(smem_addr(w_full + s), static_cast<std::uint32_t>((q / STAGES) & 1), abort_flag);
                bar_wait(smem_addr(a_full + b), static_cast<std::uint32_t>((q >> 1) & 1), abort_flag);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (lane == 0) {
                    const std::uint32_t a_tile = smem0 + b * kABufBytes;
                    const std::uint32_t b_tile = wstage0 + s * REC;
#pragma unroll
                    for (int kk = 0; kk < kWin / 16; ++kk) {
                        const std::uint64_t db = smem_desc(b_tile + kk * 256);
#pragma unroll
                        for (int sb = 0; sb < kSubBlocks; ++sb)
                            mma_bf16(tmem_base + sb * NC,
                                     smem_desc_sw128(a_tile + sb * kSubBlockBytes + (kk >> 2) * kHalfBytes + (kk & 3) * 32), db, IDESC,
                                     w > 0 || kk > 0);
                    }
                    mma_commit(smem_addr(a_empty + b));
                    mma_commit(smem_addr(w_empty + s));
                    if (w == p.windows - 1) mma_commit(smem_addr(acc_full));
                }
                __syncwarp();
            }
        }
    } else {
        // ================= loaders =================
        // Issuing a bulk copy costs its thread several hundred cycles (barrier wait, expect-tx, the
        // copy itself), so the copies of a window are spread over threads: one warp's elected lane
        // feeds the W ring, kChunkLoaders warps take the entry chunks in turn (chunk number modulo
        // kChunkLoaders); each of them walks all segments and issues only its own chunks.
        const int role = warp - kProducerWarps - 1; // 0: W slices, 1..kChunkLoaders: entry chunks
        if (role == 0) {
            if (lane == 0) {
                const long long total = my_groups * p.windows;
                for (long long q = 0; q < total; ++q) {
                    const int s = static_cast<int>(q % STAGES);
                    bar_wait(smem_addr(w_empty + s), static_cast<std::uint32_t>(((q / STAGES) & 1) ^ 1), abort_flag);
                    bar_arrive_expect_tx(smem_addr(w_full + s), REC);
                    bulk_copy_g2s(wstage0 + s * REC, p.records + static_cast<std::size_t>(q % p.windows) * REC, REC,
                                  smem_addr(w_full + s));
                }
            }
        } else {
            const int mine_mod = role - 1;
            long long qc = 0;
            for (std::int64_t gi = 0; gi < my_groups; ++gi) {
                const std::int64_t seg0 = (first_group + gi * gridDim.x) * p.windows;
                for (int wbase = 0; wbase < p.windows; wbase += 31) {
                    // segment bounds of up to 31 windows in one coalesced read
                    const int span = min(31, p.windows - wbase);
                    const std::int64_t bound = lane <= span ? __ldg(p.seg_ptr + seg0 + wbase + lane) : 0;
                    for (int j = 0; j < span; ++j) {
                        const std::int64_t lo = __shfl_sync(0xffffffffu, bound, j), hi = __shfl_sync(0xffffffffu, bound, j + 1);
                        std::int64_t at = lo;
                        do {
                            const int count = static_cast<int>(min(static_cast<std::int64_t>(kChunkEntries), hi - at));
                            if (lane == 0 && qc % kChunkLoaders == mine_mod) {
                                const int cs = static_cast<int>(qc % CS);
                                bar_wait(smem_addr(c_empty + cs), static_cast<std::uint32_t>(((qc / CS) & 1) ^ 1), abort_flag);
                                chunk_meta[cs] = (count << 1) | (at + count >= hi ? 1 : 0);
                                if (count > 0) {
                                    bar_arrive_expect_tx(smem_addr(c_full + cs), static_cast<std::uint32_t>(count) * 4u);
                                    bulk_copy_g2s(chunk0 + cs * kChunkBytes, p.entries + at, static_cast<std::uint32_t>(count) * 4u,
                                                  smem_addr(c_full + cs));
                                } else {
                                    bar_arrive(smem_addr(c_full + cs)); // an empty window still hands over one (empty) chunk
                                }
                            }
                            at += count;
                            ++qc;
                        } while (at < hi);
                    }
                }
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

template<int NC, int CS> constexpr std::size_t blocked_smem_bytes() {
    return 2 * kABufBytes + w_stages(NC, CS) * record_bytes(NC) + CS * kChunkBytes + kRows * 4 +
           (6 + 2 * w_stages(NC, CS) + 2 * CS) * sizeof(std::uint64_t) + (CS + 1) * 4 + 16;
}

template<int NC, int CS, bool BAKED>
cb200_status launch_cs(const blocked_params &p, int sm_count, cudaStream_t stream) {
    constexpr std::size_t smem = blocked_smem_bytes<NC, CS>();
    static_assert(smem <= 232448, "shared memory budget");
    static_assert(CS % kChunkLoaders == 0, "a loader always refills the same stages");
    CB200_CUDA_OK(cudaFuncSetAttribute(qcsr_fwd_blocked_kernel<NC, CS, BAKED>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(smem)));
    const std::int64_t groups = p.group_end - p.group_begin;
    const unsigned grid = static_cast<unsigned>(groups < sm_count ? groups : sm_count);
    qcsr_fwd_blocked_kernel<NC, CS, BAKED><<<grid, kThreads, smem, stream>>>(p);
    count_launch();
    CB200_CUDA_OK(cudaGetLastError());
    return CB200_STATUS_SUCCESS;
}

// Two chunk stages when a segment normally fits one 8 KB chunk (measured best on the 5 %-dense
// 33,538-gene matrix), three when segments span several chunks (the 17 %-dense 4,000-gene one).
template<int NC>
cb200_status launch_one(const blocked_params &p, bool long_segments, bool baked, int sm_count, cudaStream_t stream) {
    if (baked) return long_segments ? launch_cs<NC, 3, true>(p, sm_count, stream) : launch_cs<NC, 2, true>(p, sm_count, stream);
    return long_segments ? launch_cs<NC, 3, false>(p, sm_count, stream) : launch_cs<NC, 2, false>(p, sm_count, stream);
}

// ---------------------------------------------------------------------------------------------
// The same window kernel for baked entry words, with the scatter warps in two groups of eight that
// take alternate windows (group g owns tile buffer g and its own ring of entry chunks).  A window's
// chain -- wait for the tile, zero it, barrier, wait for the chunk, scatter, proxy fence, hand over --
// is mostly latency; with two groups the chains of consecutive windows overlap instead of following
// each other.  Measured on the 1M x 33,538 matrix (ms per launch): one group 6.86; two groups with
// (chunk entries, stages per group) (2048, 2) 6.30, (2048, 1) 6.44, (1024, 2) 6.55, (1024, 3) 6.57,
// (512, 4) 7.98; (2048, 2) with three instead of four W stages 6.45.  A matrix whose segments span
// several chunks (the 17 %-dense 4,000-gene one) is slower this way (1.30 against 1.06 ms) and keeps
// the one-group kernel.
constexpr int kGroupWarps = kProducerWarps / 2;
constexpr int kGroupThreads = kGroupWarps * 32;
constexpr int kChunk2Entries = 2048;
constexpr int kChunk2Bytes = kChunk2Entries * 4;
constexpr int kRing2 = 2; // chunk stages per scatter group
constexpr int kThreads2 = kProducerThreads + 32 * (kSubBlocks + 2); // + an MMA warp per sub-block + W loader warp + chunk loader warp
__host__ __device__ constexpr int w2_stages(int n) {
    return (232448 - 2 * kABufBytes - 2 * kRing2 * kChunk2Bytes - 1024) / (n * kWin * 2) >= kMaxWStages
               ? kMaxWStages
               : (232448 - 2 * kABufBytes - 2 * kRing2 * kChunk2Bytes - 1024) / (n * kWin * 2);
}

// TEST_HOOK: the instantiation cb200_test_arm_wait_timeout selects.  It differs in two places only: the poll limit
// of the waits comes from the launch (a few thousand instead of 2^22) and the W loader issues no copies, so
// that the waits for W run out.  Everything that happens after a wait has run out is common code.
template<int NC, bool TEST_HOOK>
__global__ void __launch_bounds__(kThreads2, 1) qcsr_fwd_blocked2_kernel(const blocked_params p) {
    constexpr int REC = record_bytes(NC);   // distance of the W records in global memory
    constexpr int WREC = NC * kWin * 2;     // the W part of a record (the decode table is not needed)
    constexpr int STAGES = w2_stages(NC);
    constexpr int CHUNKS = 2 * kRing2;
    // Who releases a window's W stage.  With more W stages than tile buffers the scatter group that sees the window's
    // tile released, one round later, passes that on (the MMA warps commit to one barrier per window).  With only as many
    // stages as buffers (N = 128) that would be a cycle -- the group waits for its next window's W, whose copy waits for
    // the release the group has not passed on yet -- so there the MMA warps commit to the stage's barrier themselves.
    constexpr bool FORWARD_W_RELEASE = STAGES > 2;
    constexpr int kTmemCols = kSubBlocks * NC < 32 ? 32 : kSubBlocks * NC;
    const std::uint32_t IDESC = p.idesc;
    extern __shared__ __align__(1024) unsigned char smem[];
    // [2][A tile] | [STAGES][W window] | [2][kRing2][entry chunk] | barriers | chunk meta | tmem | abort | scratch
    unsigned char *chunk_base = smem + 2 * kABufBytes + STAGES * WREC;
    std::uint64_t *bars = reinterpret_cast<std::uint64_t *>(chunk_base + CHUNKS * kChunk2Bytes);
    std::uint64_t *a_full = bars;                 // [2]      scatter group -> MMA (one arrival per warp of the group)
    std::uint64_t *a_empty = bars + 2;            // [2]      MMA commit -> scatter group
    std::uint64_t *w_full = bars + 4;             // [STAGES] copy engine -> MMA
    std::uint64_t *w_empty = w_full + STAGES;     // [STAGES] MMA commit -> W loader
    std::uint64_t *c_full = w_empty + STAGES;     // [CHUNKS] copy engine -> scatter group
    std::uint64_t *c_empty = c_full + CHUNKS;     // [CHUNKS] scatter group -> chunk loader (one arrival per warp)
    std::uint64_t *acc_full = c_empty + CHUNKS;   // MMA commit -> epilogue warps
    std::uint64_t *acc_empty = acc_full + 1;      // epilogue warps -> MMA
    std::uint64_t *mma_drain = acc_empty + 1;     // [2] MMA commit -> the MMA warp itself, used once, after an abort
    volatile int *chunk_meta = reinterpret_cast<volatile int *>(mma_drain + 2); // [CHUNKS] (entries << 1) | last chunk of its window
    std::uint32_t *tmem_slot = reinterpret_cast<std::uint32_t *>(const_cast<int *>(chunk_meta) + CHUNKS);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    unsigned char *scratch_slot = reinterpret_cast<unsigned char *>(tmem_slot + 2);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int limit = TEST_HOOK ? p.poll_limit : kPollLimit;
    const std::uint32_t smem0 = smem_addr(smem);
    const std::uint32_t wstage0 = smem0 + 2 * kABufBytes;
    const std::uint32_t chunk0 = wstage0 + STAGES * WREC;

    if (tid == 0) {
        for (int b = 0; b < 2; ++b) {
            bar_init(smem_addr(a_full + b), kGroupWarps);
            bar_init(smem_addr(a_empty + b), kSubBlocks); // one commit per MMA warp
        }
        for (int s = 0; s < STAGES; ++s) {
            bar_init(smem_addr(w_full + s), 1);
            bar_init(smem_addr(w_empty + s), FORWARD_W_RELEASE ? 1 : kSubBlocks);
        }
        for (int s = 0; s < CHUNKS; ++s) {
            bar_init(smem_addr(c_full + s), 1);
            bar_init(smem_addr(c_empty + s), kGroupWarps);
        }
        bar_init(smem_addr(acc_full), kSubBlocks);
        bar_init(smem_addr(acc_empty), kEpilogueWarps);
        bar_init(smem_addr(mma_drain), 1);
        bar_init(smem_addr(mma_drain + 1), 1);
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

    if (warp < kProducerWarps) {
        // ================= two scatter groups; group 0 also writes Y =================
        const int grp = warp / kGroupWarps, gtid = tid - grp * kGroupThreads;
        const int sub = tid >> 7;
        // fp16 operands were stored times powers of two: the result is divided by both again
        const float alpha = p.alpha * p.result_scale / (p.w_absmax != nullptr ? operand_scale(__uint_as_float(__ldg(p.w_absmax))) : 1.0f);
        unsigned char *tile = smem + grp * kABufBytes;
        long long q = 0;  // windows of this CTA, both groups count all of them
        long long qc = 0; // chunks this group has consumed
        for (std::int64_t gi = 0; gi < my_groups; ++gi) {
            const std::int64_t row = (first_group + gi * gridDim.x) * kRows + tid;
            for (int w = 0; w < p.windows; ++w, ++q) {
                if (static_cast<int>(q & 1) != grp) continue;
                // The window's first chunk (all of it for all but the densest matrices) goes into registers while the tile
                // is still being read by the previous window's MMAs: between the tile's release and its hand-over there
                // are then only stores.
                bool last;
                uint4 held[kChunk2Entries / (kGroupThreads * 4)];
                {
                    const int cs = grp * kRing2 + static_cast<int>(qc % kRing2);
                    bar_wait(smem_addr(c_full + cs), static_cast<std::uint32_t>((qc / kRing2) & 1), abort_flag, limit);
                    const int meta = chunk_meta[cs];
                    const int count = *abort_flag != 0 ? 0 : (meta >> 1);
                    last = (meta & 1) != 0 || *abort_flag != 0;
                    const uint4 *chunk = reinterpret_cast<const uint4 *>(chunk_base + cs * kChunk2Bytes);
#pragma unroll
                    for (int k = 0; k < kChunk2Entries / (kGroupThreads * 4); ++k) { // segments are padded to multiples of 4
                        const int i = (k * kGroupThreads + gtid) * 4;
                        held[k] = i < count ? chunk[i >> 2] : make_uint4(kInvalidEntry, kInvalidEntry, kInvalidEntry, kInvalidEntry);
                    }
                    // the words are used much later, but they must be in the registers before the stage goes back to the copy engine
                    {
                        std::uint32_t all = 0;
#pragma unroll
                        for (int k = 0; k < kChunk2Entries / (kGroupThreads * 4); ++k) all |= held[k].x | held[k].y | held[k].z | held[k].w;
                        arrive_when_loaded(smem_addr(c_empty + cs), all, lane, static_cast<std::uint32_t>(p.windows) >> 31);
                    }
                    ++qc;
                }
                // The hand-over of the tile also vouches for the window's W stage: one warp of the group waits for it here,
                // where the group has slack, and the MMA warps then wait for a single barrier per window.
                if (gtid < 32) bar_wait(smem_addr(w_full + static_cast<int>(q % STAGES)), static_cast<std::uint32_t>((q / STAGES) & 1), abort_flag, limit);
                bar_wait(smem_addr(a_empty + grp), static_cast<std::uint32_t>(((q >> 1) & 1) ^ 1), abort_flag, limit);
                // the MMAs of the group's previous window are done with the tile, hence with that window's W stage too: the
                // MMA warps commit to the tile's barrier only, and the release of the W stage is passed on from here
                if (FORWARD_W_RELEASE && gtid == 0 && q >= 2) bar_arrive(smem_addr(w_empty + static_cast<int>((q - 2) % STAGES)));
#pragma unroll
                for (int k = 0; k < kABufBytes / (kGroupThreads * 8); ++k) // 8-byte stores: a warp's 16-byte store costs 7 wavefronts of
                    *reinterpret_cast<uint2 *>(tile + k * (kGroupThreads * 8) + gtid * 8) = make_uint2(0u, 0u); // the LSU data pipe for 512 bytes, two 8-byte stores 4 (4.79 -> 4.60 ms)
                // the whole tile is zero before anyone of the group scatters (named barrier 1 or 2)
                if (grp == 0) asm volatile("bar.sync 1, %0;" ::"n"(kGroupThreads) : "memory");
                else asm volatile("bar.sync 2, %0;" ::"n"(kGroupThreads) : "memory");
#pragma unroll
                for (int k = 0; k < kChunk2Entries / (kGroupThreads * 4); ++k) {
                    const std::uint32_t e[4] = {held[k].x, held[k].y, held[k].z, held[k].w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) // padding words (top bit set) are not stored
                        if (static_cast<int>(e[j]) >= 0)
                            *reinterpret_cast<unsigned short *>(tile + (((e[j] >> 16) & 0x7fffu) << 1)) = static_cast<unsigned short>(e[j] & 0xffffu);
                }
                int guard = 0;
                while (!last && ++guard < (1 << 20)) { // further chunks of a long segment: scattered from shared memory
                    const int cs = grp * kRing2 + static_cast<int>(qc % kRing2);
                    bar_wait(smem_addr(c_full + cs), static_cast<std::uint32_t>((qc / kRing2) & 1), abort_flag, limit);
                    const int meta = chunk_meta[cs];
                    const int count = *abort_flag != 0 ? 0 : (meta >> 1);
                    last = (meta & 1) != 0 || *abort_flag != 0;
                    const uint4 *chunk = reinterpret_cast<const uint4 *>(chunk_base + cs * kChunk2Bytes);
                    for (int i = gtid * 4; i < count; i += kGroupThreads * 4) {
                        const uint4 e4 = chunk[i >> 2];
                        const std::uint32_t e[4] = {e4.x, e4.y, e4.z, e4.w};
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            unsigned char *dst = static_cast<int>(e[k]) >= 0 ? tile + (((e[k] >> 16) & 0x7fffu) << 1) : scratch_slot;
                            *reinterpret_cast<unsigned short *>(dst) = static_cast<unsigned short>(e[k] & 0xffffu);
                        }
                    }
                    __syncwarp();
                    if (lane == 0) bar_arrive(smem_addr(c_empty + cs));
                    ++qc;
                }
                fence_async_proxy(); // the tile was written with ordinary stores, the MMA reads it through the async proxy
                __syncwarp();
                if (lane == 0) bar_arrive(smem_addr(a_full + grp));
            }

            // ---- thread t < 256 (group 0) writes row t of the row group: TMEM lane = row within the sub-block
            if (grp != 0) continue;
            bar_wait(smem_addr(acc_full), static_cast<std::uint32_t>(gi & 1), abort_flag, limit);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int h = 0; h < NC / 32; ++h) {
                float v[32];
                tmem_ld32(tmem_base + (static_cast<std::uint32_t>((warp & 3) * 32) << 16) + sub * NC + h * 32, v);
                if (row < p.row_end) {
                    float *out = p.y + row * p.y_ld + h * 32;
                    store_row32(out, v, alpha, p.beta, p.bias, h * 32, p.epilogue);
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) bar_arrive(smem_addr(acc_empty));
        }
    } else if (warp < kProducerWarps + kSubBlocks) {
        // ================= MMA issuers: one warp per 128-row sub-block of the tile =================
        // One issuing thread is held to the rate at which the MMAs read their operands (the issue of a window's sixteen
        // MMAs takes about as long as their execution) and then spends half as long again on commits, waits and
        // loop overhead while the tensor pipe runs dry.  Each sub-block has its own accumulator columns, so two threads can
        // issue a window's MMAs side by side: each issues eight, and both commit to the tile's and the W stage's barriers.
        // The issue path is kept as short as it can be: a vote and a branch per window to stop early after a wait
        // has run out cost 0.7 ms of 6.3 on the 1M x 33,538 matrix.  After an abort the remaining windows are
        // therefore still issued (on stale tiles, into this CTA's own TMEM; the waits return at once) and only
        // the end of the role looks at the flag.
        const int sb = warp - kProducerWarps;
        long long q = 0;
        for (std::int64_t g = 0; g < my_groups; ++g) {
            bar_wait(smem_addr(acc_empty), static_cast<std::uint32_t>((g & 1) ^ 1), abort_flag, limit);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            for (int w = 0; w < p.windows; ++w, ++q) {
                const std::uint32_t b = static_cast<std::uint32_t>(q & 1);
                const int s = static_cast<int>(q % STAGES);
                bar_wait(smem_addr(a_full + b), static_cast<std::uint32_t>((q >> 1) & 1), abort_flag, limit); // tile and W stage
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (lane == 0) {
                    const std::uint32_t a_tile = smem0 + b * kABufBytes + sb * kSubBlockBytes;
                    const std::uint32_t b_tile = wstage0 + s * WREC;
#pragma unroll
                    for (int kk = 0; kk < kWin / 16; ++kk)
                        mma_bf16(tmem_base + sb * NC, smem_desc_sw128(a_tile + (kk >> 2) * kHalfBytes + (kk & 3) * 32), smem_desc(b_tile + kk * 256),
                                 IDESC, w > 0 || kk > 0);
                    mma_commit(smem_addr(a_empty + b));
                    if constexpr (!FORWARD_W_RELEASE) mma_commit(smem_addr(w_empty + s));
                    if (w == p.windows - 1) mma_commit(smem_addr(acc_full));
                }
                __syncwarp();
            }
        }
        // after an abort: the MMAs already issued finish before the CTA frees its TMEM and shared memory
        if (lane == 0 && *abort_flag != 0) {
            mma_commit(smem_addr(mma_drain + sb));
            bar_wait_drain(smem_addr(mma_drain + sb), 0u, limit);
        }
        __syncwarp();
    } else if (warp == kProducerWarps + kSubBlocks) {
        // ================= W loader =================
        if (lane == 0 && !(TEST_HOOK && p.withhold_w != 0)) {
            const long long total = my_groups * p.windows;
            long long q = 0;
            for (; q < total; ++q) {
                const int s = static_cast<int>(q % STAGES);
                // no new copies once a wait of the CTA has run out
                if (bar_wait(smem_addr(w_empty + s), static_cast<std::uint32_t>(((q / STAGES) & 1) ^ 1), abort_flag, limit)) break;
                bar_arrive_expect_tx(smem_addr(w_full + s), WREC);
                bulk_copy_g2s(wstage0 + s * WREC, p.records + static_cast<std::size_t>(q % p.windows) * REC, WREC, smem_addr(w_full + s));
            }
            // after an abort: let the copies still in flight land (the last one issued into each stage)
            if (q < total)
                for (long long last = q - 1; last >= 0 && last > q - 1 - STAGES; --last)
                    bar_wait_drain(smem_addr(w_full + static_cast<int>(last % STAGES)), static_cast<std::uint32_t>((last / STAGES) & 1), limit);
        }
    } else if (warp == kProducerWarps + kSubBlocks + 1) {
        // ================= entry chunks: window q goes to the ring of scatter group q & 1 =================
        long long q = 0;
        long long qc0 = 0, qc1 = 0; // chunks issued into each ring
        bool dead = false; // lane 0: a wait was given up, no copy is issued any more (the loops run out empty)
        for (std::int64_t gi = 0; gi < my_groups; ++gi) {
            const std::int64_t seg0 = (first_group + gi * gridDim.x) * p.windows;
            for (int wbase = 0; wbase < p.windows; wbase += 31) {
                const int span = min(31, p.windows - wbase); // segment bounds of up to 31 windows in one coalesced read
                const std::int64_t bound = lane <= span ? __ldg(p.seg_ptr + seg0 + wbase + lane) : 0;
                for (int j = 0; j < span; ++j, ++q) {
                    const std::int64_t lo = __shfl_sync(0xffffffffu, bound, j), hi = __shfl_sync(0xffffffffu, bound, j + 1);
                    const int ring = static_cast<int>(q & 1);
                    std::int64_t at = lo;
                    do {
                        const int count = static_cast<int>(min(static_cast<std::int64_t>(kChunk2Entries), hi - at));
                        const long long mine = ring == 0 ? qc0 : qc1;
                        if (lane == 0 && !dead) {
                            const int cs = ring * kRing2 + static_cast<int>(mine % kRing2);
                            dead = bar_wait(smem_addr(c_empty + cs), static_cast<std::uint32_t>(((mine / kRing2) & 1) ^ 1), abort_flag, limit);
                        }
                        if (lane == 0 && !dead) {
                            const int cs = ring * kRing2 + static_cast<int>(mine % kRing2);
                            chunk_meta[cs] = (count << 1) | (at + count >= hi ? 1 : 0);
                            if (count > 0) {
                                bar_arrive_expect_tx(smem_addr(c_full + cs), static_cast<std::uint32_t>(count) * 4u);
                                bulk_copy_g2s(chunk0 + cs * kChunk2Bytes, p.entries + at, static_cast<std::uint32_t>(count) * 4u,
                                              smem_addr(c_full + cs));
                            } else {
                                bar_arrive(smem_addr(c_full + cs)); // an empty window still hands over one (empty) chunk
                            }
                        }
                        at += count;
                        if (!dead) { // lane 0's counters stop with its last issued chunk (the drain below needs them)
                            if (ring == 0) ++qc0;
                            else ++qc1;
                        }
                    } while (at < hi);
                }
            }
        }
        // after an abort: let the chunk copies still in flight land (the last one issued into each stage of both rings)
        if (dead && lane == 0) {
            for (int ring = 0; ring < 2; ++ring) {
                const long long issued = ring == 0 ? qc0 : qc1;
                for (long long last = issued - 1; last >= 0 && last > issued - 1 - kRing2; --last)
                    bar_wait_drain(smem_addr(c_full + ring * kRing2 + static_cast<int>(last % kRing2)),
                                   static_cast<std::uint32_t>((last / kRing2) & 1), limit);
            }
        }
        __syncwarp();
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
    if (tid == 0 && *abort_flag != 0 && p.status != nullptr) atomicExch(p.status, 1);
}

template<int NC, bool TEST_HOOK>
cb200_status launch_blocked2_as(const blocked_params &p, int sm_count, cudaStream_t stream) {
    constexpr std::size_t smem = 2 * kABufBytes + w2_stages(NC) * NC * kWin * 2 + 2 * kRing2 * kChunk2Bytes +
                                 (8 + 2 * w2_stages(NC) + 4 * kRing2) * sizeof(std::uint64_t) + 2 * kRing2 * 4 + 24;
    static_assert(smem <= 232448, "shared memory budget");
    CB200_CUDA_OK(cudaFuncSetAttribute(qcsr_fwd_blocked2_kernel<NC, TEST_HOOK>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    const std::int64_t groups = p.group_end - p.group_begin;
    const unsigned grid = static_cast<unsigned>(groups < sm_count ? groups : sm_count);
    qcsr_fwd_blocked2_kernel<NC, TEST_HOOK><<<grid, kThreads2, smem, stream>>>(p);
    count_launch();
    CB200_CUDA_OK(cudaGetLastError());
    return CB200_STATUS_SUCCESS;
}
template<int NC>
cb200_status launch_blocked2(const blocked_params &p, int sm_count, cudaStream_t stream) {
    return p.withhold_w != 0 ? launch_blocked2_as<NC, true>(p, sm_count, stream) : launch_blocked2_as<NC, false>(p, sm_count, stream);
}
} // namespace

std::uint64_t qcsr_blocked_workspace_bytes(std::int64_t cols, std::int64_t n) {
    const std::int64_t windows = (cols + kWin - 1) / kWin;
    return static_cast<std::uint64_t>(256 + windows * record_bytes(static_cast<int>(n)));
}

bool qcsr_blocked_shape_ok(std::int64_t rows, std::int64_t cols, std::int64_t n, int bits, int dense_dtype) {
    if (bits != 8 && bits != 4) return false;
    if (n != 32 && n != 64 && n != 128) return false;
    if (dense_dtype != CB200_DTYPE_BF16 && dense_dtype != CB200_DTYPE_F32) return false; // fp32 W: split products only
    if (rows <= 0 || cols <= 0 || cols > 0x7fffffff - kWin) return false;
    const std::int64_t groups = (rows + kRows - 1) / kRows, windows = (cols + kWin - 1) / kWin;
    return groups * windows < (static_cast<std::int64_t>(1) << 31);
}

std::uint64_t qcsr_blocked_layout_bytes_bound(std::int64_t rows, std::int64_t cols, std::int64_t nnz, bool bake_lo) {
    const std::uint64_t groups = static_cast<std::uint64_t>((rows + kRows - 1) / kRows);
    const std::uint64_t segments = groups * static_cast<std::uint64_t>((cols + kWin - 1) / kWin);
    // a segment is padded to a multiple of four words: at most three more per segment
    const std::uint64_t words = static_cast<std::uint64_t>(nnz) + 3u * segments;
    return device_arena::rounded((segments + 2u) * sizeof(unsigned)) + device_arena::rounded(segments * sizeof(unsigned long long)) +
           device_arena::rounded((segments / 1024u + 2u) * sizeof(long long)) +
           device_arena::rounded((segments + 1u) * sizeof(std::int64_t)) + (bake_lo ? 2u : 1u) * device_arena::rounded(words * 4u);
}

// Builds the window-blocked copy of `x` on the current device: memory from `arena`, kernels on `stream`,
// which is waited for (the size of the copy is read back before its arrays are taken).
cb200_status build_blocked_layout(const qcsr_view &x, bool bake, bool bake_lo, bool gene_major, device_arena &arena,
                                  cudaStream_t stream, blocked_layout *out) {
    *out = blocked_layout{};
    if (x.row_ptr == nullptr || (x.nnz != 0 && (x.col_idx == nullptr || x.packed == nullptr)))
        return fail(CB200_STATUS_INVALID_ARGUMENT, "the matrix handed to prepare has null arrays");
    if (x.bits == 4 && x.packed_row_ptr == nullptr) return fail(CB200_STATUS_INVALID_ARGUMENT, "4-bit codes need packed_row_ptr");
    const std::int64_t groups = (x.rows + kRows - 1) / kRows;
    const int windows = static_cast<int>((x.cols + kWin - 1) / kWin);
    const std::int64_t segments = groups * windows;
    const int bake_mode = !bake ? 0 : (x.policy == CB200_DECODE_COLUMN_SCALE_ROW_OFFSET ? 2 : 1);
    const bool half_values = bake && !gene_major; // forward operations bake fp16 values; the transpose keeps bf16
    // two words behind the segment counters for the bound of the decoded magnitudes
    const std::uint64_t count_bytes = static_cast<std::uint64_t>(segments + 2) * sizeof(unsigned);
    const std::uint64_t cursor_bytes = static_cast<std::uint64_t>(segments) * sizeof(unsigned long long);
    const std::uint64_t seg_bytes = static_cast<std::uint64_t>(segments + 1) * sizeof(std::int64_t);
    const std::uint64_t tile_total_bytes = static_cast<std::uint64_t>((segments + kScanTile - 1) / kScanTile + 1) * sizeof(long long);
    unsigned *counts = static_cast<unsigned *>(arena.take(count_bytes));
    unsigned long long *cursor = static_cast<unsigned long long *>(arena.take(cursor_bytes));
    long long *tile_totals = static_cast<long long *>(arena.take(tile_total_bytes));
    out->seg_ptr = static_cast<std::int64_t *>(arena.take(seg_bytes));
    std::uint64_t word_bytes = 0;
    const auto give_up = [&](cb200_status st) {
        arena.give_back(out->entries_lo, word_bytes);
        arena.give_back(out->entries, word_bytes);
        arena.give_back(out->seg_ptr, seg_bytes);
        arena.give_back(tile_totals, tile_total_bytes);
        arena.give_back(cursor, cursor_bytes);
        arena.give_back(counts, count_bytes);
        *out = blocked_layout{};
        return st;
    };
    if (counts == nullptr || cursor == nullptr || tile_totals == nullptr || out->seg_ptr == nullptr)
        return give_up(fail(CB200_STATUS_INSUFFICIENT_WORKSPACE, "no device memory for the segment table of the window-blocked copy"));
    cudaError_t err = cudaMemsetAsync(counts, 0, count_bytes, stream);
    const unsigned grid = static_cast<unsigned>((x.rows + 7) / 8); // one warp per row, 8 rows per block
    std::int64_t total = 0;
    unsigned bound_bits[2] = {0u, 0u};
    if (err == cudaSuccess && half_values) {
        const bool row_policy = x.policy == CB200_DECODE_COLUMN_SCALE_ROW_OFFSET;
        const std::int64_t span = std::max<std::int64_t>(x.cols, row_policy ? x.rows : 0);
        value_bound_kernel<<<static_cast<unsigned>((span + 255) / 256), 256, 0, stream>>>(
            x.scales, row_policy ? nullptr : x.offsets, x.cols, row_policy ? x.offsets : nullptr, x.rows,
            static_cast<float>((1 << x.bits) - 1), counts + segments);
        count_launch();
        err = cudaGetLastError();
    }
    if (err == cudaSuccess) {
        if (x.bits == 8)
            blocked_pass_kernel<8, false><<<grid, 256, 0, stream>>>(x.row_ptr, x.packed_row_ptr, x.col_idx, x.packed, x.rows, x.cols, windows, counts, nullptr, nullptr, 0, nullptr, nullptr, nullptr, 0, 0.0f);
        else
            blocked_pass_kernel<4, false><<<grid, 256, 0, stream>>>(x.row_ptr, x.packed_row_ptr, x.col_idx, x.packed, x.rows, x.cols, windows, counts, nullptr, nullptr, 0, nullptr, nullptr, nullptr, 0, 0.0f);
        count_launch();
        const std::int64_t tiles = (segments + kScanTile - 1) / kScanTile;
        segment_tile_scan_kernel<<<static_cast<unsigned>(tiles), kScanTile, 0, stream>>>(counts, segments, out->seg_ptr, tile_totals);
        tile_totals_scan_kernel<<<1, kScanTile, 0, stream>>>(tile_totals, tiles, out->seg_ptr + segments);
        segment_add_base_kernel<<<static_cast<unsigned>(tiles), kScanTile, 0, stream>>>(tile_totals, segments, out->seg_ptr, cursor);
        count_launch(3);
        err = cudaGetLastError();
    }
    if (err == cudaSuccess) err = cudaMemcpyAsync(&total, out->seg_ptr + segments, sizeof(total), cudaMemcpyDeviceToHost, stream);
    if (err == cudaSuccess && half_values)
        err = cudaMemcpyAsync(bound_bits, counts + segments, sizeof(bound_bits), cudaMemcpyDeviceToHost, stream);
    if (err == cudaSuccess) err = cudaStreamSynchronize(stream);
    float bound = 0.0f, row_bound = 0.0f;
    std::memcpy(&bound, &bound_bits[0], sizeof(float));
    std::memcpy(&row_bound, &bound_bits[1], sizeof(float));
    const float half_scale = half_values ? operand_scale(bound + row_bound) : 0.0f;
    if (err == cudaSuccess && total > 0) {
        word_bytes = static_cast<std::uint64_t>(total) * sizeof(std::uint32_t);
        out->entries = static_cast<std::uint32_t *>(arena.take(word_bytes));
        if (bake && bake_lo) out->entries_lo = static_cast<std::uint32_t *>(arena.take(word_bytes));
        if (out->entries == nullptr || (bake && bake_lo && out->entries_lo == nullptr))
            return give_up(fail(CB200_STATUS_INSUFFICIENT_WORKSPACE, "no device memory for the %lld entry words of the window-blocked copy",
                                static_cast<long long>(total)));
        err = cudaMemsetAsync(out->entries, 0x80, word_bytes, stream); // padding = invalid
        if (err == cudaSuccess && out->entries_lo != nullptr) err = cudaMemsetAsync(out->entries_lo, 0x80, word_bytes, stream);
        if (err == cudaSuccess) {
            if (x.bits == 8)
                blocked_pass_kernel<8, true><<<grid, 256, 0, stream>>>(x.row_ptr, x.packed_row_ptr, x.col_idx, x.packed, x.rows, x.cols, windows, nullptr, cursor, out->entries, bake_mode, x.scales, x.offsets, out->entries_lo, gene_major ? 1 : 0, half_scale);
            else
                blocked_pass_kernel<4, true><<<grid, 256, 0, stream>>>(x.row_ptr, x.packed_row_ptr, x.col_idx, x.packed, x.rows, x.cols, windows, nullptr, cursor, out->entries, bake_mode, x.scales, x.offsets, out->entries_lo, gene_major ? 1 : 0, half_scale);
            count_launch();
            err = cudaGetLastError();
        }
    }
    if (err == cudaSuccess) err = cudaStreamSynchronize(stream);
    if (err != cudaSuccess) return give_up(fail(CB200_STATUS_CUDA_ERROR, "building the window-blocked copy: %s", cudaGetErrorString(err)));
    arena.give_back(tile_totals, tile_total_bytes);
    arena.give_back(cursor, cursor_bytes);
    arena.give_back(counts, count_bytes);
    out->groups = groups;
    out->windows = windows;
    out->total_entries = total;
    out->bytes = static_cast<std::uint64_t>(total) * (out->entries_lo != nullptr ? 8u : 4u) + static_cast<std::uint64_t>(segments + 1) * 8u;
    out->src_row_ptr = x.row_ptr;
    out->src_col_idx = x.col_idx;
    out->src_packed = x.packed;
    out->baked = bake;
    out->baked_gene_major = bake && gene_major;
    out->src_scales = x.scales;
    out->src_offsets = x.offsets;
    out->half_values = half_values;
    out->value_scale = half_values ? half_scale : 1.0f;
    return CB200_STATUS_SUCCESS;
}


cb200_status launch_qcsr_forward_blocked(const qcsr_view &x, const dense_args &d, std::int64_t row_begin,
                                         std::int64_t row_end, void *workspace, std::uint64_t workspace_bytes,
                                         const blocked_layout &layout, bool split_products, int sm_count,
                                         cudaStream_t stream, bool *taken) {
    *taken = false;
    if (row_end <= row_begin) return CB200_STATUS_SUCCESS;
    if (layout.code_tiles != nullptr) {
        if (split_products) return CB200_STATUS_SUCCESS; // one 16-bit pass only
        return launch_qcsr_forward_codes(x, d, row_begin, row_end, workspace, workspace_bytes, layout, sm_count, stream, taken);
    }
    if (layout.dense_tiles != nullptr) {
        if (split_products) return CB200_STATUS_SUCCESS; // the tiles hold bf16(value) only
        return launch_qcsr_forward_dense(x, d, row_begin, row_end, workspace, workspace_bytes, layout, sm_count, stream, taken);
    }
    if (layout.seg_ptr == nullptr || layout.baked_gene_major) return CB200_STATUS_SUCCESS; // the transpose's words are not ours
    if (!qcsr_blocked_shape_ok(x.rows, x.cols, d.n, x.bits, d.dense_dtype)) return CB200_STATUS_SUCCESS;
    const bool w_bf16 = d.dense_dtype == CB200_DTYPE_BF16;
    if (!w_bf16 && !split_products) return CB200_STATUS_SUCCESS; // one bf16 pass over an fp32 W is never asked for
    if (row_begin % kRows != 0) return CB200_STATUS_SUCCESS; // a launch starts on a group boundary, else another kernel runs
    if (reinterpret_cast<std::uintptr_t>(d.out) % 16u != 0u || (d.out_ld * 4u) % 16u != 0u) return CB200_STATUS_SUCCESS;
    if (workspace == nullptr || workspace_bytes < qcsr_blocked_workspace_bytes(x.cols, d.n)) return CB200_STATUS_SUCCESS;
    if (reinterpret_cast<std::uintptr_t>(workspace) % 256u != 0u) return CB200_STATUS_SUCCESS;
    if (x.row_ptr != layout.src_row_ptr || x.col_idx != layout.src_col_idx || x.packed != layout.src_packed ||
        (layout.baked && (x.scales != layout.src_scales || x.offsets != layout.src_offsets)))
        return fail(CB200_STATUS_STALE_STRUCTURE, "the launch's matrix is not the one the window-blocked copy was built from");
    if (layout.baked && split_products && layout.entries_lo == nullptr) return CB200_STATUS_SUCCESS; // no lo words: another kernel runs

    int *status = static_cast<int *>(workspace);
    unsigned *w_absmax = reinterpret_cast<unsigned *>(workspace) + 1; // fp16 operands: float bits of the largest |W|
    unsigned char *records = static_cast<unsigned char *>(workspace) + 256;
    const bool row_policy = x.policy == CB200_DECODE_COLUMN_SCALE_ROW_OFFSET;
    const bool half = layout.baked && layout.half_values;
    CB200_CUDA_OK(cudaMemsetAsync(status, 0, 2 * sizeof(int), stream));
    if (half) {
        const std::int64_t elements = x.cols * d.n;
        const unsigned blocks = static_cast<unsigned>(std::min<std::int64_t>((elements + 1023) / 1024, 4 * static_cast<std::int64_t>(sm_count)));
        if (w_bf16) absmax_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16 *>(d.dense), d.dense_ld, x.cols, static_cast<int>(d.n), w_absmax);
        else absmax_kernel<float><<<blocks, 256, 0, stream>>>(static_cast<const float *>(d.dense), d.dense_ld, x.cols, static_cast<int>(d.n), w_absmax);
        count_launch();
        CB200_CUDA_OK(cudaGetLastError());
    }

    blocked_params p{};
    p.entries = layout.entries; p.seg_ptr = layout.seg_ptr;
    p.row_offsets = row_policy && !layout.baked ? x.offsets : nullptr; // baked words already hold the row's offset
    p.records = records; p.y = d.out; p.y_ld = d.out_ld; p.row_end = row_end;
    p.group_begin = row_begin / kRows; p.group_end = (row_end + kRows - 1) / kRows; p.windows = layout.windows;
    p.alpha = d.alpha; p.status = status;
    p.idesc = instr_desc(static_cast<int>(d.n), half);
    p.result_scale = half ? 1.0f / layout.value_scale : 1.0f;
    p.w_absmax = half ? w_absmax : nullptr;
    p.poll_limit = kPollLimit;
    p.withhold_w = 0;
    if (const int armed = g_test_poll_limit.load(std::memory_order_relaxed)) { // test hook: see cb200_test_arm_wait_timeout
        p.poll_limit = armed;
        p.withhold_w = 1;
    }
    *taken = true;
    // One pass multiplies bf16(value) with bf16 W.  With split products the fp32 product is rebuilt
    // from bf16 pieces, value = hi + lo and (fp32 W) W = hi + lo:  bf16 W: hi*w + lo*w (two passes, exact
    // up to the 2^-17 of the value that lo leaves);  fp32 W: hi*hi + hi*lo + lo*hi (three passes,
    // ~3 * 2^-17 per product).  The passes run back to back on the stream, share the record buffer and
    // accumulate into Y (beta of the call on the first pass, 1 afterwards); every pass sums a row in
    // the same fixed order, so the result is repeatable.
    struct pass_spec { int w_part, value_part; };
    const pass_spec plain[1] = {{0, 0}}, split_bf16[2] = {{0, 0}, {0, 1}}, split_f32[3] = {{0, 0}, {1, 0}, {0, 1}};
    const pass_spec *passes = !split_products ? plain : (w_bf16 ? split_bf16 : split_f32);
    const int pass_count = !split_products ? 1 : (w_bf16 ? 2 : 3);
    int packed_part = -1;
    for (int i = 0; i < pass_count; ++i) {
        if (passes[i].w_part != packed_part) {
            const dim3 grid(static_cast<unsigned>(layout.windows), static_cast<unsigned>(d.n / kPackColumns));
            if (w_bf16)
                pack_windows_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16 *>(d.dense), d.dense_ld,
                                                                              x.cols, static_cast<int>(d.n), passes[i].w_part, x.scales,
                                                                              x.offsets, row_policy ? 0 : 1, records, half ? w_absmax : nullptr);
            else
                pack_windows_kernel<float><<<grid, 256, 0, stream>>>(static_cast<const float *>(d.dense), d.dense_ld, x.cols,
                                                                      static_cast<int>(d.n), passes[i].w_part, x.scales, x.offsets,
                                                                      row_policy ? 0 : 1, records, half ? w_absmax : nullptr);
            count_launch();
            CB200_CUDA_OK(cudaGetLastError());
            packed_part = passes[i].w_part;
        }
        p.value_part = passes[i].value_part;
        if (layout.baked) p.entries = passes[i].value_part != 0 ? layout.entries_lo : layout.entries; // baked words carry their part
        p.beta = i == 0 ? d.beta : 1.0f;
        p.bias = d.bias;
        p.epilogue = i + 1 == pass_count ? d.epilogue : CB200_EPILOGUE_NONE;
        cb200_status st;
        const bool long_segments = layout.total_entries > static_cast<std::int64_t>(kChunkEntries) * layout.groups * layout.windows;
        // two scatter groups pay when a window is a chunk or two; long segments keep one group and deeper chunks
        const bool two_groups = layout.baked && !long_segments;
        switch (d.n) {
        case 32: st = two_groups ? launch_blocked2<32>(p, sm_count, stream) : launch_one<32>(p, long_segments, layout.baked, sm_count, stream); break;
        case 64: st = two_groups ? launch_blocked2<64>(p, sm_count, stream) : launch_one<64>(p, long_segments, layout.baked, sm_count, stream); break;
        default: st = two_groups ? launch_blocked2<128>(p, sm_count, stream) : launch_one<128>(p, long_segments, layout.baked, sm_count, stream); break;
        }
        if (st != CB200_STATUS_SUCCESS) return st;
    }
    return CB200_STATUS_SUCCESS;
}

} // namespace cb200

extern "C" void cb200_test_arm_wait_timeout(uint32_t poll_limit) {
    const uint32_t clamped = poll_limit < 64u ? 64u : (poll_limit > static_cast<uint32_t>(cb200::kPollLimit) ? static_cast<uint32_t>(cb200::kPollLimit) : poll_limit);
    cb200::g_test_poll_limit.store(static_cast<int>(clamped), std::memory_order_relaxed);
}
extern "C" void cb200_test_disarm_wait_timeout(void) { cb200::g_test_poll_limit.store(0, std::memory_order_relaxed); }
