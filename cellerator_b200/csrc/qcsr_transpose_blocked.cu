// Gene-side transpose on the tensor cores from the window-blocked copy of the matrix (schedule
// "tensor_blocked" of the transpose projection), for callers whose numeric policy allows bf16
// products and who hand the device-resident matrix to prepare:
//     G'[genes, N] = alpha * deq(X)^T[genes, cells] * G[cells, N] + beta * G',   N in {32, 64}.
//
// Reference counterpart: csr_spmm_bwd_rhs_kernel_ (one scalar atomicAdd per stored entry and output
// column, src/compute/sparse/ops/kernels/base_sparse/csr_spmm_bwd_rhs_kernel_.cuh:1-22).  The exact
// kernel of this library (qcsr_transpose.cu) does the same with 128-bit vector reductions and is
// bound by the L2 atomic units: 256 bytes of reductions per stored entry.
//
// Formulation.  For a group of 256 cells and a window of 128 genes the product is a dense
// contraction over the cells:  D_w[128 genes, N] += X_gw^T[128 genes, 256 cells] * G_g[256 cells, N].
// The window-blocked copy (see qcsr_forward_blocked.cu) delivers the entries of (group, window)
// as one contiguous segment; they are decoded to bf16 and scattered into a zeroed operand tile in
// shared memory, laid out gene-major this time (M = gene, K = cell; K-major with the 128-byte
// swizzle), and sixteen 128 x N x 16 tcgen05 MMAs multiply it with the group's rows of G.  G is
// converted to bf16 once per launch into one 256 x N record per group, already in the K-major
// core-matrix operand layout (rows outside the launch's row range are written as zero, which is how a
// partial row range is honoured).  A CTA keeps the fp32 accumulators of a set of windows (four at N = 64,
// eight at N = 32; two accumulators per window, one per MMA-issuing warp, 512 TMEM columns in all) while
// it walks a run of groups, so the group's G record is fetched once per set; at the end of the run the
// two accumulators of a window are added and the sums are stored to the run's slot of a scratch array.  The
// (window set, group) pairs are dealt to the CTAs as equal contiguous runs, so two or three CTAs contribute to
// the same genes: ordered_sum_kernel adds a set's slots into G' in run order (G' is first scaled by beta by a
// small kernel), which makes G' the same bits on every launch -- vector reductions straight into G', as this
// kernel used before, are served in the order the L2 sees them.
//
// Entry words.  Prepare normally bakes them for this kernel: {bf16 value, byte position / 2 in the
// gene-major tile}, a hi array and, for the split passes, a lo array with bf16(value - hi); the scatter
// then stores words as they are (18.1 ms against 23.6 for the three split passes on the 1M x 33,538
// matrix, 6.25 against 7.93 for one bf16 pass).  Code words {code, gene, forward-tile position} are
// still decoded here when the caller's memory limit left no room for the second array.
//
// Structure of a CTA (640 threads, one CTA per SM): warps 0-15 zero, decode and scatter -- as two
// groups of eight warps on alternate tiles, each with its own tile buffer and 8 KB chunk stage, so
// that the per-tile chains of waits overlap (23.6 ms against 24.4 for the three split passes on the
// 1M x 33,538 matrix); baked words are fetched into registers before the tile is released, so that only
// stores lie between release and hand-over -- and read the accumulators back at the end of a run; warps 16
// and 17 issue the MMAs, the first and the second eight K steps of every tile (15.7 ms against 17.5 with one
// issuing warp); warp 18 feeds the G ring (2 stages of 32 KB); warp 19 deals the entry chunks.  Every barrier wait is bounded; on a
// time-out a status word is raised, waits stop blocking, and the kernel runs to completion and frees
// its TMEM.  A non-zero status means G' is not valid.
#include "kernels.cuh"
#include "sm100_primitives.cuh"

#include <algorithm>
#include <cuda_bf16.h>

namespace cb200 {
namespace {

constexpr int kWin = 128;                     // genes per window (as in the blocked copy)
constexpr int kRows = 256;                    // cells per group (as in the blocked copy)
// windows whose accumulators a CTA holds in TMEM: two sets of N columns per window (one per MMA-issuing warp, which
// take the first and the second half of a tile's K steps), 512 columns in all
__host__ __device__ constexpr int set_windows(int n) { return 256 / n; }
constexpr int kIssuers = 2;
constexpr int kProducerWarps = 16;
constexpr int kProducerThreads = kProducerWarps * 32;
constexpr int kChunkLoaders = 1;
constexpr int kThreads = kProducerThreads + 32 * (kIssuers + 1 + kChunkLoaders);
constexpr int kTileBytes = kWin * kRows * 2;  // 64 KB: [cell quarter][gene][64 cells]
constexpr int kQuarterBytes = kWin * 128;     // 16 KB: 128 genes x 64 cells
constexpr int kGStages = 2;
constexpr int kChunkEntries = 2048;
constexpr int kChunkBytes = kChunkEntries * 4;
constexpr int kChunkStages = 2;               // one per scatter group (two stages each do not fit beside the G ring)
constexpr int kGroupWarps = kProducerWarps / 2;
constexpr int kGroupThreads = kGroupWarps * 32;
constexpr int kRing = kChunkStages / 2;       // chunk stages per scatter group
static_assert(kChunkLoaders == 1 && kRing >= 1, "one loader thread deals the chunks to the two groups' rings");

__host__ __device__ constexpr int g_record_bytes(int n) { return kRows * n * 2; }

struct tb_params {
    const std::uint32_t *entries;
    const std::int64_t *seg_ptr;
    const float *scales;
    const float *gene_offsets; // per gene, per-gene-affine policy
    const float *row_offsets;  // per cell, row-offset policy
    const unsigned char *records; // G as bf16, one record per group
    float *out;
    std::int64_t out_ld;
    std::int64_t cols;
    std::int64_t group_begin, group_count;
    int windows;
    float alpha;
    int *status;
    int value_part; // 0: tile holds hi = bf16(value); 1: lo = bf16(value - hi)
    // The accumulators of a run (the consecutive units of one window set in one CTA) go to slot `global run index` of
    // this array, [run][window of the set][gene][N]; ordered_sum_kernel adds the slots of a set into G' in run order,
    // so that G' is the same bits on every launch (atomic adds of three or more CTAs' sums are not).
    float *partials;
};

// Runs of CTA b of a grid over `total` units in sets of `per_set`: it owns the units [total b / grid, total (b + 1) / grid).
__host__ __device__ inline std::int64_t runs_of_cta(std::int64_t total, std::int64_t per_set, std::int64_t grid, std::int64_t b) {
    const std::int64_t u0 = total * b / grid, u1 = total * (b + 1) / grid;
    return u1 > u0 ? (u1 - 1) / per_set - u0 / per_set + 1 : 0;
}

__device__ __forceinline__ std::int64_t dmin(std::int64_t a, std::int64_t b) { return a < b ? a : b; }
// K-major operand, no swizzle (the G record): core matrices of 8 columns x 16 bytes (8 cells); the
// 32 core matrices of 8 output columns sit side by side (LBO = 128 B), groups of 8 columns 4 KB apart.
__device__ __forceinline__ std::uint64_t smem_desc_g(std::uint32_t addr) {
    std::uint64_t d = 0;
    d |= static_cast<std::uint64_t>((addr & 0x3ffffu) >> 4);
    d |= static_cast<std::uint64_t>(128u >> 4) << 16;
    d |= static_cast<std::uint64_t>(static_cast<unsigned>(kRows * 16) >> 4) << 32;
    d |= static_cast<std::uint64_t>(1) << 46; // descriptor version of this architecture
    return d;
}
// (the tile itself is K-major with the 128-byte swizzle, 8-gene atoms of 1,024 bytes: smem_desc_sw128)
// out = beta * out (beta == 0 writes zeros without reading).
__global__ void __launch_bounds__(256) scale_output_kernel(float *out, std::int64_t rows, int n, std::int64_t ld, float beta) {
    const std::int64_t total = rows * n;
    for (std::int64_t i = static_cast<std::int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<std::int64_t>(gridDim.x) * blockDim.x) {
        float *p = out + (i / n) * ld + (i % n);
        *p = beta == 0.0f ? 0.0f : beta * *p;
    }
}

// G [cells][n] fp32 (leading dimension ld) -> one bf16 record per group of 256 cells: the n x 256
// slice of G^T in the no-swizzle K-major operand layout (byte offset of (column c, cell r) =
// (c/8)*4096 + (r/8)*128 + (c%8)*16 + (r%8)*2).  Cells outside [row_begin, row_end) are zero.
// part 0 writes hi = bf16(g); part 1 writes lo = bf16(g - hi), the next 8 bits of the mantissa.
__global__ void __launch_bounds__(256) pack_g_kernel(const float *g, std::int64_t ld, int n, std::int64_t row_begin,
                                                     std::int64_t row_end, std::int64_t group_begin, int part,
                                                     unsigned char *records) {
    const std::int64_t group = group_begin + blockIdx.x;
    unsigned char *rec = records + static_cast<std::size_t>(blockIdx.x) * g_record_bytes(n);
    // A thread makes one 16-byte piece: a column's values of eight consecutive cells.  Consecutive threads take consecutive
    // columns of the same eight cells: their loads of a cell's row are contiguous, and their pieces are too (8 columns =
    // 128 bytes of the record).
    for (int item = threadIdx.x; item < n * (kRows / 8); item += blockDim.x) {
        const int c = item % n, r8 = item / n;
        std::uint32_t packed[4];
#pragma unroll
        for (int j = 0; j < 8; j += 2) {
            float v[2];
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                const std::int64_t row = group * kRows + r8 * 8 + j + k;
                v[k] = (row >= row_begin && row < row_end) ? g[row * ld + c] : 0.0f;
            }
            __nv_bfloat16 b0 = __float2bfloat16_rn(v[0]), b1 = __float2bfloat16_rn(v[1]);
            if (part != 0) {
                b0 = __float2bfloat16_rn(v[0] - __bfloat162float(b0));
                b1 = __float2bfloat16_rn(v[1] - __bfloat162float(b1));
            }
            packed[j >> 1] = static_cast<std::uint32_t>(__bfloat16_as_ushort(b0)) | (static_cast<std::uint32_t>(__bfloat16_as_ushort(b1)) << 16);
        }
        *reinterpret_cast<uint4 *>(rec + (c >> 3) * (kRows * 16) + r8 * 128 + (c & 7) * 16) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    }
}

// BAKED: the entry words hold {bf16 value, byte position / 2 in this kernel's tile}, written at prepare
// (hi and lo arrays for the split passes): the scatter stores them as they are, no table, no arithmetic.
template<int NC, bool BAKED>
__global__ void __launch_bounds__(kThreads, 1) qcsr_transpose_blocked_kernel(const tb_params p) {
    constexpr int GREC = g_record_bytes(NC);
    constexpr int kSetWindows = set_windows(NC);
    constexpr int kTmemCols = kSetWindows * kIssuers * NC; // 512
    constexpr std::uint32_t IDESC = instr_desc(NC);
    extern __shared__ __align__(1024) unsigned char smem[];
    // [2][tile] | [kGStages][G record] | [kChunkStages][entry chunk] | tables | row offsets | barriers | ...
    unsigned char *chunk_base = smem + 2 * kTileBytes + kGStages * GREC;
    float2 *table = reinterpret_cast<float2 *>(chunk_base + kChunkStages * kChunkBytes); // [kSetWindows][kWin] {scale, offset}
    float *row_offset_s = reinterpret_cast<float *>(table + kSetWindows * kWin);         // [kRows]
    std::uint64_t *bars = reinterpret_cast<std::uint64_t *>(row_offset_s + kRows);
    std::uint64_t *a_full = bars;                      // [2]            scatter warps -> MMA (one arrival per warp)
    std::uint64_t *a_empty = bars + 2;                 // [2]            MMA commit -> scatter warps
    std::uint64_t *g_full = bars + 4;                  // [kGStages]     copy engine -> MMA
    std::uint64_t *g_empty = g_full + kGStages;        // [kGStages]     MMA commit -> loader
    std::uint64_t *c_full = g_empty + kGStages;        // [kChunkStages] copy engine -> scatter warps
    std::uint64_t *c_empty = c_full + kChunkStages;    // [kChunkStages] scatter warps -> loaders
    std::uint64_t *acc_full = c_empty + kChunkStages;  // MMA commit -> scatter warps
    std::uint64_t *acc_empty = acc_full + 1;           // scatter warps -> MMA
    volatile int *chunk_meta = reinterpret_cast<volatile int *>(acc_empty + 1); // [kChunkStages]
    std::uint32_t *tmem_slot = reinterpret_cast<std::uint32_t *>(const_cast<int *>(chunk_meta) + kChunkStages + 1);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    unsigned char *scratch_slot = reinterpret_cast<unsigned char *>(tmem_slot + 2);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const std::uint32_t smem0 = smem_addr(smem);
    const std::uint32_t grec0 = smem0 + 2 * kTileBytes;
    const std::uint32_t chunk0 = grec0 + kGStages * GREC;

    if (tid == 0) {
        for (int b = 0; b < 2; ++b) {
            bar_init(smem_addr(a_full + b), kGroupWarps);
            bar_init(smem_addr(a_empty + b), kIssuers); // one commit per MMA warp
        }
        for (int s = 0; s < kGStages; ++s) {
            bar_init(smem_addr(g_full + s), 1);
            bar_init(smem_addr(g_empty + s), kIssuers);
        }
        for (int s = 0; s < kChunkStages; ++s) {
            bar_init(smem_addr(c_full + s), 1);
            bar_init(smem_addr(c_empty + s), kGroupWarps);
        }
        bar_init(smem_addr(acc_full), kIssuers);
        bar_init(smem_addr(acc_empty), kProducerWarps);
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

    // Work: units (window set, group), numbered set * group_count + group; this CTA owns the units
    // [u0, u1).  A run = the consecutive units of one window set; it ends with the accumulators being
    // added into G'.  Every role walks the same runs.
    const std::int64_t sets = (p.windows + kSetWindows - 1) / kSetWindows;
    const std::int64_t total_units = sets * p.group_count;
    const std::int64_t u0 = total_units * blockIdx.x / gridDim.x, u1 = total_units * (blockIdx.x + 1) / gridDim.x;
    // global index of this CTA's first run: the runs of the CTAs before it (every warp adds them up for itself)
    std::int64_t first_run = 0;
    for (std::int64_t b = lane; b < static_cast<std::int64_t>(blockIdx.x); b += 32) first_run += runs_of_cta(total_units, p.group_count, gridDim.x, b);
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) first_run += __shfl_xor_sync(0xffffffffu, first_run, d);

    if (warp < kProducerWarps) {
        // ================= zero, scatter, read back =================
        // Two scatter groups of eight warps take alternate tiles (group g owns tile buffer g and chunk
        // stage g), so that the chains zero -> barrier -> chunk -> scatter -> fence of consecutive tiles overlap.
        const bool use_row_offset = p.row_offsets != nullptr;
        const int grp = warp / kGroupWarps, gtid = tid - grp * kGroupThreads;
        unsigned char *tile = smem + grp * kTileBytes;
        long long q = 0, qc = 0; // tiles of this CTA (both groups count all of them); chunks this group consumed
        int run = 0;
        for (std::int64_t u = u0; u < u1; ++run) {
            const std::int64_t set = u / p.group_count, gi0 = u % p.group_count;
            const std::int64_t count = dmin(p.group_count - gi0, u1 - u);
            const int nwin = static_cast<int>(dmin(kSetWindows, p.windows - set * kSetWindows));
            // scale / zero-point of the set's genes; nobody still reads the previous run's table
            // (baked words need neither the table nor the row offsets below)
            if constexpr (!BAKED) asm volatile("bar.sync 1, %0;" ::"n"(kProducerThreads) : "memory");
            for (int i = tid; !BAKED && i < kSetWindows * kWin; i += kProducerThreads) {
                const std::int64_t gene = set * kSetWindows * kWin + i;
                float2 so = make_float2(0.0f, 0.0f);
                if (gene < p.cols) {
                    so.x = p.scales != nullptr ? __ldg(p.scales + gene) : 1.0f;
                    so.y = p.gene_offsets != nullptr ? __ldg(p.gene_offsets + gene) : 0.0f;
                }
                table[i] = so;
            }
            if constexpr (!BAKED) asm volatile("bar.sync 1, %0;" ::"n"(kProducerThreads) : "memory");
            for (std::int64_t gi = gi0; gi < gi0 + count; ++gi) {
                const std::int64_t group = p.group_begin + gi;
                if (!BAKED && use_row_offset) {
                    asm volatile("bar.sync 1, %0;" ::"n"(kProducerThreads) : "memory"); // the previous group's scatter is over
                    if (tid < kRows) row_offset_s[tid] = __ldg(p.row_offsets + group * kRows + tid); // padded by the launcher's check
                    asm volatile("bar.sync 1, %0;" ::"n"(kProducerThreads) : "memory");
                }
                for (int wl = 0; wl < nwin; ++wl, ++q) {
                    if (static_cast<int>(q & 1) != grp) continue;
                    // Baked words: the tile's first chunk (all of it for all but the densest matrices) goes into registers
                    // while the tile is still being read by the MMAs of the group's previous tile; between the tile's release
                    // and its hand-over there are then only stores.
                    bool last = false;
                    uint4 held[kChunkEntries / (kGroupThreads * 4)];
                    if constexpr (BAKED) {
                        const int cs = grp * kRing + static_cast<int>(qc % kRing);
                        bar_wait(smem_addr(c_full + cs), static_cast<std::uint32_t>((qc / kRing) & 1), abort_flag);
                        const int meta = chunk_meta[cs];
                        const int n_entries = *abort_flag != 0 ? 0 : (meta >> 1);
                        last = (meta & 1) != 0 || *abort_flag != 0;
                        const uint4 *chunk = reinterpret_cast<const uint4 *>(chunk_base + cs * kChunkBytes);
#pragma unroll
                        for (int k = 0; k < kChunkEntries / (kGroupThreads * 4); ++k) { // segments are padded to multiples of 4
                            const int i = (k * kGroupThreads + gtid) * 4;
                            held[k] = i < n_entries ? chunk[i >> 2] : make_uint4(0x80000000u, 0x80000000u, 0x80000000u, 0x80000000u);
                        }
                        // the words are used much later, but they must be in the registers before the stage goes back to the copy engine
                        {
                            std::uint32_t all = 0;
#pragma unroll
                            for (int k = 0; k < kChunkEntries / (kGroupThreads * 4); ++k) all |= held[k].x | held[k].y | held[k].z | held[k].w;
                            arrive_when_loaded(smem_addr(c_empty + cs), all, lane, static_cast<std::uint32_t>(p.windows) >> 31);
                        }
                        ++qc;
                    }
                    bar_wait(smem_addr(a_empty + grp), static_cast<std::uint32_t>(((q >> 1) & 1) ^ 1), abort_flag);
#pragma unroll
                    for (int k = 0; k < kTileBytes / (kGroupThreads * 8); ++k) // 8-byte stores: fewer wavefronts of the LSU data pipe per byte than 16-byte ones
                        *reinterpret_cast<uint2 *>(tile + k * (kGroupThreads * 8) + gtid * 8) = make_uint2(0u, 0u);
                    // the whole tile is zero before anyone of the group scatters (named barrier 2 or 3)
                    if (grp == 0) asm volatile("bar.sync 2, %0;" ::"n"(kGroupThreads) : "memory");
                    else asm volatile("bar.sync 3, %0;" ::"n"(kGroupThreads) : "memory");
                    if constexpr (BAKED) {
#pragma unroll
                        for (int k = 0; k < kChunkEntries / (kGroupThreads * 4); ++k) {
                            const std::uint32_t e[4] = {held[k].x, held[k].y, held[k].z, held[k].w};
#pragma unroll
                            for (int j = 0; j < 4; ++j) { // padding words (top bit set) go to a scratch slot
                                unsigned char *dst = static_cast<int>(e[j]) >= 0 ? tile + (((e[j] >> 16) & 0x7fffu) << 1) : scratch_slot;
                                *reinterpret_cast<unsigned short *>(dst) = static_cast<unsigned short>(e[j] & 0xffffu);
                            }
                        }
                    }
                    const float2 *wtable = table + wl * kWin;
                    int guard = 0;
                    while (!last && ++guard < (1 << 20)) {
                        const int cs = grp * kRing + static_cast<int>(qc % kRing);
                        bar_wait(smem_addr(c_full + cs), static_cast<std::uint32_t>((qc / kRing) & 1), abort_flag);
                        const int meta = chunk_meta[cs];
                        const int n_entries = *abort_flag != 0 ? 0 : (meta >> 1);
                        last = (meta & 1) != 0 || *abort_flag != 0;
                        const uint4 *chunk = reinterpret_cast<const uint4 *>(chunk_base + cs * kChunkBytes);
                        for (int i = gtid * 4; i < n_entries; i += kGroupThreads * 4) { // segments are padded to multiples of 4
                            const uint4 e4 = chunk[i >> 2];
                            const std::uint32_t e[4] = {e4.x, e4.y, e4.z, e4.w};
                            if constexpr (BAKED) {
#pragma unroll
                                for (int k = 0; k < 4; ++k) { // padding words (top bit set) go to a scratch slot
                                    unsigned char *dst = static_cast<int>(e[k]) >= 0 ? tile + (((e[k] >> 16) & 0x7fffu) << 1) : scratch_slot;
                                    *reinterpret_cast<unsigned short *>(dst) = static_cast<unsigned short>(e[k] & 0xffffu);
                                }
                                continue;
                            }
                            float2 t[4];
#pragma unroll
                            for (int k = 0; k < 4; ++k) t[k] = wtable[(e[k] >> 8) & (kWin - 1)];
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                // the copy stores the byte position in the forward (cell-major) tile; take the cell back
                                // out of it and place the value gene-major: [cell quarter][gene][64 cells], 16-byte pieces
                                // of a gene's line permuted by gene mod 8
                                const std::uint32_t gl = (e[k] >> 8) & (kWin - 1);
                                const std::uint32_t fwd = ((e[k] >> 15) & 0x7fffu) << 1;
                                const std::uint32_t rl = ((fwd >> 15) << 7) | (((fwd >> 10) & 15u) << 3) | ((fwd >> 7) & 7u);
                                const std::uint32_t off = (rl >> 6) * kQuarterBytes + (gl >> 3) * 1024u + (gl & 7u) * 128u +
                                                          ((((rl & 63u) >> 3) ^ (gl & 7u)) << 4) + ((rl & 7u) << 1);
                                const float add = use_row_offset ? row_offset_s[rl] : t[k].y;
                                const float value = fmaf(static_cast<float>(e[k] & 0xffu), t[k].x, add);
                                // padding words (top bit set) are stored to a scratch slot instead of branching
                                unsigned char *dst = static_cast<int>(e[k]) >= 0 ? tile + off : scratch_slot;
                                __nv_bfloat16 b = __float2bfloat16_rn(value);
                                if (p.value_part != 0) b = __float2bfloat16_rn(value - __bfloat162float(b)); // the next 8 mantissa bits
                                *reinterpret_cast<__nv_bfloat16 *>(dst) = b;
                            }
                        }
                        __syncwarp();
                        if (lane == 0) bar_arrive(smem_addr(c_empty + cs));
                        ++qc;
                    }
                    fence_async_proxy(); // ordinary stores, read by the MMA through the async proxy
                    __syncwarp();
                    if (lane == 0) bar_arrive(smem_addr(a_full + grp));
                }
            }
            // ---- end of the run: add the accumulators into G'.  TMEM lane = gene within the window;
            //      a warp reads the lane quarter its number allows, for every fourth window of the set.
            bar_wait(smem_addr(acc_full), static_cast<std::uint32_t>(run & 1), abort_flag);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int quarter = warp & 3;
            for (int wl = warp >> 2; wl < kSetWindows; wl += kProducerWarps / 4) {
                if (wl >= nwin) break; // warp-uniform
                const std::int64_t gene = (set * kSetWindows + wl) * kWin + quarter * 32 + lane;
#pragma unroll
                for (int h = 0; h < NC / 32; ++h) {
                    float v[32], second[32]; // the two halves of the K steps were accumulated apart
                    tmem_ld32(tmem_base + (static_cast<std::uint32_t>(quarter * 32) << 16) + wl * kIssuers * NC + h * 32, v);
                    tmem_ld32(tmem_base + (static_cast<std::uint32_t>(quarter * 32) << 16) + (wl * kIssuers + 1) * NC + h * 32, second);
#pragma unroll
                    for (int c = 0; c < 32; ++c) v[c] += second[c];
                    if (gene < p.cols && *abort_flag == 0) {
                        float *slot = p.partials + (((first_run + run) * kSetWindows + wl) * kWin + quarter * 32 + lane) * NC + h * 32;
#pragma unroll
                        for (int c = 0; c < 32; c += 4) *reinterpret_cast<float4 *>(slot + c) = make_float4(v[c], v[c + 1], v[c + 2], v[c + 3]);
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) bar_arrive(smem_addr(acc_empty));
            u += count;
        }
    } else if (warp < kProducerWarps + kIssuers) {
        // ================= MMA issuers: warp kh issues the K steps [8 kh, 8 kh + 8) of every tile into its own accumulators.
        // One issuing thread is held to the rate at which the MMAs read their operands and then spends half as long again
        // on commits, waits and loop overhead while the tensor pipe runs dry; two threads halve the issue time of a tile. ==
        const int kh = warp - kProducerWarps;
        long long q = 0, qg = 0;
        int run = 0;
        for (std::int64_t u = u0; u < u1; ++run) {
            const std::int64_t set = u / p.group_count, gi0 = u % p.group_count;
            const std::int64_t count = dmin(p.group_count - gi0, u1 - u);
            const int nwin = static_cast<int>(dmin(kSetWindows, p.windows - set * kSetWindows));
            bar_wait(smem_addr(acc_empty), static_cast<std::uint32_t>((run & 1) ^ 1), abort_flag);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            for (std::int64_t gi = 0; gi < count; ++gi, ++qg) {
                const int gs = static_cast<int>(qg % kGStages);
                bar_wait(smem_addr(g_full + gs), static_cast<std::uint32_t>((qg / kGStages) & 1), abort_flag);
                for (int wl = 0; wl < nwin; ++wl, ++q) {
                    const std::uint32_t b = static_cast<std::uint32_t>(q & 1);
                    bar_wait(smem_addr(a_full + b), static_cast<std::uint32_t>((q >> 1) & 1), abort_flag);
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    if (lane == 0) {
                        const std::uint32_t a_tile = smem0 + b * kTileBytes;
                        const std::uint32_t g_rec = grec0 + gs * GREC;
#pragma unroll
                        for (int k8 = 0; k8 < kRows / 16 / kIssuers; ++k8) {
                            const int kk = kh * (kRows / 16 / kIssuers) + k8;
                            mma_bf16(tmem_base + (wl * kIssuers + kh) * NC, smem_desc_sw128(a_tile + (kk >> 2) * kQuarterBytes + (kk & 3) * 32),
                                     smem_desc_g(g_rec + kk * 256), IDESC, gi > 0 || k8 > 0);
                        }
                        mma_commit(smem_addr(a_empty + b));
                        if (wl == nwin - 1) mma_commit(smem_addr(g_empty + gs));
                        if (wl == nwin - 1 && gi == count - 1) mma_commit(smem_addr(acc_full));
                    }
                    __syncwarp();
                }
            }
            u += count;
        }
    } else {
        const int role = warp - kProducerWarps - kIssuers; // 0: G records, 1..kChunkLoaders: entry chunks
        if (role == 0) {
            if (lane == 0) {
                long long qg = 0;
                for (std::int64_t u = u0; u < u1; ++u, ++qg) {
                    const std::int64_t gi = u % p.group_count;
                    const int gs = static_cast<int>(qg % kGStages);
                    bar_wait(smem_addr(g_empty + gs), static_cast<std::uint32_t>(((qg / kGStages) & 1) ^ 1), abort_flag);
                    bar_arrive_expect_tx(smem_addr(g_full + gs), GREC);
                    bulk_copy_g2s(grec0 + gs * GREC, p.records + static_cast<std::size_t>(gi) * GREC, GREC, smem_addr(g_full + gs));
                }
            }
        } else {
            long long q = 0, qc0 = 0, qc1 = 0; // tiles; chunks issued into each group's ring
            for (std::int64_t u = u0; u < u1; ++u) {
                const std::int64_t set = u / p.group_count, group = p.group_begin + u % p.group_count;
                const int nwin = static_cast<int>(dmin(kSetWindows, p.windows - set * kSetWindows));
                // the unit's segments are consecutive: their bounds in one coalesced read
                const std::int64_t bound = lane <= nwin ? __ldg(p.seg_ptr + group * p.windows + set * kSetWindows + lane) : 0;
                for (int j = 0; j < nwin; ++j, ++q) {
                    const std::int64_t lo = __shfl_sync(0xffffffffu, bound, j), hi = __shfl_sync(0xffffffffu, bound, j + 1);
                    const int ring = static_cast<int>(q & 1); // tile q belongs to scatter group q & 1
                    std::int64_t at = lo;
                    do {
                        const int n_entries = static_cast<int>(dmin(kChunkEntries, hi - at));
                        const long long mine = ring == 0 ? qc0 : qc1;
                        if (lane == 0) {
                            const int cs = ring * kRing + static_cast<int>(mine % kRing);
                            bar_wait(smem_addr(c_empty + cs), static_cast<std::uint32_t>(((mine / kRing) & 1) ^ 1), abort_flag);
                            chunk_meta[cs] = (n_entries << 1) | (at + n_entries >= hi ? 1 : 0);
                            if (n_entries > 0) {
                                bar_arrive_expect_tx(smem_addr(c_full + cs), static_cast<std::uint32_t>(n_entries) * 4u);
                                bulk_copy_g2s(chunk0 + cs * kChunkBytes, p.entries + at, static_cast<std::uint32_t>(n_entries) * 4u,
                                              smem_addr(c_full + cs));
                            } else {
                                bar_arrive(smem_addr(c_full + cs)); // an empty segment still hands over one (empty) chunk
                            }
                        }
                        at += n_entries;
                        if (ring == 0) ++qc0;
                        else ++qc1;
                    } while (at < hi);
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

template<int NC> constexpr std::size_t tb_smem_bytes() {
    return 2 * kTileBytes + kGStages * g_record_bytes(NC) + kChunkStages * kChunkBytes + set_windows(NC) * kWin * 8 + kRows * 4 +
           (6 + 2 * kGStages + 2 * kChunkStages) * sizeof(std::uint64_t) + (kChunkStages + 1) * 4 + 16;
}

// G'[genes of window wl of set s] += alpha * (the sums of the runs of set s, added in run order).  Block = (set, window of
// the set); the runs of a set are those of the CTAs whose unit range meets the set, in CTA order.
template<int NC>
__global__ void __launch_bounds__(256) ordered_sum_kernel(const float *partials, float *out, std::int64_t out_ld, std::int64_t cols, int windows,
                                                          std::int64_t group_count, std::int64_t grid, float alpha) {
    constexpr int kSetWindows = set_windows(NC);
    __shared__ std::int64_t slots[512];
    __shared__ int slot_count;
    const std::int64_t set = blockIdx.x / kSetWindows;
    const int wl = static_cast<int>(blockIdx.x % kSetWindows);
    const std::int64_t window = set * kSetWindows + wl;
    if (window >= windows) return;
    const std::int64_t sets = (windows + kSetWindows - 1) / kSetWindows, total = sets * group_count;
    // thread b looks at CTA b: how many runs it has and whether one of them belongs to this set; two scans over the block
    // turn that into the global index of each CTA's first run and the place of its slot in the list (CTA order)
    __shared__ int scan[256];
    const std::int64_t b = threadIdx.x;
    const std::int64_t u0 = b < grid ? total * b / grid : 0, u1 = b < grid ? total * (b + 1) / grid : 0;
    const int runs = b < grid ? static_cast<int>(runs_of_cta(total, group_count, grid, b)) : 0;
    const int meets = (u1 > u0 && u0 < (set + 1) * group_count && u1 > set * group_count) ? 1 : 0;
    int before_runs = 0, before_meets = 0; // exclusive sums over the CTAs before b
    for (int which = 0; which < 2; ++which) {
        scan[threadIdx.x] = which == 0 ? runs : meets;
        __syncthreads();
        for (int d = 1; d < 256; d <<= 1) {
            const int add = threadIdx.x >= static_cast<unsigned>(d) ? scan[threadIdx.x - d] : 0;
            __syncthreads();
            scan[threadIdx.x] += add;
            __syncthreads();
        }
        (which == 0 ? before_runs : before_meets) = scan[threadIdx.x] - (which == 0 ? runs : meets);
        if (which == 1 && threadIdx.x == 255) slot_count = scan[255];
        __syncthreads();
    }
    if (meets) slots[before_meets] = before_runs + (set - u0 / group_count);
    __syncthreads();
    const int count = slot_count;
    for (int i = threadIdx.x; i < kWin * (NC / 4); i += blockDim.x) {
        const int gl = i / (NC / 4), c4 = i % (NC / 4);
        const std::int64_t gene = window * kWin + gl;
        if (gene >= cols) continue;
        float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (int r = 0; r < count; ++r) {
            const float4 v = *reinterpret_cast<const float4 *>(partials + ((slots[r] * kSetWindows + wl) * kWin + gl) * NC + 4 * c4);
            sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
        }
        float4 *dst = reinterpret_cast<float4 *>(out + gene * out_ld + 4 * c4);
        float4 o = *dst;
        o.x = fmaf(alpha, sum.x, o.x); o.y = fmaf(alpha, sum.y, o.y); o.z = fmaf(alpha, sum.z, o.z); o.w = fmaf(alpha, sum.w, o.w);
        *dst = o;
    }
}

template<int NC, bool BAKED>
cb200_status launch_one(const tb_params &p, int sm_count, cudaStream_t stream) {
    constexpr std::size_t smem = tb_smem_bytes<NC>();
    static_assert(smem <= 232448, "shared memory budget");
    CB200_CUDA_OK(cudaFuncSetAttribute(qcsr_transpose_blocked_kernel<NC, BAKED>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(smem)));
    const std::int64_t sets = (p.windows + set_windows(NC) - 1) / set_windows(NC);
    const std::int64_t units = sets * p.group_count;
    const unsigned grid = static_cast<unsigned>(units < sm_count ? units : sm_count);
    qcsr_transpose_blocked_kernel<NC, BAKED><<<grid, kThreads, smem, stream>>>(p);
    ordered_sum_kernel<NC><<<static_cast<unsigned>(sets * set_windows(NC)), 256, 0, stream>>>(p.partials, p.out, p.out_ld, p.cols, p.windows, p.group_count,
                                                                                             static_cast<std::int64_t>(grid), p.alpha);
    count_launch(2);
    CB200_CUDA_OK(cudaGetLastError());
    return CB200_STATUS_SUCCESS;
}

} // namespace

// status block + one bf16 record of G per group of 256 cells + the runs' sums: a run ends with its window set or with its
// CTA's share of the units, so there are fewer than sets + CTAs of them (kMaxTransposeCtas bounds the grid)
constexpr std::int64_t kMaxTransposeCtas = 256;
static std::uint64_t record_part_bytes(std::int64_t rows, std::int64_t n) {
    const std::int64_t groups = (rows + kRows - 1) / kRows;
    return (static_cast<std::uint64_t>(256 + groups * g_record_bytes(static_cast<int>(n))) + 255u) & ~static_cast<std::uint64_t>(255u);
}
std::uint64_t qcsr_transpose_blocked_workspace_bytes(std::int64_t rows, std::int64_t cols, std::int64_t n) {
    const std::int64_t per_set = n == 32 ? set_windows(32) : set_windows(64);
    const std::int64_t windows = (cols + kWin - 1) / kWin, sets = (windows + per_set - 1) / per_set;
    return record_part_bytes(rows, n) + static_cast<std::uint64_t>(sets + kMaxTransposeCtas) * per_set * kWin * n * sizeof(float);
}

bool qcsr_transpose_blocked_shape_ok(std::int64_t rows, std::int64_t cols, std::int64_t n, int bits) {
    return (bits == 8 || bits == 4) && (n == 32 || n == 64) && rows > 0 && cols > 0 && cols <= 0x7fffffff - kWin;
}

cb200_status launch_qcsr_transpose_blocked(const qcsr_view &x, const dense_args &d, std::int64_t row_begin,
                                           std::int64_t row_end, void *workspace, std::uint64_t workspace_bytes,
                                           const blocked_layout &layout, bool split_products, int sm_count,
                                           cudaStream_t stream, bool *taken) {
    *taken = false;
    if (layout.seg_ptr == nullptr || d.n == 0 || x.cols == 0) return CB200_STATUS_SUCCESS;
    if (layout.baked && (!layout.baked_gene_major || (split_products && layout.entries_lo == nullptr)))
        return CB200_STATUS_SUCCESS; // baked words of the forward tile, or no lo words for the split passes
    if (!qcsr_transpose_blocked_shape_ok(x.rows, x.cols, d.n, x.bits) || d.dense_dtype != CB200_DTYPE_F32) return CB200_STATUS_SUCCESS;
    if (reinterpret_cast<std::uintptr_t>(d.out) % 16u != 0u || (d.out_ld * 4u) % 16u != 0u) return CB200_STATUS_SUCCESS;
    if (workspace == nullptr || workspace_bytes < qcsr_transpose_blocked_workspace_bytes(x.rows, x.cols, d.n) || sm_count > kMaxTransposeCtas)
        return CB200_STATUS_SUCCESS;
    if (reinterpret_cast<std::uintptr_t>(workspace) % 256u != 0u) return CB200_STATUS_SUCCESS;
    const bool row_policy = x.policy == CB200_DECODE_COLUMN_SCALE_ROW_OFFSET;
    // the kernel reads 256 row offsets per group: the last group must not run past the array
    if (row_policy && x.offsets != nullptr && x.rows % kRows != 0) return CB200_STATUS_SUCCESS;
    if (x.row_ptr != layout.src_row_ptr || x.col_idx != layout.src_col_idx || x.packed != layout.src_packed ||
        (layout.baked && (x.scales != layout.src_scales || x.offsets != layout.src_offsets)))
        return fail(CB200_STATUS_STALE_STRUCTURE, "the launch's matrix is not the one the window-blocked copy was built from");

    *taken = true;
    // G' = beta * G', also for an empty row range
    {
        const std::int64_t total = x.cols * d.n;
        const unsigned grid = static_cast<unsigned>(std::min<std::int64_t>((total + 255) / 256, static_cast<std::int64_t>(sm_count) * 8));
        scale_output_kernel<<<grid, 256, 0, stream>>>(d.out, x.cols, static_cast<int>(d.n), d.out_ld, d.beta);
        count_launch();
        CB200_CUDA_OK(cudaGetLastError());
    }
    if (row_end <= row_begin) return CB200_STATUS_SUCCESS;

    int *status = static_cast<int *>(workspace);
    unsigned char *records = static_cast<unsigned char *>(workspace) + 256;
    const std::int64_t group_begin = row_begin / kRows, group_end = (row_end + kRows - 1) / kRows;
    CB200_CUDA_OK(cudaMemsetAsync(status, 0, sizeof(int), stream));

    tb_params p{};
    p.entries = layout.entries; p.seg_ptr = layout.seg_ptr; p.scales = x.scales;
    p.gene_offsets = row_policy ? nullptr : x.offsets; p.row_offsets = row_policy ? x.offsets : nullptr;
    p.records = records; p.out = d.out; p.out_ld = d.out_ld; p.cols = x.cols;
    p.group_begin = group_begin; p.group_count = group_end - group_begin; p.windows = layout.windows;
    p.alpha = d.alpha; p.status = status;
    p.partials = reinterpret_cast<float *>(static_cast<unsigned char *>(workspace) + record_part_bytes(x.rows, d.n));
    // One pass multiplies bf16(value) with bf16(G).  With split products the fp32 product is rebuilt
    // from three passes, hi*hi + hi*lo + lo*hi (v = hi + lo + O(2^-17 v), likewise G): relative error
    // per product about 3 * 2^-17, inside the 1e-4 bound of an fp32 dense operand.  The passes run
    // back to back on the stream, share the record buffer and add into the same G'.
    const int passes = split_products ? 3 : 1;
    int packed_part = -1;
    for (int pass = 0; pass < passes; ++pass) { // (G hi, value hi), (G hi, value lo), (G lo, value hi): G hi is packed once
        const int g_part = pass == 2 ? 1 : 0;
        p.value_part = pass == 1 ? 1 : 0;
        if (layout.baked) p.entries = pass == 1 ? layout.entries_lo : layout.entries; // baked words carry their part
        if (g_part != packed_part) {
            pack_g_kernel<<<static_cast<unsigned>(group_end - group_begin), 256, 0, stream>>>(
                static_cast<const float *>(d.dense), d.dense_ld, static_cast<int>(d.n), row_begin, row_end, group_begin, g_part,
                records);
            count_launch();
            CB200_CUDA_OK(cudaGetLastError());
            packed_part = g_part;
        }
        const cb200_status st = layout.baked ? (d.n == 64 ? launch_one<64, true>(p, sm_count, stream) : launch_one<32, true>(p, sm_count, stream))
                                             : (d.n == 64 ? launch_one<64, false>(p, sm_count, stream) : launch_one<32, false>(p, sm_count, stream));
        if (st != CB200_STATUS_SUCCESS) return st;
    }
    return CB200_STATUS_SUCCESS;
}

} // namespace cb200
