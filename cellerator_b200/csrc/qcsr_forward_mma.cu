// Quantized CSR forward projection on the tensor cores, for callers whose numeric policy allows
// bf16 products (decoded values rounded to bf16, W in bf16, fp32 accumulation):
//     Y[cells, N] = alpha * deq(X)[cells, genes] * W[genes, N] + beta * Y,   N in {32, 64, 128}.
//
// Schedule "tensor_windows": the tensor-core kernel that reads the CSR arrays as they are.  It is
// the fallback of the tensor path when prepare was not handed the matrix (with it, the kernel in
// qcsr_forward_blocked.cu streams a window-blocked copy and is ~3x faster); it beats the exact
// CUDA-core kernels only on dense matrices (>= 10 % stored entries), where prepare selects it.
//
// Why tensor cores at all.  With N = 64 every stored entry costs 64 fp32 FMAs and a 128-byte
// row of W.  On the CUDA cores that is bound by the FMA pipe and by shared-memory reads (one
// 128-byte wavefront per stored entry) at a small fraction of what HBM could deliver.  The tensor
// pipe has the arithmetic to spare even when the matrix is treated as dense: a 256-cell x 128-gene
// window holds ~1,750 stored entries of the 1M x 33,538 matrix and costs sixteen 128 x N x 16 MMAs.
// So the kernel densifies: the stored entries of a window are decoded and scattered, as bf16, into
// a zeroed operand tile in shared memory, and the tile is multiplied against the window's slice
// of W.  Entries are read once, in row order, straight from HBM.
//
// Structure of a CTA (320 threads, one CTA per SM, persistent over groups of 256 cell rows):
//   warps 0-7   one thread per cell row.  A thread brings its row's (gene, code) pairs in as aligned
//               16-byte quartets with cp.async into its own slots of a small ring in shared memory
//               (three quartets ahead, L2 prefetch 128 entries ahead), and per window zeroes its own
//               256-byte row of the A tile, then writes the entries whose gene falls into the window
//               (scale and zero-point of the window's genes come from a table that travels with the
//               W slice).  Because a thread owns its row of the tile, no two threads write the same
//               bytes and nothing is atomic.  A tiles are double buffered.  The same thread later
//               owns TMEM lane = its row and writes that row of Y.  Rows diverge (a warp runs as
//               long as its busiest row in the window) and every quartet is its own L1 request:
//               that, not HBM, bounds this kernel.
//   warp 8      one thread issues, per window, 8 K-steps x 2 row sub-blocks of tcgen05.mma
//               (M = 128, N, K = 16; fp32 accumulators in TMEM, 2 x N columns), commits the window
//               to the "A buffer free" and "W stage free" barriers and, after the last window of a
//               row group, to the "accumulators complete" barrier.
//   warp 9      one thread keeps a ring of W slices filled with bulk async copies.  A small kernel
//               beforehand writes W, per window of 128 genes, transposed into the K-major
//               core-matrix operand layout (8 x 16-byte core matrices, no swizzle) followed by the
//               window's {scale, zero-point} table, so a window is one contiguous record.
// Every barrier wait is bounded; on a time-out a status word is raised, waits stop blocking, and
// the kernel runs to completion and frees its TMEM.  A non-zero status means Y is not valid.
#include "kernels.cuh"
#include "sm100_primitives.cuh"

#include <cuda_bf16.h>

namespace cb200 {
namespace {

#ifndef CB200_MMA_WIN
#define CB200_MMA_WIN 128
#endif
#ifndef CB200_MMA_ROWS
#define CB200_MMA_ROWS 256
#endif
constexpr int kWin = CB200_MMA_WIN;    // genes per window
constexpr int kRows = CB200_MMA_ROWS;  // cell rows per row group
constexpr int kSubBlocks = kRows / 128; // one M = 128 MMA each
constexpr int kProducerWarps = kRows / 32;
constexpr int kProducerThreads = kRows;
constexpr int kThreads = kProducerThreads + 64; // + MMA warp + loader warp
constexpr int kABufBytes = kRows * kWin * 2;    // 64 KB
constexpr int kSubBlockBytes = 128 * kWin * 2;
constexpr int kRowGroupBytes = kWin * 16;       // 8 rows x kWin genes of bf16
constexpr int kPrefetchAhead = 128;             // entries a row thread asks L2 for ahead of its reads
constexpr int kRing = 4;                        // quartets per row thread in the shared-memory ring (power of 2)
constexpr int kRingBytes = kRing * kRows * 24;  // 16 bytes of gene indices + two code words per quartet
static_assert(kWin % 16 == 0 && kRows % 128 == 0, "window geometry");

__host__ __device__ constexpr int record_bytes(int n) { return n * kWin * 2 + kWin * 8; }
// stages of the W ring: as many (up to 4) as fit beside the two A tiles
__host__ __device__ constexpr int w_stages(int n) {
    return (232448 - 512 - 2 * kABufBytes - kRingBytes) / record_bytes(n) >= 4
               ? 4
               : (232448 - 512 - 2 * kABufBytes - kRingBytes) / record_bytes(n);
}

struct mma_params {
    const std::int64_t *row_ptr;
    const std::int64_t *packed_row_ptr;
    const std::int32_t *col_idx;
    const std::uint8_t *packed;
    const float *row_offsets; // per cell row, row-offset policy only
    const unsigned char *records;
    float *y;
    std::int64_t y_ld;
    std::int64_t row_begin, row_end;
    std::int64_t groups;
    int windows;
    float alpha, beta;
    const float *bias;
    int epilogue;
    int *status;
    const std::int32_t *row_order;
};

__device__ __forceinline__ void cp_async_16(std::uint32_t dst, const void *src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_4(std::uint32_t dst, const void *src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template<int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void prefetch_l2(const void *p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
// K-major operand, no swizzle: core matrices of 8 rows x 16 bytes.  The eight core matrices of a
// window's 64 genes sit side by side (LBO = 128 B between K-neighbours), groups of 8 rows follow
// each other every 1,024 B (SBO).
__device__ __forceinline__ std::uint64_t smem_desc(std::uint32_t addr) {
    std::uint64_t d = 0;
    d |= static_cast<std::uint64_t>((addr & 0x3ffffu) >> 4);
    d |= static_cast<std::uint64_t>(128u >> 4) << 16;
    d |= static_cast<std::uint64_t>(static_cast<unsigned>(kRowGroupBytes) >> 4) << 32;
    d |= static_cast<std::uint64_t>(1) << 46; // descriptor version of this architecture
    return d;
}
// W [genes][n] (leading dimension ld) -> one record per window of 64 genes: the n x 64 slice of
// W^T in operand layout (byte offset of (column c, gene e) = (c/8)*1024 + (e/8)*128 + (c%8)*16 +
// (e%8)*2, zero for genes >= cols) followed by 64 x {scale, zero-point}.
__global__ void __launch_bounds__(256) pack_windows_kernel(const __nv_bfloat16 *w, std::int64_t ld, std::int64_t cols, int n,
                                                           const float *scales, const float *offsets, int per_gene_offsets,
                                                           unsigned char *records) {
    const std::int64_t window = blockIdx.x;
    unsigned char *rec = records + window * record_bytes(n);
    __nv_bfloat16 *wt = reinterpret_cast<__nv_bfloat16 *>(rec);
    for (int i = threadIdx.x; i < n * kWin; i += blockDim.x) {
        const int e = i / n, c = i % n; // consecutive threads read consecutive columns of one gene
        const std::int64_t gene = window * kWin + e;
        const __nv_bfloat16 v = gene < cols ? w[gene * ld + c] : __float2bfloat16(0.0f);
        wt[((c >> 3) * kRowGroupBytes + (e >> 3) * 128 + (c & 7) * 16 + (e & 7) * 2) >> 1] = v;
    }
    float2 *table = reinterpret_cast<float2 *>(rec + n * kWin * 2);
    for (int e = threadIdx.x; e < kWin; e += blockDim.x) {
        const std::int64_t gene = window * kWin + e;
        float2 so = make_float2(0.0f, 0.0f);
        if (gene < cols) {
            so.x = scales != nullptr ? scales[gene] : 1.0f;
            so.y = (per_gene_offsets && offsets != nullptr) ? offsets[gene] : 0.0f;
        }
        table[e] = so;
    }
}

template<int BITS, int NC>
__global__ void __launch_bounds__(kThreads, 1) qcsr_fwd_mma_kernel(const mma_params p) {
    constexpr int REC = record_bytes(NC);
    constexpr int STAGES = w_stages(NC);
    constexpr int kTmemCols = kSubBlocks * NC < 32 ? 32 : kSubBlocks * NC; // one accumulator per row sub-block
    constexpr std::uint32_t IDESC = instr_desc(NC);
    extern __shared__ __align__(1024) unsigned char smem[];
    // [2][A tile] | [STAGES][record] | entry ring | barriers | tmem base | abort flag
    std::uint64_t *bars = reinterpret_cast<std::uint64_t *>(smem + 2 * kABufBytes + STAGES * REC + kRingBytes);
    std::uint64_t *a_full = bars;                    // [2]      row threads -> MMA   (one arrival per warp)
    std::uint64_t *a_empty = bars + 2;               // [2]      MMA commit -> row threads
    std::uint64_t *w_full = bars + 4;                // [STAGES] copy engine -> MMA, row threads
    std::uint64_t *w_empty = bars + 4 + STAGES;      // [STAGES] MMA commit -> loader
    std::uint64_t *acc_full = bars + 4 + 2 * STAGES; // MMA commit -> row threads
    std::uint64_t *acc_empty = acc_full + 1;         // row threads -> MMA   (one arrival per warp)
    std::uint32_t *tmem_slot = reinterpret_cast<std::uint32_t *>(acc_empty + 1);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const std::uint32_t smem0 = smem_addr(smem);
    const std::uint32_t wstage0 = smem0 + 2 * kABufBytes;
    const std::uint32_t ring0 = wstage0 + STAGES * REC;

    if (tid == 0) {
        for (int b = 0; b < 2; ++b) {
            bar_init(smem_addr(a_full + b), kProducerWarps);
            bar_init(smem_addr(a_empty + b), 1);
        }
        for (int s = 0; s < STAGES; ++s) {
            bar_init(smem_addr(w_full + s), 1);
            bar_init(smem_addr(w_empty + s), 1);
        }
        bar_init(smem_addr(acc_full), 1);
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

    // Row groups are taken in rounds of gridDim.x; odd rounds run through the CTAs backwards, so that
    // with a length-sorted row order every CTA receives the same mix of long and short groups.
    auto group_of_round = [&](std::int64_t round) -> std::int64_t {
        const std::int64_t pos = (round & 1) ? static_cast<std::int64_t>(gridDim.x) - 1 - blockIdx.x : blockIdx.x;
        return round * gridDim.x + pos;
    };
    const std::int64_t rounds = (p.groups + gridDim.x - 1) / gridDim.x;
    std::int64_t my_groups = 0;
    for (std::int64_t r = 0; r < rounds; ++r) my_groups += group_of_round(r) < p.groups ? 1 : 0;
    const std::int64_t rows_total = p.row_end - p.row_begin;

    if (warp < kProducerWarps) {
        // ================= one thread per cell row =================
        const int sub = tid >> 7, mp = tid & 127;
        const std::uint32_t arow_off = sub * kSubBlockBytes + (mp >> 3) * kRowGroupBytes + (mp & 7) * 16;
        long long q = 0; // windows done by this CTA
        int done_groups = 0;
        for (std::int64_t round = 0; round < rounds; ++round) {
            const std::int64_t group = group_of_round(round);
            if (group >= p.groups) continue;
            const std::int64_t pos = group * kRows + tid;
            std::int64_t row = -1;
            if (pos < rows_total)
                row = p.row_order != nullptr ? static_cast<std::int64_t>(__ldg(p.row_order + pos)) : p.row_begin + pos;

            // ---- the row's entry stream.  Gene indices travel as aligned quartets (16 bytes) counted
            //      from `origin`, the row's first entry rounded down to a multiple of 4; the first `skip`
            //      entries of the first quartet belong to the previous row.  Quartets are copied
            //      asynchronously (cp.async) into this thread's slots of a ring in shared memory,
            //      kRing - 1 quartets ahead of the one being consumed, one commit group per quartet: the
            //      thread never holds an in-flight load in a register it has to move.
            std::int64_t begin = 0, end = 0, pstart = 0;
            float row_offset = 0.0f;
            if (row >= 0) {
                begin = __ldg(p.row_ptr + row);
                end = __ldg(p.row_ptr + row + 1);
                pstart = p.packed_row_ptr != nullptr ? __ldg(p.packed_row_ptr + row) : begin;
                if (p.row_offsets != nullptr) row_offset = __ldg(p.row_offsets + row);
            }
            const bool use_row_offset = p.row_offsets != nullptr;
            const std::int64_t origin = begin & ~static_cast<std::int64_t>(3);
            const int skip = static_cast<int>(begin - origin);
            const int len_rel = static_cast<int>(end - origin); // one past the row's last entry, from origin
            const int row_len = static_cast<int>(end - begin);
            const std::int32_t *cols_o = p.col_idx + origin;
            // codes: the entry at offset i from origin is code number i - skip of the row
            const std::uint8_t *row_lo = p.packed + pstart;
            const std::uint8_t *row_hi = row_lo + (BITS == 8 ? row_len : (row_len + 1) / 2);
            // first code byte of the quartet at offset i4, and the bit offset of its first code in that byte
            auto code_byte = [&](int i4) -> const std::uint8_t * {
                const int first_code = i4 - skip; // negative only in the first quartet
                return row_lo + (BITS == 8 ? first_code : (first_code >> 1));
            };
            auto code_shift = [&](int i4) -> int {
                const int bit = BITS == 8 ? 0 : ((i4 - skip) & 1) * 4;
                return static_cast<int>(reinterpret_cast<std::uintptr_t>(code_byte(i4)) & 3u) * 8 + bit;
            };
            const std::uint32_t ring_cols = ring0 + tid * 16;                       // + slot * kRows * 16
            const std::uint32_t ring_codes = ring0 + kRing * kRows * 16 + tid * 8;  // + slot * kRows * 8
            // Copies quartet number h (offset 4h) into slot h % kRing.  The aligned 4-byte words that
            // hold its codes are copied only if they contain a byte of this row (so nothing outside
            // the matrix is read); one commit group per call, also when there is nothing to copy.
            auto issue = [&](int h) {
                const int i4 = 4 * h;
                if (i4 < len_rel) {
                    const int slot = h & (kRing - 1);
                    cp_async_16(ring_cols + slot * (kRows * 16), cols_o + i4);
                    const std::uintptr_t a = reinterpret_cast<std::uintptr_t>(code_byte(i4));
                    const std::uint8_t *word = reinterpret_cast<const std::uint8_t *>(a & ~static_cast<std::uintptr_t>(3));
                    if (word + 4 > row_lo && word < row_hi) cp_async_4(ring_codes + slot * (kRows * 8), word);
                    if (code_shift(i4) != 0 && word + 8 > row_lo && word + 4 < row_hi)
                        cp_async_4(ring_codes + slot * (kRows * 8) + 4, word + 4);
                    // pull the row's data into L2 well ahead (one 128-byte line of gene indices every 32
                    // entries, one of codes every 1024 / BITS), never past the row's end
                    if ((i4 & 31) == 0 && i4 + kPrefetchAhead < len_rel) prefetch_l2(cols_o + i4 + kPrefetchAhead);
                    if ((i4 & (1024 / BITS - 1)) == 0 && i4 - skip + kPrefetchAhead < row_len)
                        prefetch_l2(row_lo + (i4 - skip + kPrefetchAhead) * BITS / 8);
                }
                cp_async_commit();
            };
            for (int i = 32; i < kPrefetchAhead && i < len_rel; i += 32) prefetch_l2(cols_o + i);
            for (int i = 1024 / BITS; i < kPrefetchAhead && i < row_len; i += 1024 / BITS) prefetch_l2(row_lo + i * BITS / 8);
            int head = 0; // quartet being consumed; quartets head .. head + kRing - 1 are in the ring or on their way
            cp_async_wait<0>(); // nothing of the previous row is still on its way into the slots
#pragma unroll
            for (int h = 0; h < kRing; ++h) issue(h);

            for (int w = 0; w < p.windows; ++w, ++q) {
                const std::uint32_t b = static_cast<std::uint32_t>(q & 1);
                const int s = static_cast<int>(q % STAGES);
                bar_wait(smem_addr(a_empty + b), static_cast<std::uint32_t>(((q >> 1) & 1) ^ 1), abort_flag);
                bar_wait(smem_addr(w_full + s), static_cast<std::uint32_t>((q / STAGES) & 1), abort_flag);
                unsigned char *arow = smem + b * kABufBytes + arow_off;
#pragma unroll
                for (int kc = 0; kc < kWin / 8; ++kc) *reinterpret_cast<uint4 *>(arow + kc * 128) = make_uint4(0u, 0u, 0u, 0u);
                const float2 *table = reinterpret_cast<const float2 *>(smem + 2 * kABufBytes + s * REC + NC * kWin * 2);
                const int wstart = w * kWin, wend = wstart + kWin;
                // An entry is written in the window its gene falls into; a quartet is left behind once
                // its last entry lies before the window's end.  The four table reads of a quartet are
                // issued together (entries outside the window read slot 0 and store nothing).
                constexpr unsigned CM = (1u << BITS) - 1u;
                while (true) {
                    cp_async_wait<kRing - 1>(); // quartet `head` has landed
                    const int i4 = 4 * head;
                    const int slot = head & (kRing - 1);
                    int4 g;
                    unsigned lo, hi;
                    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                                 : "=r"(g.x), "=r"(g.y), "=r"(g.z), "=r"(g.w)
                                 : "r"(ring_cols + slot * (kRows * 16)));
                    asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];" : "=r"(lo), "=r"(hi) : "r"(ring_codes + slot * (kRows * 8)));
                    const unsigned c0 = __funnelshift_r(lo, hi, code_shift(i4));
                    // slots of the quartet that are entries of this row: [skip - i4, len_rel - i4) cut to 0..4
                    const int first = max(skip - i4, 0), last = min(len_rel - i4, 4);
                    const unsigned g0 = static_cast<unsigned>(g.x - wstart), g1 = static_cast<unsigned>(g.y - wstart);
                    const unsigned g2 = static_cast<unsigned>(g.z - wstart), g3 = static_cast<unsigned>(g.w - wstart);
                    const bool in0 = g0 < static_cast<unsigned>(kWin) && first <= 0 && last > 0;
                    const bool in1 = g1 < static_cast<unsigned>(kWin) && first <= 1 && last > 1;
                    const bool in2 = g2 < static_cast<unsigned>(kWin) && first <= 2 && last > 2;
                    const bool in3 = g3 < static_cast<unsigned>(kWin) && last > 3;
                    const float2 t0 = table[in0 ? g0 : 0u], t1 = table[in1 ? g1 : 0u];
                    const float2 t2 = table[in2 ? g2 : 0u], t3 = table[in3 ? g3 : 0u];
                    const float v0 = fmaf(static_cast<float>(c0 & CM), t0.x, use_row_offset ? row_offset : t0.y);
                    const float v1 = fmaf(static_cast<float>((c0 >> BITS) & CM), t1.x, use_row_offset ? row_offset : t1.y);
                    const float v2 = fmaf(static_cast<float>((c0 >> (2 * BITS)) & CM), t2.x, use_row_offset ? row_offset : t2.y);
                    const float v3 = fmaf(static_cast<float>((c0 >> (3 * BITS)) & CM), t3.x, use_row_offset ? row_offset : t3.y);
                    if (in0) *reinterpret_cast<__nv_bfloat16 *>(arow + ((g0 >> 3) << 7) + ((g0 & 7u) << 1)) = __float2bfloat16_rn(v0);
                    if (in1) *reinterpret_cast<__nv_bfloat16 *>(arow + ((g1 >> 3) << 7) + ((g1 & 7u) << 1)) = __float2bfloat16_rn(v1);
                    if (in2) *reinterpret_cast<__nv_bfloat16 *>(arow + ((g2 >> 3) << 7) + ((g2 & 7u) << 1)) = __float2bfloat16_rn(v2);
                    if (in3) *reinterpret_cast<__nv_bfloat16 *>(arow + ((g3 >> 3) << 7) + ((g3 & 7u) << 1)) = __float2bfloat16_rn(v3);
                    // move on only if the whole quartet is this row's and its last entry lies before the window's end
                    if (last < 4 || g.w >= wend) break;
                    issue(head + kRing); // refills the slot just read
                    ++head;
                }
                fence_async_proxy(); // the tile was written with ordinary stores, the MMA reads it through the async proxy
                __syncwarp();
                if (lane == 0) bar_arrive(smem_addr(a_full + b));
            }

            // ---- this thread's row of Y: TMEM lane = row within the sub-block
            bar_wait(smem_addr(acc_full), static_cast<std::uint32_t>(done_groups & 1), abort_flag);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int h = 0; h < NC / 32; ++h) {
                float v[32];
                tmem_ld32(tmem_base + (static_cast<std::uint32_t>((warp & 3) * 32) << 16) + sub * NC + h * 32, v);
                if (row >= 0) {
                    float *out = p.y + row * p.y_ld + h * 32;
                    store_row32(out, v, p.alpha, p.beta, p.bias, h * 32, p.epilogue);
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) bar_arrive(smem_addr(acc_empty));
            ++done_groups;
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
                            mma_bf16(tmem_base + sb * NC, smem_desc(a_tile + sb * kSubBlockBytes + kk * 256), db, IDESC,
                                     w > 0 || kk > 0);
                    }
                    mma_commit(smem_addr(a_empty + b));
                    mma_commit(smem_addr(w_empty + s));
                    if (w == p.windows - 1) mma_commit(smem_addr(acc_full));
                }
                __syncwarp();
            }
        }
    } else if (lane == 0) {
        // ================= W loader =================
        const long long total = my_groups * p.windows;
        for (long long q = 0; q < total; ++q) {
            const int s = static_cast<int>(q % STAGES);
            bar_wait(smem_addr(w_empty + s), static_cast<std::uint32_t>(((q / STAGES) & 1) ^ 1), abort_flag);
            bar_arrive_expect_tx(smem_addr(w_full + s), REC);
            bulk_copy_g2s(wstage0 + s * REC, p.records + static_cast<std::size_t>(q % p.windows) * REC, REC, smem_addr(w_full + s));
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

template<int NC> constexpr std::size_t mma_smem_bytes() {
    return 2 * kABufBytes + w_stages(NC) * record_bytes(NC) + kRingBytes + (6 + 2 * w_stages(NC)) * sizeof(std::uint64_t) + 16;
}

template<int BITS, int NC>
cb200_status launch_one(const mma_params &p, int sm_count, cudaStream_t stream) {
    constexpr std::size_t smem = mma_smem_bytes<NC>();
    CB200_CUDA_OK(cudaFuncSetAttribute(qcsr_fwd_mma_kernel<BITS, NC>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(smem)));
    const unsigned grid = static_cast<unsigned>(p.groups < sm_count ? p.groups : sm_count);
    qcsr_fwd_mma_kernel<BITS, NC><<<grid, kThreads, smem, stream>>>(p);
    count_launch();
    CB200_CUDA_OK(cudaGetLastError());
    return CB200_STATUS_SUCCESS;
}

template<int BITS>
cb200_status launch_n(const mma_params &p, int n, int sm_count, cudaStream_t stream) {
    switch (n) {
    case 32: return launch_one<BITS, 32>(p, sm_count, stream);
    case 64: return launch_one<BITS, 64>(p, sm_count, stream);
    default: return launch_one<BITS, 128>(p, sm_count, stream);
    }
}

} // namespace

std::uint64_t qcsr_mma_workspace_bytes(std::int64_t cols, std::int64_t n) {
    const std::int64_t windows = (cols + kWin - 1) / kWin;
    return static_cast<std::uint64_t>(256 + windows * record_bytes(static_cast<int>(n)));
}

bool qcsr_forward_mma_supported(const qcsr_view &x, const dense_args &d) {
    if (x.bits != 8 && x.bits != 4) return false;
    if (d.n != 32 && d.n != 64 && d.n != 128) return false;
    if (d.dense_dtype != CB200_DTYPE_BF16) return false;
    if (x.cols <= 0 || x.cols > 0x7fffffff - kWin) return false;
    if (x.bits == 4 && x.packed_row_ptr == nullptr) return false;
    if (reinterpret_cast<std::uintptr_t>(x.col_idx) % 16u != 0u) return false; // aligned 16-byte index loads
    if (reinterpret_cast<std::uintptr_t>(x.packed) % 8u != 0u) return false;   // aligned code words
    if (reinterpret_cast<std::uintptr_t>(d.out) % 16u != 0u || (d.out_ld * 4u) % 16u != 0u) return false;
    return true;
}

cb200_status launch_qcsr_forward_mma(const qcsr_view &x, const dense_args &d, std::int64_t row_begin,
                                     std::int64_t row_end, void *workspace, std::uint64_t workspace_bytes,
                                     const std::int32_t *row_order, int sm_count, cudaStream_t stream, bool *taken) {
    *taken = false;
    if (!qcsr_forward_mma_supported(x, d) || row_end <= row_begin) return CB200_STATUS_SUCCESS;
    if (workspace == nullptr || workspace_bytes < qcsr_mma_workspace_bytes(x.cols, d.n)) return CB200_STATUS_SUCCESS;
    if (reinterpret_cast<std::uintptr_t>(workspace) % 256u != 0u) return CB200_STATUS_SUCCESS;

    int *status = static_cast<int *>(workspace);
    unsigned char *records = static_cast<unsigned char *>(workspace) + 256;
    const int windows = static_cast<int>((x.cols + kWin - 1) / kWin);
    const bool row_policy = x.policy == CB200_DECODE_COLUMN_SCALE_ROW_OFFSET;
    CB200_CUDA_OK(cudaMemsetAsync(status, 0, sizeof(int), stream));
    pack_windows_kernel<<<static_cast<unsigned>(windows), 256, 0, stream>>>(static_cast<const __nv_bfloat16 *>(d.dense), d.dense_ld,
                                                                              x.cols, static_cast<int>(d.n), x.scales, x.offsets,
                                                                              row_policy ? 0 : 1, records);
    count_launch();
    CB200_CUDA_OK(cudaGetLastError());

    mma_params p{};
    p.row_ptr = x.row_ptr; p.packed_row_ptr = x.packed_row_ptr; p.col_idx = x.col_idx; p.packed = x.packed;
    p.row_offsets = row_policy ? x.offsets : nullptr; p.records = records; p.y = d.out; p.y_ld = d.out_ld;
    p.row_begin = row_begin; p.row_end = row_end; p.groups = (row_end - row_begin + kRows - 1) / kRows;
    p.windows = windows; p.alpha = d.alpha; p.beta = d.beta; p.bias = d.bias; p.epilogue = d.epilogue; p.status = status;
    // a row order describes the whole matrix; a partial row range runs in natural order
    p.row_order = (row_begin == 0 && row_end == x.rows) ? row_order : nullptr;
    *taken = true;
    if (x.bits == 8) return launch_n<8>(p, static_cast<int>(d.n), sm_count, stream);
    return launch_n<4>(p, static_cast<int>(d.n), sm_count, stream);
}

} // namespace cb200
