// Quantized CSR forward projection on the tensor cores from dense tiles of CODES kept at prepare
// (schedule "tensor_codes"):
//     Y[cells, N] = alpha * deq(X)[cells, genes] * W[genes, N] + beta * Y,   N in {32, 64, 128},
// for matrices dense enough that a dense tile is the smaller representation: 4-bit codes at 8 % density or more
// (the 4,000-gene, 17 %-dense configuration: 0.77 bytes per dense slot as CSR, 1 byte per slot here).
// Reference counterpart: csr_spmm_fwd over dequantised values (src/compute/sparse/ops/base_sparse.cu); the
// reference keeps no such copy, its prepared_operation only has room for one (persistent_kernel_state,
// operation_core.hh:126-129).
//
// What is kept.  For every group of 256 cells and every half window of 64 genes one 16 KB stage: a byte per
// (cell, gene), 0 where nothing is stored and code + 240 where a code is (a 4-bit code leaves room for that).
// The matrix stays QUANTIZED: the per-gene scale and zero-point are not in the copy.  They are applied at
// every launch, in registers, on the way from the byte to the fp16 operand the MMA reads, so new scales or
// offsets need no new prepare; only new codes (a new structure or value generation) do.  Against the decoded
// tiles of "tensor_dense" (2 bytes per slot, values baked in) a launch moves half the bytes.
//
// A CTA (896 threads, one per SM, row groups dealt round-robin).  Shared memory holds only what the copy engine
// brings: the decoded operand never touches it.  The decode warps write it into TENSOR MEMORY (tcgen05.st), next to
// the accumulators, and the MMA reads its A operand from there; shared-memory bandwidth, which bounds a kernel that
// stores decoded tiles to shared memory and lets the MMA read them back (16 KB in, 32 KB stored, 32 KB read per
// half window), is left to the copies and the W operand.
//   warps 0-7    write Y: a warp reads its 32 rows of the group (TMEM lane = row within the 128-row sub-block) 32
//                columns at a time, turns the block in a 4 KB shared-memory buffer so that 8 lanes write a row's
//                128 contiguous bytes, and hands the accumulators (256 columns) back as soon as they are in registers;
//   warps 8-9    one thread each issues the MMAs of one row sub-block: per window eight K = 16 steps, A from tensor
//                memory (row = lane, two fp16 per 32-bit column), B = the window's slice of W from shared memory;
//   warp 10      one thread feeds the W ring with bulk async copies (W re-laid per window into the operand
//                layout, fp16, by a small kernel before this one);
//   warp 11      one thread feeds the ring of code stages with bulk async copies (16 KB of codes and, behind them, the
//                half window's 256 bytes of {scale, zero-point} pairs and the word that allows the mask-free decode);
//   warps 12-27  decode: a warp may write the 32 tensor-memory lanes (warp mod 4), so it owns those rows of both
//                sub-blocks; the four warps of a lane quarter split a window into its two half windows and each half
//                into two pairs of 16-gene chunks, so a warp visits one code stage per window (one wait, one
//                hand-back) and decodes two chunks of it (the stage is stored chunk-major: its 16-byte loads and the
//                table's broadcast loads run without bank conflicts).  Per pair of codes a byte permute (byte ->
//                fp16 1024 + byte), a subtraction of 1264 (exact: the code, or -240 for an empty slot), a fused
//                multiply-add with the genes' {scale, zero-point} held in registers as fp16 pairs -- with max(0, .)
//                where the half window's genes allow it (pack_codes_operands_kernel), else followed by a compare that
//                gives the "something stored" mask and an AND; then one 8-column store per row into one of two operand
//                stages (a window each) of tensor memory.  The stage goes back to the copy engine behind the last use
//                of its values and a fence.
// Tensor memory: columns 0-255 accumulators (2 sub-blocks x N), 256-511 two operand stages of 2 x 64 columns.
// Every barrier wait is bounded; a role whose wait ran out stops, the loaders wait for their copies in flight and
// the MMA warp for its MMAs before the CTA frees tensor memory.  A non-zero status word means Y is not valid.
#include "blocked_tile.cuh"

#include <algorithm>

namespace cb200 {
namespace {

constexpr int kCodeStageBytes = kRows * 64;              // 16 KB: 256 rows x 64 genes, one byte per slot
constexpr int kPairTableBytes = 32 * 8;                  // a half window's 32 gene pairs x {scale pair, offset pair} as fp16
constexpr int kTableBytes = kPairTableBytes + 16;        // + a word that says whether the half window may be decoded without masks
constexpr int kPresentBias = 240;                        // a stored code is kept as code + 240 (4-bit codes: 240..255), nothing stored as 0
constexpr int kCodeSlotBytes = kCodeStageBytes + kTableBytes; // what one stage of the ring holds
constexpr int kChunkPlaneBytes = kRows * 16;             // a stage is [16-gene chunk][row][16 codes]
constexpr int kMaxCodeStages = 8;
constexpr int kOperandStages = 2;                        // decoded windows in tensor memory
constexpr int kOperandCols = kSubBlocks * 64;            // columns of one: per row sub-block 128 fp16 = 64 columns
constexpr int kOperandCol0 = 256;                        // the accumulators own the columns below
constexpr int kTmemColumns = 512;
constexpr int kDecodeWarps = 16;
constexpr int kCodeIssuers = kSubBlocks; // MMA-issuing warps: one per 128-row sub-block
constexpr int kCodesThreads = (kEpilogueWarps + kCodeIssuers + 2 + kDecodeWarps) * 32; // 896
static_assert(kSubBlocks * 128 <= kOperandCol0 && kOperandCol0 + kOperandStages * kOperandCols <= kTmemColumns, "tensor memory budget");
static_assert(kDecodeWarps == 16 && kRows == 256,
              "decode warp = (lane quarter of tensor memory it may write, 16-gene chunk); it decodes that quarter of both row sub-blocks");
__host__ __device__ constexpr int codes_w_stages(int n) { return n * kWin * 2 * 3 <= 98304 ? 3 : 98304 / (n * kWin * 2); }
constexpr int kTurnBytes = 32 * 32 * 4;                  // an epilogue warp's 32 rows x 32 columns on their way from row-per-lane to row-per-8-lanes
constexpr int kTurnRegionBytes = kEpilogueWarps * kTurnBytes;
__host__ __device__ constexpr int codes_code_stages(int n) {
    return (232448 - 512 - kTurnRegionBytes - codes_w_stages(n) * n * kWin * 2) / kCodeSlotBytes > kMaxCodeStages
               ? kMaxCodeStages
               : (232448 - 512 - kTurnRegionBytes - codes_w_stages(n) * n * kWin * 2) / kCodeSlotBytes;
}
static_assert(codes_w_stages(128) == 3 && codes_code_stages(128) == 6, "three W windows and six code stages in flight at N = 128");

// One CTA per (group, window) segment of the window-blocked copy (code words): a byte tile in shared memory,
// 0 = nothing stored, code + 240 otherwise; written out as two stages of 64 genes, each [16-gene chunk][row][16 codes].
__global__ void __launch_bounds__(512) bytify_kernel(const std::uint32_t *entries, const std::int64_t *seg_ptr, int windows,
                                                     unsigned char *stages) {
    extern __shared__ __align__(16) unsigned char tile[]; // [256 rows][128 genes]
    const std::int64_t seg = blockIdx.x;
    const int tid = threadIdx.x;
    for (int i = tid * 16; i < kRows * kWin; i += 512 * 16) *reinterpret_cast<uint4 *>(tile + i) = make_uint4(0u, 0u, 0u, 0u);
    __syncthreads();
    const std::int64_t lo = seg_ptr[seg], hi = seg_ptr[seg + 1];
    for (std::int64_t i = lo + tid; i < hi; i += 512) {
        const std::uint32_t e = entries[i];
        if (static_cast<int>(e) < 0) continue; // padding
        const std::uint32_t off = ((e >> 15) & 0x7fffu) << 1; // byte position in the fp16 operand tile: gives the row back
        const int row = static_cast<int>(((off / kSubBlockBytes) << 7) | (((off >> 10) & 15u) << 3) | ((off >> 7) & 7u));
        tile[row * kWin + ((e >> 8) & (kWin - 1))] = static_cast<unsigned char>((e & 0xffu) + kPresentBias);
    }
    __syncthreads();
    unsigned char *out = stages + static_cast<std::size_t>(seg) * (2 * kCodeStageBytes);
    for (int i = tid * 16; i < kRows * kWin; i += 512 * 16) {
        const int row = i / kWin, gene = i % kWin; // 16 consecutive genes of one row
        *reinterpret_cast<uint4 *>(out + (gene >> 6) * kCodeStageBytes + ((gene & 63) >> 4) * kChunkPlaneBytes + row * 16) =
            *reinterpret_cast<const uint4 *>(tile + i);
    }
    (void)windows;
}

// Per window: the W slice in operand layout (pack_windows_kernel's part, grid.y column groups) and, by the blocks of
// column group 0, the window's 64 gene pairs of {fp16(scale * s), fp16(offset * s)}, s = operand_scale(bound of the
// decoded magnitudes): table[pair] = {scales of genes 2p and 2p+1, offsets of genes 2p and 2p+1}; genes past the
// matrix get zeros.
__global__ void __launch_bounds__(256) pack_codes_operands_kernel(const __nv_bfloat16 *w, std::int64_t ld, std::int64_t cols, int n,
                                                                  const float *scales, const float *offsets, unsigned char *records,
                                                                  const unsigned *w_absmax, const unsigned *bound_bits, unsigned char *table) {
    const std::int64_t window = blockIdx.x;
    __half *rec = reinterpret_cast<__half *>(records + window * record_bytes(n));
    const float ws = operand_scale(__uint_as_float(*w_absmax));
    const int group_cols = n / static_cast<int>(gridDim.y), c_first = static_cast<int>(blockIdx.y) * group_cols;
    // a thread makes one 16-byte piece: a column's values of eight consecutive genes; consecutive threads take consecutive
    // columns, so that their loads of a gene's row and their pieces are contiguous
    for (int item = threadIdx.x; item < group_cols * (kWin / 8); item += blockDim.x) {
        const int e8 = item / group_cols, c = c_first + item % group_cols;
        std::uint32_t packed[4];
#pragma unroll
        for (int j = 0; j < 8; j += 2) {
            float v[2];
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                const std::int64_t gene = window * kWin + e8 * 8 + j + k;
                v[k] = gene < cols ? __bfloat162float(w[gene * ld + c]) : 0.0f;
            }
            const __half2 h = __floats2half2_rn(v[0] * ws, v[1] * ws);
            packed[j >> 1] = *reinterpret_cast<const std::uint32_t *>(&h);
        }
        *reinterpret_cast<uint4 *>(reinterpret_cast<unsigned char *>(rec) + (c >> 3) * kRowGroupBytes + e8 * 128 + (c & 7) * 16) =
            make_uint4(packed[0], packed[1], packed[2], packed[3]);
    }
    if (blockIdx.y != 0 || threadIdx.x >= kWin / 2) return; // warps 0 and 1: the pairs of the window's first and second half
    const std::int64_t pair = window * (kWin / 2) + threadIdx.x;
    const float s = operand_scale(__uint_as_float(*bound_bits));
    float sc[2], of[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const std::int64_t g = 2 * pair + i;
        sc[i] = g < cols ? (scales != nullptr ? scales[g] : 1.0f) * s : 0.0f;
        of[i] = g < cols && offsets != nullptr ? offsets[g] * s : 0.0f;
    }
    const __half2 s2 = __floats2half2_rn(sc[0], sc[1]), o2 = __floats2half2_rn(of[0], of[1]);
    unsigned char *half_table = table + (window * 2 + (threadIdx.x >> 5)) * kTableBytes;
    reinterpret_cast<uint2 *>(half_table)[threadIdx.x & 31] = make_uint2(*reinterpret_cast<const unsigned *>(&s2), *reinterpret_cast<const unsigned *>(&o2));
    // Without masks a slot decodes to max(0, (byte - 240) * scale + offset): right for a stored code when the value cannot
    // be negative (scale >= 0 and offset >= 0, as the fp16 values the kernel multiplies) and right for an empty slot
    // (byte 0) when offset - 240 * scale <= 0.  One gene that fails makes its half window take the masked form.
    bool plain = true;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const float sh = i == 0 ? __low2float(s2) : __high2float(s2), oh = i == 0 ? __low2float(o2) : __high2float(o2);
        plain = plain && sh >= 0.0f && oh >= 0.0f && oh <= static_cast<float>(kPresentBias) * sh;
    }
    const bool all_plain = __all_sync(0xffffffffu, plain);
    if ((threadIdx.x & 31) == 0) *reinterpret_cast<std::uint32_t *>(half_table + kPairTableBytes) = all_plain ? 1u : 0u;
}

struct codes_params {
    const unsigned char *stages;  // [group][window][half][16 KB]
    const unsigned char *records; // W windows in operand layout (fp16), record_bytes(N) apart
    const unsigned char *table;   // per half window kTableBytes: 32 gene pairs of {scale pair, offset pair} as fp16, then the "no masks needed" word
    float *y;
    std::int64_t y_ld;
    std::int64_t row_end; // rows >= row_end are computed but not written
    std::int64_t group_begin, group_end;
    int windows;
    float alpha, beta;
    const float *bias;
    int epilogue;
    int *status;
    const unsigned *w_absmax;    // largest |W| of this launch as float bits
    const unsigned *value_bound; // bound of the decoded magnitudes as float bits
};

// D[tmem_d] (+)= A[tmem_a] * B[descriptor]: the A operand (128 rows x 16 fp16, row = lane, two values per 32-bit
// column) is read from tensor memory, B (N x 16, K-major) from shared memory.
__device__ __forceinline__ void mma_f16_a_in_tmem(std::uint32_t tmem_d, std::uint32_t tmem_a, std::uint32_t desc_b_lo, std::uint32_t desc_b_hi,
                                                  std::uint32_t idesc, std::uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\tsetp.ne.b32 p, %4, 0;\n\tmov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %5, p;\n\t}"
        :
        : "r"(tmem_d), "r"(tmem_a), "r"(desc_b_lo), "r"(desc_b_hi), "r"(accumulate), "r"(idesc)
        : "memory");
}
// Eight 32-bit columns of this thread's lane of tensor memory (lane = 32 * (warp mod 4) + lane of the warp).
__device__ __forceinline__ void tmem_st8(std::uint32_t taddr, const std::uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]),
                 "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}

template<int NC>
__global__ void __launch_bounds__(kCodesThreads, 1) qcsr_fwd_codes_kernel(const codes_params p) {
    constexpr int SC = codes_code_stages(NC), SA = kOperandStages, SB = codes_w_stages(NC);
    constexpr int WREC = NC * kWin * 2;
    constexpr int REC = record_bytes(NC);
    constexpr std::uint32_t IDESC = instr_desc(NC, true); // fp16 operands
    extern __shared__ __align__(1024) unsigned char smem[];
    // [SB][W window] | [SC][code stage + gene table] | [epilogue warp][32 x 32 floats] | barriers | tmem slot | abort
    unsigned char *turn0 = smem + SB * WREC + SC * kCodeSlotBytes;
    std::uint64_t *bars = reinterpret_cast<std::uint64_t *>(turn0 + kTurnRegionBytes);
    std::uint64_t *c_full = bars;              // [SC] copy engine -> decode warps
    std::uint64_t *c_empty = c_full + SC;      // [SC] decode warps -> code loader (one arrival per warp)
    std::uint64_t *a_full = c_empty + SC;      // [SA] decode warps -> MMA (one arrival per warp)
    std::uint64_t *a_empty = a_full + SA;      // [SA] MMA commit -> decode warps
    std::uint64_t *b_full = a_empty + SA;      // [SB] copy engine -> MMA
    std::uint64_t *b_empty = b_full + SB;      // [SB] MMA commit -> W loader
    std::uint64_t *acc_full = b_empty + SB;    // MMA commit -> epilogue warps
    std::uint64_t *acc_empty = acc_full + 1;   // epilogue warps -> MMA (one arrival per warp)
    std::uint64_t *mma_drain = acc_empty + 1;  // [issuers] an MMA warp's own: everything it issued has finished
    std::uint32_t *tmem_slot = reinterpret_cast<std::uint32_t *>(mma_drain + kCodeIssuers);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const std::uint32_t bstage0 = smem_addr(smem);
    unsigned char *cstage0 = smem + SB * WREC;

    if (tid == 0) {
        for (int s = 0; s < SC; ++s) {
            bar_init(smem_addr(c_full + s), 1);
            bar_init(smem_addr(c_empty + s), kDecodeWarps / 2); // the warps of the stage's half window
        }
        for (int s = 0; s < SA; ++s) {
            bar_init(smem_addr(a_full + s), kDecodeWarps);
            bar_init(smem_addr(a_empty + s), kCodeIssuers); // one commit per MMA warp
        }
        for (int s = 0; s < SB; ++s) {
            bar_init(smem_addr(b_full + s), 1);
            bar_init(smem_addr(b_empty + s), kCodeIssuers);
        }
        bar_init(smem_addr(acc_full), kCodeIssuers);
        bar_init(smem_addr(acc_empty), kEpilogueWarps);
        for (int i = 0; i < kCodeIssuers; ++i) bar_init(smem_addr(mma_drain + i), 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)), "r"(kTmemColumns)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const std::uint32_t tmem_base = *tmem_slot;

    const std::int64_t first_group = p.group_begin + blockIdx.x;
    const int my_groups = first_group < p.group_end ? static_cast<int>((p.group_end - first_group + gridDim.x - 1) / gridDim.x) : 0;
    const int halves = p.windows * (kWin / 64);

    if (warp < kEpilogueWarps) {
        // ================= a warp reads its 32 rows (TMEM lane = row within the sub-block) 32 columns at a time and turns
        // them in shared memory, so that 8 lanes write the 128 contiguous bytes of a row: a store touches 4 lines instead
        // of 32.  16-byte chunk c of row r sits at chunk c ^ (r & 7): stores (a lane = a row) and loads (8 lanes = a row)
        // both spread over all banks =================
        const int sub = tid >> 7;
        unsigned char *turn = turn0 + warp * kTurnBytes;
        const int chunk = lane & 7, row_of_lane = lane >> 3; // on the way out: this lane's 4 columns, and its row among the 4 of a store
        // both operands were stored times powers of two (fp16 range): the result is divided by them again
        const float alpha = p.alpha / (operand_scale(__uint_as_float(__ldg(p.w_absmax))) * operand_scale(__uint_as_float(__ldg(p.value_bound))));
        for (int gi = 0; gi < my_groups; ++gi) {
            const std::int64_t row0 = (first_group + static_cast<std::int64_t>(gi) * gridDim.x) * kRows + sub * 128 + (warp & 3) * 32;
            if (bar_wait_sleeping(smem_addr(acc_full), static_cast<std::uint32_t>(gi & 1), abort_flag, 400u)) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
            for (int h = 0; h < NC / 32; ++h) {
                {
                    float v[32];
                    tmem_ld32(tmem_base + (static_cast<std::uint32_t>((warp & 3) * 32) << 16) + sub * NC + h * 32, v);
                    if (h == NC / 32 - 1) { // the accumulators are in registers: the next group's MMAs may start
                        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                        __syncwarp();
                        if (lane == 0) bar_arrive(smem_addr(acc_empty));
                    }
#pragma unroll
                    for (int c = 0; c < 8; ++c)
                        *reinterpret_cast<float4 *>(turn + lane * 128 + ((c ^ (lane & 7)) << 4)) =
                            make_float4(v[4 * c] * alpha, v[4 * c + 1] * alpha, v[4 * c + 2] * alpha, v[4 * c + 3] * alpha);
                }
                __syncwarp();
                float4 t[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int r = 4 * i + row_of_lane;
                    t[i] = *reinterpret_cast<const float4 *>(turn + r * 128 + ((chunk ^ (r & 7)) << 4));
                }
                __syncwarp(); // the next 32 columns may overwrite the turn buffer
                float *out = p.y + (row0 + row_of_lane) * p.y_ld + h * 32 + 4 * chunk;
                const std::int64_t rows_left = p.row_end - row0 - row_of_lane; // row 4 * i + row_of_lane is written when 4 * i < rows_left
                if (p.beta != 0.0f) {
                    float4 o[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        o[i] = 4 * i < rows_left ? *reinterpret_cast<const float4 *>(out + static_cast<std::int64_t>(4 * i) * p.y_ld) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        t[i].x = fmaf(p.beta, o[i].x, t[i].x); t[i].y = fmaf(p.beta, o[i].y, t[i].y);
                        t[i].z = fmaf(p.beta, o[i].z, t[i].z); t[i].w = fmaf(p.beta, o[i].w, t[i].w);
                    }
                }
                if (p.epilogue != CB200_EPILOGUE_NONE) {
                    const int col = h * 32 + 4 * chunk;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        t[i].x = finish_output(t[i].x, p.bias, col, p.epilogue); t[i].y = finish_output(t[i].y, p.bias, col + 1, p.epilogue);
                        t[i].z = finish_output(t[i].z, p.bias, col + 2, p.epilogue); t[i].w = finish_output(t[i].w, p.bias, col + 3, p.epilogue);
                    }
                }
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    if (4 * i < rows_left) *reinterpret_cast<float4 *>(out + static_cast<std::int64_t>(4 * i) * p.y_ld) = t[i];
            }
        }
    } else if (warp < kEpilogueWarps + kCodeIssuers) {
        // ================= MMA issuers: warp sb issues the MMAs of row sub-block sb (its own accumulator columns).  One
        // issuing thread is held to the rate of the tensor pipe and then spends half as long again on commits and waits
        // with the pipe running dry; two threads issue a window's MMAs side by side =================
        const int sb = warp - kEpilogueWarps;
        const std::uint64_t b_desc0 = smem_desc(bstage0);
        const std::uint32_t b_lo0 = static_cast<std::uint32_t>(b_desc0), b_hi = static_cast<std::uint32_t>(b_desc0 >> 32);
        int sa = 0, s = 0;
        std::uint32_t pa = 0, pb = 0;
        bool dead = false;
        for (int g = 0; g < my_groups && !dead; ++g) {
            if (bar_wait(smem_addr(acc_empty), static_cast<std::uint32_t>((g & 1) ^ 1), abort_flag)) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            for (int w = 0; w < p.windows; ++w) {
                if (bar_wait(smem_addr(b_full + s), pb, abort_flag) || bar_wait(smem_addr(a_full + sa), pa, abort_flag)) { dead = true; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (lane == 0) {
                    const std::uint32_t a_col = tmem_base + kOperandCol0 + sa * kOperandCols;
                    const std::uint32_t b_lo = b_lo0 + static_cast<std::uint32_t>((s * WREC) >> 4);
                    const std::uint32_t fresh = w != 0 ? 1u : 0u; // the group's first MMAs overwrite the accumulators
#pragma unroll
                    for (int kk = 0; kk < kWin / 16; ++kk)
                        mma_f16_a_in_tmem(tmem_base + sb * NC, a_col + sb * 64 + kk * 8, b_lo + kk * 16, b_hi, IDESC, kk == 0 ? fresh : 1u);
                    mma_commit(smem_addr(a_empty + sa));
                    mma_commit(smem_addr(b_empty + s));
                    if (w == p.windows - 1) mma_commit(smem_addr(acc_full));
                }
                __syncwarp();
                sa ^= 1;
                if (sa == 0) pa ^= 1u;
                if (++s == SB) { s = 0; pb ^= 1u; }
            }
        }
        if (*abort_flag != 0 && lane == 0) { // gave up: let the MMAs in flight finish before tensor memory is freed
            mma_commit(smem_addr(mma_drain + sb));
            bar_wait_drain(smem_addr(mma_drain + sb), 0u);
        }
    } else if (warp == kEpilogueWarps + kCodeIssuers) {
        // ================= W loader =================
        if (lane == 0) {
            int s = 0, issued = 0;
            std::uint32_t pb = 1;
            bool dead = false;
            for (int g = 0; g < my_groups && !dead; ++g)
                for (int w = 0; w < p.windows; ++w) {
                    if (bar_wait_sleeping(smem_addr(b_empty + s), pb, abort_flag, 200u)) { dead = true; break; }
                    bar_arrive_expect_tx(smem_addr(b_full + s), WREC);
                    bulk_copy_g2s(bstage0 + s * WREC, p.records + static_cast<std::size_t>(w) * REC, WREC, smem_addr(b_full + s));
                    ++issued;
                    if (++s == SB) { s = 0; pb ^= 1u; }
                }
            if (dead) // the copies still in flight land before the CTA gives up its shared memory
                for (int i = issued > SB ? issued - SB : 0; i < issued; ++i) bar_wait_drain(smem_addr(b_full + i % SB), static_cast<std::uint32_t>((i / SB) & 1));
        }
    } else if (warp == kEpilogueWarps + kCodeIssuers + 1) {
        // ================= code stages =================
        if (lane == 0) {
            int s = 0, issued = 0;
            std::uint32_t pc = 1;
            bool dead = false;
            for (int g = 0; g < my_groups && !dead; ++g) {
                const unsigned char *src = p.stages + static_cast<std::size_t>(first_group + static_cast<std::int64_t>(g) * gridDim.x) * halves * kCodeStageBytes;
                for (int h = 0; h < halves; ++h, src += kCodeStageBytes) {
                    if (bar_wait_sleeping(smem_addr(c_empty + s), pc, abort_flag, 100u)) { dead = true; break; }
                    bar_arrive_expect_tx(smem_addr(c_full + s), kCodeSlotBytes);
                    bulk_copy_g2s(smem_addr(cstage0 + s * kCodeSlotBytes), src, kCodeStageBytes, smem_addr(c_full + s));
                    bulk_copy_g2s(smem_addr(cstage0 + s * kCodeSlotBytes + kCodeStageBytes), p.table + static_cast<std::size_t>(h) * kTableBytes, kTableBytes,
                                  smem_addr(c_full + s));
                    ++issued;
                    if (++s == SC) { s = 0; pc ^= 1u; }
                }
            }
            if (dead)
                for (int i = issued > SC ? issued - SC : 0; i < issued; ++i) bar_wait_drain(smem_addr(c_full + i % SC), static_cast<std::uint32_t>((i / SC) & 1));
        }
    } else {
        // ================= decode: bytes -> fp16 operand in tensor memory =================
        // A warp may write the 32 lanes (warp mod 4) of tensor memory: rows 32 * quarter .. + 31 of both row
        // sub-blocks.  The four warps of a quarter split a window's two half windows and, within a half, its two pairs of
        // 16-gene chunks: a warp visits one code stage per window (one wait, one hand-back) and decodes two chunks of it.
        const int dw = warp - (kEpilogueWarps + kCodeIssuers + 2);
        const int quarter = warp & 3, hf = (dw >> 2) & 1, pairc = dw >> 3;
        const __half2 magic = __half2half2(__ushort_as_half(static_cast<unsigned short>(0x6400u))); // 1024: fp16(0x6400 | byte) = 1024 + byte
        const __half2 bias = __float2half2_rn(1024.0f + kPresentBias); // fp16(0x6400 | byte) - bias = the code
        const std::uint32_t lane_base = tmem_base + (static_cast<std::uint32_t>(quarter * 32) << 16) + kOperandCol0 + hf * 32 + pairc * 16;
        const int windows_total = my_groups * p.windows;
        int sa = 0;
        std::uint32_t pa = 1;
        for (int wq = 0; wq < windows_total; ++wq) {
            const int q = 2 * wq + hf; // this warp's half window in the sequence of code stages
            const int sc = q % SC;
            if (bar_wait(smem_addr(c_full + sc), static_cast<std::uint32_t>((q / SC) & 1), abort_flag)) break;
            const unsigned char *in = cstage0 + sc * kCodeSlotBytes;
            const bool plain = *reinterpret_cast<const std::uint32_t *>(in + kCodeStageBytes + kPairTableBytes) != 0u; // no masks needed
            uint4 x[2][kSubBlocks];
#pragma unroll
            for (int c = 0; c < 2; ++c)
#pragma unroll
                for (int k = 0; k < kSubBlocks; ++k)
                    x[c][k] = *reinterpret_cast<const uint4 *>(in + (pairc * 2 + c) * kChunkPlaneBytes + (k * 128 + quarter * 32 + lane) * 16);
            // a new window: its operand stage must have been read by the MMAs that used it last
            if (bar_wait(smem_addr(a_empty + sa), pa, abort_flag)) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                // the 16 genes' {scale, zero-point} pairs of this chunk: one address for the whole warp
                uint2 so[8];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint4 t = *(reinterpret_cast<const uint4 *>(in + kCodeStageBytes + (pairc * 2 + c) * 64) + j);
                    so[2 * j] = make_uint2(t.x, t.y);
                    so[2 * j + 1] = make_uint2(t.z, t.w);
                }
#pragma unroll
                for (int k = 0; k < kSubBlocks; ++k) {
                    const std::uint32_t w[4] = {x[c][k].x, x[c][k].y, x[c][k].z, x[c][k].w};
                    std::uint32_t r[8];
                    if (plain) { // two bytes -> fp16 pair 1024 + byte; minus 1264 = the code, or -240 for an empty slot; max(0, code * scale + offset)
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
#pragma unroll
                            for (int hh = 0; hh < 2; ++hh) {
                                const std::uint32_t bits = __byte_perm(w[j], 0x64646464u, hh == 0 ? 0x4140u : 0x4342u);
                                const __half2 v = __hfma2_relu(__hsub2(*reinterpret_cast<const __half2 *>(&bits), bias),
                                                               *reinterpret_cast<const __half2 *>(&so[2 * j + hh].x),
                                                               *reinterpret_cast<const __half2 *>(&so[2 * j + hh].y));
                                r[2 * j + hh] = *reinterpret_cast<const std::uint32_t *>(&v);
                            }
                        }
                    } else { // the same without the max, and 0 where the byte was 0
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
#pragma unroll
                            for (int hh = 0; hh < 2; ++hh) {
                                const std::uint32_t bits = __byte_perm(w[j], 0x64646464u, hh == 0 ? 0x4140u : 0x4342u);
                                const __half2 raw = *reinterpret_cast<const __half2 *>(&bits);
                                const __half2 v = __hfma2(__hsub2(raw, bias), *reinterpret_cast<const __half2 *>(&so[2 * j + hh].x),
                                                          *reinterpret_cast<const __half2 *>(&so[2 * j + hh].y));
                                r[2 * j + hh] = *reinterpret_cast<const std::uint32_t *>(&v) & __hne2_mask(raw, magic);
                            }
                        }
                    }
                    // columns [32 * half + 8 * chunk, + 8) of the row's 64: genes 64 * half + 16 * chunk .. + 15, the even gene in the low half
                    tmem_st8(lane_base + sa * kOperandCols + k * 64 + c * 8, r);
                }
            }
            // the stage goes back to the copy engine behind the last use of what was read from it, and behind a fence that
            // waits for this thread's loads (handed back straight after the loads, with the values not yet in their
            // registers, the stage was refilled under them)
            asm volatile("fence.acq_rel.cta;" ::: "memory");
            if (lane == 0) bar_arrive(smem_addr(c_empty + sc));
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) bar_arrive(smem_addr(a_full + sa));
            sa ^= 1;
            if (sa == 0) pa ^= 1u;
        }
        // a wait that ran out can end the loop between a store and its wait: nothing of this warp is in flight when the
        // CTA frees tensor memory
        __syncwarp();
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemColumns) : "memory");
    }
    if (tid == 0 && *abort_flag != 0 && p.status != nullptr) atomicExch(p.status, 1);
}

template<int NC>
cb200_status launch_codes(const codes_params &p, int sm_count, cudaStream_t stream) {
    constexpr int SB = codes_w_stages(NC), SC = codes_code_stages(NC);
    constexpr std::size_t smem = SB * NC * kWin * 2 + SC * kCodeSlotBytes + kTurnRegionBytes + (2 * SC + 2 * kOperandStages + 2 * SB + 2 + kCodeIssuers) * sizeof(std::uint64_t) + 16;
    static_assert(smem <= 232448, "shared memory budget");
    CB200_CUDA_OK(cudaFuncSetAttribute(qcsr_fwd_codes_kernel<NC>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    const std::int64_t groups = p.group_end - p.group_begin;
    const unsigned grid = static_cast<unsigned>(groups < sm_count ? groups : sm_count);
    qcsr_fwd_codes_kernel<NC><<<grid, kCodesThreads, smem, stream>>>(p);
    count_launch();
    CB200_CUDA_OK(cudaGetLastError());
    return CB200_STATUS_SUCCESS;
}

} // namespace

std::uint64_t qcsr_code_tile_bytes(std::int64_t rows, std::int64_t cols) {
    const std::uint64_t groups = static_cast<std::uint64_t>((rows + kRows - 1) / kRows);
    const std::uint64_t windows = static_cast<std::uint64_t>((cols + kWin - 1) / kWin);
    return groups * windows * static_cast<std::uint64_t>(2 * kCodeStageBytes);
}

std::uint64_t qcsr_codes_workspace_bytes(std::int64_t cols, std::int64_t n) {
    const std::uint64_t windows = static_cast<std::uint64_t>((cols + kWin - 1) / kWin);
    return 256u + windows * static_cast<std::uint64_t>(record_bytes(static_cast<int>(n))) + windows * 2u * kTableBytes;
}

bool qcsr_codes_shape_ok(std::int64_t rows, std::int64_t cols, std::int64_t n, int bits, int policy, int dense_dtype) {
    // a byte per slot holds code + 240 (0 = nothing stored): 4-bit codes; per-gene zero-points only
    return bits == 4 && policy == CB200_DECODE_PER_GENE_AFFINE && dense_dtype == CB200_DTYPE_BF16 &&
           qcsr_blocked_shape_ok(rows, cols, n, bits, dense_dtype);
}

// Turns the window-blocked copy (code words) into code tiles; the entry words go back to the arena.  *built is
// false, with the copy left as it was, when the arena has no room.  Waits for `stream`.
cb200_status bytify_blocked_layout(blocked_layout *layout, device_arena &arena, cudaStream_t stream, bool *built) {
    *built = false;
    if (layout == nullptr || layout->seg_ptr == nullptr || layout->baked) return CB200_STATUS_SUCCESS;
    const std::int64_t segments = layout->groups * layout->windows;
    const std::uint64_t bytes = static_cast<std::uint64_t>(segments) * (2 * kCodeStageBytes);
    unsigned char *stages = static_cast<unsigned char *>(arena.take(bytes));
    if (stages == nullptr) return CB200_STATUS_SUCCESS;
    cudaError_t err = cudaFuncSetAttribute(bytify_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kRows * kWin);
    if (err == cudaSuccess && segments > 0) {
        bytify_kernel<<<static_cast<unsigned>(segments), 512, kRows * kWin, stream>>>(layout->entries, layout->seg_ptr, layout->windows, stages);
        count_launch();
        err = cudaGetLastError();
    }
    if (err == cudaSuccess) err = cudaStreamSynchronize(stream);
    if (err != cudaSuccess) {
        arena.give_back(stages, bytes);
        return fail(CB200_STATUS_CUDA_ERROR, "building the code tiles: %s", cudaGetErrorString(err));
    }
    arena.give_back(layout->entries, static_cast<std::uint64_t>(layout->total_entries) * 4u);
    arena.give_back(layout->seg_ptr, static_cast<std::uint64_t>(segments + 1) * 8u);
    layout->entries = nullptr;
    layout->seg_ptr = nullptr;
    layout->total_entries = 0;
    layout->code_tiles = stages;
    layout->bytes = bytes;
    *built = true;
    return CB200_STATUS_SUCCESS;
}

cb200_status launch_qcsr_forward_codes(const qcsr_view &x, const dense_args &d, std::int64_t row_begin, std::int64_t row_end,
                                       void *workspace, std::uint64_t workspace_bytes, const blocked_layout &layout, int sm_count,
                                       cudaStream_t stream, bool *taken) {
    if (!qcsr_codes_shape_ok(x.rows, x.cols, d.n, x.bits, x.policy, d.dense_dtype)) return CB200_STATUS_SUCCESS;
    if (row_begin % kRows != 0) return CB200_STATUS_SUCCESS; // a launch starts on a group boundary, else another kernel runs
    if (reinterpret_cast<std::uintptr_t>(d.out) % 16u != 0u || (d.out_ld * 4u) % 16u != 0u) return CB200_STATUS_SUCCESS;
    if (workspace == nullptr || workspace_bytes < qcsr_codes_workspace_bytes(x.cols, d.n)) return CB200_STATUS_SUCCESS;
    if (reinterpret_cast<std::uintptr_t>(workspace) % 256u != 0u) return CB200_STATUS_SUCCESS;
    // the tiles hold the codes of these arrays; scales and offsets are read at launch and may be any
    if (x.row_ptr != layout.src_row_ptr || x.col_idx != layout.src_col_idx || x.packed != layout.src_packed)
        return fail(CB200_STATUS_STALE_STRUCTURE, "the launch's matrix is not the one the code tiles were built from");
    int *status = static_cast<int *>(workspace);
    unsigned *w_absmax = reinterpret_cast<unsigned *>(workspace) + 1;    // float bits of the largest |W|
    unsigned *value_bound = reinterpret_cast<unsigned *>(workspace) + 2; // [2], [3]: bounds of the decoded magnitudes
    unsigned char *records = static_cast<unsigned char *>(workspace) + 256;
    const std::int64_t windows = layout.windows;
    unsigned char *table = records + static_cast<std::size_t>(windows) * record_bytes(static_cast<int>(d.n));
    CB200_CUDA_OK(cudaMemsetAsync(status, 0, 4 * sizeof(int), stream));
    const std::int64_t elements = x.cols * d.n;
    const unsigned w_blocks = static_cast<unsigned>(std::min<std::int64_t>((elements + 1023) / 1024, 4 * static_cast<std::int64_t>(sm_count)));
    operand_bounds_kernel<<<w_blocks + static_cast<unsigned>((x.cols + 255) / 256), 256, 0, stream>>>(
        static_cast<const __nv_bfloat16 *>(d.dense), d.dense_ld, x.cols, static_cast<int>(d.n), w_blocks, x.scales, x.offsets, nullptr, 0,
        static_cast<float>((1 << x.bits) - 1), w_absmax, value_bound);
    pack_codes_operands_kernel<<<dim3(static_cast<unsigned>(windows), static_cast<unsigned>(d.n / kPackColumns)), 256, 0, stream>>>(
        static_cast<const __nv_bfloat16 *>(d.dense), d.dense_ld, x.cols, static_cast<int>(d.n), x.scales, x.offsets, records, w_absmax, value_bound,
        table);
    count_launch(2);
    CB200_CUDA_OK(cudaGetLastError());
    codes_params p{};
    p.stages = layout.code_tiles; p.records = records; p.table = table; p.y = d.out; p.y_ld = d.out_ld; p.row_end = row_end;
    p.group_begin = row_begin / kRows; p.group_end = (row_end + kRows - 1) / kRows; p.windows = layout.windows;
    p.alpha = d.alpha; p.beta = d.beta; p.bias = d.bias; p.epilogue = d.epilogue; p.status = status;
    p.w_absmax = w_absmax; p.value_bound = value_bound;
    *taken = true;
    switch (d.n) {
    case 32: return launch_codes<32>(p, sm_count, stream);
    case 64: return launch_codes<64>(p, sm_count, stream);
    default: return launch_codes<128>(p, sm_count, stream);
    }
}

} // namespace cb200
