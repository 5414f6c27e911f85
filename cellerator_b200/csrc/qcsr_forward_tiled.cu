// Gene-tiled fused dequantise + SpMM for quantized CSR: the W operand is staged through shared
// memory instead of being gathered row by row from L2.
//
// Why: at N = 64 every stored entry needs a 128-byte row of W.  Gathered from L2 that is
// ~25x the HBM bytes of the entry itself and the L2 -> SM path saturates long before HBM does.
// Here a CTA owns a group of cell rows and sweeps the gene axis in tiles: tile t of W
// (tile_genes consecutive rows, 80-96 KB) is brought into shared memory by one bulk async copy
// (cp.async.bulk, completion on an mbarrier, double buffered), the per-gene scale / zero-point
// of the tile sit beside it, and the part of every row that falls into the tile is multiplied
// (gene indices are ascending within a row, so that part is a contiguous run found by comparing
// against the tile's upper bound).  W crosses L2 -> SM once per row group instead of once per
// stored entry.
//
// Work split inside a CTA (1024 threads): a warp is cut into groups of LPN = N/8 lanes; a group
// owns two rows outright and keeps their N accumulators in registers (8 columns per lane), so no
// accumulator is replicated and nothing is reduced across lanes at the end.  In one iteration
// the LPN lanes of a group fetch and decode LPN consecutive entries of the group's row, park
// {W-row offset, value} in a per-warp staging area, and then walk them: every lane reads the
// same entry and its own 16-byte slice of that W row.  The groups of a warp run in lockstep, so
// rows are dealt out sorted by length: neighbouring ranks share a warp (similar trip counts), and
// warps get one long and one short bundle (snake order) so that all warps of the CTA reach the
// end of a tile together.  A row is worked by one lane group, so a CTA is only as fast as its
// longest row: when the caller's prepare step supplies a length-sorted row order, every CTA gets
// rows of nearly equal length and the CTAs take row groups from both ends of that order in turn.
//
// Waiting on the copy barrier is bounded: if the bound is hit a flag is raised in the status
// word (first int of the workspace) and the kernel carries on with memory-safe indices, so it
// always terminates; a non-zero status means the output is not valid.
#include "kernels.cuh"

#include <cstdlib>
#include <cstring>

namespace cb200 {
namespace {

constexpr int kWarps = 32;
constexpr int kThreads = kWarps * 32; // 1024
constexpr int kRowsPerGroup = 2;

// per instantiation: lanes per group -> groups per warp, rows per CTA, W buffer size
template<int LPN> struct tile_shape {
    static constexpr int groups_per_warp = 32 / LPN;
    static constexpr int cta_rows = kWarps * groups_per_warp * kRowsPerGroup; // 512 / 256 / 128
    static constexpr int wbuf_bytes = (LPN == 4 ? 80 : 96) * 1024;
};

struct tiled_params {
    const std::int64_t *row_ptr;
    const std::int64_t *packed_row_ptr;
    const std::int32_t *col_idx;
    const std::uint8_t *packed;
    const float *scales;
    const float *offsets;
    const void *w;
    float *y;
    std::int64_t y_ld;
    std::int64_t row_begin, row_end;
    std::int64_t groups;
    int genes;
    int tile_genes;
    int tiles;
    int n;
    int policy;
    float alpha, beta;
    const float *bias;
    int epilogue;
    int *status;
    const std::int32_t *row_order; // optional: rows in processing order (length-sorted), else natural order
};

__device__ __forceinline__ std::uint32_t smem_u32(const void *p) {
    return static_cast<std::uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(std::uint32_t bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(std::uint32_t bar, std::uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(std::uint32_t bar, std::uint32_t parity) {
    std::uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0u;
}
// One contiguous global -> shared copy by the copy engine; `bytes` and both addresses are
// multiples of 16.  Source is always this GPU's own memory.
__device__ __forceinline__ void bulk_copy_g2s(std::uint32_t dst, const void *src, std::uint32_t bytes, std::uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

#ifndef CB200_CVT_MODE
#define CB200_CVT_MODE 0
#endif
#ifndef CB200_FMA_MODE
#define CB200_FMA_MODE 0
#endif

// bf16 pair -> two floats (exact).  Three spellings (shift + mask, byte permute + mask, two byte
// permutes) and scalar vs packed FMAs were timed against each other on the 1,000,000-cell
// matrix: all within 3 % (19.7 - 20.6 ms), i.e. the kernel is not bound by the arithmetic pipes.
__device__ __forceinline__ void widen_bf16x2(std::uint32_t packed, float &lo, float &hi) {
#if CB200_CVT_MODE == 0
    lo = __uint_as_float(packed << 16);
    hi = __uint_as_float(packed & 0xffff0000u);
#elif CB200_CVT_MODE == 1
    std::uint32_t l;
    asm("prmt.b32 %0, %1, 0, 0x1044;" : "=r"(l) : "r"(packed));
    lo = __uint_as_float(l);
    hi = __uint_as_float(packed & 0xffff0000u);
#else
    std::uint32_t l, h;
    asm("prmt.b32 %0, %1, 0, 0x1044;" : "=r"(l) : "r"(packed));
    asm("prmt.b32 %0, %1, 0, 0x3244;" : "=r"(h) : "r"(packed));
    lo = __uint_as_float(l);
    hi = __uint_as_float(h);
#endif
}

__device__ __forceinline__ void fma8_packed(float (&acc)[8], float v, const float (&w)[8]) {
#if CB200_FMA_MODE == 1
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = fmaf(v, w[i], acc[i]);
    return;
#endif
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

// Shared-memory accesses by 32-bit shared-window address (keeps 64-bit pointer arithmetic out of
// the inner loop).  volatile: they stay ordered against the staging store and each other.
__device__ __forceinline__ uint4 lds_b32x4(std::uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ float2 lds_f32x2(std::uint32_t addr) {
    float2 v;
    asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts_b32x2(std::uint32_t addr, int a, float b) {
    asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(addr), "r"(a), "r"(__float_as_int(b)) : "memory");
}

// The 8 columns of a staged W row held by a lane; `addr` = row start + t * 16 for lane t of the
// group.  bf16: 8 consecutive columns (one 16-byte read).  fp32: columns [4t, 4t+4) and
// [N/2 + 4t, N/2 + 4t + 4), so that both 16-byte reads of a group are contiguous across its lanes
// (no bank conflict).
template<typename WT, int LPN>
__device__ __forceinline__ void load_w_smem(std::uint32_t addr, float (&w)[8]) {
    if constexpr (sizeof(WT) == 2) {
        const uint4 a = lds_b32x4(addr);
        widen_bf16x2(a.x, w[0], w[1]);
        widen_bf16x2(a.y, w[2], w[3]);
        widen_bf16x2(a.z, w[4], w[5]);
        widen_bf16x2(a.w, w[6], w[7]);
    } else {
        const uint4 a = lds_b32x4(addr);
        const uint4 b = lds_b32x4(addr + LPN * 16);
        w[0] = __uint_as_float(a.x); w[1] = __uint_as_float(a.y); w[2] = __uint_as_float(a.z); w[3] = __uint_as_float(a.w);
        w[4] = __uint_as_float(b.x); w[5] = __uint_as_float(b.y); w[6] = __uint_as_float(b.z); w[7] = __uint_as_float(b.w);
    }
}

template<int BITS, typename WT, int LPN>
__global__ void __launch_bounds__(kThreads, 1) qcsr_fwd_tiled_kernel(const tiled_params p) {
    using shape = tile_shape<LPN>;
    constexpr int RB = LPN * 8 * static_cast<int>(sizeof(WT)); // bytes of one W row
    constexpr int GPW = shape::groups_per_warp;
    constexpr int CTA_ROWS = shape::cta_rows;
    constexpr int WBUF = shape::wbuf_bytes;
    constexpr int BUNDLES = CTA_ROWS / GPW;                    // 2 * kWarps
    constexpr unsigned GROUP_MASK = LPN == 32 ? 0xffffffffu : ((1u << LPN) - 1u);
    extern __shared__ __align__(128) unsigned char smem[];
    const int tile_genes = p.tile_genes;
    unsigned char *wbuf = smem;                                                  // [2][WBUF]
    float2 *sc = reinterpret_cast<float2 *>(smem + 2 * WBUF);                    // [2][tile_genes] {scale, offset}
    float2 *stage = sc + 2 * tile_genes;                                         // [kWarps][40] {W row offset, value}
    int4 *meta = reinterpret_cast<int4 *>(stage + kWarps * 40);                  // [CTA_ROWS] {entry start lo, hi, length, row}
    longlong2 *meta2 = reinterpret_cast<longlong2 *>(meta + CTA_ROWS);           // [CTA_ROWS] {packed byte start, unused}
    float *rowoff = reinterpret_cast<float *>(meta2 + CTA_ROWS);                 // [CTA_ROWS]
    int *lens = reinterpret_cast<int *>(rowoff + CTA_ROWS);                      // [CTA_ROWS]
    std::uint64_t *bars = reinterpret_cast<std::uint64_t *>(lens + CTA_ROWS);    // [2]
    int *abort_flag = reinterpret_cast<int *>(bars + 2);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane / LPN, j = lane % LPN; // group within the warp, lane within the group
    const bool row_policy = p.policy == CB200_DECODE_COLUMN_SCALE_ROW_OFFSET;
    // Row groups are taken in rounds of gridDim.x; odd rounds run through the CTAs backwards, so that
    // with a length-sorted row order every CTA receives the same mix of long and short groups.
    auto group_of_round = [&](std::int64_t round) -> std::int64_t {
        const std::int64_t pos = (round & 1) ? static_cast<std::int64_t>(gridDim.x) - 1 - blockIdx.x : blockIdx.x;
        return round * gridDim.x + pos;
    };
    const std::int64_t rounds = (p.groups + gridDim.x - 1) / gridDim.x;
    std::int64_t my_groups = 0;
    for (std::int64_t r = 0; r < rounds; ++r) my_groups += group_of_round(r) < p.groups ? 1 : 0;
    const std::int64_t total_tiles = my_groups * p.tiles;
    const std::int64_t rows_total = p.row_end - p.row_begin;
    const std::uint32_t bar0 = smem_u32(bars), wbuf0 = smem_u32(wbuf);

    if (tid == 0) {
        mbar_init(bar0, 1);
        mbar_init(bar0 + 8, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    auto issue_tile = [&](std::int64_t q) { // thread 0 only
        const int t = static_cast<int>(q % p.tiles);
        const std::uint32_t b = static_cast<std::uint32_t>(q & 1);
        const int g0 = t * tile_genes;
        const int count = min(tile_genes, p.genes - g0);
        const std::uint32_t bytes = static_cast<std::uint32_t>(count) * RB;
        mbar_expect_tx(bar0 + 8 * b, bytes);
        bulk_copy_g2s(wbuf0 + b * WBUF, static_cast<const unsigned char *>(p.w) + static_cast<std::size_t>(g0) * RB, bytes,
                      bar0 + 8 * b);
    };
    if (tid == 0) {
        if (total_tiles > 0) issue_tile(0);
        if (total_tiles > 1) issue_tile(1);
    }
    // scale / zero-point of tile 0
    for (int i = tid; i < min(tile_genes, p.genes); i += kThreads)
        sc[i] = make_float2(__ldg(p.scales + i), (!row_policy && p.offsets != nullptr) ? __ldg(p.offsets + i) : 0.0f);
    __syncthreads();

    constexpr int SC_PER_THREAD = (WBUF / RB + kThreads - 1) / kThreads;
    const int slot0 = (warp * GPW + g) * kRowsPerGroup; // this group's two rows in meta[]
    // staging area of a warp: the groups' entry lists sit (LPN + 1) slots apart, so that the four
    // (two, eight) groups read entry s of their lists from distinct banks in one pass
    const std::uint32_t stage_rd = smem_u32(stage) + warp * 320 + g * (LPN + 1) * 8;
    const std::uint32_t stage_wr = stage_rd + j * 8;
    const std::uint32_t sc0 = smem_u32(sc);

    std::int64_t q = 0;
    for (std::int64_t round = 0; round < rounds; ++round) {
        const std::int64_t group = group_of_round(round);
        if (group >= p.groups) continue;
        const std::int64_t first = group * CTA_ROWS; // position of this group's first row in the processing order

        // ---- deal the rows: rank by length (longest first); GPW neighbouring ranks form a bundle
        //      that shares a warp; bundle k goes to warp k (first row) or warp BUNDLES-1-k (second)
        std::int64_t my_row = -1;
        if (tid < CTA_ROWS && first + tid < rows_total)
            my_row = p.row_order != nullptr ? static_cast<std::int64_t>(__ldg(p.row_order + first + tid)) : p.row_begin + first + tid;
        if (tid < CTA_ROWS)
            lens[tid] = my_row >= 0 ? static_cast<int>(__ldg(p.row_ptr + my_row + 1) - __ldg(p.row_ptr + my_row)) : -1;
        __syncthreads();
        if (tid < CTA_ROWS) {
            const int mine = lens[tid];
            int rank = 0;
            for (int k = 0; k < CTA_ROWS; ++k) {
                const int other = lens[k];
                rank += (other > mine || (other == mine && k < tid)) ? 1 : 0;
            }
            const int bundle = rank / GPW, gg = rank % GPW;
            const int w = bundle < kWarps ? bundle : BUNDLES - 1 - bundle;
            const int rr = bundle < kWarps ? 0 : 1;
            int4 m = make_int4(0, 0, 0, -1);
            longlong2 m2 = make_longlong2(0, 0);
            float ro = 0.0f;
            if (my_row >= 0) {
                const std::int64_t rs = __ldg(p.row_ptr + my_row);
                m.x = static_cast<int>(static_cast<std::uint64_t>(rs) & 0xffffffffu);
                m.y = static_cast<int>(static_cast<std::uint64_t>(rs) >> 32);
                m.z = mine;
                m.w = static_cast<int>(my_row - p.row_begin);
                m2.x = p.packed_row_ptr != nullptr ? __ldg(p.packed_row_ptr + my_row) : rs;
                if (row_policy && p.offsets != nullptr) ro = __ldg(p.offsets + my_row);
            }
            meta[(w * GPW + gg) * kRowsPerGroup + rr] = m;
            meta2[(w * GPW + gg) * kRowsPerGroup + rr] = m2;
            rowoff[(w * GPW + gg) * kRowsPerGroup + rr] = ro;
        }
        __syncthreads();

        // Per row of this group: cursor (entries consumed), and the (gene, code byte) of entry
        // cursor + j, fetched ahead so that no global-memory latency sits in front of a visit.
        int cur[kRowsPerGroup];
        int gene_pf[kRowsPerGroup];
        unsigned code_pf[kRowsPerGroup];
        float acc[kRowsPerGroup][8];
        auto fetch_entry = [&](const std::int32_t *cols, const std::uint8_t *codes, int len, int at, int &gene, unsigned &code) {
            gene = 0x7fffffff;
            code = 0u;
            if (at + j < len) {
                gene = __ldg(cols + at + j);
                code = __ldg(codes + (BITS == 8 ? at + j : ((at + j) >> 1)));
            }
        };
        auto row_pointers = [&](int slot, const std::int32_t *&cols, const std::uint8_t *&codes, int &len) {
            const int4 m = meta[slot];
            const std::int64_t start = static_cast<std::int64_t>((static_cast<std::uint64_t>(static_cast<std::uint32_t>(m.y)) << 32) |
                                                                 static_cast<std::uint32_t>(m.x));
            cols = p.col_idx + start;
            codes = p.packed + meta2[slot].x;
            len = m.z;
        };
#pragma unroll
        for (int rr = 0; rr < kRowsPerGroup; ++rr) {
            const std::int32_t *cols;
            const std::uint8_t *codes;
            int len;
            row_pointers(slot0 + rr, cols, codes, len);
            cur[rr] = 0;
            fetch_entry(cols, codes, len, 0, gene_pf[rr], code_pf[rr]);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[rr][i] = 0.0f;
        }

        for (int t = 0; t < p.tiles; ++t, ++q) {
            const std::uint32_t b = static_cast<std::uint32_t>(q & 1);
            const int g0 = t * tile_genes;
            const int g1 = min(p.genes, g0 + tile_genes);
            // ---- wait for the tile's bytes (bounded)
            {
                const std::uint32_t parity = static_cast<std::uint32_t>((q >> 1) & 1);
                // once any wait of the CTA has run out, later tiles do not wait again: the kernel finishes
                // promptly with memory-safe indices and reports status 1
                int spins = 0;
                while (*static_cast<volatile int *>(abort_flag) == 0 && !mbar_try_wait(bar0 + 8 * b, parity)) {
                    if (++spins > (1 << 22)) {
                        *static_cast<volatile int *>(abort_flag) = 1;
                        break;
                    }
                }
            }
            // ---- prefetch the next tile's scale / zero-point into registers
            float s_next[SC_PER_THREAD], o_next[SC_PER_THREAD];
            const bool has_next = q + 1 < total_tiles;
            const int tn = static_cast<int>((q + 1) % p.tiles);
            if (has_next) {
#pragma unroll
                for (int k = 0; k < SC_PER_THREAD; ++k) {
                    const int local = tid + k * kThreads;
                    const int gene = tn * tile_genes + local;
                    s_next[k] = 1.0f;
                    o_next[k] = 0.0f;
                    if (local < tile_genes && gene < p.genes) {
                        s_next[k] = __ldg(p.scales + gene);
                        if (!row_policy && p.offsets != nullptr) o_next[k] = __ldg(p.offsets + gene);
                    }
                }
            }
            const std::uint32_t w_lane = wbuf0 + b * WBUF + j * 16; // this lane's slice of W row 0 of the tile
            const std::uint32_t sc_addr = sc0 + b * tile_genes * 8;

            // ---- this group's two rows: the run of each that falls into [g0, g1)
#pragma unroll
            for (int rr = 0; rr < kRowsPerGroup; ++rr) {
                const std::int32_t *cols;
                const std::uint8_t *codes;
                int len;
                row_pointers(slot0 + rr, cols, codes, len);
                const float row_offset = rowoff[slot0 + rr];
                int c = cur[rr];
                int gene = gene_pf[rr];
                unsigned code_byte = code_pf[rr];
                while (true) {
                    const unsigned in_tile = __ballot_sync(0xffffffffu, gene < g1);
                    if (in_tile == 0u) break;                                  // no group of the warp has entries left here
                    const int count = __popc((in_tile >> (g * LPN)) & GROUP_MASK); // this group's entries (a prefix)
                    const int most = __reduce_max_sync(0xffffffffu, count);
                    // the window after this one; groups with nothing here keep theirs
                    int gene_n = gene;
                    unsigned code_n = code_byte;
                    if (count > 0) fetch_entry(cols, codes, len, c + count, gene_n, code_n);
                    // Decode entry c + j without branches.  Lanes past `count` stage value 0 against a
                    // row of the tile that is certainly loaded; their product adds exactly 0 for finite W.
                    const int gl = min(max(gene - g0, 0), g1 - g0 - 1);       // in-tile even for unsorted input
                    unsigned code = code_byte;
                    if constexpr (BITS == 4) code = ((c + j) & 1) ? (code_byte >> 4) : (code_byte & 0xfu);
                    const float2 so = lds_f32x2(sc_addr + gl * 8);
                    const float decoded = fmaf(static_cast<float>(code), so.x, row_policy ? row_offset : so.y);
                    __syncwarp();
                    sts_b32x2(stage_wr, gl * RB, j < count ? decoded : 0.0f);
                    __syncwarp();
#pragma unroll
                    for (int s = 0; s < LPN; ++s) {
                        if (s >= most) break;
                        const float2 e = lds_f32x2(stage_rd + s * 8);
                        float wv[8];
                        load_w_smem<WT, LPN>(w_lane + __float_as_int(e.x), wv);
                        fma8_packed(acc[rr], e.y, wv);
                    }
                    c += count;
                    gene = gene_n;
                    code_byte = code_n;
                }
                cur[rr] = c;
                gene_pf[rr] = gene;
                code_pf[rr] = code_byte;
            }

            // ---- publish the next tile's scale / zero-point, release this tile's buffer
            if (has_next) {
                float2 *sc_next = sc + (b ^ 1u) * tile_genes;
#pragma unroll
                for (int k = 0; k < SC_PER_THREAD; ++k) {
                    const int local = tid + k * kThreads;
                    if (local < tile_genes) sc_next[local] = make_float2(s_next[k], o_next[k]);
                }
            }
            __syncthreads();
            if (tid == 0 && q + 2 < total_tiles) {
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                issue_tile(q + 2);
            }
        }

        // ---- every lane writes its 8 columns of its group's two rows
#pragma unroll
        for (int rr = 0; rr < kRowsPerGroup; ++rr) {
            const int row_local = meta[slot0 + rr].w; // row - row_begin, or -1 for an empty slot
            if (row_local >= 0) {
                float *out = p.y + (p.row_begin + row_local) * p.y_ld;
                float *out_a = out + (sizeof(WT) == 2 ? j * 8 : j * 4);
                float *out_b = sizeof(WT) == 2 ? out_a + 4 : out + LPN * 4 + j * 4;
                float4 lo = make_float4(p.alpha * acc[rr][0], p.alpha * acc[rr][1], p.alpha * acc[rr][2], p.alpha * acc[rr][3]);
                float4 hi = make_float4(p.alpha * acc[rr][4], p.alpha * acc[rr][5], p.alpha * acc[rr][6], p.alpha * acc[rr][7]);
                if (p.beta != 0.0f) {
                    const float4 a = *reinterpret_cast<const float4 *>(out_a);
                    const float4 bb = *reinterpret_cast<const float4 *>(out_b);
                    lo.x = fmaf(p.beta, a.x, lo.x); lo.y = fmaf(p.beta, a.y, lo.y);
                    lo.z = fmaf(p.beta, a.z, lo.z); lo.w = fmaf(p.beta, a.w, lo.w);
                    hi.x = fmaf(p.beta, bb.x, hi.x); hi.y = fmaf(p.beta, bb.y, hi.y);
                    hi.z = fmaf(p.beta, bb.z, hi.z); hi.w = fmaf(p.beta, bb.w, hi.w);
                }
                if (p.epilogue != CB200_EPILOGUE_NONE) {
                    const int ca = static_cast<int>(out_a - out), cb = static_cast<int>(out_b - out);
                    lo.x = finish_output(lo.x, p.bias, ca + 0, p.epilogue); lo.y = finish_output(lo.y, p.bias, ca + 1, p.epilogue);
                    lo.z = finish_output(lo.z, p.bias, ca + 2, p.epilogue); lo.w = finish_output(lo.w, p.bias, ca + 3, p.epilogue);
                    hi.x = finish_output(hi.x, p.bias, cb + 0, p.epilogue); hi.y = finish_output(hi.y, p.bias, cb + 1, p.epilogue);
                    hi.z = finish_output(hi.z, p.bias, cb + 2, p.epilogue); hi.w = finish_output(hi.w, p.bias, cb + 3, p.epilogue);
                }
                *reinterpret_cast<float4 *>(out_a) = lo;
                *reinterpret_cast<float4 *>(out_b) = hi;
            }
        }
        __syncthreads(); // meta / lens are rewritten by the next group
    }
    if (tid == 0 && *abort_flag != 0 && p.status != nullptr) atomicExch(p.status, 1);
}

template<typename WT, int LPN>
constexpr std::size_t tiled_smem_bytes() {
    using shape = tile_shape<LPN>;
    constexpr int RB = LPN * 8 * static_cast<int>(sizeof(WT));
    constexpr int tile_genes = shape::wbuf_bytes / RB;
    return 2 * shape::wbuf_bytes + 2 * tile_genes * sizeof(float2) + kWarps * 40 * sizeof(float2) +
           shape::cta_rows * (sizeof(int4) + sizeof(longlong2) + sizeof(float) + sizeof(int)) + 2 * sizeof(std::uint64_t) + 16;
}

template<int BITS, typename WT, int LPN>
cb200_status launch_one(tiled_params p, int sm_count, cudaStream_t stream) {
    using shape = tile_shape<LPN>;
    constexpr int RB = LPN * 8 * static_cast<int>(sizeof(WT));
    p.tile_genes = shape::wbuf_bytes / RB;
    p.tiles = (p.genes + p.tile_genes - 1) / p.tile_genes;
    p.groups = (p.row_end - p.row_begin + shape::cta_rows - 1) / shape::cta_rows;
    constexpr std::size_t smem = tiled_smem_bytes<WT, LPN>();
    CB200_CUDA_OK(cudaFuncSetAttribute(qcsr_fwd_tiled_kernel<BITS, WT, LPN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(smem)));
    const unsigned grid = static_cast<unsigned>(p.groups < sm_count ? p.groups : sm_count);
    qcsr_fwd_tiled_kernel<BITS, WT, LPN><<<grid, kThreads, smem, stream>>>(p);
    count_launch();
    CB200_CUDA_OK(cudaGetLastError());
    return CB200_STATUS_SUCCESS;
}

template<int BITS, typename WT>
cb200_status launch_lpn(const tiled_params &p, int sm_count, cudaStream_t stream, bool *taken) {
    *taken = true;
    switch (p.n / 8) {
    case 4: return launch_one<BITS, WT, 4>(p, sm_count, stream);
    case 8: return launch_one<BITS, WT, 8>(p, sm_count, stream);
    case 16: return launch_one<BITS, WT, 16>(p, sm_count, stream);
    default: *taken = false; return CB200_STATUS_SUCCESS;
    }
}

} // namespace

// Shapes the tiled kernel covers; everything else runs the warp-per-row kernel.
bool qcsr_forward_tiled_supported(const qcsr_view &x, const dense_args &d) {
    if (x.bits != 8 && x.bits != 4) return false;
    if (d.n != 32 && d.n != 64 && d.n != 128) return false;
    if (d.dense_dtype != CB200_DTYPE_BF16 && d.dense_dtype != CB200_DTYPE_F32) return false;
    if (d.dense_dtype == CB200_DTYPE_F32 && d.n == 128) return false; // 512-byte rows: tile too short
    if (d.dense_ld != d.n) return false;                               // W tile must be one contiguous range
    if (reinterpret_cast<std::uintptr_t>(d.dense) % 16u != 0u) return false;
    if (reinterpret_cast<std::uintptr_t>(d.out) % 16u != 0u || (d.out_ld * 4u) % 16u != 0u) return false;
    if (x.scales == nullptr) return false;
    if (x.bits == 4 && x.packed_row_ptr == nullptr) return false;
    if (x.cols > 0x7fffffff) return false;
    return true;
}

cb200_status launch_qcsr_forward_tiled(const qcsr_view &x, const dense_args &d, std::int64_t row_begin,
                                       std::int64_t row_end, int *status_word, const std::int32_t *row_order,
                                       int sm_count, cudaStream_t stream, bool *taken) {
    *taken = false;
    if (!qcsr_forward_tiled_supported(x, d) || row_end <= row_begin) return CB200_STATUS_SUCCESS;
    tiled_params p{};
    p.row_ptr = x.row_ptr; p.packed_row_ptr = x.packed_row_ptr; p.col_idx = x.col_idx; p.packed = x.packed;
    p.scales = x.scales; p.offsets = x.offsets; p.w = d.dense; p.y = d.out; p.y_ld = d.out_ld;
    p.row_begin = row_begin; p.row_end = row_end; p.groups = 0; // set per instantiation
    p.genes = static_cast<int>(x.cols); p.n = static_cast<int>(d.n); p.policy = x.policy; p.alpha = d.alpha;
    p.beta = d.beta; p.bias = d.bias; p.epilogue = d.epilogue; p.status = status_word;
    // a row order describes the whole matrix; a partial row range falls back to natural order
    p.row_order = (row_begin == 0 && row_end == x.rows) ? row_order : nullptr;
    if (status_word != nullptr) CB200_CUDA_OK(cudaMemsetAsync(status_word, 0, sizeof(int), stream));
    const bool bf16 = d.dense_dtype == CB200_DTYPE_BF16;
    if (x.bits == 8) return bf16 ? launch_lpn<8, __nv_bfloat16>(p, sm_count, stream, taken) : launch_lpn<8, float>(p, sm_count, stream, taken);
    return bf16 ? launch_lpn<4, __nv_bfloat16>(p, sm_count, stream, taken) : launch_lpn<4, float>(p, sm_count, stream, taken);
}

// ---------------------------------------------------------------------------------------------
// The same kernel for callers that must not allocate device memory.
//
// The gene-tiled kernel needs a little scratch in global memory (its status block).  The
// prepared-operation path takes that from the caller's workspace.  Some callers have no way to
// provide one: code that runs where cudaMalloc is forbidden (inside a region that must stay free
// of allocator calls, or in a process whose memory budget is fixed up front and policed), and thin
// foreign-language shims that can pass pointers through but own no device allocator.  For them the
// scratch lives in a fixed array inside this library's device image.
//
// Consequences, all of them part of the contract:
//  * every GPU that loads the library carries kStaticScratchBytes of it until the process exits;
//  * the array is shared by every call on a device and keeps the previous call's contents, so each
//    call first clears (stream-ordered) the part that must start at zero, and two calls whose
//    kernels can overlap on the GPU (different streams, no ordering between them) race on it;
//  * in host code the array's name is only a host-side handle, not a device address, so the address
//    is looked up once per device with cudaGetSymbolAddress (with that device current) and cached;
//    that look-up happens in the first call on a device, which should therefore be made before any
//    stream capture begins.
namespace {

constexpr std::size_t kStaticScratchBytes = 256;
constexpr int kStaticMaxDevices = 64;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

std::atomic<void *> g_static_scratch_address[kStaticMaxDevices];

// Device address of g_static_scratch on `device` (which must be current).
cb200_status static_scratch_on(int device, void **address) {
    if (device < 0 || device >= kStaticMaxDevices)
        return fail(CB200_STATUS_INVALID_STREAM, "device ordinal %d outside 0..%d", device, kStaticMaxDevices - 1);
    void *known = g_static_scratch_address[device].load(std::memory_order_acquire);
    if (known == nullptr) {
        void *looked_up = nullptr;
        const cudaError_t err = cudaGetSymbolAddress(&looked_up, g_static_scratch);
        if (err != cudaSuccess || looked_up == nullptr)
            return fail(CB200_STATUS_CUDA_ERROR, "cudaGetSymbolAddress(static scratch) on device %d: %s", device,
                        cudaGetErrorString(err));
        g_static_scratch_address[device].store(looked_up, std::memory_order_release);
        known = looked_up;
    }
    *address = known;
    return CB200_STATUS_SUCCESS;
}

} // namespace
} // namespace cb200

extern "C" cb200_status cb200_qcsr_forward_static(const cb200_qcsr *x, const void *w, int32_t w_dtype, int64_t n,
                                                  float *y, int64_t y_ld, float alpha, float beta, int32_t device,
                                                  void *stream) {
    using namespace cb200;
    clear_error();
    if (x == nullptr || x->version != CB200_ABI_VERSION || x->size < sizeof(cb200_qcsr))
        return fail(CB200_STATUS_INVALID_ARGUMENT, "bad cb200_qcsr header");
    if (w == nullptr || y == nullptr || x->row_ptr == nullptr || (x->nnz != 0 && (x->col_idx == nullptr || x->packed_values == nullptr)))
        return fail(CB200_STATUS_INVALID_ARGUMENT, "null operand");
    if (static_cast<const void *>(y) == w) return fail(CB200_STATUS_INVALID_ARGUMENT, "output aliases the dense input");
    if (x->rows < 0 || x->cols < 0 || n <= 0 || y_ld < n) return fail(CB200_STATUS_INVALID_SHAPE, "bad shape");
    // scratch this kernel needs for this problem against what the fixed array holds
    const std::size_t needed = qcsr_tiled_workspace_bytes(); // one status block, whatever the matrix size
    static_assert(kStaticScratchBytes >= qcsr_tiled_workspace_bytes(), "the built-in array must hold the tiled kernel's scratch");
    if (needed > kStaticScratchBytes)
        return fail(CB200_STATUS_INSUFFICIENT_WORKSPACE, "needs %zu bytes of scratch, the built-in array holds %zu", needed,
                    kStaticScratchBytes);
    const qcsr_view view{x->rows, x->cols, x->nnz, x->bits, x->policy, x->row_ptr, x->packed_row_ptr,
                         x->col_idx, x->packed_values, x->scales, x->offsets};
    const dense_args d{w, n, w_dtype, y, y_ld, n, alpha, beta};
    if (!qcsr_forward_tiled_supported(view, d))
        return fail(CB200_STATUS_UNSUPPORTED,
                    "outside what the allocation-free entry covers: 8/4-bit codes with per-gene scales, N in {32,64,128} "
                    "(fp32 W: 32 or 64), W contiguous (ld == N) and 16-byte aligned, Y rows 16-byte aligned; got bits=%d N=%lld",
                    x->bits, static_cast<long long>(n));
    if (x->rows == 0) return CB200_STATUS_SUCCESS;
    device_scope scope(device);
    CB200_CUDA_OK(scope.status);
    void *scratch = nullptr;
    const cb200_status found = static_scratch_on(device, &scratch);
    if (found != CB200_STATUS_SUCCESS) return found;
    int sm_count = 0;
    CB200_CUDA_OK(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device));
    bool taken = false;
    // clears the status word on the stream, then launches; nothing here allocates
    const cb200_status st = launch_qcsr_forward_tiled(view, d, 0, x->rows, static_cast<int *>(scratch), nullptr, sm_count,
                                                      static_cast<cudaStream_t>(stream), &taken);
    if (st != CB200_STATUS_SUCCESS) return st;
    if (!taken) return fail(CB200_STATUS_INTERNAL_ERROR, "tiled kernel declined a shape it reports as supported");
    return CB200_STATUS_SUCCESS;
}

extern "C" cb200_status cb200_qcsr_forward_static_status(int32_t device, void *stream, int32_t *host_word) {
    using namespace cb200;
    clear_error();
    if (host_word == nullptr) return fail(CB200_STATUS_INVALID_ARGUMENT, "status needs an output");
    *host_word = 0;
    if (device < 0 || device >= kStaticMaxDevices)
        return fail(CB200_STATUS_INVALID_STREAM, "device ordinal %d outside 0..%d", device, kStaticMaxDevices - 1);
    // the address cached by the first static call on this device; nothing is looked up or allocated here
    void *scratch = g_static_scratch_address[device].load(std::memory_order_acquire);
    if (scratch == nullptr)
        return fail(CB200_STATUS_INVALID_ARGUMENT, "no cb200_qcsr_forward_static call has run on device %d yet", device);
    device_scope scope(device);
    CB200_CUDA_OK(scope.status);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    CB200_CUDA_OK(cudaMemcpyAsync(host_word, scratch, sizeof(int32_t), cudaMemcpyDeviceToHost, s));
    CB200_CUDA_OK(cudaStreamSynchronize(s));
    if (*host_word != 0)
        return fail(CB200_STATUS_DEVICE_WAIT_TIMEOUT, "the last static forward call on device %d gave up a bounded wait: its output is not valid", device);
    return CB200_STATUS_SUCCESS;
}
