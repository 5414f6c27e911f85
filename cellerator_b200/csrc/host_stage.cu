// Forward projection of a quantized CSR matrix that lives in HOST memory: the row range is cut into
// chunks that travel host -> device -> host through a small ring of device buffers, so that the copy
// in, the multiply and the copy out of neighbouring chunks overlap and the device never holds more
// than `chunk_buffers` chunks.  The reference's callers do the same by hand before every projection
// (operands are copied in, the projection runs, the result is copied out: src/abi/abi.cu:278-340);
// here it is one call of the C ABI.
//
// Streams: one for host -> device copies, one for the kernels, one for device -> host copies, tied by
// events per ring buffer.  A chunk's row pointers arrive with their absolute offsets and are rebased on
// the device (one small kernel), so the chunk is a matrix of its own for the projection kernel.  The
// kernels are the CSR schedules that read codes and indices at launch (gene-tiled where the shape allows,
// else warp per row): the values arrive with the call, so nothing prepared from them can be used.
//
// The call is bound by the host -> device link (5 bytes per stored entry: a code and a 32-bit gene index), so the
// indices travel in a shorter form: a small pool of host threads rewrites a chunk's indices into a pinned staging
// buffer while the previous chunk is on the link, and a kernel restores the 32-bit indices on the device.
//   gaps (any k): one byte per entry, gene - previous gene of the row - 1 (the row's first entry: its gene); an entry
//     whose gap does not fit (255 or more, or a row whose genes do not ascend) is sent as the byte 255 plus a record
//     {position, gene} in a short list.  2 bytes per entry on the link.  A warp per row restores the genes with a
//     prefix sum.
//   16-bit words (k <= 65,536): 3 bytes per entry on the link.  A chunk that holds an index outside [0, k) is copied as
//     it is (the kernels leave such entries out; narrowed they would alias another gene).
// In the default mode the host rewrites only the share of a chunk's rows that keeps it and the link busy for the same
// time (the first rewritten chunks of a call are timed), and the other rows' 32-bit indices are enqueued first; a host
// that is very slow (few cores, or many processes sharing them) sends 32-bit indices for the rest of the call and the
// next few calls.
#include "kernels.cuh"

#include <algorithm>
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstring>
#include <mutex>
#include <new>
#include <thread>
#include <vector>

#include <immintrin.h>
#include <sched.h>

using namespace cb200;

namespace {

constexpr int kMaxBuffers = 4;

__global__ void __launch_bounds__(256) rebase_kernel(std::int64_t *ptr, std::int64_t count, std::int64_t base) {
    const std::int64_t i = static_cast<std::int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < count) ptr[i] -= base;
}

// 16-bit gene indices -> the 32-bit ones the kernels read; eight per thread (the buffers are 16-byte aligned and
// padded to a multiple of eight entries)
__global__ void __launch_bounds__(256) widen_indices_kernel(const uint4 *narrow, int4 *wide, std::int64_t groups_of_eight) {
    const std::int64_t i = static_cast<std::int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= groups_of_eight) return;
    const uint4 v = narrow[i];
    wide[2 * i] = make_int4(static_cast<int>(v.x & 0xffffu), static_cast<int>(v.x >> 16), static_cast<int>(v.y & 0xffffu), static_cast<int>(v.y >> 16));
    wide[2 * i + 1] = make_int4(static_cast<int>(v.z & 0xffffu), static_cast<int>(v.z >> 16), static_cast<int>(v.w & 0xffffu), static_cast<int>(v.w >> 16));
}

// Gap bytes -> 32-bit gene indices, a warp per row: gene = previous gene + gap + 1, the row's first gap counted from
// -1.  The byte 255 marks an entry whose gene is in `exceptions` ({position in the chunk, gene}, ascending positions).
__global__ void __launch_bounds__(256) gaps_to_indices_kernel(const std::uint8_t *gaps, const std::int64_t *row_ptr, std::int64_t rows,
                                                              const int2 *exceptions, int exception_count, std::int32_t *col_idx) {
    const int lane = threadIdx.x & 31;
    const std::int64_t r = static_cast<std::int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= rows) return; // warp-uniform
    const std::int64_t begin = row_ptr[r], end = row_ptr[r + 1];
    int carry = -1;
    for (std::int64_t base = begin; base < end; base += 32) {
        const std::int64_t i = base + lane;
        const unsigned byte = i < end ? gaps[i] : 0u;
        const bool marked = i < end && byte == 255u;
        int sum = i < end && !marked ? static_cast<int>(byte) + 1 : 0;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int up = __shfl_up_sync(0xffffffffu, sum, d);
            if (lane >= d) sum += up;
        }
        int gene = carry + sum;
        unsigned todo = __ballot_sync(0xffffffffu, marked);
        while (todo != 0u) { // rare: the marked entry's gene comes from the list, and the entries behind it count on from there
            const int m = __ffs(static_cast<int>(todo)) - 1;
            todo &= todo - 1u;
            const int position = static_cast<int>(base - 0) + m; // positions are chunk-local, like row_ptr after its rebase
            int lo = 0, hi = exception_count - 1, found = 0;
            while (lo <= hi) {
                const int mid = (lo + hi) >> 1;
                const int at = exceptions[mid].x;
                if (at == position) { found = exceptions[mid].y; break; }
                if (at < position) lo = mid + 1;
                else hi = mid - 1;
            }
            const int shift = found - __shfl_sync(0xffffffffu, gene, m);
            if (lane >= m) gene += shift;
        }
        if (i < end) col_idx[i] = gene;
        carry = __shfl_sync(0xffffffffu, gene, 31);
    }
}

// One row's genes -> gap bytes at out[0..len); an entry that needs it is appended to the job's exception list through
// `except(position in the row, gene)`.
template<typename Except>
inline void gaps_of_row_scalar(const std::int32_t *genes, std::int64_t from, std::int64_t to, std::uint8_t *out, Except &&except) {
    for (std::int64_t i = from; i < to; ++i) {
        const std::int64_t gap = static_cast<std::int64_t>(genes[i]) - (i == 0 ? -1 : static_cast<std::int64_t>(genes[i - 1])) - 1;
        if (gap < 0 || gap >= 255) {
            out[i] = 255u;
            except(i, genes[i]);
        } else {
            out[i] = static_cast<std::uint8_t>(gap);
        }
    }
}
template<typename Except>
__attribute__((target("avx2"))) inline void gaps_of_row_avx2(const std::int32_t *genes, std::int64_t len, std::uint8_t *out, Except &&except) {
    if (len <= 0) return;
    // entries up to the first 32-byte boundary of the output one by one (at least the row's first, which has no
    // predecessor): the vector loop then writes whole aligned lines around the cache, which the copy engine reads next
    std::int64_t i = std::min<std::int64_t>(len, 1 + static_cast<std::int64_t>((32u - ((reinterpret_cast<std::uintptr_t>(out) + 1u) & 31u)) & 31u));
    gaps_of_row_scalar(genes, 0, i, out, except);
    const __m256i one = _mm256_set1_epi32(1), top = _mm256_set1_epi32(254);
    const __m256i order = _mm256_setr_epi32(0, 4, 1, 5, 2, 6, 3, 7);
    for (; i + 32 <= len; i += 32) {
        __m256i d[4];
        __m256i over = _mm256_setzero_si256();
        for (int j = 0; j < 4; ++j) { // (four iterations: the host compiler unrolls them)
            const __m256i a = _mm256_loadu_si256(reinterpret_cast<const __m256i *>(genes + i + 8 * j));
            const __m256i b = _mm256_loadu_si256(reinterpret_cast<const __m256i *>(genes + i + 8 * j - 1));
            d[j] = _mm256_sub_epi32(_mm256_sub_epi32(a, b), one);
            over = _mm256_or_si256(over, _mm256_xor_si256(_mm256_max_epu32(d[j], top), top)); // non-zero where a gap, as unsigned, exceeds 254
        }
        if (!_mm256_testz_si256(over, over)) {
            gaps_of_row_scalar(genes, i, i + 32, out, except);
            continue;
        }
        // 32-bit -> 16-bit -> 8-bit packs interleave the 128-bit halves: one permutation of 32-bit words puts them back
        const __m256i bytes = _mm256_packus_epi16(_mm256_packus_epi32(d[0], d[1]), _mm256_packus_epi32(d[2], d[3]));
        _mm256_stream_si256(reinterpret_cast<__m256i *>(out + i), _mm256_permutevar8x32_epi32(bytes, order));
    }
    _mm_sfence();
    gaps_of_row_scalar(genes, i, len, out, except);
}

// Narrows src[0..n) to 16 bits; returns false if an index lies outside [0, k) (dst is then not to be used).
// With AVX2: sixteen indices per step, written around the cache (dst is 32-byte aligned: the staging buffer is, and
// blocks start at multiples of kNarrowBlock); the copy engine reads them from memory next, no core does.
__attribute__((target("avx2"))) bool narrow_block_avx2(const std::int32_t *src, std::uint16_t *dst, std::int64_t n, std::uint32_t k) {
    const __m256i limit = _mm256_set1_epi32(static_cast<int>(k - 1u));
    __m256i above = _mm256_setzero_si256(); // non-zero where an index, as unsigned, exceeds k - 1
    std::int64_t i = 0;
    if ((reinterpret_cast<std::uintptr_t>(dst) & 31u) == 0u) {
        for (; i + 16 <= n; i += 16) {
            const __m256i a = _mm256_loadu_si256(reinterpret_cast<const __m256i *>(src + i));
            const __m256i b = _mm256_loadu_si256(reinterpret_cast<const __m256i *>(src + i + 8));
            above = _mm256_or_si256(above, _mm256_xor_si256(_mm256_max_epu32(a, limit), limit));
            above = _mm256_or_si256(above, _mm256_xor_si256(_mm256_max_epu32(b, limit), limit));
            // the pack interleaves the two sources' 128-bit halves: put them back in order
            _mm256_stream_si256(reinterpret_cast<__m256i *>(dst + i), _mm256_permute4x64_epi64(_mm256_packus_epi32(a, b), 0xd8));
        }
        _mm_sfence();
    }
    std::uint32_t outside = _mm256_testz_si256(above, above) ? 0u : 1u;
    for (; i < n; ++i) {
        const std::uint32_t v = static_cast<std::uint32_t>(src[i]);
        outside |= v >= k ? 1u : 0u;
        dst[i] = static_cast<std::uint16_t>(v);
    }
    return outside == 0u;
}
bool narrow_block(const std::int32_t *src, std::uint16_t *dst, std::int64_t n, std::uint32_t k) {
    static const bool avx2 = __builtin_cpu_supports("avx2") != 0;
    if (avx2) return narrow_block_avx2(src, dst, n, k);
    std::uint32_t outside = 0;
    for (std::int64_t i = 0; i < n; ++i) {
        const std::uint32_t v = static_cast<std::uint32_t>(src[i]);
        outside |= v >= k ? 1u : 0u;
        dst[i] = static_cast<std::uint16_t>(v);
    }
    return outside == 0u;
}

// A few host threads that rewrite one chunk's indices at a time, in blocks claimed with an atomic counter (kNarrowBlock
// entries of the 16-bit form, kGapRows rows of the gap form); the calling thread takes blocks too and returns when every
// block is done.
constexpr std::int64_t kNarrowBlock = 1 << 18;
constexpr std::int64_t kGapRows = 64;
struct narrow_pool {
    std::vector<std::thread> workers;
    std::mutex m;
    std::condition_variable wake, done;
    bool stop = false;
    int active = 0; // workers inside work(): a new job is set up only when none is
    std::uint64_t generation = 0;
    // the job
    const std::int32_t *src = nullptr;
    std::uint16_t *dst = nullptr;
    std::int64_t n = 0;
    std::uint32_t k = 0;
    std::atomic<std::int64_t> next{0};
    std::atomic<std::int64_t> blocks_left{0};
    std::atomic<int> all_inside{1};
    // the gap form's job: rows [0, rows) of the chunk, row_ptr with the caller's absolute offsets (first = row_ptr[0])
    bool gaps = false;
    const std::int64_t *row_ptr = nullptr;
    std::int64_t rows = 0;
    std::uint8_t *dst8 = nullptr;
    // exception records per block of rows: a block is rewritten by one thread, row after row, so its records ascend by
    // position, and the blocks' lists joined in block order are the chunk's list in ascending order
    std::vector<std::vector<int2>> block_exceptions;

    void gap_rows(std::int64_t block, std::int64_t r0, std::int64_t r1) {
        static const bool avx2 = __builtin_cpu_supports("avx2") != 0;
        const std::int64_t first = row_ptr[0];
        std::vector<int2> &list = block_exceptions[static_cast<std::size_t>(block)];
        for (std::int64_t r = r0; r < r1; ++r) {
            const std::int64_t at = row_ptr[r] - first, len = row_ptr[r + 1] - row_ptr[r];
            auto except = [&](std::int64_t i, std::int32_t gene) { list.push_back(make_int2(static_cast<int>(at + i), gene)); };
            if (avx2) gaps_of_row_avx2(src + at, len, dst8 + at, except);
            else gaps_of_row_scalar(src + at, 0, len, dst8 + at, except);
        }
    }
    void work() {
        for (;;) {
            const std::int64_t b = next.fetch_add(1, std::memory_order_relaxed);
            if (gaps) {
                const std::int64_t r0 = b * kGapRows;
                if (r0 >= rows) return;
                gap_rows(b, r0, std::min(rows, r0 + kGapRows));
            } else {
                const std::int64_t lo = b * kNarrowBlock;
                if (lo >= n) return;
                const std::int64_t len = std::min<std::int64_t>(kNarrowBlock, n - lo);
                if (!narrow_block(src + lo, dst + lo, len, k)) all_inside.store(0, std::memory_order_relaxed);
            }
            if (blocks_left.fetch_sub(1, std::memory_order_acq_rel) == 1) {
                std::lock_guard<std::mutex> lock(m);
                done.notify_all();
            }
        }
    }
    void loop() {
        std::uint64_t seen = 0;
        for (;;) {
            {
                std::unique_lock<std::mutex> lock(m);
                wake.wait(lock, [&] { return stop || generation != seen; });
                if (stop) return;
                seen = generation;
                ++active;
            }
            work();
            {
                std::lock_guard<std::mutex> lock(m);
                --active;
            }
            done.notify_all();
        }
    }
    void start(int threads) {
        for (int i = 0; i < threads; ++i) workers.emplace_back([this] { loop(); });
    }
    // The job's fields change only under the lock and only while no worker is inside work(): a worker that wakes late
    // for an earlier job finds that job's counter run out, or this job complete with all its fields.
    template<typename Setup>
    void run_job(std::int64_t blocks, Setup &&setup) {
        {
            std::unique_lock<std::mutex> lock(m);
            done.wait(lock, [&] { return active == 0; });
            setup();
            next.store(0, std::memory_order_relaxed);
            blocks_left.store(blocks, std::memory_order_relaxed);
            ++generation;
        }
        wake.notify_all();
        work();
        std::unique_lock<std::mutex> lock(m);
        done.wait(lock, [&] { return blocks_left.load(std::memory_order_acquire) <= 0; });
    }
    // 16-bit words; false: an index outside [0, genes)
    bool run(const std::int32_t *from, std::uint16_t *to, std::int64_t count, std::uint32_t genes) {
        if (count <= 0) return true;
        run_job((count + kNarrowBlock - 1) / kNarrowBlock, [&] {
            gaps = false; src = from; dst = to; n = count; k = genes;
            all_inside.store(1, std::memory_order_relaxed);
        });
        return all_inside.load(std::memory_order_relaxed) != 0;
    }
    // gap bytes of the chunk's rows (ptr = the chunk's row pointers, absolute; from = the chunk's first index); returns the
    // number of exception records, sorted by position, or -1 if the list has no room for them
    int run_gaps(const std::int32_t *from, const std::int64_t *ptr, std::int64_t row_count, std::uint8_t *to, int2 *list, int room) {
        if (row_count <= 0) return 0;
        const std::int64_t blocks = (row_count + kGapRows - 1) / kGapRows;
        run_job(blocks, [&] {
            gaps = true; src = from; row_ptr = ptr; rows = row_count; dst8 = to;
            if (block_exceptions.size() < static_cast<std::size_t>(blocks)) block_exceptions.resize(static_cast<std::size_t>(blocks));
            for (std::int64_t b = 0; b < blocks; ++b) block_exceptions[static_cast<std::size_t>(b)].clear();
        });
        std::size_t count = 0;
        for (std::int64_t b = 0; b < blocks; ++b) count += block_exceptions[static_cast<std::size_t>(b)].size();
        if (count > static_cast<std::size_t>(room)) return -1;
        for (std::int64_t b = 0; b < blocks; ++b) {
            const std::vector<int2> &part = block_exceptions[static_cast<std::size_t>(b)];
            if (!part.empty()) std::memcpy(list, part.data(), part.size() * sizeof(int2));
            list += part.size();
        }
        return static_cast<int>(count);
    }
    ~narrow_pool() {
        {
            std::lock_guard<std::mutex> lock(m);
            stop = true;
        }
        wake.notify_all();
        for (std::thread &t : workers) t.join();
    }
};

int usable_host_threads() {
    cpu_set_t set;
    CPU_ZERO(&set);
    if (sched_getaffinity(0, sizeof(set), &set) == 0) return std::max(1, CPU_COUNT(&set));
    return std::max(1u, std::thread::hardware_concurrency());
}

struct chunk_buffer {
    std::int64_t *row_ptr = nullptr;
    std::int64_t *packed_row_ptr = nullptr; // 4-bit codes only
    std::int32_t *col_idx = nullptr;
    unsigned char *narrow_idx = nullptr;     // device: the chunk's gap bytes or 16-bit indices as they arrive
    unsigned char *narrow_host = nullptr;    // pinned host staging of the same
    int2 *exceptions = nullptr;              // device: {position, gene} of the gap form's entries that do not fit a byte
    int2 *exceptions_host = nullptr;         // pinned host staging of the same
    std::uint8_t *packed = nullptr;
    float *row_offsets = nullptr;           // row-offset policy only
    float *y = nullptr;
    void *workspace = nullptr;
    cudaEvent_t copied_in = nullptr, computed = nullptr, copied_out = nullptr;
};

} // namespace

struct cb200_host_stage {
    cb200_host_stage_options o{};
    int sm_count = 0;
    fwd_schedule schedule = fwd_schedule::warp_per_row;
    cudaStream_t h2d = nullptr, compute = nullptr, d2h = nullptr;
    void *w = nullptr;
    float *scales = nullptr, *offsets = nullptr;
    cudaEvent_t shared_in = nullptr;
    chunk_buffer ring[kMaxBuffers];
    std::uint64_t device_bytes = 0;
    std::uint64_t workspace_bytes = 0;
    narrow_pool *pool = nullptr; // non-null: gene indices may travel in a shorter form
    bool words16 = false;        // the shorter form is 16-bit words (else gap bytes)
    int exception_room = 0;      // records the exception lists hold
    int narrow_pause = 0;        // calls that still copy 32-bit indices after one in which the host narrowed too slowly
    double rewrite_share = 1.0;  // gap form: share of a chunk's entries the host rewrites (the rest go as 32-bit indices)
};

namespace {

template<typename T>
cudaError_t device_alloc(T **p, std::uint64_t count, std::uint64_t *total) {
    const std::uint64_t bytes = std::max<std::uint64_t>(count, 1u) * sizeof(T);
    *total += bytes;
    return cudaMalloc(reinterpret_cast<void **>(p), bytes);
}

} // namespace

extern "C" {

void cb200_host_stage_destroy(cb200_host_stage *s) {
    if (s == nullptr) return;
    device_scope scope(s->o.device);
    for (cudaStream_t st : {s->h2d, s->compute, s->d2h})
        if (st != nullptr) cudaStreamSynchronize(st);
    for (chunk_buffer &b : s->ring) {
        cudaFree(b.row_ptr); cudaFree(b.packed_row_ptr); cudaFree(b.col_idx); cudaFree(b.packed); cudaFree(b.narrow_idx); cudaFree(b.exceptions);
        if (b.narrow_host != nullptr) cudaFreeHost(b.narrow_host);
        if (b.exceptions_host != nullptr) cudaFreeHost(b.exceptions_host);
        cudaFree(b.row_offsets); cudaFree(b.y); cudaFree(b.workspace);
        for (cudaEvent_t e : {b.copied_in, b.computed, b.copied_out})
            if (e != nullptr) cudaEventDestroy(e);
    }
    cudaFree(s->w); cudaFree(s->scales); cudaFree(s->offsets);
    if (s->shared_in != nullptr) cudaEventDestroy(s->shared_in);
    for (cudaStream_t st : {s->h2d, s->compute, s->d2h})
        if (st != nullptr) cudaStreamDestroy(st);
    delete s->pool;
    delete s;
}

cb200_status cb200_host_stage_create(const cb200_host_stage_options *o, cb200_host_stage **out) {
    clear_error();
    if (out == nullptr) return fail(CB200_STATUS_INVALID_ARGUMENT, "host_stage_create needs an output handle");
    *out = nullptr;
    if (o == nullptr || o->version != CB200_ABI_VERSION || o->size < sizeof(cb200_host_stage_options))
        return fail(CB200_STATUS_INVALID_ARGUMENT, "bad cb200_host_stage_options header");
    if (o->k <= 0 || o->n <= 0 || o->max_chunk_rows <= 0 || o->max_chunk_nnz <= 0 || o->max_chunk_rows > 0x7fffffffll)
        return fail(CB200_STATUS_INVALID_SHAPE, "a stage needs positive k, n and chunk capacities");
    if (o->bits != 8 && o->bits != 4) return fail(CB200_STATUS_UNSUPPORTED, "bits must be 4 or 8, got %d", o->bits);
    if (o->policy != CB200_DECODE_PER_GENE_AFFINE && o->policy != CB200_DECODE_COLUMN_SCALE_ROW_OFFSET)
        return fail(CB200_STATUS_UNSUPPORTED, "unknown decode policy %d", o->policy);
    if (o->dense_dtype != CB200_DTYPE_F32 && o->dense_dtype != CB200_DTYPE_BF16) return fail(CB200_STATUS_UNSUPPORTED, "W must be fp32 or bf16");
    if (o->chunk_buffers < 2 || o->chunk_buffers > kMaxBuffers) return fail(CB200_STATUS_INVALID_ARGUMENT, "2..%d chunk buffers", kMaxBuffers);
    int visible = 0, major = 0;
    CB200_CUDA_OK(cudaGetDeviceCount(&visible));
    if (o->device < 0 || o->device >= visible) return fail(CB200_STATUS_INVALID_STREAM, "device %d not present (%d visible)", o->device, visible);
    CB200_CUDA_OK(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, o->device));
    if (major != 10) return fail(CB200_STATUS_UNSUPPORTED, "this library is built for sm_100a only");
    device_scope scope(o->device);
    CB200_CUDA_OK(scope.status);
    cb200_host_stage *s = new (std::nothrow) cb200_host_stage{};
    if (s == nullptr) return fail(CB200_STATUS_INTERNAL_ERROR, "out of host memory");
    s->o = *o;
    cudaError_t err = cudaDeviceGetAttribute(&s->sm_count, cudaDevAttrMultiProcessorCount, o->device);
    const std::uint64_t elem = o->dense_dtype == CB200_DTYPE_BF16 ? 2u : 4u;
    // the gene-tiled kernel where the shape allows it (its fixed cost per visit needs rows of some length,
    // which a chunk of a single-cell matrix has); else one warp per row
    const std::int64_t row_bytes = o->n * static_cast<std::int64_t>(elem);
    const bool tiled_shape = (o->n == 32 || o->n == 64 || o->n == 128) && row_bytes <= 256;
    const double mean = static_cast<double>(o->max_chunk_nnz) / static_cast<double>(o->max_chunk_rows);
    const double per_visit = mean * (98304.0 / static_cast<double>(row_bytes)) / static_cast<double>(o->k);
    s->schedule = tiled_shape && per_visit >= 6.0 ? fwd_schedule::gene_tiled : fwd_schedule::warp_per_row;
    s->workspace_bytes = qcsr_tiled_workspace_bytes();
    for (cudaStream_t *st : {&s->h2d, &s->compute, &s->d2h})
        if (err == cudaSuccess) err = cudaStreamCreateWithFlags(st, cudaStreamNonBlocking);
    if (err == cudaSuccess) err = cudaEventCreateWithFlags(&s->shared_in, cudaEventDisableTiming);
    unsigned char *w_bytes = nullptr;
    if (err == cudaSuccess) err = device_alloc(&w_bytes, static_cast<std::uint64_t>(o->k) * o->n * elem, &s->device_bytes);
    s->w = w_bytes;
    if (err == cudaSuccess) err = device_alloc(&s->scales, o->k, &s->device_bytes);
    if (err == cudaSuccess && o->policy == CB200_DECODE_PER_GENE_AFFINE) err = device_alloc(&s->offsets, o->k, &s->device_bytes);
    for (int b = 0; b < o->chunk_buffers && err == cudaSuccess; ++b) {
        chunk_buffer &c = s->ring[b];
        err = device_alloc(&c.row_ptr, o->max_chunk_rows + 1, &s->device_bytes);
        if (err == cudaSuccess && o->bits == 4) err = device_alloc(&c.packed_row_ptr, o->max_chunk_rows + 1, &s->device_bytes);
        if (err == cudaSuccess) err = device_alloc(&c.col_idx, o->max_chunk_nnz + 8, &s->device_bytes);
        // 4-bit rows are padded to whole bytes: at most one byte per row on top of nnz / 2
        const std::uint64_t code_bytes = o->bits == 8 ? static_cast<std::uint64_t>(o->max_chunk_nnz)
                                                      : static_cast<std::uint64_t>(o->max_chunk_nnz) / 2u + static_cast<std::uint64_t>(o->max_chunk_rows);
        if (err == cudaSuccess) err = device_alloc(&c.packed, code_bytes + 16u, &s->device_bytes);
        if (err == cudaSuccess && o->policy == CB200_DECODE_COLUMN_SCALE_ROW_OFFSET) err = device_alloc(&c.row_offsets, o->max_chunk_rows, &s->device_bytes);
        if (err == cudaSuccess) err = device_alloc(&c.y, static_cast<std::uint64_t>(o->max_chunk_rows) * o->n, &s->device_bytes);
        unsigned char *ws = nullptr;
        if (err == cudaSuccess) err = device_alloc(&ws, s->workspace_bytes, &s->device_bytes);
        c.workspace = ws;
        for (cudaEvent_t *e : {&c.copied_in, &c.computed, &c.copied_out})
            if (err == cudaSuccess) err = cudaEventCreateWithFlags(e, cudaEventDisableTiming);
    }
    // a shorter form of the gene indices on the link: needs host threads to rewrite them with
    const int host_threads = std::min(o->host_threads > 0 ? o->host_threads : usable_host_threads(), 16);
    if (o->narrow_indices < -1 || o->narrow_indices > 2 || o->host_threads < 0) {
        cb200_host_stage_destroy(s);
        return fail(CB200_STATUS_INVALID_ARGUMENT, "narrow_indices is -1, 0, 1 or 2, host_threads is not negative");
    }
    const bool want_words = o->narrow_indices == 1 && o->k <= 65536;
    const bool want_gaps = o->narrow_indices == 2 || (o->narrow_indices == 0 && host_threads >= 4);
    if (err == cudaSuccess && (want_words || want_gaps) && o->max_chunk_nnz < 0x7fffff00ll) {
        s->words16 = want_words;
        s->exception_room = static_cast<int>(std::max<std::int64_t>(4096, o->max_chunk_nnz / 128));
        const std::uint64_t bytes = (static_cast<std::uint64_t>(o->max_chunk_nnz) + 64u) * (want_words ? 2u : 1u);
        for (int b = 0; b < o->chunk_buffers && err == cudaSuccess; ++b) {
            chunk_buffer &c = s->ring[b];
            err = device_alloc(&c.narrow_idx, bytes, &s->device_bytes);
            if (err == cudaSuccess) err = cudaHostAlloc(reinterpret_cast<void **>(&c.narrow_host), bytes, cudaHostAllocDefault);
            if (err == cudaSuccess && !want_words) {
                err = device_alloc(&c.exceptions, static_cast<std::uint64_t>(s->exception_room), &s->device_bytes);
                if (err == cudaSuccess)
                    err = cudaHostAlloc(reinterpret_cast<void **>(&c.exceptions_host), static_cast<std::size_t>(s->exception_room) * sizeof(int2), cudaHostAllocDefault);
            }
        }
        if (err == cudaSuccess) {
            s->pool = new (std::nothrow) narrow_pool{};
            if (s->pool != nullptr) s->pool->start(std::max(host_threads - 1, 0)); // the calling thread rewrites too
        } else if (o->narrow_indices == 0) {
            // no room for the staging buffers (pinned host memory, mostly): the stage works without the shorter form
            cudaGetLastError();
            err = cudaSuccess;
            for (int b = 0; b < o->chunk_buffers; ++b) {
                chunk_buffer &c = s->ring[b];
                cudaFree(c.narrow_idx); cudaFree(c.exceptions);
                if (c.narrow_host != nullptr) cudaFreeHost(c.narrow_host);
                if (c.exceptions_host != nullptr) cudaFreeHost(c.exceptions_host);
                c.narrow_idx = nullptr; c.exceptions = nullptr; c.narrow_host = nullptr; c.exceptions_host = nullptr;
            }
            cudaGetLastError();
        }
    }
    if (err != cudaSuccess) {
        cudaGetLastError();
        cb200_host_stage_destroy(s);
        return fail(CB200_STATUS_CUDA_ERROR, "host stage: %s", cudaGetErrorString(err));
    }
    *out = s;
    return CB200_STATUS_SUCCESS;
}

uint64_t cb200_host_stage_device_bytes(const cb200_host_stage *s) { return s != nullptr ? s->device_bytes : 0u; }

int64_t cb200_host_encode_gene_gaps(const int32_t *col_idx, const int64_t *row_ptr, int64_t rows, uint8_t *gaps, int32_t *exception_positions,
                                    int32_t *exception_genes, int64_t room, int32_t threads) {
    clear_error();
    if (rows < 0 || room < 0 || threads < 1 || threads > 64 || row_ptr == nullptr || (rows > 0 && row_ptr[rows] > row_ptr[0] && (col_idx == nullptr || gaps == nullptr)) ||
        (room > 0 && (exception_positions == nullptr || exception_genes == nullptr))) {
        fail(CB200_STATUS_INVALID_ARGUMENT, "encode_gene_gaps: null arrays, or rows / room / threads out of range");
        return -2;
    }
    if (rows == 0 || row_ptr[rows] - row_ptr[0] >= 0x7fffff00ll) return rows == 0 ? 0 : -2;
    const int capped = static_cast<int>(std::min<std::int64_t>(room, 0x7fffffff));
    std::vector<int2> list(static_cast<std::size_t>(capped));
    narrow_pool pool;
    pool.start(threads - 1);
    const int count = pool.run_gaps(col_idx + row_ptr[0], row_ptr, rows, gaps, list.data(), capped);
    for (int i = 0; i < count; ++i) {
        exception_positions[i] = list[static_cast<std::size_t>(i)].x;
        exception_genes[i] = list[static_cast<std::size_t>(i)].y;
    }
    return count;
}

cb200_status cb200_host_forward(cb200_host_stage *s, const cb200_qcsr *x, const void *w, int64_t w_ld, float *y, int64_t y_ld,
                                float alpha, uint64_t *h2d_bytes, uint64_t *d2h_bytes) {
    clear_error();
    if (s == nullptr) return fail(CB200_STATUS_INVALID_ARGUMENT, "null host stage");
    if (x == nullptr || x->version != CB200_ABI_VERSION || x->size < sizeof(cb200_qcsr)) return fail(CB200_STATUS_INVALID_ARGUMENT, "bad cb200_qcsr header");
    const cb200_host_stage_options &o = s->o;
    if (x->cols != o.k || x->bits != o.bits || x->policy != o.policy) return fail(CB200_STATUS_INVALID_SHAPE, "the matrix disagrees with the stage");
    if (x->rows < 0 || w_ld != o.n || y_ld < o.n) return fail(CB200_STATUS_INVALID_SHAPE, "W must be contiguous (ld == n) and y_ld >= n");
    if (x->row_ptr == nullptr || w == nullptr || (x->rows != 0 && y == nullptr) || x->scales == nullptr ||
        (x->nnz != 0 && (x->col_idx == nullptr || x->packed_values == nullptr)) || (o.bits == 4 && x->packed_row_ptr == nullptr))
        return fail(CB200_STATUS_INVALID_ARGUMENT, "the host matrix has null arrays (scales are required; 4-bit codes need packed_row_ptr)");
    const bool row_policy = o.policy == CB200_DECODE_COLUMN_SCALE_ROW_OFFSET;
    const std::int64_t *rp = x->row_ptr;
    const std::int64_t *prp = o.bits == 8 ? x->row_ptr : x->packed_row_ptr;
    // chunk plan: as many rows as fit the buffers, at least one
    std::vector<std::int64_t> bounds{0};
    for (std::int64_t r = 0; r < x->rows;) {
        std::int64_t hi = std::min<std::int64_t>(x->rows, r + o.max_chunk_rows);
        // largest end with rp[end] - rp[r] <= max_chunk_nnz (row pointers ascend)
        const std::int64_t *cut = std::upper_bound(rp + r, rp + hi + 1, rp[r] + o.max_chunk_nnz);
        hi = std::min<std::int64_t>(hi, static_cast<std::int64_t>(cut - rp) - 1);
        if (hi <= r) return fail(CB200_STATUS_INSUFFICIENT_WORKSPACE, "row %lld holds %lld entries, a chunk buffer %lld", (long long)r,
                                 (long long)(rp[r + 1] - rp[r]), (long long)o.max_chunk_nnz);
        bounds.push_back(hi);
        r = hi;
    }
    device_scope scope(o.device);
    CB200_CUDA_OK(scope.status);
    const std::uint64_t elem = o.dense_dtype == CB200_DTYPE_BF16 ? 2u : 4u;
    std::uint64_t in_bytes = 0, out_bytes = 0;
    // operands every chunk shares
    const std::uint64_t w_bytes = static_cast<std::uint64_t>(o.k) * o.n * elem;
    CB200_CUDA_OK(cudaMemcpyAsync(s->w, w, w_bytes, cudaMemcpyHostToDevice, s->h2d));
    CB200_CUDA_OK(cudaMemcpyAsync(s->scales, x->scales, static_cast<std::uint64_t>(o.k) * 4u, cudaMemcpyHostToDevice, s->h2d));
    in_bytes += w_bytes + static_cast<std::uint64_t>(o.k) * 4u;
    if (!row_policy && x->offsets != nullptr) {
        CB200_CUDA_OK(cudaMemcpyAsync(s->offsets, x->offsets, static_cast<std::uint64_t>(o.k) * 4u, cudaMemcpyHostToDevice, s->h2d));
        in_bytes += static_cast<std::uint64_t>(o.k) * 4u;
    }
    CB200_CUDA_OK(cudaEventRecord(s->shared_in, s->h2d));
    CB200_CUDA_OK(cudaStreamWaitEvent(s->compute, s->shared_in, 0));

    const int buffers = o.chunk_buffers;
    // The host rewrites while the link moves: per entry the link carries 2 bytes of a rewritten entry (gap and code) and 5
    // of one that goes as it is, and the host spends 1 / R on a rewritten one (R = its rewriting rate).  Both are busy
    // for the same time when the host rewrites the share 5 R / (L + 3 R) of the entries, L = the link's rate, and the rest
    // of a chunk's rows go as 32-bit indices, enqueued first so that the link has them to move while the host works.  At
    // R = 19 G entries/s and L = 50 GB/s that is 0.89 of the entries and 21 G entries/s for the call; a host that rewrites
    // 8 G/s rewrites 0.54 of them for 15 G/s, where 32-bit indices alone give 10.  The better of the first two rewritten
    // chunks of a call sets the share for the rest of the call and for the next call; a host below kRewriteMinRate (or
    // rows whose genes do not ascend) sends 32-bit indices for the rest of this call and the next few.
    bool narrow = s->pool != nullptr;
    int timed_chunks = 0;        // rewritten chunks of this call whose rate has been looked at (the first starts the threads cold)
    double best_rate = 0.0;
    constexpr double kRewriteMinRate = 3.0e9, kLinkRate = 50.0e9;
    constexpr int kNarrowPauseCalls = 8; // a call that found the host too slow is not the only one to pay for finding out
    if (narrow && o.narrow_indices == 0 && s->narrow_pause > 0) {
        --s->narrow_pause;
        narrow = false;
    }
    double share = o.narrow_indices == 0 && !s->words16 ? s->rewrite_share : 1.0;
    for (std::size_t c = 0; c + 1 < bounds.size(); ++c) {
        chunk_buffer &b = s->ring[c % static_cast<std::size_t>(buffers)];
        const std::int64_t r0 = bounds[c], r1 = bounds[c + 1], rows = r1 - r0;
        const std::int64_t n0 = rp[r0], nnz = rp[r1] - n0, p0 = prp[r0], code_bytes = prp[r1] - p0;
        // ---- in: one copy per array, once the buffer's previous chunk has been multiplied
        if (c >= static_cast<std::size_t>(buffers)) CB200_CUDA_OK(cudaStreamWaitEvent(s->h2d, b.computed, 0));
        CB200_CUDA_OK(cudaMemcpyAsync(b.row_ptr, rp + r0, static_cast<std::uint64_t>(rows + 1) * 8u, cudaMemcpyHostToDevice, s->h2d));
        in_bytes += static_cast<std::uint64_t>(rows + 1) * 8u;
        if (o.bits == 4) {
            CB200_CUDA_OK(cudaMemcpyAsync(b.packed_row_ptr, prp + r0, static_cast<std::uint64_t>(rows + 1) * 8u, cudaMemcpyHostToDevice, s->h2d));
            in_bytes += static_cast<std::uint64_t>(rows + 1) * 8u;
        }
        bool narrowed = false;
        int exception_count = 0;
        std::int64_t head_rows = rows, head_nnz = nnz; // what the host rewrites: the chunk's first rows
        if (nnz > 0) {
            if (narrow && share < 1.0) {
                const std::int64_t target = n0 + static_cast<std::int64_t>(share * static_cast<double>(nnz));
                head_rows = std::min<std::int64_t>(rows, std::max<std::int64_t>(0, (std::upper_bound(rp + r0, rp + r1 + 1, target) - (rp + r0)) - 1));
                head_nnz = rp[r0 + head_rows] - n0;
            }
            // what needs no work of the host goes first: the codes, and the indices of the rows that are not rewritten
            CB200_CUDA_OK(cudaMemcpyAsync(b.packed, x->packed_values + p0, static_cast<std::uint64_t>(code_bytes), cudaMemcpyHostToDevice, s->h2d));
            in_bytes += static_cast<std::uint64_t>(code_bytes);
            if (narrow && head_nnz < nnz) {
                CB200_CUDA_OK(cudaMemcpyAsync(b.col_idx + head_nnz, x->col_idx + n0 + head_nnz, static_cast<std::uint64_t>(nnz - head_nnz) * 4u, cudaMemcpyHostToDevice, s->h2d));
                in_bytes += static_cast<std::uint64_t>(nnz - head_nnz) * 4u;
            }
            if (narrow && head_nnz > 0) {
                // the staging buffer's previous copy (buffers chunks ago) has left it
                if (c >= static_cast<std::size_t>(buffers)) CB200_CUDA_OK(cudaEventSynchronize(b.copied_in));
                const auto t0 = std::chrono::steady_clock::now();
                if (s->words16) {
                    narrowed = s->pool->run(x->col_idx + n0, reinterpret_cast<std::uint16_t *>(b.narrow_host), nnz, static_cast<std::uint32_t>(o.k));
                } else {
                    exception_count = s->pool->run_gaps(x->col_idx + n0, rp + r0, head_rows, b.narrow_host, b.exceptions_host, s->exception_room);
                    // worth it while the list is short: with one record per eight entries the form costs as much as 16-bit words
                    narrowed = exception_count >= 0 && static_cast<std::int64_t>(exception_count) * 8 <= head_nnz;
                    if (!narrowed) exception_count = 0;
                }
                const double seconds = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
                best_rate = std::max(best_rate, static_cast<double>(head_nnz) / std::max(seconds, 1e-9));
                ++timed_chunks;
                const bool last_chunk = c + 2 == bounds.size();
                if (o.narrow_indices == 0 && (timed_chunks == 2 || last_chunk || !narrowed)) {
                    if (!narrowed || best_rate < kRewriteMinRate) {
                        narrow = false; // 32-bit copies from the next chunk on, and for the next calls
                        s->narrow_pause = kNarrowPauseCalls;
                    } else if (!s->words16 && timed_chunks <= 2) {
                        share = std::min(1.0, std::max(0.25, 5.0 * best_rate / (kLinkRate + 3.0 * best_rate)));
                        s->rewrite_share = share;
                    }
                }
            }
            if (narrowed) {
                const std::uint64_t bytes = (static_cast<std::uint64_t>(head_nnz) * (s->words16 ? 2u : 1u) + 15u) & ~static_cast<std::uint64_t>(15u);
                CB200_CUDA_OK(cudaMemcpyAsync(b.narrow_idx, b.narrow_host, bytes, cudaMemcpyHostToDevice, s->h2d));
                in_bytes += bytes;
                if (exception_count > 0) {
                    CB200_CUDA_OK(cudaMemcpyAsync(b.exceptions, b.exceptions_host, static_cast<std::uint64_t>(exception_count) * sizeof(int2), cudaMemcpyHostToDevice, s->h2d));
                    in_bytes += static_cast<std::uint64_t>(exception_count) * sizeof(int2);
                }
            } else {
                // (all of the chunk's indices, or the rows that were to be rewritten and could not be)
                const std::int64_t plain = narrow || head_nnz < nnz ? head_nnz : nnz;
                CB200_CUDA_OK(cudaMemcpyAsync(b.col_idx, x->col_idx + n0, static_cast<std::uint64_t>(plain) * 4u, cudaMemcpyHostToDevice, s->h2d));
                in_bytes += static_cast<std::uint64_t>(plain) * 4u;
            }
        }
        if (row_policy && x->offsets != nullptr) {
            CB200_CUDA_OK(cudaMemcpyAsync(b.row_offsets, x->offsets + r0, static_cast<std::uint64_t>(rows) * 4u, cudaMemcpyHostToDevice, s->h2d));
            in_bytes += static_cast<std::uint64_t>(rows) * 4u;
        }
        CB200_CUDA_OK(cudaEventRecord(b.copied_in, s->h2d));
        // ---- multiply, once the chunk is in and the buffer's previous result is out
        CB200_CUDA_OK(cudaStreamWaitEvent(s->compute, b.copied_in, 0));
        if (c >= static_cast<std::size_t>(buffers)) CB200_CUDA_OK(cudaStreamWaitEvent(s->compute, b.copied_out, 0));
        const unsigned grid = static_cast<unsigned>((rows + 1 + 255) / 256);
        rebase_kernel<<<grid, 256, 0, s->compute>>>(b.row_ptr, rows + 1, n0);
        if (o.bits == 4) rebase_kernel<<<grid, 256, 0, s->compute>>>(b.packed_row_ptr, rows + 1, p0);
        count_launch(o.bits == 4 ? 2 : 1);
        if (narrowed && s->words16) {
            const std::int64_t eights = (nnz + 7) / 8;
            widen_indices_kernel<<<static_cast<unsigned>((eights + 255) / 256), 256, 0, s->compute>>>(
                reinterpret_cast<const uint4 *>(b.narrow_idx), reinterpret_cast<int4 *>(b.col_idx), eights);
            count_launch();
        } else if (narrowed) { // after the rebase: the kernel reads the chunk's own row pointers
            gaps_to_indices_kernel<<<static_cast<unsigned>((head_rows + 7) / 8), 256, 0, s->compute>>>(b.narrow_idx, b.row_ptr, head_rows, b.exceptions,
                                                                                                     exception_count, b.col_idx);
            count_launch();
        }
        CB200_CUDA_OK(cudaGetLastError());
        const qcsr_view view{rows, o.k, nnz, o.bits, o.policy, b.row_ptr, o.bits == 4 ? b.packed_row_ptr : nullptr, b.col_idx, b.packed,
                             s->scales, row_policy ? (x->offsets != nullptr ? b.row_offsets : nullptr) : (x->offsets != nullptr ? s->offsets : nullptr)};
        const dense_args d{s->w, o.n, o.dense_dtype, b.y, o.n, o.n, alpha, 0.0f};
        const cb200_status st = launch_qcsr_forward(view, d, 0, rows, s->schedule, nullptr, nullptr, false, b.workspace, s->workspace_bytes,
                                                    s->sm_count, s->compute);
        if (st != CB200_STATUS_SUCCESS) return st;
        CB200_CUDA_OK(cudaEventRecord(b.computed, s->compute));
        // ---- out
        CB200_CUDA_OK(cudaStreamWaitEvent(s->d2h, b.computed, 0));
        if (y_ld == o.n) {
            CB200_CUDA_OK(cudaMemcpyAsync(y + r0 * y_ld, b.y, static_cast<std::uint64_t>(rows) * o.n * 4u, cudaMemcpyDeviceToHost, s->d2h));
        } else {
            CB200_CUDA_OK(cudaMemcpy2DAsync(y + r0 * y_ld, static_cast<std::size_t>(y_ld) * 4u, b.y, static_cast<std::size_t>(o.n) * 4u,
                                            static_cast<std::size_t>(o.n) * 4u, static_cast<std::size_t>(rows), cudaMemcpyDeviceToHost, s->d2h));
        }
        out_bytes += static_cast<std::uint64_t>(rows) * o.n * 4u;
        CB200_CUDA_OK(cudaEventRecord(b.copied_out, s->d2h));
    }
    CB200_CUDA_OK(cudaStreamSynchronize(s->d2h));
    CB200_CUDA_OK(cudaStreamSynchronize(s->compute));
    CB200_CUDA_OK(cudaStreamSynchronize(s->h2d));
    // the kernels' bounded waits: a status word per ring buffer, all of them zero unless a wait ran out
    const std::size_t used = std::min<std::size_t>(bounds.size() - 1u, static_cast<std::size_t>(buffers));
    for (std::size_t b = 0; b < used; ++b) {
        int word = 0;
        CB200_CUDA_OK(cudaMemcpy(&word, s->ring[b].workspace, sizeof(int), cudaMemcpyDeviceToHost));
        if (word != 0) return fail(CB200_STATUS_DEVICE_WAIT_TIMEOUT, "a kernel of the call gave up a bounded wait: y is not valid");
    }
    if (h2d_bytes != nullptr) *h2d_bytes = in_bytes;
    if (d2h_bytes != nullptr) *d2h_bytes = out_bytes;
    return CB200_STATUS_SUCCESS;
}

} // extern "C"
