// CSR -> physical Blocked-ELL lowering on the device, under a row order and a feature order.
//
// Reference counterpart (host loops): query_bell_candidates_host / evaluate
// (src/compute/math/physical_bell_candidates.cc:131-238), validate (src/compute/math/physical_bell.cc:27-80)
// and materialize_bell_candidate_host (physical_bell.cc:98-200).  Same geometry, metrics, column indices
// and value placement, bit for bit; the reference's FNV-1a identity chains are sequential host work over
// arrays the caller already owns and stay with the caller.
//
// Conventions (physical_bell.cc:44-58): feature_permutation[execution] = canonical,
// inverse_feature_permutation[canonical] = execution, row_permutation[execution row] = canonical row.
// Every semantic feature block of the execution order is padded on its own to a multiple of the
// block size, so a physical block column never spans two semantic blocks.
//
// One CTA per block row (8, 16 or 32 execution rows).  The block columns a block row touches are a
// bitmap in shared memory (one bit per physical block column): the lanes of a warp read a row's
// feature ids coalesced, map each to its physical block column and set the bit.  The number of set
// bits is the block row's ELL demand (query); the rank of a bit among the set bits -- a word-level
// exclusive scan plus a popcount -- is the slot of that block column, ascending as in the reference
// (materialize), and tells every stored value where it goes.
#include "kernels.cuh"

#include <algorithm>
#include <vector>

namespace cb200 {
namespace {

constexpr int kLowerThreads = 256;
constexpr std::size_t kMaxBitmapBytes = 96 * 1024; // two arrays of this size at most: bitmap and ranks

struct lowering_params {
    const std::uint32_t *row_offsets, *feature_ids;
    const unsigned char *values;
    const std::uint32_t *fb_offsets;    // device copy, fb_count + 1
    const std::uint32_t *block_offsets; // physical block column of the first column of every semantic block
    const std::uint32_t *finv, *rperm;
    std::uint32_t rows, features, fb_count, value_size, words; // words of the bitmap
    std::uint32_t ell_blocks;
    int values_layout;
    unsigned long long row_stride_bytes;
    std::int32_t *column_indices;
    unsigned char *values_out;
    unsigned int *max_active;
    unsigned long long *occupied;
};

__device__ __forceinline__ std::uint32_t semantic_block(const lowering_params &p, std::uint32_t execution) {
    std::uint32_t first = 0u, last = p.fb_count;
    while (first + 1u < last) {
        const std::uint32_t middle = first + (last - first) / 2u;
        if (__ldg(p.fb_offsets + middle) <= execution) first = middle;
        else last = middle;
    }
    return first;
}

// physical block column of an execution feature, and its column within that block
template<int BS>
__device__ __forceinline__ std::uint32_t physical_block(const lowering_params &p, std::uint32_t execution, std::uint32_t *local) {
    const std::uint32_t semantic = p.fb_count == 1u ? 0u : semantic_block(p, execution);
    const std::uint32_t within = execution - __ldg(p.fb_offsets + semantic);
    *local = within % BS;
    return __ldg(p.block_offsets + semantic) + within / BS;
}

// Sets, in the shared bitmap, the physical block columns that block row `br` touches.
template<int BS>
__device__ __forceinline__ void mark_block_row(const lowering_params &p, std::uint32_t br, unsigned *bitmap) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    for (std::uint32_t w = threadIdx.x; w < p.words; w += blockDim.x) bitmap[w] = 0u;
    __syncthreads();
    const std::uint32_t begin = br * BS, end = min(p.rows, begin + BS);
    for (std::uint32_t er = begin + warp; er < end; er += warps) {
        const std::uint32_t r = __ldg(p.rperm + er);
        const std::uint32_t lo = __ldg(p.row_offsets + r), hi = __ldg(p.row_offsets + r + 1u);
        for (std::uint32_t i = lo + lane; i < hi; i += 32u) {
            std::uint32_t local;
            const std::uint32_t pb = physical_block<BS>(p, __ldg(p.finv + __ldg(p.feature_ids + i)), &local);
            atomicOr(bitmap + (pb >> 5), 1u << (pb & 31u));
        }
    }
    __syncthreads();
}

template<int BS>
__global__ void __launch_bounds__(kLowerThreads) lowering_count_kernel(const lowering_params p) {
    extern __shared__ unsigned lowering_smem[];
    __shared__ unsigned warp_sums[kLowerThreads / 32];
    mark_block_row<BS>(p, blockIdx.x, lowering_smem);
    unsigned active = 0u;
    for (std::uint32_t w = threadIdx.x; w < p.words; w += blockDim.x) active += __popc(lowering_smem[w]);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) active += __shfl_xor_sync(0xffffffffu, active, off);
    if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = active;
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned total = 0u;
        for (int w = 0; w < kLowerThreads / 32; ++w) total += warp_sums[w];
        atomicMax(p.max_active, total);
        atomicAdd(p.occupied, static_cast<unsigned long long>(total));
    }
}

template<int VS>
__device__ __forceinline__ void copy_value(unsigned char *dst, const unsigned char *src, std::uint32_t value_size) {
    if constexpr (VS == 1) *dst = *src;
    else if constexpr (VS == 2) *reinterpret_cast<unsigned short *>(dst) = *reinterpret_cast<const unsigned short *>(src);
    else if constexpr (VS == 4) *reinterpret_cast<unsigned *>(dst) = *reinterpret_cast<const unsigned *>(src);
    else if constexpr (VS == 8) *reinterpret_cast<uint2 *>(dst) = *reinterpret_cast<const uint2 *>(src);
    else
        for (std::uint32_t b = 0; b < value_size; ++b) dst[b] = src[b];
}

template<int BS, int VS>
__global__ void __launch_bounds__(kLowerThreads) lowering_fill_kernel(const lowering_params p) {
    extern __shared__ unsigned lowering_smem[];
    __shared__ unsigned chunk_sums[kLowerThreads];
    unsigned *bitmap = lowering_smem, *ranks = lowering_smem + p.words; // ranks[w]: set bits in words before w
    const std::uint32_t br = blockIdx.x;
    mark_block_row<BS>(p, br, bitmap);
    // exclusive scan of the words' popcounts: every thread owns a contiguous run of words
    const std::uint32_t per = (p.words + blockDim.x - 1u) / blockDim.x;
    const std::uint32_t w0 = min(p.words, per * threadIdx.x), w1 = min(p.words, w0 + per);
    unsigned sum = 0u;
    for (std::uint32_t w = w0; w < w1; ++w) sum += __popc(bitmap[w]);
    chunk_sums[threadIdx.x] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned run = 0u;
        for (int t = 0; t < kLowerThreads; ++t) {
            const unsigned v = chunk_sums[t];
            chunk_sums[t] = run;
            run += v;
        }
    }
    __syncthreads();
    unsigned at = chunk_sums[threadIdx.x];
    for (std::uint32_t w = w0; w < w1; ++w) {
        ranks[w] = at;
        unsigned bits = bitmap[w];
        while (bits != 0u) { // slots in ascending physical block column
            const int b = __ffs(static_cast<int>(bits)) - 1;
            bits &= bits - 1u;
            if (at < p.ell_blocks) p.column_indices[static_cast<std::size_t>(br) * p.ell_blocks + at] = static_cast<std::int32_t>(w * 32u + b);
            ++at;
        }
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const std::uint32_t begin = br * BS, end = min(p.rows, begin + BS);
    for (std::uint32_t er = begin + warp; er < end; er += warps) {
        const std::uint32_t r = __ldg(p.rperm + er);
        const std::uint32_t lo = __ldg(p.row_offsets + r), hi = __ldg(p.row_offsets + r + 1u);
        for (std::uint32_t i = lo + lane; i < hi; i += 32u) {
            std::uint32_t local;
            const std::uint32_t pb = physical_block<BS>(p, __ldg(p.finv + __ldg(p.feature_ids + i)), &local);
            const unsigned long long slot = ranks[pb >> 5] + __popc(bitmap[pb >> 5] & ((1u << (pb & 31u)) - 1u));
            if (slot >= p.ell_blocks) continue; // a stale geometry: never write outside the buffers
            const unsigned long long at_byte =
                p.values_layout == 1
                    ? static_cast<unsigned long long>(er) * p.row_stride_bytes + (slot * BS + local) * p.value_size
                    : ((static_cast<unsigned long long>(br) * p.ell_blocks + slot) * BS * BS +
                       static_cast<unsigned long long>(er - begin) * BS + local) * p.value_size;
            copy_value<VS>(p.values_out + at_byte, p.values + static_cast<unsigned long long>(i) * p.value_size, p.value_size);
        }
    }
}

// flags: 1 = feature maps are not inverses, 2 = row maps are not inverses, 4 = CSR invalid
__global__ void __launch_bounds__(256) lowering_validate_kernel(const std::uint32_t *row_offsets, const std::uint32_t *feature_ids,
                                                                const std::uint32_t *fperm, const std::uint32_t *finv,
                                                                const std::uint32_t *rperm, const std::uint32_t *rinv,
                                                                std::uint32_t rows, std::uint32_t features, std::uint32_t nnz,
                                                                unsigned *flags) {
    const std::uint32_t stride = gridDim.x * blockDim.x, first = blockIdx.x * blockDim.x + threadIdx.x;
    unsigned bad = 0u;
    for (std::uint32_t e = first; e < features; e += stride) {
        const std::uint32_t c = fperm[e];
        if (c >= features || finv[c] != e) bad |= 1u; // in range and finv o fperm = id: fperm is a bijection
    }
    for (std::uint32_t e = first; e < rows; e += stride) {
        const std::uint32_t c = rperm[e];
        if (c >= rows || rinv[c] != e) bad |= 2u;
    }
    if (first == 0u && (row_offsets[0] != 0u || row_offsets[rows] != nnz)) bad |= 4u;
    for (std::uint32_t r = first; r < rows; r += stride) {
        const std::uint32_t lo = row_offsets[r], hi = row_offsets[r + 1u];
        if (lo > hi || hi > nnz) {
            bad |= 4u;
            continue;
        }
        for (std::uint32_t i = lo; i < hi; ++i)
            if (feature_ids[i] >= features || (i != lo && feature_ids[i] <= feature_ids[i - 1u])) bad |= 4u;
    }
    if (bad != 0u) atomicOr(flags, bad);
}

struct host_plan {
    std::vector<std::uint32_t> block_offsets; // fb_count + 1
    std::uint64_t physical_blocks = 0;
};

// physical_bell_candidates.cc:96-110
bool fill_physical_offsets(const cb200_bell_lowering_input &in, std::uint32_t bs, host_plan *plan) {
    plan->block_offsets.assign(static_cast<std::size_t>(in.feature_block_count) + 1u, 0u);
    std::uint64_t count = 0;
    for (std::uint32_t b = 0; b < in.feature_block_count; ++b) {
        const std::uint64_t width = in.feature_block_offsets[b + 1u] - in.feature_block_offsets[b];
        count += (width + bs - 1u) / bs;
        if (count > 0x7fffffffull) return false;
        plan->block_offsets[b + 1u] = static_cast<std::uint32_t>(count);
    }
    plan->physical_blocks = count;
    return true;
}

cb200_status check_input(const cb200_bell_lowering_input *in, std::uint32_t bs) {
    if (in == nullptr || in->version != CB200_ABI_VERSION || in->size < sizeof(cb200_bell_lowering_input))
        return fail(CB200_STATUS_INVALID_ARGUMENT, "bad cb200_bell_lowering_input header");
    if (bs != 8u && bs != 16u && bs != 32u) return fail(CB200_STATUS_INVALID_ARGUMENT, "block size %u is not 8, 16 or 32", bs);
    if (in->features == 0u || in->feature_block_count == 0u || in->feature_block_offsets == nullptr ||
        in->feature_permutation == nullptr || in->inverse_feature_permutation == nullptr)
        return fail(CB200_STATUS_INVALID_ARGUMENT, "incompatible plan: semantic plan is incomplete");
    if (in->value_size_bytes == 0u || in->value_size_bytes > 16u || in->row_offsets == nullptr ||
        (in->nnz != 0u && (in->feature_ids == nullptr || in->values == nullptr)))
        return fail(CB200_STATUS_INVALID_ARGUMENT, "invalid source: canonical CSR is invalid");
    if (in->row_permutation == nullptr || in->inverse_row_permutation == nullptr)
        return fail(CB200_STATUS_INVALID_ARGUMENT, "incompatible order: row maps are missing");
    if (in->feature_block_offsets[0] != 0u || in->feature_block_offsets[in->feature_block_count] != in->features)
        return fail(CB200_STATUS_INVALID_ARGUMENT, "incompatible plan: feature-block endpoints are invalid");
    for (std::uint32_t b = 0; b < in->feature_block_count; ++b)
        if (in->feature_block_offsets[b] >= in->feature_block_offsets[b + 1u])
            return fail(CB200_STATUS_INVALID_ARGUMENT, "incompatible plan: feature block is empty");
    return CB200_STATUS_SUCCESS;
}

std::uint64_t workspace_need(const cb200_bell_lowering_input &in) {
    return 256u + 2u * ((static_cast<std::uint64_t>(in.feature_block_count) + 1u) * 4u + 252u) / 256u * 256u;
}

// Uploads the plan's small arrays into the workspace and fills the kernel parameters.
cb200_status stage(const cb200_bell_lowering_input &in, std::uint32_t bs, const host_plan &plan, void *workspace,
                   std::uint64_t workspace_bytes, cudaStream_t stream, lowering_params *p) {
    if (workspace == nullptr || workspace_bytes < workspace_need(in) || reinterpret_cast<std::uintptr_t>(workspace) % 16u != 0u)
        return fail(CB200_STATUS_INSUFFICIENT_WORKSPACE, "the lowering needs %llu bytes of 16-byte aligned workspace",
                    static_cast<unsigned long long>(workspace_need(in)));
    const std::uint64_t words = (plan.physical_blocks + 31u) / 32u;
    if (words * 4u > kMaxBitmapBytes)
        return fail(CB200_STATUS_UNSUPPORTED, "%llu block columns exceed the shared-memory bitmap of the lowering kernels",
                    static_cast<unsigned long long>(plan.physical_blocks));
    unsigned char *base = static_cast<unsigned char *>(workspace);
    const std::size_t table = ((static_cast<std::size_t>(in.feature_block_count) + 1u) * 4u + 252u) / 256u * 256u;
    std::uint32_t *d_fb = reinterpret_cast<std::uint32_t *>(base + 256), *d_bo = reinterpret_cast<std::uint32_t *>(base + 256 + table);
    const std::size_t bytes = (static_cast<std::size_t>(in.feature_block_count) + 1u) * 4u;
    CB200_CUDA_OK(cudaMemsetAsync(base, 0, 256, stream));
    CB200_CUDA_OK(cudaMemcpyAsync(d_fb, in.feature_block_offsets, bytes, cudaMemcpyHostToDevice, stream));
    CB200_CUDA_OK(cudaMemcpyAsync(d_bo, plan.block_offsets.data(), bytes, cudaMemcpyHostToDevice, stream));
    *p = lowering_params{};
    p->row_offsets = in.row_offsets; p->feature_ids = in.feature_ids; p->values = static_cast<const unsigned char *>(in.values);
    p->fb_offsets = d_fb; p->block_offsets = d_bo; p->finv = in.inverse_feature_permutation; p->rperm = in.row_permutation;
    p->rows = in.rows; p->features = in.features; p->fb_count = in.feature_block_count; p->value_size = in.value_size_bytes;
    p->words = static_cast<std::uint32_t>(words);
    p->max_active = reinterpret_cast<unsigned int *>(base);
    p->occupied = reinterpret_cast<unsigned long long *>(base + 8);
    (void)bs;
    return CB200_STATUS_SUCCESS;
}

template<int BS, int VS>
cb200_status launch_fill(const lowering_params &p, unsigned grid, std::size_t smem, cudaStream_t stream) {
    if (smem > 48u * 1024u)
        CB200_CUDA_OK(cudaFuncSetAttribute(lowering_fill_kernel<BS, VS>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    lowering_fill_kernel<BS, VS><<<grid, kLowerThreads, smem, stream>>>(p);
    count_launch();
    CB200_CUDA_OK(cudaGetLastError());
    return CB200_STATUS_SUCCESS;
}

// Typed copies need both arrays aligned to the value size; anything else is copied byte by byte.
template<int BS>
cb200_status launch_fill_vs(const lowering_params &p, unsigned grid, std::size_t smem, cudaStream_t stream) {
    const std::uintptr_t vs = p.value_size;
    const bool aligned = reinterpret_cast<std::uintptr_t>(p.values) % vs == 0u && reinterpret_cast<std::uintptr_t>(p.values_out) % vs == 0u &&
                         (p.values_layout != 1 || p.row_stride_bytes % vs == 0u);
    if (!aligned) return launch_fill<BS, 0>(p, grid, smem, stream);
    switch (p.value_size) {
    case 1: return launch_fill<BS, 1>(p, grid, smem, stream);
    case 2: return launch_fill<BS, 2>(p, grid, smem, stream);
    case 4: return launch_fill<BS, 4>(p, grid, smem, stream);
    case 8: return launch_fill<BS, 8>(p, grid, smem, stream);
    default: return launch_fill<BS, 0>(p, grid, smem, stream);
    }
}

template<int BS>
cb200_status launch_count(const lowering_params &p, unsigned grid, std::size_t smem, cudaStream_t stream) {
    if (smem > 48u * 1024u)
        CB200_CUDA_OK(cudaFuncSetAttribute(lowering_count_kernel<BS>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    lowering_count_kernel<BS><<<grid, kLowerThreads, smem, stream>>>(p);
    count_launch();
    CB200_CUDA_OK(cudaGetLastError());
    return CB200_STATUS_SUCCESS;
}

} // namespace
} // namespace cb200

extern "C" cb200_status cb200_bell_lowering_workspace(const cb200_bell_lowering_input *in, uint64_t *bytes) {
    using namespace cb200;
    clear_error();
    if (in == nullptr || bytes == nullptr) return fail(CB200_STATUS_INVALID_ARGUMENT, "null argument");
    *bytes = workspace_need(*in);
    return CB200_STATUS_SUCCESS;
}

extern "C" cb200_status cb200_bell_lowering_query(const cb200_bell_lowering_input *in, uint32_t block_size,
                                                  const cb200_bell_lowering_policy *policy, void *workspace,
                                                  uint64_t workspace_bytes, void *stream_handle, cb200_bell_geometry *out) {
    using namespace cb200;
    clear_error();
    if (out == nullptr || policy == nullptr) return fail(CB200_STATUS_INVALID_ARGUMENT, "null argument");
    if (!(policy->maximum_value_slot_expansion > 0.0) || !(policy->maximum_storage_expansion > 0.0) ||
        policy->maximum_value_slot_expansion > 1.0e300 || policy->maximum_storage_expansion > 1.0e300)
        return fail(CB200_STATUS_INVALID_ARGUMENT, "candidate policy is invalid");
    cb200_status st = check_input(in, block_size);
    if (st != CB200_STATUS_SUCCESS) return st;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
    device_scope scope(in->device);
    CB200_CUDA_OK(scope.status);

    *out = cb200_bell_geometry{};
    out->version = CB200_ABI_VERSION;
    out->size = sizeof(*out);
    out->state = CB200_BELL_STATE_OVERFLOW;
    out->block_size = block_size;
    out->rows = in->rows;
    out->features = in->features;
    out->feature_block_offset_count = static_cast<std::uint64_t>(in->feature_block_count) + 1u;
    host_plan plan;
    if (!fill_physical_offsets(*in, block_size, &plan)) return CB200_STATUS_SUCCESS; // state = overflow, as the reference
    const std::uint64_t block_rows = (static_cast<std::uint64_t>(in->rows) + block_size - 1u) / block_size;
    const std::uint64_t padded_rows = block_rows * block_size, padded_features = plan.physical_blocks * block_size;
    if (padded_rows > 0xffffffffull || padded_features > 0xffffffffull) return CB200_STATUS_SUCCESS;
    out->block_rows = static_cast<std::uint32_t>(block_rows);
    out->padded_rows = static_cast<std::uint32_t>(padded_rows);
    out->padded_features = static_cast<std::uint32_t>(padded_features);

    lowering_params p;
    st = stage(*in, block_size, plan, workspace, workspace_bytes, stream, &p);
    if (st != CB200_STATUS_SUCCESS) return st;
    unsigned *flags = reinterpret_cast<unsigned *>(static_cast<unsigned char *>(workspace) + 16);
    const unsigned vgrid = static_cast<unsigned>(std::min<std::uint64_t>(
        (std::max<std::uint64_t>(in->rows, in->features) + 255u) / 256u + 1u, 4096u));
    lowering_validate_kernel<<<vgrid, 256, 0, stream>>>(in->row_offsets, in->feature_ids, in->feature_permutation,
                                                        in->inverse_feature_permutation, in->row_permutation,
                                                        in->inverse_row_permutation, in->rows, in->features, in->nnz, flags);
    count_launch();
    CB200_CUDA_OK(cudaGetLastError());
    unsigned host_flags = 0u;
    CB200_CUDA_OK(cudaMemcpyAsync(&host_flags, flags, sizeof host_flags, cudaMemcpyDeviceToHost, stream));
    CB200_CUDA_OK(cudaStreamSynchronize(stream));
    if (host_flags & 1u) return fail(CB200_STATUS_INVALID_ARGUMENT, "incompatible plan: feature maps are not inverses");
    if (host_flags & 2u) return fail(CB200_STATUS_INVALID_ARGUMENT, "incompatible order: row maps are not inverses");
    if (host_flags & 4u) return fail(CB200_STATUS_INVALID_ARGUMENT, "invalid source: CSR offsets or features are not sorted and in range");

    if (block_rows > 0u) {
        const std::size_t smem = static_cast<std::size_t>(p.words) * 4u;
        const unsigned grid = static_cast<unsigned>(block_rows);
        st = block_size == 8u ? launch_count<8>(p, grid, smem, stream)
                              : (block_size == 16u ? launch_count<16>(p, grid, smem, stream) : launch_count<32>(p, grid, smem, stream));
        if (st != CB200_STATUS_SUCCESS) return st;
    }
    unsigned maximum = 0u;
    unsigned long long occupied = 0u;
    CB200_CUDA_OK(cudaMemcpyAsync(&maximum, p.max_active, sizeof maximum, cudaMemcpyDeviceToHost, stream));
    CB200_CUDA_OK(cudaMemcpyAsync(&occupied, p.occupied, sizeof occupied, cudaMemcpyDeviceToHost, stream));
    CB200_CUDA_OK(cudaStreamSynchronize(stream));

    // physical_bell_candidates.cc:167-207
    const std::uint64_t stored = block_rows * maximum;
    const std::uint64_t slots = stored * block_size * block_size;
    const std::uint64_t bytes = slots * in->value_size_bytes;
    const std::uint64_t persistent = stored * 4u + bytes + out->feature_block_offset_count * 4u;
    const std::uint64_t source_bytes = (static_cast<std::uint64_t>(in->rows) + 1u) * 4u +
                                       static_cast<std::uint64_t>(in->nnz) * (4u + in->value_size_bytes);
    out->ell_blocks_per_row = maximum;
    out->ell_columns = maximum * block_size;
    out->column_index_count = stored;
    out->value_bytes = bytes;
    out->occupied_blocks = occupied;
    out->stored_blocks = stored;
    out->dense_value_slots = slots;
    out->persistent_bytes = persistent;
    out->source_bytes = source_bytes;
    out->scalar_occupancy = slots == 0u ? 0.0 : static_cast<double>(in->nnz) / static_cast<double>(slots);
    out->ell_slot_utilization = stored == 0u ? 0.0 : static_cast<double>(occupied) / static_cast<double>(stored);
    out->value_slot_expansion = in->nnz == 0u ? 0.0 : static_cast<double>(slots) / in->nnz;
    out->storage_expansion = source_bytes == 0u ? 0.0 : static_cast<double>(persistent) / static_cast<double>(source_bytes);
    if (in->nnz == 0u) out->state = CB200_BELL_STATE_EMPTY_SOURCE;
    else if (out->value_slot_expansion > policy->maximum_value_slot_expansion) out->state = CB200_BELL_STATE_VALUE_EXPANSION_EXCEEDED;
    else if (out->storage_expansion > policy->maximum_storage_expansion) out->state = CB200_BELL_STATE_STORAGE_EXPANSION_EXCEEDED;
    else if (persistent > policy->maximum_persistent_bytes) out->state = CB200_BELL_STATE_PERSISTENT_BYTES_EXCEEDED;
    else out->state = CB200_BELL_STATE_LEGAL;
    return CB200_STATUS_SUCCESS;
}

extern "C" cb200_status cb200_bell_lowering_materialize(const cb200_bell_lowering_input *in, const cb200_bell_geometry *geometry,
                                                        int32_t values_layout, uint64_t row_stride_bytes,
                                                        uint32_t *padded_feature_block_offsets, int32_t *column_indices,
                                                        void *values, void *workspace, uint64_t workspace_bytes,
                                                        void *stream_handle) {
    using namespace cb200;
    clear_error();
    if (geometry == nullptr || geometry->version != CB200_ABI_VERSION || geometry->size < sizeof(cb200_bell_geometry))
        return fail(CB200_STATUS_INVALID_ARGUMENT, "bad cb200_bell_geometry header");
    cb200_status st = check_input(in, geometry->block_size);
    if (st != CB200_STATUS_SUCCESS) return st;
    if (geometry->state != CB200_BELL_STATE_LEGAL) return fail(CB200_STATUS_UNSUPPORTED, "candidate rejected: state %d", geometry->state);
    const std::uint32_t bs = geometry->block_size;
    host_plan plan;
    if (!fill_physical_offsets(*in, bs, &plan)) return fail(CB200_STATUS_INVALID_SHAPE, "physical feature padding overflowed");
    const std::uint64_t block_rows = (static_cast<std::uint64_t>(in->rows) + bs - 1u) / bs;
    if (geometry->rows != in->rows || geometry->features != in->features || geometry->block_rows != block_rows ||
        geometry->padded_rows != block_rows * bs || geometry->padded_features != plan.physical_blocks * bs ||
        geometry->ell_columns != geometry->ell_blocks_per_row * bs ||
        geometry->column_index_count != block_rows * geometry->ell_blocks_per_row ||
        geometry->value_bytes != geometry->column_index_count * bs * bs * in->value_size_bytes)
        return fail(CB200_STATUS_STALE_STRUCTURE, "candidate mismatch: the geometry is not the one queried for this input");
    if (values_layout != CB200_BELL_VALUES_BLOCK_MAJOR && values_layout != CB200_BELL_VALUES_ROW_MAJOR)
        return fail(CB200_STATUS_INVALID_ARGUMENT, "unknown values layout %d", values_layout);
    if (values_layout == CB200_BELL_VALUES_ROW_MAJOR &&
        row_stride_bytes < static_cast<std::uint64_t>(geometry->ell_columns) * in->value_size_bytes)
        return fail(CB200_STATUS_INVALID_SHAPE, "row stride smaller than a row of the Blocked-ELL matrix");
    if (padded_feature_block_offsets == nullptr || (geometry->column_index_count != 0u && column_indices == nullptr) ||
        (geometry->value_bytes != 0u && values == nullptr))
        return fail(CB200_STATUS_INVALID_ARGUMENT, "insufficient capacity: null output buffer");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
    device_scope scope(in->device);
    CB200_CUDA_OK(scope.status);

    lowering_params p;
    st = stage(*in, bs, plan, workspace, workspace_bytes, stream, &p);
    if (st != CB200_STATUS_SUCCESS) return st;
    std::vector<std::uint32_t> padded(plan.block_offsets.size());
    for (std::size_t b = 0; b < padded.size(); ++b) padded[b] = plan.block_offsets[b] * bs;
    CB200_CUDA_OK(cudaMemcpyAsync(padded_feature_block_offsets, padded.data(), padded.size() * 4u, cudaMemcpyHostToDevice, stream));
    const std::uint64_t value_bytes = values_layout == CB200_BELL_VALUES_ROW_MAJOR
                                          ? static_cast<std::uint64_t>(geometry->padded_rows) * row_stride_bytes
                                          : geometry->value_bytes;
    if (geometry->column_index_count != 0u)
        CB200_CUDA_OK(cudaMemsetAsync(column_indices, 0xff, geometry->column_index_count * sizeof(std::int32_t), stream)); // -1 = empty
    if (value_bytes != 0u) CB200_CUDA_OK(cudaMemsetAsync(values, 0, value_bytes, stream));
    if (block_rows == 0u || geometry->ell_blocks_per_row == 0u) return CB200_STATUS_SUCCESS;
    p.ell_blocks = geometry->ell_blocks_per_row;
    p.values_layout = values_layout;
    p.row_stride_bytes = row_stride_bytes;
    p.column_indices = column_indices;
    p.values_out = static_cast<unsigned char *>(values);
    const std::size_t smem = static_cast<std::size_t>(p.words) * 8u;
    const unsigned grid = static_cast<unsigned>(block_rows);
    return bs == 8u ? launch_fill_vs<8>(p, grid, smem, stream)
                    : (bs == 16u ? launch_fill_vs<16>(p, grid, smem, stream) : launch_fill_vs<32>(p, grid, smem, stream));
}

// ---------------------------------------------------------------------------------------------
// Feature-order pack of a dense operand (the W that goes with a lowered matrix):
//     packed[execution][column] = source[feature_permutation[execution]][column],
// contiguous row-major.  Reference counterpart: pack_dense_operand_cuda
// (src/compute/math/packed_dense_operand.cu:131-170,227-262; one thread per element, grid-stride).
// Here a row-major source whose rows are 16-byte aligned moves as 16-byte pieces (a bf16 row of 64
// columns is 8 of them), anything else element by element.
namespace cb200 {
namespace {

template<typename T>
__global__ void __launch_bounds__(256) pack_dense_kernel(const std::uint32_t *fperm, const T *source, std::uint32_t rows,
                                                         std::uint64_t columns, std::uint64_t ld, int col_major,
                                                         std::uint32_t features, T *packed, unsigned *flags) {
    const std::uint64_t count = static_cast<std::uint64_t>(rows) * columns;
    for (std::uint64_t i = static_cast<std::uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count;
         i += static_cast<std::uint64_t>(blockDim.x) * gridDim.x) {
        const std::uint32_t execution = static_cast<std::uint32_t>(i / columns);
        const std::uint64_t column = i - static_cast<std::uint64_t>(execution) * columns;
        const std::uint32_t feature = __ldg(fperm + execution);
        if (feature >= features) { // physical_view_status invalid_geometry; nothing is read out of range
            if (column == 0u) atomicOr(flags, 1u);
            continue;
        }
        packed[i] = source[col_major ? column * ld + feature : static_cast<std::uint64_t>(feature) * ld + column];
    }
}

struct bytes16 { uint4 v; };
struct bytes_n { unsigned char b; };

template<typename T>
cb200_status launch_pack(const std::uint32_t *fperm, const void *source, std::uint32_t rows, std::uint64_t columns,
                         std::uint64_t ld, int col_major, std::uint32_t features, void *packed, unsigned *flags,
                         cudaStream_t stream) {
    const std::uint64_t count = static_cast<std::uint64_t>(rows) * columns;
    if (count == 0u) return CB200_STATUS_SUCCESS;
    const unsigned grid = static_cast<unsigned>(std::min<std::uint64_t>((count + 255u) / 256u, 148u * 32u));
    pack_dense_kernel<T><<<grid, 256, 0, stream>>>(fperm, static_cast<const T *>(source), rows, columns, ld, col_major, features,
                                                   static_cast<T *>(packed), flags);
    count_launch();
    CB200_CUDA_OK(cudaGetLastError());
    return CB200_STATUS_SUCCESS;
}

} // namespace
} // namespace cb200

extern "C" cb200_status cb200_pack_dense_operand(const cb200_dense_pack *d, void *stream_handle) {
    using namespace cb200;
    clear_error();
    if (d == nullptr || d->version != CB200_ABI_VERSION || d->size < sizeof(cb200_dense_pack))
        return fail(CB200_STATUS_INVALID_ARGUMENT, "bad cb200_dense_pack header");
    const std::uint32_t vs = d->value_size_bytes;
    if (vs != 1u && vs != 2u && vs != 4u && vs != 8u && vs != 16u)
        return fail(CB200_STATUS_UNSUPPORTED, "value size %u is not 1, 2, 4, 8 or 16 bytes", vs);
    if (d->feature_permutation == nullptr || d->status_word == nullptr ||
        (d->features != 0u && d->columns != 0u && (d->source == nullptr || d->packed == nullptr)))
        return fail(CB200_STATUS_INVALID_ARGUMENT, "null argument");
    if (d->packed == d->source && d->source != nullptr) return fail(CB200_STATUS_INVALID_ARGUMENT, "packed output aliases its source");
    if (d->leading_dimension < (d->source_col_major ? d->features : d->columns))
        return fail(CB200_STATUS_INVALID_SHAPE, "leading dimension smaller than the contiguous extent");
    const std::uint32_t blocks = d->feature_block_count;
    std::uint64_t packed_rows = d->features;
    if (blocks != 0u) {
        if (d->feature_block_offsets == nullptr || d->padded_feature_block_offsets == nullptr)
            return fail(CB200_STATUS_INVALID_ARGUMENT, "feature blocks without their offsets");
        if (d->feature_block_offsets[0] != 0u || d->feature_block_offsets[blocks] != d->features || d->padded_feature_block_offsets[0] != 0u)
            return fail(CB200_STATUS_INVALID_SHAPE, "feature-block endpoints are invalid");
        for (std::uint32_t b = 0; b < blocks; ++b)
            if (d->feature_block_offsets[b + 1u] <= d->feature_block_offsets[b] ||
                d->padded_feature_block_offsets[b + 1u] - d->padded_feature_block_offsets[b] <
                    d->feature_block_offsets[b + 1u] - d->feature_block_offsets[b])
                return fail(CB200_STATUS_INVALID_SHAPE, "a padded feature block is narrower than the block it pads");
        packed_rows = d->padded_feature_block_offsets[blocks];
    }
    const std::uint64_t need = packed_rows * d->columns * vs;
    if (d->packed_capacity_bytes < need)
        return fail(CB200_STATUS_INSUFFICIENT_WORKSPACE, "packed operand needs %llu bytes, %llu given",
                    static_cast<unsigned long long>(need), static_cast<unsigned long long>(d->packed_capacity_bytes));
    cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
    device_scope scope(d->device);
    CB200_CUDA_OK(scope.status);
    CB200_CUDA_OK(cudaMemsetAsync(d->status_word, 0, sizeof(unsigned), stream));
    if (blocks != 0u && need != 0u) CB200_CUDA_OK(cudaMemsetAsync(d->packed, 0, need, stream)); // rows of the padding

    // a row-major source with 16-byte aligned rows moves as 16-byte pieces
    const std::uint64_t row_bytes = d->columns * vs;
    const bool wide = !d->source_col_major && row_bytes % 16u == 0u && (d->leading_dimension * vs) % 16u == 0u &&
                      reinterpret_cast<std::uintptr_t>(d->source) % 16u == 0u && reinterpret_cast<std::uintptr_t>(d->packed) % 16u == 0u;
    const std::uint32_t piece = wide ? 16u : vs;
    const std::uint64_t columns = row_bytes / piece, ld = d->leading_dimension * vs / piece;
    const std::uint32_t runs = blocks == 0u ? 1u : blocks;
    for (std::uint32_t b = 0; b < runs; ++b) {
        const std::uint32_t first = blocks == 0u ? 0u : d->feature_block_offsets[b];
        const std::uint32_t rows = blocks == 0u ? d->features : d->feature_block_offsets[b + 1u] - first;
        const std::uint64_t row0 = blocks == 0u ? 0u : d->padded_feature_block_offsets[b];
        void *dst = static_cast<unsigned char *>(d->packed) + row0 * row_bytes;
        const std::uint32_t *perm = d->feature_permutation + first;
        unsigned *flags = static_cast<unsigned *>(d->status_word);
        cb200_status st;
        switch (piece) {
        case 1: st = launch_pack<unsigned char>(perm, d->source, rows, columns, ld, d->source_col_major, d->features, dst, flags, stream); break;
        case 2: st = launch_pack<unsigned short>(perm, d->source, rows, columns, ld, d->source_col_major, d->features, dst, flags, stream); break;
        case 4: st = launch_pack<unsigned>(perm, d->source, rows, columns, ld, d->source_col_major, d->features, dst, flags, stream); break;
        case 8: st = launch_pack<uint2>(perm, d->source, rows, columns, ld, d->source_col_major, d->features, dst, flags, stream); break;
        default: st = launch_pack<uint4>(perm, d->source, rows, columns, ld, d->source_col_major, d->features, dst, flags, stream); break;
        }
        if (st != CB200_STATUS_SUCCESS) return st;
    }
    return CB200_STATUS_SUCCESS;
}

// ---------------------------------------------------------------------------------------------
// Execution-order feature ids of an ordered plan partition (the CSR a packed-order projection or the
// lowering above consumes): execution = feature_block_offsets[block] + local.  Reference counterpart:
// the loop of build_execution_csr_view_host (src/compute/math/physical_csr.cc:47-75).  One warp per
// row; the ascending check inside a row compares neighbours through a shuffle.
namespace cb200 {
namespace {

// flags: 1 = geometry (offsets, block or local out of range), 2 = identity (canonical id or order)
__global__ void __launch_bounds__(256) execution_ids_kernel(const std::uint32_t *row_offsets, const std::uint32_t *block_ids,
                                                            const std::uint32_t *local_ids, const std::uint32_t *canonical_ids,
                                                            const std::uint32_t *fb_offsets, const std::uint32_t *fperm,
                                                            std::uint32_t rows, std::uint32_t nnz, std::uint32_t fb_count,
                                                            std::uint32_t *execution_ids, unsigned *flags) {
    const int lane = threadIdx.x & 31;
    const std::uint32_t row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const std::uint32_t begin = row_offsets[row], end = row_offsets[row + 1u];
    unsigned bad = 0u;
    if (end < begin || end > nnz || (row == 0u && begin != 0u) || (row + 1u == rows && end != nnz)) {
        if (lane == 0) atomicOr(flags, 1u);
        return;
    }
    std::uint32_t carry = 0xffffffffu; // execution id of the entry before this batch
    for (std::uint32_t base = begin; base < end; base += 32u) {
        const std::uint32_t i = base + lane;
        std::uint32_t execution = 0xffffffffu;
        bool geometry_ok = true;
        if (i < end) {
            const std::uint32_t block = block_ids[i];
            if (block >= fb_count) geometry_ok = false;
            else {
                const std::uint32_t block_begin = __ldg(fb_offsets + block), block_end = __ldg(fb_offsets + block + 1u);
                if (local_ids[i] >= block_end - block_begin) geometry_ok = false;
                else execution = block_begin + local_ids[i];
            }
            if (!geometry_ok) bad |= 1u;
            else if (__ldg(fperm + execution) != canonical_ids[i]) bad |= 2u;
        }
        std::uint32_t previous = __shfl_up_sync(0xffffffffu, execution, 1);
        if (lane == 0) previous = carry;
        if (i < end && geometry_ok) {
            if (i != begin && previous != 0xffffffffu && execution <= previous) bad |= 2u;
            execution_ids[i] = execution;
        }
        carry = __shfl_sync(0xffffffffu, execution, 31);
    }
    if (bad != 0u) atomicOr(flags, bad);
}

} // namespace
} // namespace cb200

extern "C" cb200_status cb200_build_execution_csr(const cb200_execution_csr *e, void *stream_handle) {
    using namespace cb200;
    clear_error();
    if (e == nullptr || e->version != CB200_ABI_VERSION || e->size < sizeof(cb200_execution_csr))
        return fail(CB200_STATUS_INVALID_ARGUMENT, "bad cb200_execution_csr header");
    if (e->feature_block_count == 0u || e->feature_block_offsets == nullptr || (e->features != 0u && e->feature_permutation == nullptr) ||
        e->feature_block_offsets[0] != 0u || e->feature_block_offsets[e->feature_block_count] != e->features)
        return fail(CB200_STATUS_INVALID_ARGUMENT, "invalid argument: execution CSR requires a valid frozen plan view");
    if (e->row_offsets == nullptr || e->status_word == nullptr ||
        (e->nnz != 0u && (e->block_ids == nullptr || e->local_feature_ids == nullptr || e->canonical_feature_ids == nullptr)))
        return fail(CB200_STATUS_INVALID_ARGUMENT, "incompatible identity: ordered partition disagrees with the frozen feature plan");
    if (e->nnz != 0u && e->execution_feature_ids == nullptr)
        return fail(CB200_STATUS_INSUFFICIENT_WORKSPACE, "insufficient capacity: execution feature buffer is missing");
    const std::uint64_t table = (static_cast<std::uint64_t>(e->feature_block_count) + 1u) * 4u;
    if (e->workspace == nullptr || e->workspace_bytes < table || reinterpret_cast<std::uintptr_t>(e->workspace) % 4u != 0u)
        return fail(CB200_STATUS_INSUFFICIENT_WORKSPACE, "the feature-block offsets need %llu bytes of device workspace",
                    static_cast<unsigned long long>(table));
    cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
    device_scope scope(e->device);
    CB200_CUDA_OK(scope.status);
    CB200_CUDA_OK(cudaMemsetAsync(e->status_word, 0, sizeof(unsigned), stream));
    CB200_CUDA_OK(cudaMemcpyAsync(e->workspace, e->feature_block_offsets, table, cudaMemcpyHostToDevice, stream));
    if (e->rows == 0u) return CB200_STATUS_SUCCESS;
    execution_ids_kernel<<<(e->rows + 7u) / 8u, 256, 0, stream>>>(e->row_offsets, e->block_ids, e->local_feature_ids,
                                                                 e->canonical_feature_ids, static_cast<const std::uint32_t *>(e->workspace),
                                                                 e->feature_permutation, e->rows, e->nnz, e->feature_block_count,
                                                                 e->execution_feature_ids, static_cast<unsigned *>(e->status_word));
    count_launch();
    CB200_CUDA_OK(cudaGetLastError());
    return CB200_STATUS_SUCCESS;
}
