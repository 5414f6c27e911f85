// Multi-GPU layer of the C ABI: a fleet of device slots with their streams and scratch, the uniform
// row partition, per-slot launch loops for the forward and the transpose projection, and the NCCL
// all-reduce that combines the transpose partials.
//
// Reference counterparts: fleet_context / discover_fleet / request_fleet_scratch / synchronize_slots
// (src/compute/runtime/runtime.hh:47-87, runtime.cu:96-199), reduce_sum_to_leader_f32
// (src/compute/runtime/reduce.cu:147-294), nccl_communicator with init_local / init_ranked and
// communicator_allreduce (include/Cellerator/dist/nccl_communicator.cuh:12-22,109-156,290-315), and the
// dist::launch_* loops (src/compute/sparse/project/project.cu:321-341,
// src/compute/sparse/ops/kernels/dist_sparse.cu:24-32,177-197).
//
// Differences by design: NCCL is bound at run time (dlopen), so the library loads on hosts without it and
// shares the copy a process already holds; the collective is enqueued on the slots' compute streams with
// no host synchronisation in front of it (stream order carries the dependency; the reference waits for
// every slot first, reduce.cu:164); and a communicator that is not ready is reported as a status instead
// of falling back to peer copies and adds.  The only peer traffic is NCCL's: this file issues no load or
// copy of another GPU's memory.
#include "kernels.cuh"

#include <dlfcn.h>
#include <nccl.h> // types and enums only; every function is reached through dlsym

#include <cstring>
#include <new>

using namespace cb200;

namespace {

constexpr int kMaxSlots = 16;

struct nccl_api {
    void *handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommInitAll)(ncclComm_t *, int, const int *) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
    bool ready() const { return handle != nullptr; }
};

// Binds the eight NCCL entry points this file uses.  false (with the reason in `why`) when the library or
// one of the symbols cannot be had.
bool load_nccl(const char *library, nccl_api *api, char *why, std::size_t why_bytes) {
    const char *name = (library != nullptr && library[0] != '\0') ? library : "libnccl.so.2";
    void *h = dlopen(name, RTLD_NOW | RTLD_LOCAL);
    if (h == nullptr) {
        const char *e = dlerror();
        std::snprintf(why, why_bytes, "dlopen(%s): %s", name, e != nullptr ? e : "failed");
        return false;
    }
    const auto bind = [&](const char *symbol, void **slot) {
        *slot = dlsym(h, symbol);
        return *slot != nullptr;
    };
    nccl_api a;
    const bool ok = bind("ncclGetUniqueId", reinterpret_cast<void **>(&a.GetUniqueId)) &&
                    bind("ncclCommInitRank", reinterpret_cast<void **>(&a.CommInitRank)) &&
                    bind("ncclCommInitAll", reinterpret_cast<void **>(&a.CommInitAll)) &&
                    bind("ncclCommDestroy", reinterpret_cast<void **>(&a.CommDestroy)) &&
                    bind("ncclAllReduce", reinterpret_cast<void **>(&a.AllReduce)) &&
                    bind("ncclGroupStart", reinterpret_cast<void **>(&a.GroupStart)) &&
                    bind("ncclGroupEnd", reinterpret_cast<void **>(&a.GroupEnd)) &&
                    bind("ncclGetErrorString", reinterpret_cast<void **>(&a.GetErrorString));
    if (!ok) {
        std::snprintf(why, why_bytes, "%s lacks an NCCL entry point", name);
        dlclose(h);
        return false;
    }
    a.handle = h;
    *api = a;
    return true;
}

} // namespace

struct cb200_fleet {
    int slot_count = 0;
    int devices[kMaxSlots] = {};
    cudaStream_t streams[kMaxSlots] = {};
    bool owns_stream[kMaxSlots] = {};
    void *scratch[kMaxSlots] = {};
    std::uint64_t scratch_bytes[kMaxSlots] = {};
    int world_size = 1;
    int world_rank = 0;
    nccl_api nccl;
    ncclComm_t comms[kMaxSlots] = {};
    bool comm_ready = false;
    char comm_error[256] = "";
};

namespace {

bool slot_ok(const cb200_fleet *f, std::uint32_t slot) { return f != nullptr && slot < static_cast<std::uint32_t>(f->slot_count); }

cb200_status require_slots(const cb200_fleet *f, const std::uint32_t *slots, std::uint32_t count) {
    if (f == nullptr) return fail(CB200_STATUS_INVALID_ARGUMENT, "null fleet");
    if (slots == nullptr && count != 0u) return fail(CB200_STATUS_INVALID_ARGUMENT, "a distributed launch needs its slot list");
    if (count > static_cast<std::uint32_t>(kMaxSlots)) return fail(CB200_STATUS_INVALID_ARGUMENT, "more slots than a fleet can hold");
    for (std::uint32_t i = 0; i < count; ++i) {
        if (!slot_ok(f, slots[i])) return fail(CB200_STATUS_INVALID_ARGUMENT, "slot %u is not part of the fleet", slots[i]);
        for (std::uint32_t j = 0; j < i; ++j)
            if (slots[j] == slots[i]) return fail(CB200_STATUS_INVALID_ARGUMENT, "slot %u is listed twice", slots[i]);
    }
    return CB200_STATUS_SUCCESS;
}

// A collective over the whole job: every local slot has to take part, once, and the communicator must be ready.
cb200_status require_collective(const cb200_fleet *f, std::uint32_t slot_count) {
    if (f->world_size == 1 && f->slot_count == 1) return CB200_STATUS_SUCCESS; // a job of one rank: the sum is the partial
    if (slot_count != static_cast<std::uint32_t>(f->slot_count))
        return fail(CB200_STATUS_INVALID_ARGUMENT, "a collective needs every slot of the fleet (%d), %u listed", f->slot_count, slot_count);
    if (!f->comm_ready)
        return fail(CB200_STATUS_COMM_NOT_READY, "the NCCL communicator of this fleet is not ready (%s); nothing falls back to peer copies",
                    f->comm_error[0] != '\0' ? f->comm_error : "not initialised");
    return CB200_STATUS_SUCCESS;
}

// One grouped ncclAllReduce(float32, sum) per listed slot, on the slots' streams.
cb200_status grouped_allreduce(cb200_fleet *f, const std::uint32_t *slots, std::uint32_t slot_count, const float *const *send,
                               float *const *recv, std::uint64_t count) {
    if (count == 0u) return CB200_STATUS_SUCCESS;
    if (f->world_size == 1 && f->slot_count == 1) {
        if (send[0] != recv[0]) {
            device_scope scope(f->devices[slots[0]]);
            CB200_CUDA_OK(scope.status);
            CB200_CUDA_OK(cudaMemcpyAsync(recv[0], send[0], count * sizeof(float), cudaMemcpyDeviceToDevice, f->streams[slots[0]]));
        }
        return CB200_STATUS_SUCCESS;
    }
    ncclResult_t result = f->nccl.GroupStart();
    if (result != ncclSuccess) return fail(CB200_STATUS_COMM_NOT_READY, "ncclGroupStart: %s", f->nccl.GetErrorString(result));
    for (std::uint32_t i = 0; i < slot_count; ++i) {
        const std::uint32_t slot = slots[i];
        result = f->nccl.AllReduce(send[i], recv[i], static_cast<size_t>(count), ncclFloat32, ncclSum, f->comms[slot], f->streams[slot]);
        if (result != ncclSuccess) {
            f->nccl.GroupEnd();
            return fail(CB200_STATUS_INTERNAL_ERROR, "ncclAllReduce on slot %u: %s", slot, f->nccl.GetErrorString(result));
        }
    }
    result = f->nccl.GroupEnd();
    if (result != ncclSuccess) return fail(CB200_STATUS_INTERNAL_ERROR, "ncclGroupEnd: %s", f->nccl.GetErrorString(result));
    return CB200_STATUS_SUCCESS;
}

} // namespace

extern "C" {

cb200_status cb200_fleet_unique_id(const char *nccl_library, void *unique_id_128) {
    clear_error();
    if (unique_id_128 == nullptr) return fail(CB200_STATUS_INVALID_ARGUMENT, "unique_id needs 128 bytes of output");
    static_assert(sizeof(ncclUniqueId) == 128, "the unique id travels as 128 bytes");
    nccl_api api;
    char why[256];
    if (!load_nccl(nccl_library, &api, why, sizeof(why))) return fail(CB200_STATUS_COMM_NOT_READY, "%s", why);
    ncclUniqueId id;
    const ncclResult_t result = api.GetUniqueId(&id);
    if (result != ncclSuccess) return fail(CB200_STATUS_COMM_NOT_READY, "ncclGetUniqueId: %s", api.GetErrorString(result));
    std::memcpy(unique_id_128, &id, sizeof(id));
    return CB200_STATUS_SUCCESS;
}

cb200_status cb200_fleet_create(const cb200_fleet_options *o, cb200_fleet **out) {
    clear_error();
    if (out == nullptr) return fail(CB200_STATUS_INVALID_ARGUMENT, "fleet_create needs an output handle");
    *out = nullptr;
    if (o == nullptr || o->version != CB200_ABI_VERSION || o->size < sizeof(cb200_fleet_options))
        return fail(CB200_STATUS_INVALID_ARGUMENT, "bad cb200_fleet_options header");
    if (o->device_count < 1 || o->device_count > kMaxSlots) return fail(CB200_STATUS_INVALID_ARGUMENT, "a fleet has 1..%d slots", kMaxSlots);
    const int world = o->world_size == 0 ? o->device_count : o->world_size;
    if (world < o->device_count || o->world_rank < 0 || o->world_rank + o->device_count > world)
        return fail(CB200_STATUS_INVALID_ARGUMENT, "ranks %d..%d do not fit a job of %d", o->world_rank, o->world_rank + o->device_count - 1, world);
    if (world > o->device_count && o->nccl_unique_id == nullptr)
        return fail(CB200_STATUS_INVALID_ARGUMENT, "a job that spans processes needs the NCCL unique id of its rank 0");
    int visible = 0;
    CB200_CUDA_OK(cudaGetDeviceCount(&visible));
    cb200_fleet *f = new (std::nothrow) cb200_fleet{};
    if (f == nullptr) return fail(CB200_STATUS_INTERNAL_ERROR, "out of host memory");
    f->slot_count = o->device_count;
    f->world_size = world;
    f->world_rank = o->world_rank;
    for (int i = 0; i < f->slot_count; ++i) {
        f->devices[i] = o->devices != nullptr ? o->devices[i] : i;
        if (f->devices[i] < 0 || f->devices[i] >= visible) {
            const int bad = f->devices[i];
            delete f;
            return fail(CB200_STATUS_INVALID_STREAM, "device %d not present (%d visible)", bad, visible);
        }
        for (int j = 0; j < i; ++j) {
            if (f->devices[j] == f->devices[i]) {
                delete f;
                return fail(CB200_STATUS_INVALID_ARGUMENT, "a device can hold one slot only");
            }
        }
    }
    int previous = -1;
    cudaGetDevice(&previous);
    // streams: the caller's, or one non-blocking stream per slot (discover_fleet's default)
    for (int i = 0; i < f->slot_count; ++i) {
        if (o->streams != nullptr) {
            f->streams[i] = static_cast<cudaStream_t>(o->streams[i]);
            continue;
        }
        cudaError_t err = cudaSetDevice(f->devices[i]);
        if (err == cudaSuccess) err = cudaStreamCreateWithFlags(&f->streams[i], cudaStreamNonBlocking);
        if (err != cudaSuccess) {
            if (previous >= 0) cudaSetDevice(previous);
            cb200_fleet_destroy(f);
            return fail(CB200_STATUS_CUDA_ERROR, "stream of slot %d: %s", i, cudaGetErrorString(err));
        }
        f->owns_stream[i] = true;
    }
    if (o->enable_peer_access != 0) {
        for (int i = 0; i < f->slot_count; ++i) {
            for (int j = 0; j < f->slot_count; ++j) {
                int can = 0;
                if (i == j || cudaDeviceCanAccessPeer(&can, f->devices[i], f->devices[j]) != cudaSuccess || can == 0) continue;
                if (cudaSetDevice(f->devices[i]) != cudaSuccess) continue;
                const cudaError_t err = cudaDeviceEnablePeerAccess(f->devices[j], 0);
                if (err != cudaSuccess) cudaGetLastError(); // already enabled, or not possible: NCCL finds its own path
            }
        }
    }
    // the communicator: not needed by a job of one rank; otherwise its absence is remembered, not fatal
    if (!(world == 1 && f->slot_count == 1)) {
        if (!load_nccl(o->nccl_library, &f->nccl, f->comm_error, sizeof(f->comm_error))) {
            f->comm_ready = false;
        } else {
            ncclResult_t result = ncclSuccess;
            if (o->nccl_unique_id == nullptr) {
                result = f->nccl.CommInitAll(f->comms, f->slot_count, f->devices);
            } else {
                ncclUniqueId id;
                std::memcpy(&id, o->nccl_unique_id, sizeof(id));
                result = f->nccl.GroupStart();
                for (int i = 0; i < f->slot_count && result == ncclSuccess; ++i) {
                    if (cudaSetDevice(f->devices[i]) != cudaSuccess) {
                        result = ncclUnhandledCudaError;
                        break;
                    }
                    result = f->nccl.CommInitRank(&f->comms[i], world, id, f->world_rank + i);
                }
                const ncclResult_t ended = f->nccl.GroupEnd();
                if (result == ncclSuccess) result = ended;
            }
            f->comm_ready = result == ncclSuccess;
            if (!f->comm_ready) {
                std::snprintf(f->comm_error, sizeof(f->comm_error), "NCCL communicator init: %s", f->nccl.GetErrorString(result));
                for (int i = 0; i < f->slot_count; ++i) f->comms[i] = nullptr;
            }
        }
    }
    if (previous >= 0) cudaSetDevice(previous);
    *out = f;
    return CB200_STATUS_SUCCESS;
}

void cb200_fleet_destroy(cb200_fleet *f) {
    if (f == nullptr) return;
    int previous = -1;
    cudaGetDevice(&previous);
    for (int i = 0; i < f->slot_count; ++i) {
        if (cudaSetDevice(f->devices[i]) != cudaSuccess) continue;
        if (f->comm_ready && f->comms[i] != nullptr) f->nccl.CommDestroy(f->comms[i]);
        if (f->scratch[i] != nullptr) cudaFree(f->scratch[i]);
        if (f->owns_stream[i] && f->streams[i] != nullptr) cudaStreamDestroy(f->streams[i]);
    }
    if (previous >= 0) cudaSetDevice(previous);
    // the NCCL library stays loaded: other fleets, or the process's own NCCL user, may still hold it
    delete f;
}

int32_t cb200_fleet_slot_count(const cb200_fleet *f) { return f != nullptr ? f->slot_count : 0; }
int32_t cb200_fleet_world_size(const cb200_fleet *f) { return f != nullptr ? f->world_size : 0; }
int32_t cb200_fleet_device(const cb200_fleet *f, uint32_t slot) { return slot_ok(f, slot) ? f->devices[slot] : -1; }
void *cb200_fleet_stream(const cb200_fleet *f, uint32_t slot) { return slot_ok(f, slot) ? f->streams[slot] : nullptr; }
int32_t cb200_fleet_communicator_ready(const cb200_fleet *f) {
    if (f == nullptr) return 0;
    return (f->world_size == 1 && f->slot_count == 1) || f->comm_ready ? 1 : 0;
}

cb200_status cb200_fleet_request_scratch(cb200_fleet *f, uint32_t slot, uint64_t bytes, void **scratch) {
    clear_error();
    if (!slot_ok(f, slot) || scratch == nullptr) return fail(CB200_STATUS_INVALID_ARGUMENT, "request_scratch needs a slot of the fleet and an output");
    *scratch = nullptr;
    if (bytes > f->scratch_bytes[slot]) {
        device_scope scope(f->devices[slot]);
        CB200_CUDA_OK(scope.status);
        void *grown = nullptr;
        CB200_CUDA_OK(cudaMalloc(&grown, bytes));
        if (f->scratch[slot] != nullptr) {
            // launches that still read the old block have to finish before it goes away
            CB200_CUDA_OK(cudaStreamSynchronize(f->streams[slot]));
            cudaFree(f->scratch[slot]);
        }
        f->scratch[slot] = grown;
        f->scratch_bytes[slot] = bytes;
    }
    *scratch = f->scratch[slot];
    return CB200_STATUS_SUCCESS;
}

cb200_status cb200_fleet_synchronize(cb200_fleet *f, const uint32_t *slots, uint32_t slot_count) {
    clear_error();
    const cb200_status ok = require_slots(f, slots, slot_count);
    if (ok != CB200_STATUS_SUCCESS) return ok;
    for (uint32_t i = 0; i < slot_count; ++i) {
        device_scope scope(f->devices[slots[i]]);
        CB200_CUDA_OK(scope.status);
        CB200_CUDA_OK(cudaStreamSynchronize(f->streams[slots[i]]));
    }
    return CB200_STATUS_SUCCESS;
}

cb200_status cb200_fleet_partition(int64_t rows, int32_t parts, const int64_t *row_ptr, const int64_t *packed_row_ptr,
                                   cb200_csr_block *blocks) {
    clear_error();
    if (rows < 0 || parts < 1 || row_ptr == nullptr || blocks == nullptr)
        return fail(CB200_STATUS_INVALID_ARGUMENT, "partition needs rows >= 0, parts >= 1, row_ptr and an output");
    const int64_t *packed = packed_row_ptr != nullptr ? packed_row_ptr : row_ptr;
    // the reference's rule: blocks of ceil(rows / parts) rows, the last one clipped; read back through get_block
    const int64_t per = rows == 0 ? 1 : (rows + parts - 1) / parts;
    const int64_t count = cb200_block_count_for_rows(rows, per);
    int64_t bounds[kMaxSlots * 16 + 1];
    if (parts > kMaxSlots * 16) return fail(CB200_STATUS_INVALID_ARGUMENT, "at most %d parts", kMaxSlots * 16);
    if (cb200_build_uniform_block_row_ptr(rows, per, bounds) != count) return fail(CB200_STATUS_INTERNAL_ERROR, "uniform partition failed");
    for (int32_t b = 0; b < parts; ++b) {
        if (b < count) {
            const cb200_status st = cb200_get_block(rows, row_ptr, packed, bounds, count, b, &blocks[b]);
            if (st != CB200_STATUS_SUCCESS) return st;
        } else { // rows did not fill every part: an empty shard at the end of the matrix
            blocks[b].block_index = b;
            blocks[b].row_begin = blocks[b].row_end = rows;
            blocks[b].nnz_begin = blocks[b].nnz_end = row_ptr[rows];
            blocks[b].packed_begin = blocks[b].packed_end = packed[rows];
        }
    }
    return CB200_STATUS_SUCCESS;
}

cb200_status cb200_fleet_run_forward(cb200_fleet *f, const uint32_t *slots, uint32_t slot_count, cb200_prepared *const *prepared,
                                     cb200_launch *launches) {
    clear_error();
    const cb200_status ok = require_slots(f, slots, slot_count);
    if (ok != CB200_STATUS_SUCCESS) return ok;
    if (slot_count != 0u && (prepared == nullptr || launches == nullptr))
        return fail(CB200_STATUS_INVALID_ARGUMENT, "run_forward needs one prepared operation and one launch per slot");
    for (uint32_t i = 0; i < slot_count; ++i) { // serial host loop over the slots, like the reference's
        launches[i].device = f->devices[slots[i]];
        launches[i].stream = f->streams[slots[i]];
        const cb200_status st = cb200_spmm_run(prepared[i], &launches[i]);
        if (st != CB200_STATUS_SUCCESS) return st;
    }
    return CB200_STATUS_SUCCESS;
}

cb200_status cb200_fleet_run_transpose(cb200_fleet *f, const uint32_t *slots, uint32_t slot_count, cb200_prepared *const *prepared,
                                       cb200_launch *launches) {
    clear_error();
    cb200_status st = require_slots(f, slots, slot_count);
    if (st != CB200_STATUS_SUCCESS) return st;
    if (slot_count == 0u) return CB200_STATUS_SUCCESS;
    if (prepared == nullptr || launches == nullptr)
        return fail(CB200_STATUS_INVALID_ARGUMENT, "run_transpose needs one prepared operation and one launch per slot");
    st = require_collective(f, slot_count); // before any kernel is enqueued
    if (st != CB200_STATUS_SUCCESS) return st;
    uint64_t k = 0, n = 0;
    for (uint32_t i = 0; i < slot_count; ++i) {
        uint64_t rows = 0, cols = 0;
        if (prepared[i] == nullptr || cb200_prepared_output_shape(prepared[i], &rows, &cols) != CB200_STATUS_SUCCESS)
            return fail(CB200_STATUS_INVALID_ARGUMENT, "slot %u has no prepared operation", slots[i]);
        if (i == 0) { k = rows; n = cols; }
        if (rows != k || cols != n) return fail(CB200_STATUS_INVALID_SHAPE, "the slots' partials differ in shape");
        if (launches[i].out_ld != static_cast<int64_t>(n))
            return fail(CB200_STATUS_INVALID_SHAPE, "the all-reduce takes a contiguous partial: out_ld must equal n");
    }
    for (uint32_t i = 0; i < slot_count; ++i) {
        launches[i].device = f->devices[slots[i]];
        launches[i].stream = f->streams[slots[i]];
        st = cb200_spmm_run(prepared[i], &launches[i]);
        if (st != CB200_STATUS_SUCCESS) return st;
    }
    const float *send[kMaxSlots];
    float *recv[kMaxSlots];
    for (uint32_t i = 0; i < slot_count; ++i) send[i] = recv[i] = launches[i].out;
    return grouped_allreduce(f, slots, slot_count, send, recv, k * n);
}

cb200_status cb200_fleet_allreduce_sum_f32(cb200_fleet *f, const uint32_t *slots, uint32_t slot_count, const float *const *partials,
                                           float *const *outs, uint64_t count) {
    clear_error();
    cb200_status st = require_slots(f, slots, slot_count);
    if (st != CB200_STATUS_SUCCESS) return st;
    if (slot_count == 0u || count == 0u) return CB200_STATUS_SUCCESS;
    if (partials == nullptr || outs == nullptr) return fail(CB200_STATUS_INVALID_ARGUMENT, "all-reduce needs the partials and the outputs");
    for (uint32_t i = 0; i < slot_count; ++i)
        if (partials[i] == nullptr || outs[i] == nullptr) return fail(CB200_STATUS_INVALID_ARGUMENT, "null buffer for slot %u", slots[i]);
    st = require_collective(f, slot_count);
    if (st != CB200_STATUS_SUCCESS) return st;
    return grouped_allreduce(f, slots, slot_count, partials, outs, count);
}

} // extern "C"
