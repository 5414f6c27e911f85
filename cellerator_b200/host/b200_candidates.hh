// Cellerator operation-core candidates backed by libcellerator_b200.so.
//
// This header and b200_candidates.cc are the host side of the backend in the reference's own
// language and against the reference's own contracts: they compile against the Cellerator
// headers (-I<cellerator>/include) and fill core::operation_candidate records
// (include/Cellerator/compute/math/operation_core/operation_core.hh:195-207) whose
// supports_numeric / prepare / run call the C ABI of include/cellerator_b200.h.  They are what a
// Cellerator maintainer adds to the tree to register the backend; nothing in them is a copy of
// Cellerator code.
//
// The operation core passes no shapes to prepare() -- only identities -- so the binding keeps a
// small projection catalog: the owner of a structure registers, under the projection's runtime
// handle, the dimensions and axis identities of the operation; prepare() looks them up.
#pragma once

#include <Cellerator/compute/math/operation_core/operation_core.hh>
#include <Cellerator/planner/end_to_end_planner.hh>

#include <cellerator_b200.h>

#include <cstdint>

namespace cellerator_b200::host {

namespace core = ::cellerator::compute::math::core;
namespace ex = ::cellerator::execution;

// Device arrays of a quantized CSR structure: what sparse_relation_view.projection_data points at
// for the CSR and transpose projections (operands.hh:97-107).
struct csr_projection_data {
    std::int64_t rows, cols, nnz;
    const std::int64_t *row_ptr;
    const std::int64_t *packed_row_ptr; // null for 8-bit codes
    const std::int32_t *col_idx;
};

// Same for the Blocked-ELL projection.
struct bell_projection_data {
    std::int64_t rows, cols;
    std::int32_t block_size, ell_cols;
    std::int64_t row_stride_bytes;
    const std::uint32_t *block_col_idx;
};

// One catalog entry = everything prepare() needs that the operation core does not carry.
struct projection_catalog_entry {
    ex::projection_handle projection{}; // key
    std::int32_t projection_kind = 0;   // CB200_PROJECTION_*
    std::int64_t m = 0, k = 0, n = 0, nnz = 0;
    std::int32_t bits = 8;
    std::int32_t decode_policy = CB200_DECODE_PER_GENE_AFFINE;
    std::int32_t dense_dtype = CB200_DTYPE_BF16;
    std::int32_t device = 0;
    const std::int64_t *host_row_ptr = nullptr; // optional, for the row schedule
    // optional: the device-resident matrix (final contents).  With numeric_policy.multiply == bf16 and
    // prepare_policy.allow_persistent_preprocessing, prepare builds the window-blocked copy from it
    const cb200_qcsr *device_matrix = nullptr;
    // generation of the value plane whose codes, scales and offsets device_matrix points at.  A copy that
    // prepare builds from them is only valid for that generation: a launch binding another one is refused
    // as a stale value (the reference does not freeze values in prepared state, lifetimes.hh:80-81)
    ex::value_generation device_matrix_generation{};
    // optional: one schedule by name (cb200_spmm_problem.schedule_hint): how a planner that keeps one candidate
    // per schedule pins its choice; null lets prepare choose
    const char *schedule_hint = nullptr;
    // optional: persistent memory of the execution session (reserve_persistent before seal_session,
    // include/Cellerator/runtime/session.cuh:141) that prepare builds its copies in instead of allocating,
    // sized by cb200_spmm_persistent_requirement, and the stream prepare works on
    void *persistent = nullptr;
    std::uint64_t persistent_bytes = 0u;
    void *prepare_stream = nullptr;
    // how the result meets the destination (output_effect_contract, launch_bindings.hh:19-33): overwrite
    // (out = product), accumulate (out += product; the destination must be initialised) or
    // affine_accumulate (out = alpha * product + beta * out, alpha and beta bound per launch as f32 or
    // f64 scalars under these two binding ids)
    ex::output_update_kind output_update = ex::output_update_kind::overwrite;
    std::uint32_t alpha_binding_id = ex::invalid_scalar_binding_id, beta_binding_id = ex::invalid_scalar_binding_id;
    // epilogue the operation composes into the projection (cb200_epilogue; epilogue_kind of the
    // request, operation.hh:49-61).  Anything but none is served by the composed-epilogue
    // candidates only; the bias kinds bind the bias vector (latent axis, fp32) as third input.
    std::int32_t epilogue = CB200_EPILOGUE_NONE;
    ex::axis_identity cells{}, genes{}, latent{};
};

inline constexpr std::uint32_t projection_catalog_capacity = 64u;

// Returns false when the catalog is full or the handle is invalid.  Re-registering a handle
// replaces its entry.  Callers serialise mutation (the reference's registries do the same).
bool register_projection(const projection_catalog_entry &entry) noexcept;
void clear_projection_catalog() noexcept;

core::operation_candidate quantized_csr_forward_candidate() noexcept;
core::operation_candidate quantized_csr_transpose_candidate() noexcept;
core::operation_candidate quantized_blocked_ell_candidate() noexcept;
// The forward projections with the catalog entry's epilogue applied in the kernel's output stage:
// out = act(product + bias[latent]).  They carry candidate_composed_epilogue, so
// prepare_policy.allow_composed_epilogue == false rejects them (operation_core.cc:226-230).
core::operation_candidate quantized_csr_forward_epilogue_candidate() noexcept;
core::operation_candidate quantized_blocked_ell_epilogue_candidate() noexcept;

// The transpose with a fixed order of its fp32 sums (bitwise identical runs): it carries
// candidate_deterministic, so a deterministic prepare_policy selects it where the atomic-order
// transpose is rejected (operation_core.cc:210-214), and candidate_persistent_preprocessing for the
// gene-major copy it builds from the catalog entry's device matrix.
core::operation_candidate quantized_csr_transpose_ordered_candidate() noexcept;

// Registers the six candidates; returns the first failing status.
core::operation_status register_all(core::candidate_registry *registry) noexcept;

// Releases what prepare() attached to a prepared operation (the cb200_prepared handle and the
// binding-contract arrays).  The operation core has no destroy hook: the plan owner calls this.
void release_prepared(core::prepared_operation *prepared) noexcept;

// Kernel schedule the backend chose at prepare time ("gene_tiled", "tensor_blocked", ...), "" when the
// prepared operation is not one of this library's.
const char *prepared_schedule(const core::prepared_operation &prepared) noexcept;

// Kernel schedules as projection variants.  projection_key.variant (operation_core.hh:94-100) tells two physical
// forms of one projection apart, and the planner caches its winner by (candidate identity, projection identity,
// variant) (end_to_end_planner.cc find_candidate_index).  Variant 0 leaves the choice to the backend's prepare;
// the others name one schedule, which prepare() passes on as cb200_spmm_problem.schedule_hint.
enum schedule_variant : std::uint32_t {
    schedule_backend_choice = 0u,
    schedule_warp_per_row = 1u,
    schedule_gene_tiled = 2u,
    schedule_tensor_windows = 3u,
    schedule_tensor_blocked = 4u,     // forward: one bf16 pass, or split passes when fp32 products are asked for; transpose alike
    schedule_tensor_dense = 5u,
    schedule_vector_reductions = 6u,  // transpose, fp32 FMA + vector reductions
    schedule_gene_gather = 7u,        // transpose, fixed order of the sums
    schedule_tcgen05_block_rows = 8u, // Blocked-ELL
    schedule_cuda_cores = 9u,
    schedule_tensor_codes = 10u,      // forward, 4-bit codes on dense matrices: tiles of codes, decoded at launch
    schedule_variant_count = 11u
};
const char *schedule_name(std::uint32_t variant) noexcept; // "" for the backend's choice or an unknown variant

// One planner_candidate per (operation candidate, schedule): identity and operation are the candidate's, the
// projection key carries the schedule as its variant, the analytical phase costs come from the algorithmic
// bytes of the shape, the fraction of the HBM roofline the schedule was measured at on B200 (kernel_ns), the
// bytes cb200_spmm_persistent_requirement reports for it (persistent_bytes, and the prepare time of building
// them), and the workspace of the schedule (transient_bytes).  `multiply` is the request's numeric_policy.multiply
// as a cb200_dtype: it decides between the one-pass and the split-product forms of the tensor schedules.
::cellerator::planner::planner_candidate make_schedule_candidate(const core::operation_candidate &candidate,
                                                                 const core::projection_key &projection,
                                                                 const projection_catalog_entry &shape, std::uint32_t variant,
                                                                 std::int32_t multiply, double hbm_bytes_per_ns) noexcept;

// planner_candidate record (end_to_end_planner.hh:118-126) with analytical phase costs from a
// bandwidth model: kernel time = algorithmic bytes / `hbm_bytes_per_ns`, scaled by the fraction
// of the roofline the kernel reaches.
::cellerator::planner::planner_candidate make_planner_candidate(const core::operation_candidate &candidate,
                                                                const core::projection_key &projection,
                                                                const projection_catalog_entry &shape,
                                                                double hbm_bytes_per_ns,
                                                                double roofline_fraction) noexcept;

} // namespace cellerator_b200::host
