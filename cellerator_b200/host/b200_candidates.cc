// Implementation of the Cellerator operation-core candidates over the cellerator_b200 C ABI.
// See b200_candidates.hh.  Everything is noexcept and reports through operation_status, like the
// rest of the operation core (operation_core.hh:133-157); messages are static strings or the
// library's thread-local last-error text.
#include "b200_candidates.hh"

#include <cmath>
#include <cstring>
#include <new>

namespace cellerator_b200::host {
namespace {

projection_catalog_entry g_catalog[projection_catalog_capacity];
std::uint32_t g_catalog_size = 0u;

const projection_catalog_entry *find_projection(ex::projection_handle handle) noexcept {
    for (std::uint32_t i = 0u; i < g_catalog_size; ++i)
        if (ex::same_handle(g_catalog[i].projection, handle)) return &g_catalog[i];
    return nullptr;
}

int dtype_of(ex::numeric_type type) noexcept { return static_cast<int>(type); } // same enum values

core::operation_status status(core::operation_status_code code, const char *message) noexcept {
    return {code, ex::binding_validation_code::ok, message};
}

bool query(int projection, const core::numeric_policy &n) noexcept {
    cb200_numeric_policy p{};
    p.version = CB200_ABI_VERSION;
    p.size = sizeof p;
    p.sparse_storage = dtype_of(n.sparse_storage);
    p.dense_storage = dtype_of(n.dense_storage);
    p.output_storage = dtype_of(n.output_storage);
    p.multiply = dtype_of(n.multiply);
    p.accumulation = dtype_of(n.accumulation);
    p.quantized = n.quantization != core::quantization_granularity::none;
    cb200_capability cap{};
    return cb200_backend_query(projection, &p, &cap) == CB200_STATUS_SUCCESS && cap.supported != 0;
}

bool bias_epilogue(int kind) noexcept { return kind == CB200_EPILOGUE_BIAS || kind >= CB200_EPILOGUE_BIAS_RELU; }

bool supports_csr(const core::numeric_policy &n) noexcept { return query(CB200_PROJECTION_CSR, n); }
bool supports_transpose(const core::numeric_policy &n) noexcept { return query(CB200_PROJECTION_TRANSPOSE, n); }
bool supports_bell(const core::numeric_policy &n) noexcept { return query(CB200_PROJECTION_BLOCKED_ELL, n); }

// What prepared.persistent.data points at: the library handle plus the arrays the binding
// contract refers to (they must outlive the prepared operation, OPERATION_CORE.md:17-25).
struct prepared_state {
    cb200_prepared *handle = nullptr;
    std::int32_t projection_kind = 0;
    std::int32_t bits = 8;
    std::int32_t decode_policy = CB200_DECODE_PER_GENE_AFFINE;
    std::int32_t epilogue = CB200_EPILOGUE_NONE;
    ex::output_update_kind update = ex::output_update_kind::overwrite;
    std::uint32_t alpha_id = ex::invalid_scalar_binding_id, beta_id = ex::invalid_scalar_binding_id;
    ex::operand_axis_contract inputs[3]{}; // X, dense, and the bias vector of a bias epilogue
    ex::operand_axis_contract outputs[1]{};
    ex::output_axis_contract orders[2]{};
    ex::output_effect_contract effects[1]{};
};

ex::operand_axis_contract axis_contract(ex::operand_kind kind, const ex::axis_identity &a,
                                        const ex::axis_identity &b) noexcept {
    ex::operand_axis_contract c{};
    c.kind = kind;
    c.rank = 2u;
    c.axes[0] = a;
    c.axes[1] = b;
    return c;
}

ex::output_axis_contract preserve_order(const ex::axis_identity &axis, std::uint8_t axis_index) noexcept {
    ex::output_axis_contract c{};
    c.input_axis = axis;
    c.output_axis = axis;
    c.transition = ex::order_transition_kind::preserve;
    c.axis_index = axis_index;
    c.operand_index = 0u;
    return c;
}

core::operation_status run(const core::prepared_operation &prepared, const ex::launch_bindings &launch) noexcept {
    // run_prepared_operation has already applied validate_launch_bindings (operation_core.cc:133-147).
    const auto *state = static_cast<const prepared_state *>(prepared.persistent.data);
    if (state == nullptr || state->handle == nullptr)
        return status(core::operation_status_code::execution_failed, "prepared operation carries no backend state");
    if (launch.value_count < 1u || launch.values[0].plane == nullptr)
        return {core::operation_status_code::invalid_launch_bindings, ex::binding_validation_code::stale_value,
                "the quantized value plane is not bound"};
    const ex::sparse_relation_view &rel = launch.inputs[0].storage.relation;
    const ex::dense_tensor_view &dense = launch.inputs[1].storage.dense;
    const ex::dense_tensor_view &out = launch.outputs[0].storage.dense;
    const ex::value_plane &plane = *launch.values[0].plane;
    if (rel.projection_data == nullptr)
        return status(core::operation_status_code::execution_failed, "sparse relation has no projection data");

    cb200_launch l{};
    l.version = CB200_ABI_VERSION;
    l.size = sizeof l;
    cb200_qcsr csr{};
    cb200_qbell bell{};
    if (state->projection_kind == CB200_PROJECTION_BLOCKED_ELL) {
        const auto *proj = static_cast<const bell_projection_data *>(rel.projection_data);
        bell.version = CB200_ABI_VERSION;
        bell.size = sizeof bell;
        bell.rows = proj->rows;
        bell.cols = proj->cols;
        bell.block_size = proj->block_size;
        bell.ell_cols = proj->ell_cols;
        bell.row_stride_bytes = proj->row_stride_bytes;
        bell.bits = state->bits;
        bell.policy = state->decode_policy;
        bell.block_col_idx = proj->block_col_idx;
        bell.packed_values = static_cast<const std::uint8_t *>(plane.values);
        bell.scales = static_cast<const float *>(plane.quantization.scales);
        bell.offsets = static_cast<const float *>(plane.quantization.offsets);
        l.bell = &bell;
    } else {
        const auto *proj = static_cast<const csr_projection_data *>(rel.projection_data);
        csr.version = CB200_ABI_VERSION;
        csr.size = sizeof csr;
        csr.rows = proj->rows;
        csr.cols = proj->cols;
        csr.nnz = proj->nnz;
        csr.bits = state->bits;
        csr.policy = state->decode_policy;
        csr.row_ptr = proj->row_ptr;
        csr.packed_row_ptr = proj->packed_row_ptr;
        csr.col_idx = proj->col_idx;
        csr.packed_values = static_cast<const std::uint8_t *>(plane.values);
        csr.scales = static_cast<const float *>(plane.quantization.scales);
        csr.offsets = static_cast<const float *>(plane.quantization.offsets);
        l.csr = &csr;
    }
    l.dense = dense.data;
    l.dense_ld = dense.stride[0];
    l.out = static_cast<float *>(out.data);
    l.out_ld = out.stride[0];
    // the output effect of the contract: overwrite (out = product), accumulate (out += product) or
    // affine_accumulate with the launch's scalars (validate_launch_bindings has checked that they are bound)
    l.alpha = 1.0f;
    l.beta = state->update == ex::output_update_kind::overwrite ? 0.0f : 1.0f;
    if (state->update == ex::output_update_kind::affine_accumulate) {
        bool have_alpha = false, have_beta = false;
        for (std::uint32_t i = 0u; i < launch.scalars.count && i < ex::maximum_scalar_bindings; ++i) {
            const ex::scalar_binding &s = launch.scalars.values[i];
            float value;
            if (s.type == ex::numeric_type::f32) {
                const std::uint32_t bits = static_cast<std::uint32_t>(s.bits);
                std::memcpy(&value, &bits, sizeof value);
            } else if (s.type == ex::numeric_type::f64) {
                double wide;
                std::memcpy(&wide, &s.bits, sizeof wide);
                value = static_cast<float>(wide);
            } else {
                continue;
            }
            if (s.binding_id == state->alpha_id) { l.alpha = value; have_alpha = true; }
            if (s.binding_id == state->beta_id) { l.beta = value; have_beta = true; }
        }
        if (!have_alpha || !have_beta)
            return {core::operation_status_code::invalid_launch_bindings, ex::binding_validation_code::ok,
                    "alpha and beta must be bound as f32 or f64 scalars"};
    }
    l.value_generation = plane.generation.value;
    l.epilogue = state->epilogue;
    if (bias_epilogue(state->epilogue)) {
        if (launch.input_count < 3u || launch.inputs[2].storage.dense.data == nullptr)
            return {core::operation_status_code::invalid_launch_bindings, ex::binding_validation_code::ok,
                    "the bias vector of the composed epilogue is not bound"};
        l.bias = static_cast<const float *>(launch.inputs[2].storage.dense.data);
    }
    l.structure_epoch = launch.structures[0].epoch.value;
    l.row_begin = 0; // the operation core binds whole operands; shards are separate structures
    l.row_end = CB200_ALL_ROWS;
    l.stream = launch.stream.stream;
    l.device = launch.stream.device_ordinal;
    l.workspace = launch.workspace.data;
    l.workspace_bytes = launch.workspace.bytes;
    l.workspace_device = launch.workspace.location.device_ordinal;
    switch (cb200_spmm_run(state->handle, &l)) {
    case CB200_STATUS_SUCCESS: return {};
    case CB200_STATUS_STALE_STRUCTURE:
        return {core::operation_status_code::stale_structure, ex::binding_validation_code::stale_structure, cb200_last_error()};
    case CB200_STATUS_INSUFFICIENT_WORKSPACE:
        return {core::operation_status_code::invalid_launch_bindings, ex::binding_validation_code::insufficient_workspace,
                cb200_last_error()};
    case CB200_STATUS_STALE_VALUE:
        return {core::operation_status_code::invalid_launch_bindings, ex::binding_validation_code::stale_value, cb200_last_error()};
    case CB200_STATUS_INVALID_STREAM:
        return {core::operation_status_code::invalid_launch_bindings, ex::binding_validation_code::invalid_stream,
                cb200_last_error()};
    default: return status(core::operation_status_code::execution_failed, cb200_last_error());
    }
}

core::operation_status prepare_any(int projection_kind, bool composed, bool ordered, const core::operation_candidate &candidate,
                                   const core::operation_problem &problem, const core::structure_set_key &structures,
                                   const core::projection_key &projection, const core::numeric_policy &numeric,
                                   const core::prepare_policy &policy, core::prepared_operation *out) noexcept {
    const projection_catalog_entry *shape = find_projection(projection.runtime);
    if (shape == nullptr || shape->projection_kind != projection_kind)
        return status(core::operation_status_code::unsupported_projection, "projection is not in the backend catalog");
    if (structures.count != 1u)
        return status(core::operation_status_code::unsupported_problem, "the quantized projections bind one structure");
    if (!composed && shape->epilogue != CB200_EPILOGUE_NONE)
        return status(core::operation_status_code::unsupported_problem,
                      "the projection composes an epilogue: prepare the composed-epilogue candidate");
    if (composed && (shape->epilogue <= CB200_EPILOGUE_NONE || shape->epilogue > CB200_EPILOGUE_BIAS_GELU_TANH))
        return status(core::operation_status_code::unsupported_problem, "the projection names no epilogue to compose");
    const bool with_bias = composed && bias_epilogue(shape->epilogue);
    if (with_bias && numeric.bias != ex::numeric_type::f32)
        return status(core::operation_status_code::unsupported_numeric_policy, "the bias vector is fp32");
    const std::uint32_t input_count = with_bias ? 3u : 2u;
    if (problem.input_count != input_count || problem.output_count != 1u)
        return status(core::operation_status_code::unsupported_problem,
                      with_bias ? "expected inputs {X, dense, bias} and one output"
                                : "expected inputs {X, dense} and one output");

    cb200_spmm_problem p{};
    p.version = CB200_ABI_VERSION;
    p.size = sizeof p;
    p.projection = projection_kind;
    p.m = shape->m;
    p.k = shape->k;
    p.n = shape->n;
    p.nnz = shape->nnz;
    p.bits = shape->bits;
    p.policy = shape->decode_policy;
    p.dense_dtype = dtype_of(numeric.dense_storage);
    p.device = shape->device;
    p.structure_epoch = structures.structures[0].epoch.value;
    // the optional length-sorted row order is persistent preprocessing: only when the policy allows it
    p.host_row_ptr = policy.allow_persistent_preprocessing ? shape->host_row_ptr : nullptr;
    // the ordered transpose always asks for the fixed order; it gathers from a gene-major copy that
    // prepare builds from the device matrix of the catalog entry
    if (ordered && shape->device_matrix == nullptr)
        return status(core::operation_status_code::unsupported_problem,
                      "the ordered transpose needs the device matrix in the projection's catalog entry");
    p.deterministic = (policy.deterministic || ordered) ? 1 : 0;
    // bf16 products (tensor-core schedules) only when the request's numeric policy says so
    p.multiply = dtype_of(numeric.multiply);
    p.device_matrix = policy.allow_persistent_preprocessing ? shape->device_matrix : nullptr;
    p.persistent_limit_bytes = policy.persistent_memory_limit;
    p.value_generation = p.device_matrix != nullptr ? shape->device_matrix_generation.value : 0u;
    // the planner's choice travels as the projection's variant; the catalog entry may pin one as well
    p.schedule_hint = projection.variant != schedule_backend_choice ? schedule_name(projection.variant) : shape->schedule_hint;
    // persistent memory the session reserved for this operation (borrowed, OPERATION_CORE.md:17-25), and its stream
    p.persistent = shape->persistent;
    p.persistent_bytes = shape->persistent_bytes;
    p.prepare_stream = shape->prepare_stream;

    auto *state = new (std::nothrow) prepared_state;
    if (state == nullptr) return status(core::operation_status_code::preparation_failed, "out of host memory");
    if (cb200_spmm_prepare(&p, &state->handle) != CB200_STATUS_SUCCESS) {
        delete state;
        return status(core::operation_status_code::preparation_failed, cb200_last_error());
    }
    state->projection_kind = projection_kind;
    state->bits = shape->bits;
    state->decode_policy = shape->decode_policy;
    state->epilogue = composed ? shape->epilogue : CB200_EPILOGUE_NONE;
    state->update = shape->output_update;
    state->alpha_id = shape->alpha_binding_id;
    state->beta_id = shape->beta_binding_id;
    const bool transpose = projection_kind == CB200_PROJECTION_TRANSPOSE;
    // forward / Blocked-ELL: X(cells, genes) . W(genes, latent) -> Y(cells, latent)
    // transpose:             X(cells, genes)^T . G(cells, latent) -> G'(genes, latent)
    state->inputs[0] = axis_contract(ex::operand_kind::sparse_relation, shape->cells, shape->genes);
    state->inputs[1] = axis_contract(ex::operand_kind::dense_tensor, transpose ? shape->cells : shape->genes, shape->latent);
    if (with_bias) {
        state->inputs[2] = {};
        state->inputs[2].kind = ex::operand_kind::dense_tensor;
        state->inputs[2].rank = 1u;
        state->inputs[2].axes[0] = shape->latent;
    }
    state->outputs[0] = axis_contract(ex::operand_kind::dense_tensor, transpose ? shape->genes : shape->cells, shape->latent);
    state->orders[0] = preserve_order(transpose ? shape->genes : shape->cells, 0u);
    state->orders[1] = preserve_order(shape->latent, 1u);
    switch (shape->output_update) {
    case ex::output_update_kind::overwrite:
        state->effects[0] = {ex::output_update_kind::overwrite, false, false, 0u, ex::invalid_scalar_binding_id,
                             ex::invalid_scalar_binding_id};
        break;
    case ex::output_update_kind::accumulate:
        state->effects[0] = {ex::output_update_kind::accumulate, true, false, 0u, ex::invalid_scalar_binding_id,
                             ex::invalid_scalar_binding_id};
        break;
    case ex::output_update_kind::affine_accumulate:
        state->effects[0] = {ex::output_update_kind::affine_accumulate, true, false, 0u, shape->alpha_binding_id,
                             shape->beta_binding_id};
        break;
    default:
        cb200_prepared_destroy(state->handle);
        delete state;
        return status(core::operation_status_code::unsupported_problem, "partial writes are addressed by row ranges, not by an output effect");
    }

    core::prepared_operation prepared{};
    prepared.problem = problem;
    prepared.structures = structures;
    prepared.projection = projection;
    prepared.numeric = numeric;
    prepared.kernel = {candidate.identity.low ^ 0x6b65726e656cull, candidate.identity.high};
    prepared.backend = core::backend_kind::native_direct;
    prepared.capability_flags = candidate.capability_flags;
    prepared.persistent = {state, sizeof(prepared_state)};
    prepared.binding_contract.structures[0] = {structures.structures[0].runtime, structures.structures[0].epoch};
    prepared.binding_contract.structure_count = 1u;
    prepared.binding_contract.inputs = state->inputs;
    prepared.binding_contract.outputs = state->outputs;
    prepared.binding_contract.output_orders = state->orders;
    prepared.binding_contract.output_effects = state->effects;
    prepared.binding_contract.input_count = input_count;
    prepared.binding_contract.output_count = 1u;
    prepared.binding_contract.output_order_count = 2u;
    prepared.binding_contract.output_effect_count = 1u;
    std::uint64_t bytes = 0u;
    std::uint32_t alignment = 256u;
    cb200_prepared_workspace(state->handle, &bytes, &alignment);
    prepared.binding_contract.workspace = {bytes, alignment, 0u};
    prepared.run = &run;
    const core::operation_status valid = core::validate_prepared_operation(prepared);
    if (!valid) {
        cb200_prepared_destroy(state->handle);
        delete state;
        return valid;
    }
    *out = prepared;
    return {};
}

core::operation_status prepare_csr(const core::operation_candidate &c, const core::operation_problem &pr,
                                   const core::structure_set_key &s, const core::projection_key &pj,
                                   const core::numeric_policy &n, const core::prepare_policy &po,
                                   core::prepared_operation *out) noexcept {
    return prepare_any(CB200_PROJECTION_CSR, false, false, c, pr, s, pj, n, po, out);
}
core::operation_status prepare_csr_epilogue(const core::operation_candidate &c, const core::operation_problem &pr,
                                            const core::structure_set_key &s, const core::projection_key &pj,
                                            const core::numeric_policy &n, const core::prepare_policy &po,
                                            core::prepared_operation *out) noexcept {
    return prepare_any(CB200_PROJECTION_CSR, true, false, c, pr, s, pj, n, po, out);
}
core::operation_status prepare_bell_epilogue(const core::operation_candidate &c, const core::operation_problem &pr,
                                             const core::structure_set_key &s, const core::projection_key &pj,
                                             const core::numeric_policy &n, const core::prepare_policy &po,
                                             core::prepared_operation *out) noexcept {
    return prepare_any(CB200_PROJECTION_BLOCKED_ELL, true, false, c, pr, s, pj, n, po, out);
}
core::operation_status prepare_transpose(const core::operation_candidate &c, const core::operation_problem &pr,
                                         const core::structure_set_key &s, const core::projection_key &pj,
                                         const core::numeric_policy &n, const core::prepare_policy &po,
                                         core::prepared_operation *out) noexcept {
    return prepare_any(CB200_PROJECTION_TRANSPOSE, false, false, c, pr, s, pj, n, po, out);
}
core::operation_status prepare_transpose_ordered(const core::operation_candidate &c, const core::operation_problem &pr,
                                                 const core::structure_set_key &s, const core::projection_key &pj,
                                                 const core::numeric_policy &n, const core::prepare_policy &po,
                                                 core::prepared_operation *out) noexcept {
    return prepare_any(CB200_PROJECTION_TRANSPOSE, false, true, c, pr, s, pj, n, po, out);
}
core::operation_status prepare_bell(const core::operation_candidate &c, const core::operation_problem &pr,
                                    const core::structure_set_key &s, const core::projection_key &pj,
                                    const core::numeric_policy &n, const core::prepare_policy &po,
                                    core::prepared_operation *out) noexcept {
    return prepare_any(CB200_PROJECTION_BLOCKED_ELL, false, false, c, pr, s, pj, n, po, out);
}

core::operation_candidate make_candidate(std::uint64_t id, const char *name, core::projection_kind projection,
                                         std::uint32_t flags, core::numeric_support_function supports,
                                         core::prepare_function prepare, std::uint64_t transient) noexcept {
    core::operation_candidate c;
    c.identity = {id, 0xb200ull};
    c.name = name;
    c.operation = core::operation_kind::sparse_dense_multiply;
    c.projection = projection;
    c.backend = core::backend_kind::native_direct;
    c.capability_flags = flags;
    c.persistent_bytes = 0u;
    c.transient_bytes = transient;
    c.supports_numeric = supports;
    c.prepare = prepare;
    return c;
}

} // namespace

bool register_projection(const projection_catalog_entry &entry) noexcept {
    if (!ex::valid_handle(entry.projection)) return false;
    for (std::uint32_t i = 0u; i < g_catalog_size; ++i)
        if (ex::same_handle(g_catalog[i].projection, entry.projection)) {
            g_catalog[i] = entry;
            return true;
        }
    if (g_catalog_size == projection_catalog_capacity) return false;
    g_catalog[g_catalog_size++] = entry;
    return true;
}

void clear_projection_catalog() noexcept { g_catalog_size = 0u; }

core::operation_candidate quantized_csr_forward_candidate() noexcept {
    // one lane group owns a row and sums in a fixed order: repeated runs are bitwise identical
    return make_candidate(0xcb200c5a00000001ull, "cb200.qcsr.forward.sm100a", core::projection_kind::csr,
                          core::candidate_deterministic | core::candidate_graph_capture, &supports_csr, &prepare_csr, 256u);
}

core::operation_candidate quantized_csr_transpose_candidate() noexcept {
    // floating-point reductions into G' in no fixed order: never deterministic
    return make_candidate(0xcb200c5a00000002ull, "cb200.qcsr.transpose.sm100a", core::projection_kind::transpose_or_backward,
                          core::candidate_graph_capture, &supports_transpose, &prepare_transpose, 0u);
}

core::operation_candidate quantized_csr_transpose_ordered_candidate() noexcept {
    // gathers gene by gene from a gene-major copy built at prepare time; the fp32 sums have a fixed
    // order, so repeated runs are bitwise identical.  The copy is persistent preprocessing.
    return make_candidate(0xcb200c5a00000006ull, "cb200.qcsr.transpose.ordered.sm100a", core::projection_kind::transpose_or_backward,
                          core::candidate_deterministic | core::candidate_graph_capture | core::candidate_persistent_preprocessing,
                          &supports_transpose, &prepare_transpose_ordered, 256u);
}

core::operation_candidate quantized_blocked_ell_candidate() noexcept {
    return make_candidate(0xcb200c5a00000003ull, "cb200.qbell.forward.sm100a", core::projection_kind::blocked_ell,
                          core::candidate_deterministic | core::candidate_graph_capture, &supports_bell, &prepare_bell, 0u);
}

core::operation_candidate quantized_csr_forward_epilogue_candidate() noexcept {
    return make_candidate(0xcb200c5a00000004ull, "cb200.qcsr.forward.epilogue.sm100a", core::projection_kind::csr,
                          core::candidate_deterministic | core::candidate_graph_capture | core::candidate_composed_epilogue,
                          &supports_csr, &prepare_csr_epilogue, 256u);
}

core::operation_candidate quantized_blocked_ell_epilogue_candidate() noexcept {
    return make_candidate(0xcb200c5a00000005ull, "cb200.qbell.forward.epilogue.sm100a", core::projection_kind::blocked_ell,
                          core::candidate_deterministic | core::candidate_graph_capture | core::candidate_composed_epilogue,
                          &supports_bell, &prepare_bell_epilogue, 0u);
}

core::operation_status register_all(core::candidate_registry *registry) noexcept {
    const core::operation_candidate all[] = {quantized_csr_forward_candidate(), quantized_csr_transpose_candidate(),
                                             quantized_blocked_ell_candidate(), quantized_csr_forward_epilogue_candidate(),
                                             quantized_blocked_ell_epilogue_candidate(),
                                             quantized_csr_transpose_ordered_candidate()};
    for (const core::operation_candidate &c : all) {
        const core::operation_status s = core::register_candidate(registry, c);
        if (!s) return s;
    }
    return {};
}

void release_prepared(core::prepared_operation *prepared) noexcept {
    if (prepared == nullptr || prepared->persistent.data == nullptr) return;
    auto *state = const_cast<prepared_state *>(static_cast<const prepared_state *>(prepared->persistent.data));
    cb200_prepared_destroy(state->handle);
    delete state;
    prepared->persistent = {};
    prepared->run = nullptr;
}

const char *prepared_schedule(const core::prepared_operation &prepared) noexcept {
    const auto *state = static_cast<const prepared_state *>(prepared.persistent.data);
    return state != nullptr && state->handle != nullptr ? cb200_prepared_schedule(state->handle) : "";
}

::cellerator::planner::planner_candidate make_planner_candidate(const core::operation_candidate &candidate,
                                                                const core::projection_key &projection,
                                                                const projection_catalog_entry &shape,
                                                                double hbm_bytes_per_ns, double roofline_fraction) noexcept {
    namespace pl = ::cellerator::planner;
    pl::planner_candidate record;
    record.identity = candidate.identity;
    record.name = candidate.name;
    record.operation = &candidate;
    record.projection = projection;
    const double dense_bytes = shape.dense_dtype == CB200_DTYPE_BF16 ? 2.0 : 4.0;
    const double m = static_cast<double>(shape.m), k = static_cast<double>(shape.k), n = static_cast<double>(shape.n);
    double bytes = static_cast<double>(shape.nnz) * (shape.bits / 8.0 + 4.0) + (m + 1.0) * 8.0 + k * 8.0;
    if (shape.projection_kind == CB200_PROJECTION_TRANSPOSE) bytes += m * n * 4.0 + k * n * 4.0;
    else if (shape.projection_kind == CB200_PROJECTION_BLOCKED_ELL)
        bytes = static_cast<double>(shape.nnz) * shape.bits / 8.0 + m * n * 4.0 + k * n * dense_bytes + k * 8.0;
    else bytes += m * n * 4.0 + k * n * dense_bytes;
    const double rate = hbm_bytes_per_ns * (roofline_fraction > 0.0 ? roofline_fraction : 1.0);
    record.analytical.kernel_ns = rate > 0.0 ? bytes / rate : 0.0;
    record.analytical.backend_prepare_ns = shape.host_row_ptr != nullptr ? 60.0 * m : 2.0e4; // row-order sort
    record.analytical.persistent_bytes = shape.host_row_ptr != nullptr ? static_cast<std::uint64_t>(shape.m) * 4u : 0u;
    record.analytical.transient_bytes = candidate.transient_bytes;
    record.flags = pl::planner_candidate_correct | pl::planner_candidate_graph_capture |
                   ((candidate.capability_flags & core::candidate_deterministic) ? pl::planner_candidate_deterministic : 0u);
    return record;
}

const char *schedule_name(std::uint32_t variant) noexcept {
    static const char *const names[schedule_variant_count] = {"", "warp_per_row", "gene_tiled", "tensor_windows", "tensor_blocked",
                                                               "tensor_dense", "vector_reductions", "gene_gather",
                                                               "tcgen05_block_rows", "cuda_cores", "tensor_codes"};
    return variant < schedule_variant_count ? names[variant] : "";
}

::cellerator::planner::planner_candidate make_schedule_candidate(const core::operation_candidate &candidate,
                                                                 const core::projection_key &projection,
                                                                 const projection_catalog_entry &shape, std::uint32_t variant,
                                                                 std::int32_t multiply, double hbm_bytes_per_ns) noexcept {
    namespace pl = ::cellerator::planner;
    const bool transpose = shape.projection_kind == CB200_PROJECTION_TRANSPOSE;
    const bool split = multiply != CB200_DTYPE_BF16;
    // Fraction of the measured HBM copy bandwidth each schedule reached on B200 on the benchmark configurations
    // (1M x 33,538 cells x genes at 5.4 % density; 500k x 4,000 at 17 % for the dense and the code tiles; 250k x 8,192 Blocked-ELL).
    double fraction = 0.05;
    switch (variant) {
    case schedule_warp_per_row: fraction = 0.05; break;
    case schedule_gene_tiled: fraction = 0.070; break;
    case schedule_tensor_windows: fraction = 0.062; break;
    case schedule_tensor_blocked:
        fraction = transpose ? (split ? 0.092 : 0.275) : (split ? (shape.dense_dtype == CB200_DTYPE_BF16 ? 0.150 : 0.100) : 0.300);
        break;
    case schedule_tensor_dense: fraction = 0.395; break;
    case schedule_tensor_codes: fraction = 0.570; break;
    case schedule_vector_reductions: fraction = 0.013; break;
    case schedule_gene_gather: fraction = 0.047; break;
    case schedule_tcgen05_block_rows: fraction = 0.267; break;
    case schedule_cuda_cores: fraction = 0.013; break;
    default: break;
    }
    pl::planner_candidate record = make_planner_candidate(candidate, projection, shape, hbm_bytes_per_ns, fraction);
    record.projection.variant = variant;
    // what prepare would keep on the device for this schedule, from the backend itself (host arithmetic only)
    cb200_spmm_problem p{};
    p.version = CB200_ABI_VERSION;
    p.size = sizeof p;
    p.projection = shape.projection_kind;
    p.m = shape.m; p.k = shape.k; p.n = shape.n; p.nnz = shape.nnz;
    p.bits = shape.bits; p.policy = shape.decode_policy; p.dense_dtype = shape.dense_dtype; p.device = shape.device;
    p.structure_epoch = 1u;
    p.host_row_ptr = shape.host_row_ptr;
    p.deterministic = variant == schedule_gene_gather ? 1 : 0;
    p.multiply = multiply;
    p.device_matrix = shape.device_matrix;
    p.schedule_hint = schedule_name(variant);
    std::uint64_t persistent = 0u;
    if (cb200_spmm_persistent_requirement(&p, &persistent) != CB200_STATUS_SUCCESS) persistent = 0u;
    record.analytical.persistent_bytes = persistent;
    // building the copies: measured 18 ms of kernels for the 7.2 GB window-blocked copy of the 1M x 33,538 matrix
    // (two passes over the matrix with an atomic per run of entries), i.e. 0.06 of the copy bandwidth per byte kept
    record.analytical.backend_prepare_ns = 2.0e4 + static_cast<double>(persistent) / (hbm_bytes_per_ns * 0.06);
    return record;
}

} // namespace cellerator_b200::host
